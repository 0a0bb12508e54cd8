"""ascb200_gemm_mxfp4_noalloc: the MXFP4 Matmul for hosts that cannot allocate device memory.

Such a host has given the whole GPU to its own memory pool, or sits in a loop where cudaMalloc's
device-wide synchronisation is unacceptable, so neither ascb200_init nor the scratch growth inside
ascb200_gemm is available to it.  This entry point keeps its status word and the re-tiled scale
factors in an array inside the library image instead.  The checks below go through the C ABI:
its int8 and bf16 outputs must equal ascb200_gemm's byte for byte on two calls in a row (the
second on a different shape, so it runs over whatever the first left in the shared array) and
match the CPU oracle; the largest documented problem (8192 x 8192 x 8192) must be accepted and give
ascb200_gemm's bytes; a problem whose scales do not fit the array must be refused without a
launch; the status latch must read zero after clean runs.

This file is named so that pytest collects it last.
"""
import numpy as np
import pytest

import ctypes as C

import ascb200 as ab
import oracle as orc
from gpu_util import mx_quantize, quant_params

pytestmark = pytest.mark.gpu


def _problem(m, n, k, seed):
    rng = np.random.default_rng(seed)
    a, sa = mx_quantize(rng.standard_normal((m, k)).astype(np.float32))
    b, sb = mx_quantize(rng.standard_normal((n, k)).astype(np.float32))
    q = quant_params((rng.uniform(0.5, 2.0, n) * 40.0 / np.sqrt(k)).astype(np.float32))
    return [ab.to_dev(x) for x in (a, b, sa, sb, q)] + [(a, sa, b, sb, q)]


def _run(m, n, k, bufs, noalloc):
    a, b, sa, sb, q = bufs[:5]
    c, c2 = ab.empty((m, n), np.int8), ab.empty((m, n), np.uint16)
    c.fill(0x55)
    c2.fill(0x55)
    ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, a, b, c, ab.S8, epilogue=ab.EPI_FIXPIPE_QUANT, trans_b=True, scale_a=sa, scale_b=sb,
                     quant=q, c2=c2, c2_dtype=ab.BF16, noalloc=noalloc), "mxfp4 gemm")
    ab.check(ab.lib().ascb200_stream_sync(None), "sync")
    return c.download(), c2.download()


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    shapes = [(384, 512, 1024, 5), (200, 256, 320, 6)]
    problems = [(m, n, k, _problem(m, n, k, seed)) for m, n, k, seed in shapes]
    # the allocation-free calls come first and back to back: they need no ascb200_init
    got = [_run(m, n, k, bufs, noalloc=True) for m, n, k, bufs in problems]
    st = C.c_uint32(0xFFFFFFFF)
    assert ab.lib().ascb200_noalloc_status(None, C.byref(st)) == 0 and st.value == 0   # needs no ascb200_init either
    ab.init(0)
    for (m, n, k, bufs), (q_na, bf_na) in zip(problems, got):
        q_ref, bf_ref = _run(m, n, k, bufs, noalloc=False)
        assert (q_na == q_ref).all() and (bf_na == bf_ref).all()
        assert (q_ref != 0x55).any()  # the kernel really wrote the buffers
        # and against the CPU oracle: the bf16 tensor within the GEMM tolerance, the int8 tensor at most one step away from
        # the oracle's (its accumulators differ from the tensor cores' in the last bits) and equal on nearly all elements
        a, sa, b, sb, q = bufs[5]
        acc = orc.gemm_mxf4(a, sa, b, sb, base_k=256)
        assert np.allclose(orc.bf16_bits_to_f32(bf_na), acc, rtol=1e-2, atol=1e-3)
        d = np.abs(q_na.astype(np.int32) - orc.fixpipe_qf322b8(acc, q).astype(np.int32))
        assert d.max() <= 1 and (d != 0).mean() < 2e-3


def test_noalloc_accepts_the_largest_documented_problem():
    """m = n = k = 8192: (64 + 64 + 2) blocks x 64 chunks x 512 bytes of re-tiled scales fit the array.  Operands are random
    fp4 codes and scale bytes near 127 (no quantiser run: this checks sizes and plumbing); outputs must be ascb200_gemm's."""
    m = n = k = 8192
    need = ((m + 127) // 128 + (n + 127) // 128 + 2) * 2 * ((k + 255) // 256) * 512
    assert need == 4259840
    rng = np.random.default_rng(8192)
    a = rng.integers(0, 256, (m, k // 2), dtype=np.uint8)
    b = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    sa = rng.integers(124, 131, (m, k // 32), dtype=np.uint8)
    sb = rng.integers(124, 131, (n, k // 32), dtype=np.uint8)
    bufs = [ab.to_dev(x) for x in (a, b, sa, sb)]
    outs = []
    ab.init(0)
    for noalloc in (True, False):
        c = ab.empty((m, n), np.uint16)
        c.fill(0x55)
        ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, bufs[0], bufs[1], c, ab.BF16, trans_b=True, scale_a=bufs[2], scale_b=bufs[3], noalloc=noalloc),
                 "mxfp4 gemm 8192^3")
        ab.check(ab.lib().ascb200_stream_sync(None), "sync")
        outs.append(c.download())
        c.free()
    assert (outs[0] == outs[1]).all()
    st = C.c_uint32(0)
    assert ab.lib().ascb200_noalloc_status(None, C.byref(st)) == 0 and st.value == 0


def test_noalloc_rejects_what_does_not_fit_and_other_kinds():
    m = n = 8192
    k = 16384  # scales would need 8.1 MiB of the 4.5 MiB array
    dummy = ab.DevBuf(1024)
    assert ab.gemm(ab.KIND_MXFP4, m, n, k, dummy, dummy, dummy, ab.F32, trans_b=True, scale_a=dummy, scale_b=dummy, noalloc=True) == -7
    assert ab.gemm(ab.KIND_S8, 128, 128, 128, dummy, dummy, dummy, ab.S32, trans_b=True, noalloc=True) == -3
