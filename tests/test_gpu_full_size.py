"""The three GEMM configurations at their full baseline sizes: the oracle on sampled rows (it needs seconds, not minutes,
for a few dozen rows) plus properties that cover every output element whatever the size - an exact checksum of the int32
accumulators, exact power-of-two scaling of the block-scaled product."""
import numpy as np
import pytest

import oracle as orc
from gpu_util import dev, mx_quantize, quant_params
from sharding import dirichlet_counts

pytestmark = pytest.mark.gpu


def test_a8w8_full_size_checksum_and_sampled_rows():
    ab = dev()
    M, K, N = 4096, 4096, 11008
    rng = np.random.default_rng(0xA5C00002)
    a = rng.integers(-127, 128, (M, K), dtype=np.int8)
    b = rng.integers(-127, 128, (N, K), dtype=np.int8)
    tok = rng.uniform(1e-3, 1e-2, M).astype(np.float32)
    ch = rng.uniform(1e-3, 1e-2, N).astype(np.float32)
    d_a, d_b = ab.to_dev(a), ab.to_dev(b)
    # (1) int32 accumulators of all 45 M outputs: every row sum equals a[m,:] . colsum(b), exactly, in int64
    d_acc = ab.empty((M, N), np.int32)
    ab.check(ab.gemm(ab.KIND_S8, M, N, K, d_a, d_b, d_acc, ab.S32, trans_b=True))
    ab.sync()
    acc = d_acc.download().reshape(M, N)
    assert (acc.sum(axis=1, dtype=np.int64) == a.astype(np.int64) @ b.astype(np.int64).sum(axis=0)).all()
    assert (acc.sum(axis=0, dtype=np.int64) == b.astype(np.int64) @ a.astype(np.int64).sum(axis=0)).all()
    # (2) the timed epilogue, bit exact on sampled rows of the whole width
    rows = np.sort(rng.choice(M, 24, replace=False))
    d_c = ab.empty((M, N), np.uint16)
    ab.check(ab.gemm(ab.KIND_S8, M, N, K, d_a, d_b, d_c, ab.BF16, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=True, tok=ab.to_dev(tok),
                     ch=ab.to_dev(ch)))
    ab.sync()
    ref = orc.dequant_tok_ch(orc.gemm_i8(a[rows], b, trans_b=True), tok[rows], ch, orc.BF16)
    assert (acc[rows] == orc.gemm_i8(a[rows], b, trans_b=True)).all()
    assert (d_c.download().reshape(M, N)[rows] == ref).all()


def test_grouped_full_size_sampled_rows_of_every_group():
    ab = dev()
    G, M, K, N = 64, 32768, 7168, 2048
    counts = dirichlet_counts(G, M, seed=0xA5C00003)
    assert counts.sum() == M
    rng = np.random.default_rng(0xA5C00003)
    x = rng.integers(-127, 128, (M, K), dtype=np.int8)
    w = rng.integers(-127, 128, (G, N, K), dtype=np.int8)
    tok = rng.uniform(1e-3, 1e-2, M).astype(np.float32)
    ch = rng.uniform(1e-3, 1e-2, (G, N)).astype(np.float32)
    d_y = ab.empty((M, N), np.uint16)
    d_y.fill(0x5A)
    ab.check(ab.gemm(ab.KIND_S8, M, N, K, ab.to_dev(x), ab.to_dev(w), d_y, ab.BF16, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=True,
                     tok=ab.to_dev(tok), ch=ab.to_dev(ch), group_counts=ab.to_dev(counts), groups=G))
    ab.sync()
    y = d_y.download().reshape(M, N)
    start = np.concatenate([[0], np.cumsum(counts)])
    for g in range(G):
        if counts[g] == 0:
            continue
        rows = np.unique([start[g], start[g] + counts[g] // 2, start[g + 1] - 1])  # first, middle and last row of the group
        ref = orc.dequant_tok_ch(orc.gemm_i8(x[rows], w[g], trans_b=True), tok[rows], ch[g], orc.BF16)
        assert (y[rows] == ref).all(), f"group {g}"


def test_mxfp4_full_size_sampled_rows_and_exact_scaling():
    ab = dev()
    M = N = K = 8192
    rng = np.random.default_rng(0xA5C00004)
    a, sa = mx_quantize(rng.standard_normal((M, K), dtype=np.float32))
    b, sb = mx_quantize(rng.standard_normal((N, K), dtype=np.float32))
    d_a, d_b, d_sb = ab.to_dev(a), ab.to_dev(b), ab.to_dev(sb)
    d_c = ab.empty((M, N), np.float32)
    ab.check(ab.gemm(ab.KIND_MXFP4, M, N, K, d_a, d_b, d_c, ab.F32, trans_b=True, scale_a=ab.to_dev(sa), scale_b=d_sb))
    ab.sync()
    c = d_c.download().reshape(M, N)
    rows = np.sort(rng.choice(M, 16, replace=False))
    ref = orc.gemm_mxf4(a[rows], sa[rows], b, sb, base_k=256)
    assert np.allclose(c[rows], ref, rtol=1e-2, atol=1e-3)
    assert np.abs(c[rows] - ref).max() <= 2e-4 * np.abs(ref).max()   # both sides accumulate in fp32
    # every scale of A two exponent steps up: each product, each partial sum and so every output is exactly four times as large
    d_c4 = ab.empty((M, N), np.float32)
    ab.check(ab.gemm(ab.KIND_MXFP4, M, N, K, d_a, d_b, d_c4, ab.F32, trans_b=True, scale_a=ab.to_dev((sa + 2).astype(np.uint8)), scale_b=d_sb))
    ab.sync()
    assert (d_c4.download().reshape(M, N) == 4.0 * c).all()
    # the timed configuration's pair of outputs on the sampled rows
    q = quant_params(rng.uniform(0.5, 2.0, N).astype(np.float32) * np.float32(127.0 / (4.0 * np.abs(ref).max())))
    d_q, d_bf = ab.empty((M, N), np.int8), ab.empty((M, N), np.uint16)
    ab.check(ab.gemm(ab.KIND_MXFP4, M, N, K, d_a, d_b, d_q, ab.S8, epilogue=ab.EPI_FIXPIPE_QUANT, trans_b=True, scale_a=ab.to_dev(sa), scale_b=d_sb,
                     quant=ab.to_dev(q), c2=d_bf, c2_dtype=ab.BF16))
    ab.sync()
    got_q = d_q.download().reshape(M, N)[rows].astype(np.int32)
    ref_q = orc.fixpipe_qf322b8(c[rows], q).astype(np.int32)   # the stage applied to the GPU's own accumulators: bit exact
    assert (got_q == ref_q).all()
    assert (d_bf.download().reshape(M, N)[rows] == orc.cast_f32(c[rows], orc.BF16)).all()
