"""The optional all-gather of C slabs (NCCL + a local re-layout kernel) through the C ABI: the re-layout on a faked four-rank
buffer, the whole call on a one-rank communicator, and on two GPUs driven from this process when the box has two."""
import ctypes as C

import numpy as np
import pytest

from gpu_util import dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("elem_bytes,n_loc,pad", [(2, 1376, 0), (1, 2048, 0), (2, 344, 8), (1, 173, 3), (4, 50, 0), (2, 7, 1)])
def test_interleave_slabs_faked_four_ranks(elem_bytes, n_loc, pad):
    """[ranks][m][n_loc] -> row-major [m][ranks * n_loc (+ pad)]; shapes cover the 16-byte, 4-byte and single-byte copy paths."""
    ab = dev()
    ranks, m = 4, 301
    rng = np.random.default_rng(n_loc)
    src = rng.integers(0, 256, (ranks, m, n_loc * elem_bytes), dtype=np.uint8)
    ld = ranks * n_loc + pad
    d_src = ab.to_dev(src)
    d_dst = ab.DevBuf(m * ld * elem_bytes + 64)
    d_dst.fill(0xEE)
    ab.check(ab.lib().ascb200_interleave_slabs(d_src.ptr, d_dst.ptr, ranks, m, n_loc, ld if pad else 0, elem_bytes, None))
    ab.sync()
    got = d_dst.download(shape=(m * ld * elem_bytes + 64,), dtype=np.uint8)
    assert (got[m * ld * elem_bytes:] == 0xEE).all()
    got = got[:m * ld * elem_bytes].reshape(m, ld * elem_bytes)
    want = np.full((m, ld * elem_bytes), 0xEE, np.uint8)
    for r in range(ranks):
        want[:, r * n_loc * elem_bytes:(r + 1) * n_loc * elem_bytes] = src[r]
    assert (got == want).all()


def test_allgather_slabs_on_a_one_rank_communicator():
    ab = dev()
    comm = C.c_void_p()
    rc = ab.lib().ascb200_comm_init_all(C.byref(comm), 1, None)
    if rc == ab.EUNSUPPORTED:
        pytest.skip("no NCCL library on this box")
    ab.check(rc, "comm_init_all")
    m, n_loc = 256, 1376
    slab = np.random.default_rng(1).integers(0, 65536, (m, n_loc), dtype=np.uint16)
    d_slab, d_gath, d_full = ab.to_dev(slab), ab.empty((1, m, n_loc), np.uint16), ab.empty((m, n_loc), np.uint16)
    ab.check(ab.lib().ascb200_allgather_slabs(comm, 1, d_slab.ptr, m, n_loc, 2, d_gath.ptr, d_full.ptr, 0, None), "allgather")
    ab.sync()
    assert (d_gath.download()[0] == slab).all() and (d_full.download() == slab).all()
    ab.check(ab.lib().ascb200_comm_destroy(comm))


def test_allgather_slabs_on_two_gpus():
    """Two devices, one process: each device holds its column slab of C; after the call both hold the whole row-major C."""
    ab = dev()
    if ab.lib().ascb200_init(1) != 0:
        ab.check(ab.lib().ascb200_init(0))
        pytest.skip("one GPU visible")
    comms = (C.c_void_p * 2)()
    rc = ab.lib().ascb200_comm_init_all(comms, 2, None)
    if rc == ab.EUNSUPPORTED:
        ab.check(ab.lib().ascb200_init(0))
        pytest.skip("no NCCL library on this box")
    ab.check(rc, "comm_init_all")
    m, n_loc = 512, 688
    full = np.random.default_rng(2).integers(0, 65536, (m, 2 * n_loc), dtype=np.uint16)
    bufs = []
    try:
        _two_gpu_body(ab, comms, m, n_loc, full, bufs)
    finally:
        ab.check(ab.lib().ascb200_init(0))   # the other tests expect device 0 to be current


def _two_gpu_body(ab, comms, m, n_loc, full, bufs):
    for d in range(2):
        ab.check(ab.lib().ascb200_init(d))   # makes device d current
        bufs.append((ab.to_dev(np.ascontiguousarray(full[:, d * n_loc:(d + 1) * n_loc])), ab.empty((2, m, n_loc), np.uint16),
                     ab.empty((m, 2 * n_loc), np.uint16)))
    ab.check(ab.lib().ascb200_group_start())
    for d in range(2):
        ab.check(ab.lib().ascb200_init(d))
        slab, gath, out = bufs[d]
        # inside a group NCCL only records the call: the re-layout is issued after the group has been closed
        ab.check(ab.lib().ascb200_allgather_slabs(comms[d], 2, slab.ptr, m, n_loc, 2, gath.ptr, None, 0, None), "allgather")
    ab.check(ab.lib().ascb200_group_end())
    for d in range(2):
        ab.check(ab.lib().ascb200_init(d))
        ab.check(ab.lib().ascb200_interleave_slabs(bufs[d][1].ptr, bufs[d][2].ptr, 2, m, n_loc, 0, 2, None), "interleave")
        ab.sync()
        assert (bufs[d][2].download() == full).all(), f"device {d}"
        for b in bufs[d]:
            b.free()
        ab.check(ab.lib().ascb200_comm_destroy(comms[d]))
