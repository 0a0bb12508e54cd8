"""GPU parity of SoftMax / AscendQuant / AscendDequant against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

import oracle as orc
from gpu_util import dev, f16_bits, bf16_bits

pytestmark = pytest.mark.gpu

HALF_STEP = 2.0 ** -24  # one subnormal half step


def _softmax_case(m, k, dtype, brc, seed, sigma=3.0):
    ab = dev()
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k)).astype(np.float32) * sigma
    xin = f16_bits(x) if dtype == ab.F16 else x
    d_x = ab.to_dev(xin)
    d_y = ab.empty((m, k), xin.dtype)
    rep = 8 if brc else 1
    d_sum, d_max = ab.empty((m, rep), np.float32), ab.empty((m, rep), np.float32)
    ab.check(ab.softmax(d_x, d_y, d_sum, d_max, m, k, dtype, brc), "softmax")
    ab.sync()
    y, s, mx = d_y.download(), d_sum.download(), d_max.download()
    ry, rmx, rs = orc.softmax(xin, dtype, brc=brc)
    if not brc:
        rmx, rs = rmx[:, None], rs[:, None]
    assert (mx == rmx).all()
    # the oracle adds k terms one after another in fp32; its own rounding error grows with k
    assert np.allclose(s, rs, rtol=1e-5 if k <= 4096 else 1e-4, atol=0)
    if dtype == ab.F16:
        yf, rf = orc.f16_bits_to_f32(y), orc.f16_bits_to_f32(ry)
        # north-star tolerance: 1e-3 relative; plus one subnormal half step where fp16 itself is coarser
        assert (np.abs(yf - rf) <= 1e-3 * np.abs(rf) + HALF_STEP).all()
        assert (y != ry).mean() < 0.02
    else:
        assert np.allclose(y, ry, rtol=1e-5 if k <= 4096 else 1e-4, atol=1e-30)
    return xin, y


@pytest.mark.parametrize("m,k", [(1, 16), (7, 48), (33, 256), (64, 2048), (5, 4096), (3, 16384), (2, 65536), (4096, 2048)])
def test_softmax_f16(m, k):
    _softmax_case(m, k, 1, False, seed=m * 131 + k)


@pytest.mark.parametrize("m,k", [(32, 32), (9, 8), (17, 1024), (6, 8192), (3, 32768)])
def test_softmax_f32_brc(m, k):
    _softmax_case(m, k, 0, True, seed=m * 17 + k)


def test_softmax_reference_example_edge_rows():
    """Row of FLT_MIN values (the reference example's first row) and a row with one dominant element."""
    ab = dev()
    x = np.random.default_rng(3).uniform(-1, 1, (32, 32)).astype(np.float32)
    x[0, :] = np.finfo(np.float32).min
    x[1, :] = -30.0
    x[1, 5] = 30.0
    d_x, d_y = ab.to_dev(x), ab.empty((32, 32), np.float32)
    d_s, d_m = ab.empty((32, 8), np.float32), ab.empty((32, 8), np.float32)
    ab.check(ab.softmax(d_x, d_y, d_s, d_m, 32, 32, ab.F32, True))
    ab.sync()
    ry, rm, rs = orc.softmax(x, orc.F32, brc=True)
    assert np.allclose(d_y.download(), ry, rtol=1e-5, atol=1e-30)
    assert (d_m.download() == rm).all()


def test_softmax_argument_errors():
    ab = dev()
    d = ab.empty((4, 64), np.uint16)
    s = ab.empty((4,), np.float32)
    assert ab.softmax(d, d, s, s, 4, 24, ab.F16) == -2      # 48 bytes: not a 32-byte multiple
    assert ab.softmax(None, d, s, s, 4, 64, ab.F16) == -1
    assert ab.softmax(d, d, s, s, 4, 64, ab.S8) == -3
    assert ab.softmax(d, d, s, s, 0, 64, ab.F16) == 0       # empty input


@pytest.mark.parametrize("dtype", [1, 2, 0])
@pytest.mark.parametrize("n", [32, 1024, 8 * 1000 + 32, 1 << 20])
def test_quant_per_tensor(dtype, n):
    ab = dev()
    rng = np.random.default_rng(n + dtype)
    x = rng.uniform(-4, 4, n).astype(np.float32)
    x[:8] = [0.05, -0.05, 63.55, -64.45, 1e4, -1e4, 0.3, 0.8]
    xin = f16_bits(x) if dtype == ab.F16 else bf16_bits(x) if dtype == ab.BF16 else x
    d_x, d_q = ab.to_dev(xin), ab.empty((n,), np.int8)
    ab.check(ab.quant_per_tensor(d_x, d_q, n, dtype, 2.0, 0.9))
    ab.sync()
    assert (d_q.download() == orc.quant_per_tensor(xin, dtype, 2.0, 0.9)).all()


@pytest.mark.parametrize("dtype", [1, 2, 0])
@pytest.mark.parametrize("rows,k,offset_tensor", [(4, 32, False), (37, 2048, True), (128, 96, True), (3, 40, False)])
def test_quant_per_channel(dtype, rows, k, offset_tensor):
    ab = dev()
    rng = np.random.default_rng(rows * k + dtype)
    x = rng.uniform(-1, 1, (rows, k)).astype(np.float32)
    sc = rng.uniform(30, 250, k).astype(np.float32)
    of = rng.uniform(-3, 3, k).astype(np.float32)
    conv = (lambda a: f16_bits(a)) if dtype == ab.F16 else (lambda a: bf16_bits(a)) if dtype == ab.BF16 else (lambda a: a)
    xin, scin, ofin = conv(x), conv(sc), conv(of)
    d_x, d_s, d_o, d_q = ab.to_dev(xin), ab.to_dev(scin), ab.to_dev(ofin), ab.empty((rows, k), np.int8)
    ab.check(ab.quant_per_channel(d_x, d_q, rows, k, dtype, d_s, d_o if offset_tensor else None, 0.25))
    ab.sync()
    ref = orc.quant_per_channel(xin, dtype, scin, ofin if offset_tensor else 0.25)
    assert (d_q.download() == ref).all()


@pytest.mark.parametrize("dst_dtype", [0, 1, 2])
@pytest.mark.parametrize("m,n,cal,scale_kind", [(128, 32, 32, "f32"), (33, 256, 200, "bf16"), (5, 40, 40, "scalar"), (7, 24, 10, "f32")])
def test_dequant(dst_dtype, m, n, cal, scale_kind):
    ab = dev()
    rng = np.random.default_rng(m * n + dst_dtype)
    src = rng.integers(-100000, 100000, (m, n)).astype(np.int32)
    scale = rng.uniform(-3, 3, cal).astype(np.float32)
    esz = 4 if dst_dtype == ab.F32 else 2
    n_dst = -(-n * esz // 32) * 32 // esz
    d_src = ab.to_dev(src)
    d_dst = ab.empty((m, n_dst), np.float32 if dst_dtype == ab.F32 else np.uint16)
    d_dst.fill(0)
    if scale_kind == "scalar":
        ab.check(ab.dequant(d_src, d_dst, m, n, cal, n_dst, dst_dtype, None, ab.F32, 0.37))
        ref = orc.dequant(src, 0.37, dst_dtype, cal_count=cal, n_dst=n_dst)
    elif scale_kind == "bf16":
        sb = bf16_bits(scale)
        ab.check(ab.dequant(d_src, d_dst, m, n, cal, n_dst, dst_dtype, ab.to_dev(sb), ab.BF16, 0.0))
        ref = orc.dequant(src, sb, dst_dtype, orc.BF16, cal_count=cal, n_dst=n_dst)
    else:
        ab.check(ab.dequant(d_src, d_dst, m, n, cal, n_dst, dst_dtype, ab.to_dev(scale), ab.F32, 0.0))
        ref = orc.dequant(src, scale, dst_dtype, cal_count=cal, n_dst=n_dst)
    ab.sync()
    assert (d_dst.download() == ref).all()  # one fp32 multiply and one rounding: bit exact


def test_softmax_quant_fused_full_size():
    """BASELINE config: X[4096,2048] fp16 ~ N(0, 3^2), per-channel int8 quant of the SoftMax output.

    Scales: u ~ U[0.5,2); AscendQuant multiplies by its scale, so the parity-bearing run uses the
    reciprocal of the dequant scale u/127 (127/u); the literal scale u/127 is checked to give all zeros."""
    ab = dev()
    m, k = 4096, 2048
    rng = np.random.default_rng(0xA5C00001)
    x = f16_bits(rng.standard_normal((m, k)).astype(np.float32) * 3.0)
    u = rng.uniform(0.5, 2.0, k).astype(np.float32)
    d_x = ab.to_dev(x)
    d_y, d_q = ab.empty((m, k), np.uint16), ab.empty((m, k), np.int8)
    d_s, d_m = ab.empty((m,), np.float32), ab.empty((m,), np.float32)
    for scale in (127.0 / u, u / 127.0):
        sc = f16_bits(scale)
        d_sc = ab.to_dev(sc)
        ab.check(ab.softmax_quant(d_x, d_y, d_s, d_m, d_q, d_sc, None, 0.0, m, k))
        ab.sync()
        y, q = d_y.download(), d_q.download()
        ry, rmx, rs = orc.softmax(x, orc.F16)
        yf, rf = orc.f16_bits_to_f32(y), orc.f16_bits_to_f32(ry)
        assert (np.abs(yf - rf) <= 1e-3 * np.abs(rf) + HALF_STEP).all()
        assert (d_m.download() == rmx).all() and np.allclose(d_s.download(), rs, rtol=1e-5)
        # stage-wise bit exactness: the int8 tensor is exactly AscendQuant of the fp16 tensor the kernel wrote
        assert (q == orc.quant_per_channel(y, orc.F16, sc, 0.0)).all()
        # and it agrees with the all-oracle pipeline except where the fp16 softmax value itself differs by one step
        rq = orc.quant_per_channel(ry, orc.F16, sc, 0.0)
        assert np.abs(q.astype(np.int32) - rq.astype(np.int32)).max() <= 1
        assert ((q != rq) & (y == ry)).sum() == 0
        # unfused pair gives the same bytes as the fused kernel
        d_y2, d_q2 = ab.empty((m, k), np.uint16), ab.empty((m, k), np.int8)
        ab.check(ab.softmax(d_x, d_y2, d_s, d_m, m, k, ab.F16))
        ab.check(ab.quant_per_channel(d_y2, d_q2, m, k, ab.F16, d_sc, None, 0.0))
        ab.sync()
        assert (d_y2.download() == y).all() and (d_q2.download() == q).all()
    assert (q == 0).all()  # literal scale: softmax <= 1 times <= 0.0158 rounds to zero everywhere


def _as_stored(x, dtype):
    return x.astype(np.float32) if dtype == 0 else (f16_bits(x) if dtype == 1 else bf16_bits(x))


@pytest.mark.parametrize("dst_dtype", [3, 6, 7])          # int8, fp8 e4m3, fp8 e5m2
@pytest.mark.parametrize("src_dtype,scale_dtype", [(1, 0), (2, 0), (0, 0), (1, 1), (2, 2)])
@pytest.mark.parametrize("m,n,has_offset", [(64, 256, True), (37, 200, False), (5, 33, True)])
def test_quant_per_token_policy(m, n, has_offset, src_dtype, scale_dtype, dst_dtype):
    """AscendQuant PER_TOKEN: one scale (and offset) per row; bit exact against the oracle."""
    ab = dev()
    rng = np.random.default_rng(m * n + 7 * src_dtype + dst_dtype)
    x = _as_stored(rng.standard_normal((m, n)).astype(np.float32) * 3, src_dtype)
    scale = _as_stored(rng.uniform(2.0, 40.0, m).astype(np.float32), scale_dtype)
    offset = _as_stored(rng.uniform(-8, 8, m).astype(np.float32), scale_dtype)
    d_q = ab.empty((m, n), np.uint8)
    d_q.fill(0x5A)
    ab.check(ab.quant_policy(ab.to_dev(x), d_q, m, n, src_dtype, scale_dtype, dst_dtype, ab.QUANT_PER_TOKEN, ab.to_dev(scale),
                             offset=ab.to_dev(offset) if has_offset else None, has_offset=has_offset))
    ab.sync()
    ref = orc.quant_policy(x, scale, src_dtype, scale_dtype, dst_dtype, 2, offset=offset if has_offset else None, has_offset=has_offset)
    got = d_q.download().reshape(m, n)
    assert (got == ref).all(), f"{(got != ref).sum()} of {ref.size} differ; first {np.argwhere(got != ref)[:4].tolist()}"


@pytest.mark.parametrize("round_mode", [0, 1, 2, 3, 4, 5])   # RoundMode: NONE, RINT, FLOOR, CEIL, ROUND, TRUNC
@pytest.mark.parametrize("policy,src_dtype,scale_dtype", [(2, 1, 0), (3, 0, 0), (2, 2, 2)])
def test_quant_policy_round_modes(round_mode, policy, src_dtype, scale_dtype):
    """config.roundMode of the policy AscendQuant on int8 destinations: values that land on and next to halves (also negative and
    saturating ones), bit exact against the oracle; fp8 destinations take nearest-even only."""
    ab = dev()
    m, n, group = 24, 256, 64
    rng = np.random.default_rng(round_mode * 10 + policy)
    base = rng.integers(-140, 141, (m, n)).astype(np.float32)
    frac = rng.choice(np.array([0.0, 0.25, 0.5, 0.75], np.float32), (m, n))
    x = _as_stored((base + frac) / 4.0, src_dtype)          # scale 4 puts the products on quarters
    shape = (m,) if policy == 2 else (m, n // group)
    scale = _as_stored(np.full(shape, 4.0, np.float32), scale_dtype)
    d_q = ab.empty((m, n), np.uint8)
    ab.check(ab.quant_policy(ab.to_dev(x), d_q, m, n, src_dtype, scale_dtype, ab.S8, policy, ab.to_dev(scale), k_dim=1, group_size=group if policy == 3 else 0,
                             round_mode=round_mode))
    ab.sync()
    ref = orc.quant_policy(x, scale, src_dtype, scale_dtype, orc.S8, policy, k_dim=1, group_size=group if policy == 3 else 0, round_mode=round_mode or 1)
    got = d_q.download().reshape(m, n)
    assert (got == ref).all(), f"{(got != ref).sum()} differ; first {np.argwhere(got != ref)[:4].tolist()}"
    if round_mode in (2, 3, 4, 5):
        rint = orc.quant_policy(x, scale, src_dtype, scale_dtype, orc.S8, policy, k_dim=1, group_size=group if policy == 3 else 0)
        assert (rint != ref).any()   # the mode really changes results on this data
        assert ab.quant_policy(ab.to_dev(x), d_q, m, n, src_dtype, scale_dtype, ab.FP8_E4M3, policy, ab.to_dev(scale), k_dim=1,
                               group_size=group if policy == 3 else 0, round_mode=round_mode) == ab.EUNSUPPORTED
    assert ab.quant_policy(ab.to_dev(x), d_q, m, n, src_dtype, scale_dtype, ab.S8, policy, ab.to_dev(scale), k_dim=1,
                           group_size=group if policy == 3 else 0, round_mode=6) == ab.EUNSUPPORTED


@pytest.mark.parametrize("dst_dtype", [3, 6, 5])          # int8, fp8 e4m3, packed fp4 e2m1
@pytest.mark.parametrize("src_dtype,scale_dtype", [(1, 0), (2, 0), (0, 0), (1, 1)])
@pytest.mark.parametrize("m,n,group,k_dim", [(48, 256, 32, 1), (40, 320, 64, 1), (70, 96, 32, 0), (9, 250, 128, 1)])
def test_quant_per_group_policy(m, n, group, k_dim, src_dtype, scale_dtype, dst_dtype):
    """AscendQuant PER_GROUP along columns (kDim = 1) or rows (kDim = 0), incl. the fp4 destination that feeds block-scaled GEMMs."""
    ab = dev()
    rng = np.random.default_rng(m + n + group + 3 * src_dtype + dst_dtype)
    x = _as_stored(rng.standard_normal((m, n)).astype(np.float32), src_dtype)
    sshape = (m, -(-n // group)) if k_dim == 1 else (-(-m // group), n)
    amp = 1.5 if dst_dtype == 5 else 30.0
    scale = _as_stored(rng.uniform(0.5 * amp, amp, sshape).astype(np.float32), scale_dtype)
    has_offset = dst_dtype != 5
    d_q = ab.empty((m, n // 2) if dst_dtype == 5 else (m, n), np.uint8)
    ab.check(ab.quant_policy(ab.to_dev(x), d_q, m, n, src_dtype, scale_dtype, dst_dtype, ab.QUANT_PER_GROUP, ab.to_dev(scale), k_dim=k_dim,
                             group_size=group, offset_scalar=1.5, has_offset=has_offset))
    ab.sync()
    ref = orc.quant_policy(x, scale, src_dtype, scale_dtype, dst_dtype, 3, k_dim=k_dim, group_size=group, offset_scalar=1.5, has_offset=has_offset)
    got = d_q.download().reshape(ref.shape)
    assert (got == ref).all(), f"{(got != ref).sum()} of {ref.size} differ; first {np.argwhere(got != ref)[:4].tolist()}"


def test_quant_policy_argument_errors():
    ab = dev()
    x = ab.to_dev(np.zeros((4, 64), np.float32))
    s = ab.to_dev(np.ones(4, np.float32))
    q = ab.empty((4, 64), np.uint8)
    assert ab.quant_policy(x, q, 4, 64, ab.F32, ab.F32, ab.S8, 1, s) == ab.EUNSUPPORTED                      # PER_CHANNEL has its own entry point
    assert ab.quant_policy(x, q, 4, 64, ab.F32, ab.F32, ab.S8, ab.QUANT_PER_GROUP, s, group_size=48) == ab.EINVAL  # groups are multiples of 32
    assert ab.quant_policy(x, q, 4, 64, ab.F32, ab.F32, ab.FP4, ab.QUANT_PER_TOKEN, s) == ab.EUNSUPPORTED   # fp4 only per group
    assert ab.quant_policy(x, q, 4, 64, ab.F32, ab.F16, ab.S8, ab.QUANT_PER_TOKEN, s) == ab.EUNSUPPORTED    # 16-bit scale needs the same source type


@pytest.mark.parametrize("dst_dtype", [0, 1, 2])
@pytest.mark.parametrize("src_f32,scale_dtype", [(False, 0), (False, 2), (True, 1), (True, 0)])
@pytest.mark.parametrize("m,n,policy,group,k_dim", [(33, 256, 0, 0, 1), (48, 320, 1, 64, 1), (70, 96, 1, 32, 0), (5, 33, 0, 0, 1)])
def test_dequant_policies(m, n, policy, group, k_dim, src_f32, scale_dtype, dst_dtype):
    """AscendDequant PER_TOKEN / PER_GROUP: float(src) * float(scale), one rounding to the destination type; bit exact."""
    ab = dev()
    rng = np.random.default_rng(m * 31 + n + policy + scale_dtype + dst_dtype)
    src = (rng.standard_normal((m, n)) * 1000).astype(np.float32) if src_f32 else rng.integers(-2**20, 2**20, (m, n)).astype(np.int32)
    sshape = (m,) if policy == 0 else ((m, -(-n // group)) if k_dim == 1 else (-(-m // group), n))
    scale = _as_stored(rng.uniform(1e-3, 1e-2, sshape).astype(np.float32), scale_dtype)
    out_np = np.float32 if dst_dtype == 0 else np.uint16
    d_out = ab.empty((m, n), out_np)
    ab.check(ab.dequant_policy(ab.to_dev(src), d_out, m, n, ab.F32 if src_f32 else ab.S32, scale_dtype, dst_dtype, policy, ab.to_dev(scale),
                               k_dim=k_dim, group_size=group))
    ab.sync()
    ref = orc.dequant_policy(src, scale, scale_dtype, dst_dtype, policy, k_dim=k_dim, group_size=group)
    got = d_out.download().reshape(m, n)
    assert (got.view(np.uint32 if dst_dtype == 0 else np.uint16) == ref.view(np.uint32 if dst_dtype == 0 else np.uint16)).all()


def _to_f32(a, dtype):
    return a.astype(np.float32) if dtype == 0 else orc.f16_bits_to_f32(a)


@pytest.mark.parametrize("dtype,stats_dtype", [(1, 0), (1, 1), (0, 0)])
@pytest.mark.parametrize("m,k,brc", [(64, 128, True), (37, 2048, True), (8, 4096, False), (3, 16, True)])
def test_softmax_flash_v2_two_steps(m, k, brc, dtype, stats_dtype):
    """Two SoftmaxFlashV2 steps over two K tiles (first without, then with update) against the oracle, and the online-softmax
    identity: sum_2 equals the sum of exp(x - max_2) over both tiles."""
    ab = dev()
    rng = np.random.default_rng(m + k + dtype * 3 + stats_dtype)
    x1 = (rng.standard_normal((m, k)) * 2).astype(np.float32)
    x2 = (rng.standard_normal((m, k)) * 2 + 1).astype(np.float32)
    s1, s2 = _as_stored(x1, dtype), _as_stored(x2, dtype)
    srep = (32 // (2 if stats_dtype == 1 else 4)) if brc else 1
    erep = (32 // (2 if dtype == 1 else 4)) if brc else 1
    np_d, np_s = (np.float32 if dtype == 0 else np.uint16), (np.float32 if stats_dtype == 0 else np.uint16)
    d_y, d_sum, d_max, d_em = ab.empty((m, k), np_d), ab.empty((m, srep), np_s), ab.empty((m, srep), np_s), ab.empty((m, erep), np_d)
    ab.check(ab.softmax_flash_v2(ab.to_dev(s1), d_y, d_sum, d_max, None, None, None, m, k, dtype, stats_dtype, False, brc))
    ab.sync()
    y_r, sum_r, max_r, _ = orc.softmax_flash_v2(s1, dtype, stats_dtype, brc=brc)
    sum1, max1 = d_sum.download().reshape(m, srep), d_max.download().reshape(m, srep)
    assert (max1 == max_r).all()
    assert np.allclose(_to_f32(sum1, stats_dtype), _to_f32(sum_r, stats_dtype), rtol=2e-3)
    assert np.allclose(_to_f32(d_y.download().reshape(m, k), dtype), _to_f32(y_r, dtype), rtol=1e-3, atol=1e-6)
    # second tile, update: the inputs are the first step's device outputs
    d_sum2, d_max2 = ab.empty((m, srep), np_s), ab.empty((m, srep), np_s)
    ab.check(ab.softmax_flash_v2(ab.to_dev(s2), d_y, d_sum2, d_max2, d_em, d_sum, d_max, m, k, dtype, stats_dtype, True, brc))
    ab.sync()
    y2_r, sum2_r, max2_r, em_r = orc.softmax_flash_v2(s2, dtype, stats_dtype, in_sum=sum1, in_max=max1, brc=brc)
    sum2, max2 = d_sum2.download().reshape(m, srep), d_max2.download().reshape(m, srep)
    assert (max2 == max2_r).all()
    assert np.allclose(_to_f32(sum2, stats_dtype), _to_f32(sum2_r, stats_dtype), rtol=2e-3)
    assert np.allclose(_to_f32(d_em.download().reshape(m, erep), dtype), _to_f32(em_r, dtype), rtol=2e-3, atol=1e-6)
    assert np.allclose(_to_f32(d_y.download().reshape(m, k), dtype), _to_f32(y2_r, dtype), rtol=1e-3, atol=1e-6)
    both = np.concatenate([_to_f32(s1, dtype), _to_f32(s2, dtype)], axis=1).astype(np.float64)
    ident = np.exp(both - _to_f32(max2, stats_dtype)[:, :1].astype(np.float64)).sum(axis=1)
    assert np.allclose(_to_f32(sum2, stats_dtype)[:, 0], ident, rtol=4e-3 if stats_dtype == 1 else 1e-3)


@pytest.mark.parametrize("dtype", [1, 0])
@pytest.mark.parametrize("m,k,brc", [(1, 16, True), (37, 2048, True), (64, 4096, False), (5, 16384, True), (2, 32768, True), (4096, 2048, True),
                                     (300, 64, False)])
def test_log_softmax(m, k, brc, dtype):
    """LogSoftMax against the oracle: max bit exact, sum and y within 1e-3; statistics in the source dtype."""
    ab = dev()
    rng = np.random.default_rng(m * 7 + k + dtype)
    x = (rng.standard_normal((m, k)) * 3).astype(np.float32)
    xin = _as_stored(x, dtype)
    rep = (16 if dtype == 1 else 8) if brc else 1
    d_y, d_sum, d_max = ab.empty((m, k), xin.dtype), ab.empty((m, rep), xin.dtype), ab.empty((m, rep), xin.dtype)
    ab.check(ab.log_softmax(ab.to_dev(xin), d_y, d_sum, d_max, m, k, dtype, brc), "log_softmax")
    ab.sync()
    ry, rmx, rs = orc.log_softmax(xin, dtype, brc=brc)
    y, s, mx = d_y.download().reshape(m, k), d_sum.download().reshape(m, rep), d_max.download().reshape(m, rep)
    assert (mx == rmx.reshape(m, rep)).all()
    assert np.allclose(_to_f32(s, dtype), _to_f32(rs.reshape(m, rep), dtype), rtol=2e-3 if dtype == 1 else 1e-4)
    yf, rf = _to_f32(y, dtype), _to_f32(ry, dtype)
    assert (np.abs(yf - rf) <= 1e-3 * np.abs(rf) + (2e-3 if dtype == 1 else 1e-5)).all()
    # against the reference's golden formula (log10 of the softmax) in float64
    xs = _to_f32(xin, dtype).astype(np.float64)
    e = np.exp(xs - xs.max(axis=1, keepdims=True))
    gold = np.log10(e / e.sum(axis=1, keepdims=True))
    assert (np.abs(yf - gold) <= 1e-3 * np.abs(gold) + (4e-3 if dtype == 1 else 1e-4)).all()


def test_log_softmax_underflow_and_errors():
    """Entries far below the row maximum underflow exp() to 0 and give -inf like the reference's ln(0); argument checks as SoftMax."""
    ab = dev()
    x = np.zeros((4, 64), np.float32)
    x[:, 0] = 200.0
    d_y, d_s, d_m = ab.empty((4, 64), np.float32), ab.empty((4, 8), np.float32), ab.empty((4, 8), np.float32)
    ab.check(ab.log_softmax(ab.to_dev(x), d_y, d_s, d_m, 4, 64, 0, True))
    ab.sync()
    y = d_y.download().reshape(4, 64)
    assert (y[:, 0] == 0).all() and np.isneginf(y[:, 1:]).all()
    assert (d_s.download() == 1).all() and (d_m.download() == 200).all()
    assert ab.log_softmax(ab.to_dev(x), d_y, d_s, d_m, 4, 60, 0, True) == ab.EALIGN      # 60 floats: not whole 32-byte blocks
    assert ab.log_softmax(ab.to_dev(x), d_y, d_s, d_m, 4, 64, 2, True) == ab.EUNSUPPORTED  # bf16 is not a LogSoftMax type
    assert ab.log_softmax(None, d_y, d_s, d_m, 4, 64, 0, True) == ab.EINVAL
    assert ab.log_softmax(ab.to_dev(x), d_y, d_s, d_m, 0, 64, 0, True) == 0


@pytest.mark.parametrize("dtype,stats_dtype", [(1, 0), (1, 1), (0, 0)])
@pytest.mark.parametrize("m,k,brc", [(1, 16, True), (37, 2048, True), (64, 4096, False), (3, 32768, True), (4096, 2048, True), (301, 80, False)])
def test_simple_softmax(m, k, brc, dtype, stats_dtype):
    """SimpleSoftMax with the statistics of a SoftMax over the same rows: equals the oracle within 1e-3 and reproduces SoftMax itself."""
    ab = dev()
    rng = np.random.default_rng(m * 3 + k + dtype + stats_dtype)
    x = (rng.standard_normal((m, k)) * 3).astype(np.float32)
    xin = _as_stored(x, dtype)
    xf = _to_f32(xin, dtype)
    mx = xf.max(axis=1)
    sm = np.exp(xf - mx[:, None]).sum(axis=1, dtype=np.float64).astype(np.float32)
    rep = (16 if stats_dtype == 1 else 8) if brc else 1
    mx_s, sm_s = _as_stored(np.repeat(mx[:, None], rep, 1), stats_dtype), _as_stored(np.repeat(sm[:, None], rep, 1), stats_dtype)
    d_y = ab.empty((m, k), xin.dtype)
    ab.check(ab.simple_softmax(ab.to_dev(xin), d_y, ab.to_dev(sm_s), ab.to_dev(mx_s), m, k, dtype, stats_dtype, brc), "simple_softmax")
    ab.sync()
    y = _to_f32(d_y.download().reshape(m, k), dtype)
    ref = _to_f32(orc.simple_softmax(xin, sm_s, mx_s, dtype, stats_dtype), dtype)
    assert (np.abs(y - ref) <= 1e-3 * np.abs(ref) + (HALF_STEP if dtype == 1 else 1e-30)).all()
    if stats_dtype == 0:  # exact statistics: the two-pass result is the softmax
        gold = np.exp(xf.astype(np.float64) - mx[:, None]) / sm[:, None].astype(np.float64)
        assert (np.abs(y - gold) <= 1e-3 * gold + (HALF_STEP if dtype == 1 else 1e-30)).all()


def test_simple_softmax_argument_errors():
    ab = dev()
    x, y, st = ab.empty((4, 64), np.float32), ab.empty((4, 64), np.float32), ab.empty((4, 8), np.float32)
    assert ab.simple_softmax(x, y, st, st, 0, 64, ab.F32, ab.F32) == 0
    assert ab.simple_softmax(x, y, None, st, 4, 64, ab.F32, ab.F32) == ab.EINVAL
    assert ab.simple_softmax(x, y, st, st, 4, 60, ab.F32, ab.F32) == ab.EALIGN
    assert ab.simple_softmax(x, y, st, st, 4, 64, ab.F32, ab.F16) == ab.EUNSUPPORTED   # half statistics beside float data: no such overload
    assert ab.simple_softmax(x, y, st, st, 4, 64, ab.BF16, ab.F32) == ab.EUNSUPPORTED


@pytest.mark.parametrize("dtype", [1, 0])
@pytest.mark.parametrize("front", [False, True])
@pytest.mark.parametrize("m,k", [(1, 16), (37, 2048), (64, 4096), (5, 16384), (2, 32768), (4096, 2048), (301, 960)])
def test_softmax_grad(m, k, front, dtype):
    """SoftmaxGrad / SoftmaxGradFront against the oracle: the row sum within fp32 reordering, the output within 1e-3."""
    ab = dev()
    rng = np.random.default_rng(m * 5 + k + dtype)
    grad = _as_stored(rng.uniform(-1, 1, (m, k)).astype(np.float32), dtype)
    x = rng.standard_normal((m, k)) * 2
    y = np.exp(x - x.max(axis=1, keepdims=True))
    src = _as_stored((y / y.sum(axis=1, keepdims=True)).astype(np.float32), dtype)   # a softmax output, as in a backward pass
    rep = 16 if dtype == 1 else 8
    d_out = ab.empty((m, rep) if front else (m, k), grad.dtype)
    ab.check(ab.softmax_grad(ab.to_dev(grad), ab.to_dev(src), d_out, m, k, dtype, front), "softmax_grad")
    ab.sync()
    got = _to_f32(d_out.download().reshape(m, -1), dtype)
    ref = _to_f32(orc.softmax_grad(grad, src, dtype, front=front), dtype)
    scale = np.abs(_to_f32(grad, dtype)).max() * np.abs(_to_f32(src, dtype)).max(axis=1, keepdims=True)
    tol = 1e-3 * np.abs(ref) + (1e-3 if dtype == 1 else 1e-5) * (1.0 if front else scale) + (HALF_STEP if dtype == 1 else 0)
    assert (np.abs(got - ref) <= tol).all()
    if front:
        assert (got == got[:, :1]).all()


def test_softmax_grad_argument_errors():
    ab = dev()
    g, y, o = ab.empty((4, 64), np.float32), ab.empty((4, 64), np.float32), ab.empty((4, 64), np.float32)
    assert ab.softmax_grad(g, y, o, 0, 64, ab.F32) == 0
    assert ab.softmax_grad(g, None, o, 4, 64, ab.F32) == ab.EINVAL
    assert ab.softmax_grad(g, y, o, 4, 60, ab.F32) == ab.EALIGN
    assert ab.softmax_grad(g, y, o, 4, 64, ab.BF16) == ab.EUNSUPPORTED
    assert ab.softmax_grad(g, y, o, 4, 1 << 20, ab.F32) == ab.ETOOBIG


@pytest.mark.parametrize("dtype,stats_dtype", [(1, 0), (1, 1), (0, 0)])
@pytest.mark.parametrize("m,k,brc", [(64, 128, True), (37, 2048, True), (8, 4096, False), (3, 16, True)])
def test_softmax_flash_first_version_two_steps(m, k, brc, dtype, stats_dtype):
    """SoftmaxFlash (the normalising first version): both steps against the oracle, and the identity that tile 1 rescaled by expMax
    next to tile 2 is the softmax of the whole row."""
    ab = dev()
    rng = np.random.default_rng(m + k + dtype * 5 + stats_dtype)
    x1 = (rng.standard_normal((m, k)) * 2).astype(np.float32)
    x2 = (rng.standard_normal((m, k)) * 2 + 1).astype(np.float32)
    s1, s2 = _as_stored(x1, dtype), _as_stored(x2, dtype)
    srep = (32 // (2 if stats_dtype == 1 else 4)) if brc else 1
    erep = (32 // (2 if dtype == 1 else 4)) if brc else 1
    np_d, np_s = (np.float32 if dtype == 0 else np.uint16), (np.float32 if stats_dtype == 0 else np.uint16)
    d_y1, d_sum, d_max, d_em = ab.empty((m, k), np_d), ab.empty((m, srep), np_s), ab.empty((m, srep), np_s), ab.empty((m, erep), np_d)
    ab.check(ab.softmax_flash(ab.to_dev(s1), d_y1, d_sum, d_max, None, None, None, m, k, dtype, stats_dtype, False, brc))
    ab.sync()
    y_r, sum_r, max_r, _ = orc.softmax_flash(s1, dtype, stats_dtype, brc=brc)
    sum1, max1 = d_sum.download().reshape(m, srep), d_max.download().reshape(m, srep)
    y1 = _to_f32(d_y1.download().reshape(m, k), dtype)
    assert (max1 == max_r).all()
    assert np.allclose(_to_f32(sum1, stats_dtype), _to_f32(sum_r, stats_dtype), rtol=2e-3)
    assert (np.abs(y1 - _to_f32(y_r, dtype)) <= 1e-3 * _to_f32(y_r, dtype) + (HALF_STEP if dtype == 1 else 1e-30)).all()
    d_y2, d_sum2, d_max2 = ab.empty((m, k), np_d), ab.empty((m, srep), np_s), ab.empty((m, srep), np_s)
    ab.check(ab.softmax_flash(ab.to_dev(s2), d_y2, d_sum2, d_max2, d_em, d_sum, d_max, m, k, dtype, stats_dtype, True, brc))
    ab.sync()
    y2_r, sum2_r, max2_r, em_r = orc.softmax_flash(s2, dtype, stats_dtype, in_sum=sum1, in_max=max1, brc=brc)
    y2, em = _to_f32(d_y2.download().reshape(m, k), dtype), _to_f32(d_em.download().reshape(m, erep), dtype)
    assert (d_max2.download().reshape(m, srep) == max2_r).all()
    assert np.allclose(_to_f32(d_sum2.download().reshape(m, srep), stats_dtype), _to_f32(sum2_r, stats_dtype), rtol=2e-3)
    assert np.allclose(em, _to_f32(em_r, dtype), rtol=3e-3, atol=1e-6)
    assert (np.abs(y2 - _to_f32(y2_r, dtype)) <= 2e-3 * _to_f32(y2_r, dtype) + (HALF_STEP if dtype == 1 else 1e-30)).all()
    both = np.concatenate([_to_f32(s1, dtype), _to_f32(s2, dtype)], axis=1).astype(np.float64)
    e = np.exp(both - both.max(axis=1, keepdims=True))
    whole = e / e.sum(axis=1, keepdims=True)
    got = np.concatenate([y1 * em[:, :1], y2], axis=1)
    rt = 1.2e-2 if stats_dtype == 1 else (6e-3 if dtype == 1 else 1e-4)   # half statistics carry 2^-11 each
    assert (np.abs(got - whole) <= rt * whole + (2 * HALF_STEP if dtype == 1 else 1e-12)).all()


@pytest.mark.parametrize("dst_dtype", [1, 2])
@pytest.mark.parametrize("mode,with_offset", [(0, True), (1, True), (1, False), (2, True), (2, False)])
@pytest.mark.parametrize("rows,cols", [(8, 128), (37, 2048), (300, 96), (1, 32)])
def test_antiquant(rows, cols, mode, with_offset, dst_dtype):
    """AscendAntiQuant int8 -> half / bfloat16: bit exact against the oracle in every mode (the arithmetic type is part of the contract)."""
    ab = dev()
    rng = np.random.default_rng(rows + cols * 3 + mode * 7 + dst_dtype)
    src = rng.integers(-128, 128, (rows, cols), dtype=np.int8)
    npar = cols if mode == 1 else rows
    sc = _as_stored(rng.uniform(-4, 4, npar).astype(np.float32), dst_dtype)
    of = _as_stored(rng.uniform(-10, 10, npar).astype(np.float32), dst_dtype)
    d_out = ab.empty((rows, cols), np.uint16)
    kw = dict(scale_scalar=0.37, offset_scalar=-2.25 if with_offset else 0.0)
    if mode == 0:
        ab.check(ab.antiquant(ab.to_dev(src), d_out, rows, cols, dst_dtype, 0, **kw))
        ref = orc.antiquant(src, dst_dtype, 0, **kw)
    else:
        ab.check(ab.antiquant(ab.to_dev(src), d_out, rows, cols, dst_dtype, mode, ab.to_dev(sc), ab.to_dev(of) if with_offset else None))
        ref = orc.antiquant(src, dst_dtype, mode, scale=sc, offset=of if with_offset else None)
    ab.sync()
    got = d_out.download().reshape(rows, cols)
    assert (got == ref).all(), f"{(got != ref).sum()} of {got.size} differ"


def test_antiquant_argument_errors():
    ab = dev()
    s, d, p = ab.empty((4, 64), np.int8), ab.empty((4, 64), np.uint16), ab.empty((64,), np.uint16)
    assert ab.antiquant(s, d, 0, 64, ab.F16, 0) == 0
    assert ab.antiquant(s, d, 4, 48, ab.F16, 0) == ab.EALIGN          # rows are whole 32-byte blocks
    assert ab.antiquant(s, d, 4, 64, ab.F32, 0) == ab.EUNSUPPORTED    # half / bfloat16 outputs only
    assert ab.antiquant(s, d, 4, 64, ab.F16, 1) == ab.EINVAL          # per channel needs the scale tensor
    assert ab.antiquant(s, d, 4, 64, ab.F16, 3, p) == ab.EINVAL


def test_new_entry_points_edge_cases():
    """Zero extents succeed without touching memory; bad extents, types and alignments are refused with the documented codes."""
    ab = dev()
    x = ab.to_dev(np.zeros((4, 64), np.float32))
    s = ab.to_dev(np.ones(4, np.float32))
    q = ab.empty((4, 64), np.uint8)
    assert ab.quant_policy(x, q, 0, 64, ab.F32, ab.F32, ab.S8, ab.QUANT_PER_TOKEN, s) == 0
    assert ab.quant_policy(x, q, 4, 0, ab.F32, ab.F32, ab.S8, ab.QUANT_PER_TOKEN, s) == 0
    assert ab.quant_policy(None, q, 4, 64, ab.F32, ab.F32, ab.S8, ab.QUANT_PER_TOKEN, s) == ab.EINVAL
    assert ab.dequant_policy(x, q, 0, 64, ab.F32, ab.F32, ab.F32, ab.DEQUANT_PER_TOKEN, s) == 0
    assert ab.dequant_policy(x, q, 4, 64, ab.F16, ab.F32, ab.F32, ab.DEQUANT_PER_TOKEN, s) == ab.EUNSUPPORTED   # source is int32 or fp32
    assert ab.dequant_policy(x, q, 4, 64, ab.F32, ab.F32, ab.F32, 2, s) == ab.EUNSUPPORTED                     # PER_CHANNEL_PER_GROUP
    assert ab.dequant_policy(x, q, 4, 64, ab.F32, ab.F32, ab.F32, ab.DEQUANT_PER_GROUP, s, group_size=0) == ab.EINVAL
    st = ab.empty((4, 8), np.float32)
    y = ab.empty((4, 64), np.float32)
    assert ab.softmax_flash_v2(x, y, st, st, None, None, None, 0, 64, ab.F32, ab.F32, False, True) == 0
    assert ab.softmax_flash_v2(x, y, st, st, None, None, None, 4, 64, ab.F32, ab.F32, True, True) == ab.EINVAL       # update needs the previous statistics
    assert ab.softmax_flash_v2(x, y, st, st, None, None, None, 4, 64, ab.F32, ab.F16, False, True) == ab.EUNSUPPORTED
    assert ab.softmax_flash_v2(x, y, st, st, None, None, None, 4, 60, ab.F32, ab.F32, False, True) == ab.EALIGN       # rows are multiples of 32 bytes
    w = ab.empty((1, 64, 32), np.int8)
    assert ab.nz_unpack(w, w, 0, 64, 32, 1, True) == 0
    assert ab.nz_unpack(w, w, 1, 60, 32, 1, True) == ab.EINVAL      # whole fractal blocks only
    assert ab.nz_unpack(w, w, 1, 64, 32, 4, True) == ab.EUNSUPPORTED
    ab.sync()


def _guarded(ab, nbytes):
    buf = ab.DevBuf(nbytes + 512)
    buf.fill(0x5A)
    return buf


def test_row_kernels_write_nothing_past_their_outputs():
    """Outputs sized exactly, followed by a guard area: ragged extents must not spill over the end of any destination."""
    ab = dev()
    rng = np.random.default_rng(11)

    def tail_intact(buf, used):
        host = np.zeros(buf.nbytes, np.uint8)
        ab.check(ab.lib().ascb200_memcpy_d2h(host.ctypes.data, buf.ptr, buf.nbytes, None))
        ab.sync()
        return bool((host[used:] == 0x5A).all())

    for m, n, dst, policy, group in [(37, 200, ab.S8, ab.QUANT_PER_TOKEN, 0), (5, 250, ab.FP4, ab.QUANT_PER_GROUP, 32), (9, 264, ab.FP8_E4M3, ab.QUANT_PER_GROUP, 64),
                                     (1029, 32, ab.S8, ab.QUANT_PER_TOKEN, 0)]:
        x = ab.to_dev(f16_bits(rng.standard_normal((m, n)).astype(np.float32)))
        sshape = (m,) if policy == ab.QUANT_PER_TOKEN else (m, -(-n // group))
        s = ab.to_dev(np.ones(sshape, np.float32))
        used = m * n // 2 if dst == ab.FP4 else m * n
        q = _guarded(ab, used)
        ab.check(ab.quant_policy(x, q, m, n, ab.F16, ab.F32, dst, policy, s, k_dim=1, group_size=group))
        ab.sync()
        assert tail_intact(q, used), ("quant_policy", m, n)
    for m, n, dst_dtype, esz in [(33, 200, ab.BF16, 2), (7, 24, ab.F32, 4), (5, 33, ab.F16, 2)]:
        src = ab.to_dev(rng.integers(-1000, 1000, (m, n)).astype(np.int32))
        s = ab.to_dev(np.ones(m, np.float32))
        out = _guarded(ab, m * n * esz)
        ab.check(ab.dequant_policy(src, out, m, n, ab.S32, ab.F32, dst_dtype, ab.DEQUANT_PER_TOKEN, s))
        ab.sync()
        assert tail_intact(out, m * n * esz), ("dequant_policy", m, n)
    for rows, cols in [(37, 2048), (3, 64), (1025, 8)]:
        x = ab.to_dev(f16_bits(rng.standard_normal((rows, cols)).astype(np.float32)))
        sc = ab.to_dev(f16_bits(np.ones(cols, np.float32)))
        q = _guarded(ab, rows * cols)
        ab.check(ab.quant_per_channel(x, q, rows, cols, ab.F16, sc, None, 0.0))
        ab.sync()
        assert tail_intact(q, rows * cols), ("quant_per_channel", rows, cols)
    for m, k in [(5, 2048), (131, 64), (3, 4096)]:
        x = ab.to_dev(f16_bits(rng.standard_normal((m, k)).astype(np.float32)))
        y, sm, mx = _guarded(ab, m * k * 2), _guarded(ab, m * 32), _guarded(ab, m * 32)
        ab.check(ab.softmax_flash_v2(x, y, sm, mx, None, None, None, m, k, ab.F16, ab.F32, False, True))
        ab.sync()
        assert tail_intact(y, m * k * 2) and tail_intact(sm, m * 32) and tail_intact(mx, m * 32), ("softmax_flash_v2", m, k)
    # the softmax family added beside SoftMax, and AscendAntiQuant: ragged row counts at every launch shape
    for m, k in [(5, 2048), (131, 64), (3, 4096), (2, 16384)]:
        x = ab.to_dev(f16_bits(rng.standard_normal((m, k)).astype(np.float32)))
        g = ab.to_dev(f16_bits(rng.uniform(-1, 1, (m, k)).astype(np.float32)))
        st = ab.to_dev(f16_bits(np.ones((m, 16), np.float32)))
        y, sm, mx = _guarded(ab, m * k * 2), _guarded(ab, m * 32), _guarded(ab, m * 32)
        ab.check(ab.log_softmax(x, y, sm, mx, m, k, ab.F16, True))
        ab.sync()
        assert tail_intact(y, m * k * 2) and tail_intact(sm, m * 32) and tail_intact(mx, m * 32), ("log_softmax", m, k)
        y = _guarded(ab, m * k * 2)
        ab.check(ab.simple_softmax(x, y, st, st, m, k, ab.F16, ab.F16, True))
        ab.sync()
        assert tail_intact(y, m * k * 2), ("simple_softmax", m, k)
        y, fr = _guarded(ab, m * k * 2), _guarded(ab, m * 32)
        ab.check(ab.softmax_grad(g, x, y, m, k, ab.F16, False))
        ab.check(ab.softmax_grad(g, x, fr, m, k, ab.F16, True))
        ab.sync()
        assert tail_intact(y, m * k * 2) and tail_intact(fr, m * 32), ("softmax_grad", m, k)
        y, em = _guarded(ab, m * k * 2), _guarded(ab, m * 32)
        sm2, mx2 = _guarded(ab, m * 32), _guarded(ab, m * 32)
        ab.check(ab.softmax_flash(x, y, sm2, mx2, em, st, st, m, k, ab.F16, ab.F16, True, True))
        ab.sync()
        assert tail_intact(y, m * k * 2) and tail_intact(em, m * 32) and tail_intact(sm2, m * 32) and tail_intact(mx2, m * 32), ("softmax_flash", m, k)
    for rows, cols, mode in [(37, 2048, 1), (9, 96, 1), (1025, 32, 2), (5, 160, 0)]:
        src = ab.to_dev(rng.integers(-128, 128, (rows, cols), dtype=np.int8))
        par = ab.to_dev(f16_bits(np.ones(max(rows, cols), np.float32)))
        out = _guarded(ab, rows * cols * 2)
        ab.check(ab.antiquant(src, out, rows, cols, ab.F16, mode, par, par))
        ab.sync()
        assert tail_intact(out, rows * cols * 2), ("antiquant", rows, cols, mode)
