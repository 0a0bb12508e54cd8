"""GPU parity of the tensor-core Matmul path (fp16 / bf16 / int8 / MXFP4, grouped) against the CPU oracle."""
import numpy as np
import pytest

import oracle as orc
from gpu_util import NP_OUT, bf16_bits, dev, f16_bits, mx_quantize, out_to_f32, quant_params

pytestmark = pytest.mark.gpu

# north-star tolerance for floating-point GEMM outputs
RTOL, ATOL = 1e-2, 1e-3


def run_f16(m, n, k, trans_a=False, trans_b=False, bf16=False, bias=True, c_dtype=0, seed=0, relu=False):
    ab = dev()
    rng = np.random.default_rng(seed)
    conv = bf16_bits if bf16 else f16_bits
    a = conv(rng.uniform(-1, 1, (k, m) if trans_a else (m, k)).astype(np.float32))
    b = conv(rng.uniform(-1, 1, (n, k) if trans_b else (k, n)).astype(np.float32))
    bias_h = rng.uniform(-1, 1, n).astype(np.float32) if bias else None
    d_c = ab.empty((m, n), NP_OUT[c_dtype])
    d_c.fill(0xFF)
    rc = ab.gemm(ab.KIND_BF16 if bf16 else ab.KIND_F16, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, c_dtype, trans_a=trans_a,
                 trans_b=trans_b, bias=ab.to_dev(bias_h) if bias else None, relu=relu)
    ab.check(rc, "gemm")
    ab.sync()
    got = out_to_f32(d_c.download(), c_dtype)
    acc = orc.gemm_f16(a, b, bias_h, trans_a=trans_a, trans_b=trans_b, is_bf16=bf16, base_k=64)
    ref = out_to_f32(orc.cast_f32(acc, c_dtype, relu=relu), c_dtype)
    err = np.abs(got - ref)
    assert np.isfinite(got).all(), f"non-finite outputs: {(~np.isfinite(got)).sum()}"
    assert (err <= ATOL + RTOL * np.abs(ref)).all(), f"max err {err.max()} at {np.unravel_index(err.argmax(), err.shape)}"
    # far tighter in practice: both sides accumulate in fp32
    assert err.max() <= 1e-3 * max(1.0, np.abs(ref).max()) * (8 if c_dtype else 1)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 64, 256), (256, 512, 512), (200, 328, 264), (64, 504, 248), (8, 8, 8)])
@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False), (True, True)])
def test_gemm_f16_layouts(m, n, k, trans_a, trans_b):
    run_f16(m, n, k, trans_a, trans_b, seed=m + n + k)


def test_gemm_f16_baseline_config():
    """A[512,512] fp16 ND, B[512,1024] fp16 ND, bias[1024] fp32, C fp32 (the reference Matmul example shape family)."""
    run_f16(512, 1024, 512, False, False, bias=True, c_dtype=0, seed=0xA5C00000)


@pytest.mark.parametrize("c_dtype", [0, 1, 2])
def test_gemm_bf16_outputs(c_dtype):
    run_f16(384, 640, 320, False, True, bf16=True, c_dtype=c_dtype, seed=5, relu=(c_dtype == 2))


def test_gemm_f16_many_tiles_persistent():
    run_f16(2048, 4352, 256, False, True, bias=False, c_dtype=2, seed=9)  # 16 x 17 tiles > SM count: several tiles per CTA


def _i8_inputs(m, n, k, trans_a, trans_b, seed, lo=-127, hi=128):
    rng = np.random.default_rng(seed)
    a = rng.integers(lo, hi, (k, m) if trans_a else (m, k)).astype(np.int8)
    b = rng.integers(lo, hi, (n, k) if trans_b else (k, n)).astype(np.int8)
    return rng, a, b


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 64, 512), (512, 1024, 1024), (144, 272, 400), (80, 48, 16)])
@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, True)])
def test_gemm_i8_int32_exact(m, n, k, trans_a, trans_b):
    ab = dev()
    rng, a, b = _i8_inputs(m, n, k, trans_a, trans_b, m * 7 + n + k)
    bias = rng.integers(-1000, 1000, n).astype(np.int32)
    d_c = ab.empty((m, n), np.int32)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.S32, trans_a=trans_a, trans_b=trans_b,
                     bias=ab.to_dev(bias)))
    ab.sync()
    ref = orc.gemm_i8(a, b, bias, trans_a=trans_a, trans_b=trans_b)
    got = d_c.download()
    assert (got == ref).all(), f"{(got != ref).sum()} of {ref.size} differ; first {np.argwhere(got != ref)[:5].tolist()}"


@pytest.mark.parametrize("m,n,k,trans_a,trans_b", [(2304, 2560, 256, False, True), (2304, 2560, 256, False, False), (2048, 2816, 384, True, True),
                                                    (2200, 2568, 272, False, True)])
def test_gemm_i8_cta_pair_exact(m, n, k, trans_a, trans_b):
    """Shapes with at least one 256 x 256 tile per pair of SMs take the two-CTA kernel; ragged edges included."""
    ab = dev()
    rng, a, b = _i8_inputs(m, n, k, trans_a, trans_b, m + 3 * n + k)
    bias = rng.integers(-1000, 1000, n).astype(np.int32)
    d_c = ab.empty((m, n), np.int32)
    d_c.fill(0x5A)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.S32, trans_a=trans_a, trans_b=trans_b, bias=ab.to_dev(bias)))
    ab.sync()
    ref = orc.gemm_i8(a, b, bias, trans_a=trans_a, trans_b=trans_b)
    got = d_c.download()
    assert (got == ref).all(), f"{(got != ref).sum()} of {ref.size} differ; first {np.argwhere(got != ref)[:5].tolist()}"


@pytest.mark.parametrize("band", [1, 2, 4, 7])
@pytest.mark.parametrize("m,n,k,no_pair", [(2200, 2568, 272, False), (1100, 712, 144, True)])
def test_gemm_i8_banded_tile_order_exact(m, n, k, no_pair, band, monkeypatch):
    """The banded tile order (bands of `band` row blocks, the last band narrower) that large A operands take by themselves,
    forced here on small shapes: every tile is still computed exactly once, on CTA pairs and on single CTAs."""
    monkeypatch.setenv("ASCB200_BAND_M", str(band))
    if no_pair:
        monkeypatch.setenv("ASCB200_NO_PAIR", "1")
    ab = dev()
    rng, a, b = _i8_inputs(m, n, k, False, True, m + band)
    d_c = ab.empty((m, n), np.int32)
    d_c.fill(0x5A)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.S32, trans_b=True))
    ab.sync()
    ref = orc.gemm_i8(a, b, None, trans_b=True)
    got = d_c.download()
    assert (got == ref).all(), f"{(got != ref).sum()} of {ref.size} differ; first {np.argwhere(got != ref)[:5].tolist()}"


@pytest.mark.parametrize("split", [2, 4])
@pytest.mark.parametrize("m,n,k,trans_b", [(128, 64, 2048, True), (300, 200, 1664, True), (100, 336, 1152, False), (512, 512, 4096, True), (40, 320, 8192, True)])
def test_gemm_i8_split_k_over_a_cluster_exact(m, n, k, trans_b, split, monkeypatch):
    """Few tiles, long K: the CTAs of a cluster split the K blocks of each tile and the leader adds their accumulators
    (through its shared memory).  Integer sums: bit exact, also with a ragged last K block and with bias."""
    monkeypatch.setenv("ASCB200_SPLIT_K", str(split))
    monkeypatch.setenv("ASCB200_NO_PAIR", "1")
    ab = dev()
    rng, a, b = _i8_inputs(m, n, k, False, trans_b, m + split)
    bias = rng.integers(-1000, 1000, n).astype(np.int32)
    d_c = ab.empty((m, n), np.int32)
    d_c.fill(0x5A)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.S32, trans_b=trans_b, bias=ab.to_dev(bias)))
    ab.sync()
    ref = orc.gemm_i8(a, b, bias, trans_b=trans_b)
    got = d_c.download()
    assert (got == ref).all(), f"{(got != ref).sum()} of {ref.size} differ; first {np.argwhere(got != ref)[:5].tolist()}"


@pytest.mark.parametrize("split", [0, 2, 4])
def test_gemm_f16_split_k_over_a_cluster(split, monkeypatch):
    """The fp16 baseline configuration (512 x 512 x 1024 + bias -> fp32) with the K blocks split over clusters of 2 and 4
    CTAs, and as one chain: fp32 sums are added in rank order, inside the tolerance of the configuration."""
    monkeypatch.setenv("ASCB200_SPLIT_K", str(split))
    run_f16(512, 512, 1024, False, True, bias=True, c_dtype=0, seed=11)


@pytest.mark.parametrize("trans_a,trans_b", [(True, False), (True, True), (False, False)])
@pytest.mark.parametrize("c_dtype", [0, 1])
def test_gemm_f16_split_k_with_untransposed_operands(trans_a, trans_b, c_dtype, monkeypatch):
    """M- / N-contiguous operands arrive as several 64-wide boxes per tile whose distance is part of the shared-memory
    descriptor; every CTA of the cluster builds its descriptors from its own shared-memory offset."""
    monkeypatch.setenv("ASCB200_SPLIT_K", "2")
    run_f16(256, 192, 1024, trans_a, trans_b, bias=True, c_dtype=c_dtype, seed=13)
    monkeypatch.setenv("ASCB200_SPLIT_K", "4")
    run_f16(128, 256, 2048, trans_a, trans_b, bf16=True, bias=False, c_dtype=c_dtype, seed=14)


@pytest.mark.parametrize("mode", ["dequant_bf16", "req8", "s32_atomic_add"])
def test_gemm_i8_split_k_chosen_by_itself_with_fused_epilogues(mode):
    """A long K and few tiles: the library splits K by itself (no switch set); the fused stages after the sum are unchanged."""
    ab = dev()
    m, n, k = 128, 512, 8192
    rng, a, b = _i8_inputs(m, n, k, False, True, 31)
    acc = orc.gemm_i8(a, b, None, trans_b=True)
    if mode == "dequant_bf16":
        tok = rng.uniform(1e-3, 1e-2, m).astype(np.float32); ch = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
        d_c = ab.empty((m, n), np.uint16)
        ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.BF16, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=True,
                         tok=ab.to_dev(tok), ch=ab.to_dev(ch)))
        ref = orc.dequant_tok_ch(acc, tok, ch, ab.BF16)
    elif mode == "req8":
        scales = rng.uniform(2e-5, 6e-5, n).astype(np.float32)
        q = quant_params(scales)
        d_c = ab.empty((m, n), np.int8)
        ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.S8, epilogue=ab.EPI_FIXPIPE_QUANT, trans_b=True, quant=ab.to_dev(q)))
        ref = orc.fixpipe_req8(acc, q)
    else:
        start = rng.integers(-1000, 1000, (m, n)).astype(np.int32)
        d_c = ab.to_dev(start)
        ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.S32, trans_b=True, atomic=1))
        ref = start + acc
    ab.sync()
    assert (d_c.download() == ref).all()


def test_gemm_mxfp4_split_k_over_a_cluster(monkeypatch):
    """Block-scaled fp4 with the K blocks (and their scale chunks) split over a cluster of two CTAs."""
    monkeypatch.setenv("ASCB200_SPLIT_K", "2")
    monkeypatch.setenv("ASCB200_NO_PAIR", "1")
    ab = dev()
    m, n, k = 256, 384, 4096
    rng, a, sa, b, sb = _mx_case(m, n, k, 21)
    d_c = ab.empty((m, n), np.float32)
    ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.F32, trans_b=True, scale_a=ab.to_dev(sa), scale_b=ab.to_dev(sb)))
    ab.sync()
    ref = orc.gemm_mxf4(a, sa, b, sb, base_k=256)
    err = np.abs(d_c.download() - ref)
    assert (err <= ATOL + RTOL * np.abs(ref)).all() and err.max() <= 1e-3 * np.abs(ref).max()


@pytest.mark.parametrize("trans_a,trans_b", [(False, True), (False, False), (True, False)])
def test_gemm_f16_cta_pair(trans_a, trans_b):
    run_f16(2304, 2560, 192, trans_a, trans_b, bias=True, c_dtype=0, seed=31)


def test_gemm_a8w8_cta_pair_token_channel_dequant():
    ab = dev()
    m, n, k = 2100, 2576, 512
    rng, a, b = _i8_inputs(m, n, k, False, True, 5)
    tok = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    ch = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    d_c = ab.empty((m, n), np.uint16)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.BF16, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=True,
                     tok=ab.to_dev(tok), ch=ab.to_dev(ch)))
    ab.sync()
    assert (d_c.download() == orc.dequant_tok_ch(orc.gemm_i8(a, b, trans_b=True), tok, ch, orc.BF16)).all()


@pytest.mark.parametrize("pair_n", [240, 208, 176, 144, 112, 80, 48])
def test_gemm_i8_cta_pair_tile_widths(pair_n, monkeypatch):
    """The CTA-pair kernel takes any tile width that is a multiple of 16; a half-owned 32-column chunk at the tile edge is stored
    from registers, whole chunks by bulk stores.  int32 (direct), bf16 dequant and int8 requant (staged) outputs."""
    monkeypatch.setenv("ASCB200_PAIR_N", str(pair_n))
    ab = dev()
    m, n, k = 520, 1000, 384
    rng, a, b = _i8_inputs(m, n, k, False, True, pair_n)
    acc = orc.gemm_i8(a, b, trans_b=True)
    d_a, d_b = ab.to_dev(a), ab.to_dev(b)
    d_c = ab.empty((m, n), np.int32)
    d_c.fill(0x5A)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, d_a, d_b, d_c, ab.S32, trans_b=True))
    ab.sync()
    assert (d_c.download() == acc).all()
    tok = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    ch = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    d_y = ab.empty((m, n), np.uint16)
    d_y.fill(0x5A)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, d_a, d_b, d_y, ab.BF16, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=True, tok=ab.to_dev(tok),
                     ch=ab.to_dev(ch)))
    ab.sync()
    assert (d_y.download() == orc.dequant_tok_ch(acc, tok, ch, orc.BF16)).all()
    q = quant_params(rng.uniform(2e-5, 2e-4, n).astype(np.float32), rng.integers(-20, 20, n))
    d_q = ab.empty((m, n), np.int8)
    d_q.fill(0x5A)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, d_a, d_b, d_q, ab.S8, epilogue=ab.EPI_FIXPIPE_QUANT, trans_b=True, quant=ab.to_dev(q)))
    ab.sync()
    assert (d_q.download() == orc.fixpipe_req8(acc, q)).all()


@pytest.mark.parametrize("pair_n", [224, 96])
def test_gemm_f16_cta_pair_tile_widths(pair_n, monkeypatch):
    monkeypatch.setenv("ASCB200_PAIR_N", str(pair_n))
    run_f16(300, 1336, 192, False, True, bias=True, c_dtype=1, seed=pair_n)


@pytest.mark.parametrize("mode", ["req8", "req8_scalar_relu", "deqf16", "qs322bf16"])
def test_gemm_i8_fixpipe_quant(mode):
    ab = dev()
    m, n, k = 256, 384, 256
    rng, a, b = _i8_inputs(m, n, k, False, False, 21, -10, 10)
    acc = orc.gemm_i8(a, b)
    scales = rng.uniform(0.005, 0.05, n).astype(np.float32)
    offsets = rng.integers(-20, 20, n)
    q = quant_params(scales, offsets)
    kw = dict(epilogue=ab.EPI_FIXPIPE_QUANT)
    if mode == "req8":
        c_dtype, ref = ab.S8, orc.fixpipe_req8(acc, q)
        kw["quant"] = ab.to_dev(q)
    elif mode == "req8_scalar_relu":
        c_dtype, ref = ab.S8, orc.fixpipe_req8(acc, q[3], relu=True)
        kw.update(quant_scalar=int(q[3]), relu=True)
    elif mode == "deqf16":
        c_dtype, ref = ab.F16, orc.fixpipe_deqf16(acc, q)
        kw["quant"] = ab.to_dev(q)
    else:
        c_dtype, ref = ab.BF16, orc.fixpipe_qs322bf16(acc, q)
        kw["quant"] = ab.to_dev(q)
    d_c = ab.empty((m, n), NP_OUT[c_dtype])
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, c_dtype, **kw))
    ab.sync()
    assert (d_c.download() == ref).all()  # integer accumulators, one fp32 multiply, one rounding: bit exact


@pytest.mark.parametrize("m,n,k,c_dtype", [(256, 512, 512, 2), (300, 200, 384, 1), (128, 1376, 1024, 2)])
def test_gemm_a8w8_token_channel_dequant(m, n, k, c_dtype):
    """The A8W8 baseline path: bf16((float(acc) * ch_scale[n]) * tok_scale[m]), B stored K-major."""
    ab = dev()
    rng, a, b = _i8_inputs(m, n, k, False, True, m + n)
    tok = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    ch = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    d_c = ab.empty((m, n), np.uint16)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, c_dtype, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL,
                     trans_b=True, tok=ab.to_dev(tok), ch=ab.to_dev(ch)))
    ab.sync()
    ref = orc.dequant_tok_ch(orc.gemm_i8(a, b, trans_b=True), tok, ch, c_dtype)
    assert (d_c.download() == ref).all()


@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (200, 328, 128)])   # staged bulk stores / stores from registers at the ragged edge
def test_gemm_a8w8_dequant_to_half_saturates_and_keeps_nan(m, n, k):
    """fp16 output of the dequant epilogue: products beyond the half range (and infinite ones) become +-65504 like the
    reference's saturating cast, a NaN scale stays NaN; everything else bit exact."""
    ab = dev()
    rng, a, b = _i8_inputs(m, n, k, False, True, 77)
    tok = rng.uniform(0.5, 2.0, m).astype(np.float32)
    ch = rng.uniform(0.5, 2.0, n).astype(np.float32)   # |acc| reaches 1e5 and more: many products overflow half
    ch[3] = np.inf
    ch[n - 2] = np.nan
    tok[5] = 3.0e38                                   # overflows fp32 in the second product
    d_c = ab.empty((m, n), np.uint16)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.F16, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL,
                     trans_b=True, tok=ab.to_dev(tok), ch=ab.to_dev(ch)))
    ab.sync()
    got = d_c.download()
    ref = orc.dequant_tok_ch(orc.gemm_i8(a, b, trans_b=True), tok, ch, ab.F16)
    nan = (ref & 0x7FFF) > 0x7C00
    assert nan.any() and ((ref & 0x7FFF) == 0x7BFF).any() and not ((ref & 0x7FFF) == 0x7C00).any()
    assert (((got & 0x7FFF) > 0x7C00) == nan).all()
    assert (got[~nan] == ref[~nan]).all()


@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("counts", [[40, 0, 7, 300], [128, 128], [1, 1, 1, 1, 1, 500, 0, 0, 3]])
def test_grouped_a8w8(counts, trans_b):
    ab = dev()
    counts = np.array(counts, np.int64)
    G, k, n = len(counts), 384, 320
    m = int(counts.sum())
    rng = np.random.default_rng(G * 100 + m)
    x = rng.integers(-127, 128, (m, k)).astype(np.int8)
    w = rng.integers(-127, 128, (G, n, k) if trans_b else (G, k, n)).astype(np.int8)
    tok = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    ch = rng.uniform(1e-3, 1e-2, (G, n)).astype(np.float32)
    d_c = ab.empty((m, n), np.uint16)
    d_c.fill(0)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(x), ab.to_dev(w), d_c, ab.BF16, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL,
                     trans_b=trans_b, tok=ab.to_dev(tok), ch=ab.to_dev(ch), group_counts=ab.to_dev(counts), groups=G))
    ab.sync()
    ref = orc.grouped_i8(x, w, counts, tok, ch, orc.BF16, trans_b=trans_b)
    assert (d_c.download() == ref).all()


@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("counts", [[300, 0, 517, 256, 1, 999, 130], [512, 512, 512], [1500, 40]])
def test_grouped_a8w8_cta_pairs(counts, trans_b, monkeypatch):
    """Grouped problems on the CTA-pair kernel (chosen by itself only for long groups, forced here): 256-row tiles whose tail
    reaches into the next group (or past the matrix) must store only the group's own rows; groups of zero rows are skipped."""
    monkeypatch.setenv("ASCB200_PAIR_N", "256" if not trans_b else "176")
    ab = dev()
    counts = np.array(counts, np.int64)
    G, k, n = len(counts), 256, 608
    m = int(counts.sum())
    rng = np.random.default_rng(G * 1000 + m)
    x = rng.integers(-127, 128, (m, k)).astype(np.int8)
    w = rng.integers(-127, 128, (G, n, k) if trans_b else (G, k, n)).astype(np.int8)
    tok = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    ch = rng.uniform(1e-3, 1e-2, (G, n)).astype(np.float32)
    d_c = ab.empty((m, n), np.uint16)
    d_c.fill(0)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(x), ab.to_dev(w), d_c, ab.BF16, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL,
                     trans_b=trans_b, tok=ab.to_dev(tok), ch=ab.to_dev(ch), group_counts=ab.to_dev(counts), groups=G))
    ab.sync()
    ref = orc.grouped_i8(x, w, counts, tok, ch, orc.BF16, trans_b=trans_b)
    got = d_c.download()
    assert (got == ref).all(), f"{(got != ref).sum()} differ; first {np.argwhere(got != ref)[:5].tolist()}"


@pytest.mark.parametrize("trans_b", [True, False])
@pytest.mark.parametrize("c_dtype", [0, 1, 2])
def test_grouped_a8w8_swapped_tail_blocks(trans_b, c_dtype, monkeypatch):
    """CTA pairs multiply a group's partial last 256-row block with the operand roles swapped (weights on the M side, the
    block's rows, rounded up to 16, on the N side).  Group sizes cover every box count of the narrow operand, tails that end on
    and next to multiples of 16 and 32, whole blocks before a tail, and a column count that is no multiple of the tile width."""
    monkeypatch.setenv("ASCB200_PAIR_N", "256")
    ab = dev()
    counts = np.array([1, 15, 16, 17, 0, 63, 64, 65, 96, 97, 128, 129, 191, 193, 240, 241, 255, 256, 257, 512 + 33, 768], np.int64)
    G, k, n = len(counts), 384, 608
    m = int(counts.sum())
    rng = np.random.default_rng(4242 + c_dtype)
    x = rng.integers(-127, 128, (m, k)).astype(np.int8)
    w = rng.integers(-127, 128, (G, n, k) if trans_b else (G, k, n)).astype(np.int8)
    tok = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    ch = rng.uniform(1e-3, 1e-2, (G, n)).astype(np.float32)
    esz = 4 if c_dtype == ab.F32 else 2
    d_c = ab.DevBuf(m * n * esz + 256)
    d_c.fill(0x5A)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(x), ab.to_dev(w), d_c, c_dtype, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL,
                     trans_b=trans_b, tok=ab.to_dev(tok), ch=ab.to_dev(ch), group_counts=ab.to_dev(counts), groups=G))
    ab.sync()
    host = d_c.download(shape=(m * n * esz + 256,), dtype=np.uint8)
    assert (host[m * n * esz:] == 0x5A).all(), "wrote past the end"
    ref = orc.grouped_i8(x, w, counts, tok, ch, c_dtype, trans_b=trans_b)
    got = host[:m * n * esz].view(ref.dtype).reshape(m, n)
    if c_dtype == ab.F32:
        assert (got.view(np.uint32) == ref.view(np.uint32)).all()
    else:
        assert (got == ref).all(), f"{(got != ref).sum()} differ; first {np.argwhere(got != ref)[:5].tolist()}"


def test_grouped_matches_reference_recipe(golden_dir):
    """The grouped example's own numpy recipe incl. FasterGelu and fp16 output (tests/golden/grouped.npz)."""
    import os
    ab = dev()
    g = np.load(os.path.join(golden_dir, "grouped.npz"))
    x, w, counts = g["x"], g["w"], g["counts"]
    m, k = x.shape
    G, _, n = w.shape
    d_c = ab.empty((m, n), np.uint16)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(x), ab.to_dev(w), d_c, ab.F16, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL,
                     trans_b=False, tok=ab.to_dev(g["tok"]), ch=ab.to_dev(g["scale"]), group_counts=ab.to_dev(counts), groups=G, act=1))
    ab.sync()
    got = orc.f16_bits_to_f32(d_c.download())
    ok = np.isclose(got, g["golden_gelu"].astype(np.float32), rtol=1e-3, atol=1e-3)
    assert (~ok).mean() <= 1e-4  # the example's acceptance rule (verify_result.py:19-41)


def _mx_case(m, n, k, seed):
    rng = np.random.default_rng(seed)
    a, sa = mx_quantize(rng.standard_normal((m, k)).astype(np.float32))
    b, sb = mx_quantize(rng.standard_normal((n, k)).astype(np.float32))
    return rng, a, sa, b, sb


@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (128, 256, 512), (384, 512, 1024), (100, 200, 192), (256, 1024, 2048),
                                   (2048, 2560, 512), (2000, 2600, 320)])  # the last two take the 192-column tile
def test_gemm_mxfp4_fp32(m, n, k):
    ab = dev()
    rng, a, sa, b, sb = _mx_case(m, n, k, m + n + k)
    d_c = ab.empty((m, n), np.float32)
    ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.F32, trans_b=True, scale_a=ab.to_dev(sa),
                     scale_b=ab.to_dev(sb)))
    ab.sync()
    got = d_c.download()
    ref = orc.gemm_mxf4(a, sa, b, sb, base_k=256)
    err = np.abs(got - ref)
    print(f"mxfp4 {m}x{n}x{k}: max abs err {err.max():.3e}, max |ref| {np.abs(ref).max():.3e}, ratio {err.max() / np.abs(ref).max():.3e}")
    assert (err <= ATOL + RTOL * np.abs(ref)).all(), f"max err {err.max()} ref {np.abs(ref).max()}"
    assert err.max() <= 1e-3 * np.abs(ref).max()  # every product is exact in fp32; only the summation differs


@pytest.mark.parametrize("m,n,k", [(384, 512, 1024), (2048, 2560, 512), (100, 200, 192)])
def test_gemm_mxfp4_prepacked_scales(m, n, k):
    """Scale tensors re-tiled once with ascb200_mx_scale_prepack (the weights' scales do not change between calls) give the
    same bytes as scales re-tiled inside the call, for either operand and for both."""
    ab = dev()
    rng, a, sa, b, sb = _mx_case(m, n, k, 5 * m + n)
    d_a, d_b, d_sa, d_sb = ab.to_dev(a), ab.to_dev(b), ab.to_dev(sa), ab.to_dev(sb)
    pa, pb = ab.mx_scale_prepack(d_sa, m, k), ab.mx_scale_prepack(d_sb, n, k)
    assert pa.nbytes == ab.lib().ascb200_mx_scale_prepacked_bytes(m, k) == ((m + 127) // 128 + 2) * 2 * ((k + 255) // 256) * 512
    outs = []
    for flags, s_a, s_b in ((0, d_sa, d_sb), (ab.SCALE_B_PREPACKED, d_sa, pb), (ab.SCALE_A_PREPACKED, pa, d_sb),
                            (ab.SCALE_A_PREPACKED | ab.SCALE_B_PREPACKED, pa, pb)):
        d_c = ab.empty((m, n), np.float32)
        d_c.fill(0xFF)
        ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, d_a, d_b, d_c, ab.F32, trans_b=True, scale_a=s_a, scale_b=s_b, scale_flags=flags))
        ab.sync()
        outs.append(d_c.download().view(np.uint32))
    for o in outs[1:]:
        assert (o == outs[0]).all()
    ref = orc.gemm_mxf4(a, sa, b, sb, base_k=256)
    assert np.allclose(outs[0].view(np.float32), ref, rtol=RTOL, atol=ATOL)
    assert ab.gemm(ab.KIND_MXFP4, m, n, k, d_a, d_b, d_c, ab.F32, trans_b=True, scale_a=d_sa, scale_b=d_sb, scale_flags=16) == ab.EINVAL


def test_gemm_mxfp4_two_streams_with_different_scales():
    """Two MXFP4 calls with different scale tensors, issued on two streams without any ordering between them, many times
    over: the re-tiled scales of one call must never be read by the other (each stream has its own scratch)."""
    import ctypes as C
    ab = dev()
    m, n, k = 1024, 1024, 2048
    rng, a, sa, b, sb = _mx_case(m, n, k, 99)
    sa2 = (sa.astype(np.int32) + rng.integers(-3, 4, sa.shape)).clip(1, 250).astype(np.uint8)
    sb2 = (sb.astype(np.int32) + rng.integers(-3, 4, sb.shape)).clip(1, 250).astype(np.uint8)
    d_a, d_b = ab.to_dev(a), ab.to_dev(b)
    sets = [(ab.to_dev(sa), ab.to_dev(sb), ab.empty((m, n), np.float32)), (ab.to_dev(sa2), ab.to_dev(sb2), ab.empty((m, n), np.float32))]
    streams = []
    for _ in range(2):
        p = C.c_void_p()
        ab.check(ab.lib().ascb200_stream_create(C.byref(p)))
        streams.append(p.value)
    refs = []
    for (s_a, s_b, d_c) in sets:   # one call at a time gives the expected bytes of each
        ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, d_a, d_b, d_c, ab.F32, trans_b=True, scale_a=s_a, scale_b=s_b))
        ab.sync()
        refs.append(d_c.download().view(np.uint32).copy())
    assert (refs[0] != refs[1]).any()
    for rep in range(20):
        for i, (s_a, s_b, d_c) in enumerate(sets):
            d_c.fill(0, streams[i])
            ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, d_a, d_b, d_c, ab.F32, trans_b=True, scale_a=s_a, scale_b=s_b, stream=streams[i]))
    for i in range(2):
        ab.sync(streams[i])
    for i, (_, _, d_c) in enumerate(sets):
        assert (d_c.download().view(np.uint32) == refs[i]).all(), f"stream {i} read the other call's scales"
    for sp in streams:
        ab.lib().ascb200_stream_destroy(sp)


def test_gemm_mxfp4_reference_layouts_of_untransposed_operands(golden_dir):
    """MX Matmul in the layouts the reference's examples write: B [K, N] (two N-neighbours per byte) with scaleB [sK/2, N, 2],
    and a transposed A [K, M] with scaleA in the same pair order.  Every combination gives the bytes of the K-major call."""
    import os
    ab = dev()
    g = np.load(os.path.join(golden_dir, "mxfp4_nd.npz"))
    m, n, k = g["a"].shape[0], g["b_kmajor"].shape[0], g["a"].shape[1] * 2
    d = {key: ab.to_dev(g[key]) for key in ("a", "a_t", "b_nd", "b_kmajor", "sa", "sa_paired", "sb", "sb_paired")}

    def run(a, ta, sa, fa, b, tb, sb, fb):
        d_c = ab.empty((m, n), np.float32)
        d_c.fill(0xFF)
        ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, d[a], d[b], d_c, ab.F32, trans_a=ta, trans_b=tb, scale_a=d[sa], scale_b=d[sb], scale_flags=fa | fb))
        ab.sync()
        return d_c.download()

    base = run("a", False, "sa", 0, "b_kmajor", True, "sb", 0)
    assert np.allclose(base, g["golden_f64"], rtol=RTOL, atol=ATOL)
    for args in (("a", False, "sa", 0, "b_nd", False, "sb_paired", ab.SCALE_B_PAIRED),
                 ("a_t", True, "sa_paired", ab.SCALE_A_PAIRED, "b_kmajor", True, "sb", 0),
                 ("a_t", True, "sa_paired", ab.SCALE_A_PAIRED, "b_nd", False, "sb_paired", ab.SCALE_B_PAIRED),
                 ("a", False, "sa", 0, "b_nd", False, "sb", 0)):   # ND operand with plain scales
        assert (run(*args).view(np.uint32) == base.view(np.uint32)).all(), args
    # prepacked from the pair order
    pb = ab.mx_scale_prepack(d["sb_paired"], n, k, paired=True)
    d_c = ab.empty((m, n), np.float32)
    ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, d["a"], d["b_nd"], d_c, ab.F32, trans_b=False, scale_a=d["sa"], scale_b=pb, scale_flags=ab.SCALE_B_PREPACKED))
    ab.sync()
    assert (d_c.download().view(np.uint32) == base.view(np.uint32)).all()


@pytest.mark.parametrize("rows,cols", [(256, 64), (512, 192), (300, 70), (64, 2), (2, 130), (1024, 1000)])
def test_fp4_transpose(rows, cols):
    ab = dev()
    rng = np.random.default_rng(rows + cols)
    codes = rng.integers(0, 16, (rows, cols), dtype=np.uint8)
    src = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    want = (codes.T[:, 0::2] | (codes.T[:, 1::2] << 4)).astype(np.uint8)
    d_dst = ab.DevBuf(want.size + 64)
    d_dst.fill(0xEE)
    ab.check(ab.lib().ascb200_fp4_transpose(ab.to_dev(src).ptr, d_dst.ptr, rows, cols, None))
    ab.sync()
    got = d_dst.download(shape=(want.size + 64,), dtype=np.uint8)
    assert (got[want.size:] == 0xEE).all()
    assert (got[:want.size].reshape(want.shape) == want).all()
    assert ab.lib().ascb200_fp4_transpose(ab.to_dev(src).ptr, d_dst.ptr, rows + 1, cols, None) == ab.EINVAL


@pytest.mark.parametrize("layout", [1, 2])
@pytest.mark.parametrize("case", ["f16_f32", "f16_f16", "i8_s32", "i8_bf16_dequant", "i8_s8_req8", "f16_pair"])
def test_gemm_output_layouts_column_major_and_nz(layout, case):
    """C written column-major (CubeFormat::COLUMN_MAJOR) or fractal (CubeFormat::NZ: blocks of 16 columns, 32 for 1-byte outputs,
    row-major inside a block) holds the values of the row-major result, nothing beyond its last element is written."""
    ab = dev()
    rng = np.random.default_rng(layout * 10 + len(case))
    m, n, k = (200, 328, 256) if case != "f16_pair" else (2304, 2560, 128)
    kw = {}
    if case.startswith("f16"):
        a = f16_bits(rng.uniform(-1, 1, (m, k)).astype(np.float32))
        b = f16_bits(rng.uniform(-1, 1, (n, k)).astype(np.float32))
        kind, c_dtype = ab.KIND_F16, (ab.F16 if case == "f16_f16" else ab.F32)
    else:
        a = rng.integers(-127, 128, (m, k), dtype=np.int8)
        b = rng.integers(-127, 128, (n, k), dtype=np.int8)
        kind = ab.KIND_S8
        if case == "i8_s32":
            c_dtype = ab.S32
        elif case == "i8_bf16_dequant":
            c_dtype = ab.BF16
            kw = dict(epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, tok=ab.to_dev(rng.uniform(1e-3, 1e-2, m).astype(np.float32)),
                      ch=ab.to_dev(rng.uniform(1e-3, 1e-2, n).astype(np.float32)))
        else:
            c_dtype = ab.S8
            kw = dict(epilogue=ab.EPI_FIXPIPE_QUANT, quant=ab.to_dev(quant_params(rng.uniform(1e-4, 3e-4, n).astype(np.float32))))
    np_t = NP_OUT[c_dtype]
    esz = np.dtype(np_t).itemsize
    d_a, d_b = ab.to_dev(a), ab.to_dev(b)
    d_ref = ab.empty((m, n), np_t)
    ab.check(ab.gemm(kind, m, n, k, d_a, d_b, d_ref, c_dtype, trans_b=True, **kw))
    ab.sync()
    ref = d_ref.download()
    c0 = 32 if esz == 1 else 16
    blocks = (n + c0 - 1) // c0
    elems = m * n if layout == 1 else blocks * m * c0
    d_c = ab.DevBuf(elems * esz + 64)
    d_c.fill(0x5A)
    ab.check(ab.gemm(kind, m, n, k, d_a, d_b, d_c, c_dtype, trans_b=True, c_layout=layout, **kw))
    ab.sync()
    raw = d_c.download(shape=(elems * esz + 64,), dtype=np.uint8)
    assert (raw[elems * esz:] == 0x5A).all()
    got = raw[:elems * esz].view(np_t)
    if layout == 1:
        assert np.ascontiguousarray(got.reshape(n, m).T).tobytes() == np.ascontiguousarray(ref).tobytes()
    else:
        nz = got.reshape(blocks, m, c0)
        back = nz.transpose(1, 0, 2).reshape(m, blocks * c0)[:, :n]
        assert np.ascontiguousarray(back).tobytes() == np.ascontiguousarray(ref).tobytes()
        if n % c0:   # the padding columns of the last block are left untouched
            pad = nz[-1][:, n % c0:]
            assert (np.ascontiguousarray(pad).view(np.uint8) == 0x5A).all()


def _fp8_codes(rng, shape, e5m2):
    """Random finite fp8 codes of moderate magnitude (|x| <= 8) so that sums of a few thousand products stay well inside fp32."""
    import ml_dtypes
    t = ml_dtypes.float8_e5m2 if e5m2 else ml_dtypes.float8_e4m3fn
    return (rng.standard_normal(shape) * 2).clip(-8, 8).astype(np.float32).astype(t).view(np.uint8)


def test_gemm_mxfp8_reference_example(golden_dir):
    """The reference's matmul_mx example as its generator writes it: e5m2 A [32, 128], B [128, 128] stored [K, N], scaleA [M, K/32],
    scaleB in the pair order [K/64][N][2]; fp32 output against the generator's golden."""
    import os
    ab = dev()
    g = np.load(os.path.join(golden_dir, "mxfp8.npz"))
    m, k = g["a"].shape
    n = g["b_kn"].shape[1]
    d_c = ab.empty((m, n), np.float32)
    ab.check(ab.gemm(ab.KIND_MXFP8_E5M2, m, n, k, ab.to_dev(g["a"]), ab.to_dev(g["b_kn"]), d_c, ab.F32, trans_b=False, scale_a=ab.to_dev(g["sa"]),
                     scale_b=ab.to_dev(g["sb_paired"]), scale_flags=ab.SCALE_B_PAIRED))
    ab.sync()
    assert np.allclose(d_c.download(), g["golden"], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("e5m2", [False, True])
@pytest.mark.parametrize("m,n,k,trans_a,trans_b", [(128, 128, 128, False, True), (384, 512, 1024, False, True), (100, 200, 192, False, True),
                                                   (256, 640, 512, False, False), (208, 264, 320, True, True), (1024, 2304, 256, False, True)])
def test_gemm_mxfp8(m, n, k, trans_a, trans_b, e5m2):
    """MX Matmul with fp8 operands (e4m3fn / e5m2) and e8m0 scales per 32 K elements against the oracle, K-major and transposed
    operand layouts, fp32 and bf16 outputs."""
    ab = dev()
    rng = np.random.default_rng(m + n + k + int(e5m2))
    a = _fp8_codes(rng, (m, k), e5m2)
    b = _fp8_codes(rng, (n, k), e5m2)
    sa = rng.integers(123, 131, (m, k // 32), dtype=np.uint8)
    sb = rng.integers(123, 131, (n, k // 32), dtype=np.uint8)
    ref = orc.gemm_mxf8(a, sa, b, sb, e5m2, base_k=128)
    a_dev = ab.to_dev(np.ascontiguousarray(a.T) if trans_a else a)
    b_dev = ab.to_dev(b if trans_b else np.ascontiguousarray(b.T))
    kind = ab.KIND_MXFP8_E5M2 if e5m2 else ab.KIND_MXFP8_E4M3
    d_c = ab.empty((m, n), np.float32)
    d_c.fill(0xFF)
    ab.check(ab.gemm(kind, m, n, k, a_dev, b_dev, d_c, ab.F32, trans_a=trans_a, trans_b=trans_b, scale_a=ab.to_dev(sa), scale_b=ab.to_dev(sb)))
    ab.sync()
    got = d_c.download()
    err = np.abs(got - ref)
    assert (err <= ATOL + RTOL * np.abs(ref)).all(), f"max err {err.max()} ref {np.abs(ref).max()}"
    assert err.max() <= 1e-3 * np.abs(ref).max()   # every product is exact in fp32; only the summation order differs
    d_bf = ab.empty((m, n), np.uint16)
    ab.check(ab.gemm(kind, m, n, k, a_dev, b_dev, d_bf, ab.BF16, trans_a=trans_a, trans_b=trans_b, scale_a=ab.to_dev(sa), scale_b=ab.to_dev(sb)))
    ab.sync()
    assert (d_bf.download() == orc.cast_f32(got, orc.BF16)).all()   # the cast applied to the GPU's own accumulators: bit exact


def test_gemm_mxfp4_requant_and_bf16():
    """MXFP4 baseline epilogue: int8 via per-channel VQF322B8_PRE plus the bf16 cast of the same accumulators."""
    ab = dev()
    m, n, k = 256, 512, 1024
    rng, a, sa, b, sb = _mx_case(m, n, k, 77)
    ref_acc = orc.gemm_mxf4(a, sa, b, sb, base_k=256)
    sigma = ref_acc.std()
    scales = (rng.uniform(0.5, 2.0, n) * 40.0 / sigma).astype(np.float32)
    q = quant_params(scales)
    d_c, d_c2, d_acc = ab.empty((m, n), np.int8), ab.empty((m, n), np.uint16), ab.empty((m, n), np.float32)
    args = (ab.KIND_MXFP4, m, n, k, ab.to_dev(a), ab.to_dev(b))
    kw = dict(trans_b=True, scale_a=ab.to_dev(sa), scale_b=ab.to_dev(sb))
    ab.check(ab.gemm(*args, d_c, ab.S8, epilogue=ab.EPI_FIXPIPE_QUANT, quant=ab.to_dev(q), c2=d_c2, c2_dtype=ab.BF16, **kw))
    ab.check(ab.gemm(*args, d_acc, ab.F32, **kw))
    ab.sync()
    acc_gpu = d_acc.download()
    # stage-wise: the epilogue applied to the accumulators the tensor cores produced is bit exact
    assert (d_c.download() == orc.fixpipe_qf322b8(acc_gpu, q)).all()
    assert (d_c2.download() == orc.cast_f32(acc_gpu, orc.BF16)).all()
    # end to end against the all-oracle pipeline: int8 may differ by one step only at rounding boundaries
    ref_q = orc.fixpipe_qf322b8(ref_acc, q)
    diff = np.abs(d_c.download().astype(np.int32) - ref_q.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3, f"int8 mismatches: {(diff != 0).sum()} of {diff.size}"
    bf = orc.bf16_bits_to_f32(d_c2.download())
    assert (np.abs(bf - ref_acc) <= ATOL + RTOL * np.abs(ref_acc)).all()


def test_gemm_argument_errors():
    ab = dev()
    buf = ab.empty((256, 256), np.int8)
    out = ab.empty((256, 256), np.float32)
    assert ab.gemm(ab.KIND_S8, 128, 128, 128, buf, buf, out, ab.F32) == -3                # int32 accumulators cannot be cast to fp32 without a scale
    assert ab.gemm(ab.KIND_S8, 128, 128, 100, buf, buf, out, ab.S32, trans_b=True) == -2  # K-major rows must be 16-byte multiples
    assert ab.gemm(ab.KIND_F16, 128, 128, 128, None, buf, out, ab.F32) == -1
    assert ab.gemm(ab.KIND_MXFP4, 128, 128, 96, buf, buf, out, ab.F32, trans_b=True, scale_a=buf, scale_b=buf) == -1  # K % 64
    assert ab.gemm(ab.KIND_F16, 0, 128, 128, buf, buf, out, ab.F32) == 0                  # empty problem
    assert ab.gemm(7, 128, 128, 128, buf, buf, out, ab.F32) == -1


@pytest.mark.parametrize("e5m2", [False, True])
def test_gemm_f16_fixpipe_fp8_output(e5m2):
    """QF322FP8_PRE: fp32 accumulator x per-channel scale -> fp8 (round to nearest even, saturating)."""
    ab = dev()
    m, n, k = 300, 416, 256
    rng = np.random.default_rng(77 + e5m2)
    a = f16_bits(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    b = f16_bits(rng.uniform(-1, 1, (n, k)).astype(np.float32))
    q = quant_params(rng.uniform(0.5, 60.0, n).astype(np.float32), np.zeros(n, np.int64))
    d_c = ab.empty((m, n), np.uint8)
    ab.check(ab.gemm(ab.KIND_F16, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.FP8_E5M2 if e5m2 else ab.FP8_E4M3, epilogue=ab.EPI_FIXPIPE_QUANT,
                     trans_b=True, quant=ab.to_dev(q)))
    ab.sync()
    acc = orc.gemm_f16(a, b, None, trans_b=True, base_k=64)
    ref = orc.fixpipe_qf322fp8(acc, q, e5m2=e5m2)
    got = d_c.download()
    # the two accumulations differ in the last fp32 bits, which can move a value across an fp8 rounding boundary
    diff = got != ref
    assert diff.mean() < 2e-3, f"{diff.sum()} of {diff.size} differ"
    step = np.abs(got[diff].astype(np.int16) - ref[diff].astype(np.int16))
    assert (step <= 1).all()
    if not e5m2:
        assert ((ref & 0x7F) == 0x7E).any(), "the e4m3 case must reach saturation (448)"


def test_gemm_mxfp4_fp8_output():
    ab = dev()
    m, n, k = 256, 384, 512
    rng, a, sa, b, sb = _mx_case(m, n, k, 99)
    q = quant_params(rng.uniform(0.05, 0.5, n).astype(np.float32), np.zeros(n, np.int64))
    d_c = ab.empty((m, n), np.uint8)
    ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.FP8_E4M3, epilogue=ab.EPI_FIXPIPE_QUANT, trans_b=True,
                     scale_a=ab.to_dev(sa), scale_b=ab.to_dev(sb), quant=ab.to_dev(q)))
    ab.sync()
    ref = orc.fixpipe_qf322fp8(orc.gemm_mxf4(a, sa, b, sb, base_k=256), q)
    got = d_c.download()
    diff = got != ref
    assert diff.mean() < 5e-3 and (np.abs(got[diff].astype(np.int16) - ref[diff].astype(np.int16)) <= 1).all()


@pytest.mark.parametrize("c_dtype", [0, 1, 2])
def test_gemm_f16_atomic_add(c_dtype):
    """enAtomic = 1: the result is added into C (bulk reducing stores for fp16 / bf16, reductions per element for fp32)."""
    ab = dev()
    m, n, k = 200, 328, 128   # ragged: edge chunks take the per-element path
    rng = np.random.default_rng(3 + c_dtype)
    a = f16_bits(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    b = f16_bits(rng.uniform(-1, 1, (n, k)).astype(np.float32))
    base = rng.integers(-8, 8, (m, n)).astype(np.float32)  # exactly representable in every output type
    c0 = base if c_dtype == 0 else (f16_bits(base) if c_dtype == 1 else bf16_bits(base))
    d_c = ab.to_dev(c0)
    ab.check(ab.gemm(ab.KIND_F16, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, c_dtype, trans_b=True, atomic=1))
    ab.sync()
    got = out_to_f32(d_c.download().reshape(m, n), c_dtype)
    acc = orc.gemm_f16(a, b, None, trans_b=True, base_k=64)
    part = out_to_f32(orc.cast_f32(acc, c_dtype), c_dtype)          # the value that is added, in the output type
    ref = out_to_f32(orc.cast_f32(base + part, c_dtype), c_dtype)   # one rounding of the sum
    tol = 1e-5 if c_dtype == 0 else (2e-2 if c_dtype == 1 else 0.13)
    assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())


def test_gemm_i8_atomic_add_int32_exact():
    ab = dev()
    m, n, k = 256, 320, 256
    rng, a, b = _i8_inputs(m, n, k, False, True, 8)
    base = rng.integers(-1000, 1000, (m, n)).astype(np.int32)
    d_c = ab.to_dev(base)
    for _ in range(2):
        ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.S32, trans_b=True, atomic=1))
    ab.sync()
    assert (d_c.download().reshape(m, n) == base + 2 * orc.gemm_i8(a, b, trans_b=True)).all()


@pytest.mark.parametrize("op", [2, 3])
@pytest.mark.parametrize("c_dtype", [0, 1, 2])
def test_gemm_f16_atomic_max_min(c_dtype, op):
    """enAtomic = 2 / 3: C = max(C, result) / min(C, result); exact, since a maximum involves no rounding beyond the cast of the result."""
    ab = dev()
    m, n, k = 200, 328, 128   # ragged: edge chunks take the per-element path
    rng = np.random.default_rng(31 + c_dtype * 2 + op)
    a = f16_bits(rng.uniform(-1, 1, (m, k)).astype(np.float32))
    b = f16_bits(rng.uniform(-1, 1, (n, k)).astype(np.float32))
    base = rng.integers(-4, 5, (m, n)).astype(np.float32)   # results spread over about +-8: both signs on both sides
    c0 = base if c_dtype == 0 else (f16_bits(base) if c_dtype == 1 else bf16_bits(base))
    d_c = ab.to_dev(c0)
    ab.check(ab.gemm(ab.KIND_F16, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, c_dtype, trans_b=True, atomic=op))
    ab.sync()
    d_p = ab.empty((m, n), c0.dtype)
    ab.check(ab.gemm(ab.KIND_F16, m, n, k, ab.to_dev(a), ab.to_dev(b), d_p, c_dtype, trans_b=True))
    ab.sync()
    part = out_to_f32(d_p.download().reshape(m, n), c_dtype)   # the plain result in the output type
    got = out_to_f32(d_c.download().reshape(m, n), c_dtype)
    ref = np.maximum(base, part) if op == 2 else np.minimum(base, part)
    assert (got == ref).all()
    assert (got != base).any() and (got == base).any()


@pytest.mark.parametrize("op", [2, 3])
def test_gemm_i8_atomic_max_min_int32(op):
    ab = dev()
    m, n, k = 256, 320, 256
    rng, a, b = _i8_inputs(m, n, k, False, True, 18)
    acc = orc.gemm_i8(a, b, trans_b=True)
    base = rng.integers(-100000, 100000, (m, n)).astype(np.int32)
    d_c = ab.to_dev(base)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.S32, trans_b=True, atomic=op))
    ab.sync()
    assert (d_c.download().reshape(m, n) == (np.maximum(base, acc) if op == 2 else np.minimum(base, acc))).all()


def test_gemm_atomic_rejects_int8_output():
    ab = dev()
    a = ab.to_dev(np.zeros((128, 128), np.int8))
    c = ab.empty((128, 128), np.int8)
    assert ab.gemm(ab.KIND_S8, 128, 128, 128, a, a, c, ab.S8, epilogue=ab.EPI_FIXPIPE_QUANT, trans_b=True, quant_scalar=0x3F800000, atomic=1) == ab.EUNSUPPORTED
    c32 = ab.empty((128, 128), np.int32)
    assert ab.gemm(ab.KIND_S8, 128, 128, 128, a, a, c32, ab.S32, trans_b=True, atomic=4) == ab.EUNSUPPORTED   # enAtomic stops at 3


@pytest.mark.parametrize("esz,to_nk", [(1, True), (1, False), (2, True), (2, False)])
def test_nz_unpack(esz, to_nk):
    """Fractal NZ weights as the grouped example writes them -> row-major [G,N,K] or [G,K,N], bit exact."""
    ab = dev()
    G, k, n = 3, 304, 192
    c0 = 32 // esz
    rng = np.random.default_rng(esz * 2 + to_nk)
    w = rng.integers(-128, 128, (G, k, n)).astype(np.int8) if esz == 1 else rng.integers(0, 65536, (G, k, n)).astype(np.uint16)
    nz = orc.nz_pack(w, c0)
    d_out = ab.empty((G, n, k) if to_nk else (G, k, n), w.dtype)
    d_out.fill(0x5A)
    ab.check(ab.nz_unpack(ab.to_dev(nz), d_out, G, k, n, esz, to_nk))
    ab.sync()
    got = d_out.download().reshape((G, n, k) if to_nk else (G, k, n))
    assert (got == (w.transpose(0, 2, 1) if to_nk else w)).all()


def test_grouped_reference_recipe_nz_weights(golden_dir):
    """The grouped example end to end with its NZ-stored weights: unpack once, then the grouped kernel on K-major weights."""
    import os
    ab = dev()
    g = np.load(os.path.join(golden_dir, "grouped.npz"))
    x, w, counts = g["x"], g["w"], g["counts"]
    m, k = x.shape
    G, _, n = w.shape
    d_w = ab.empty((G, n, k), np.int8)
    ab.check(ab.nz_unpack(ab.to_dev(orc.nz_pack(w, 32)), d_w, G, k, n, 1, True))
    d_c = ab.empty((m, n), np.uint16)
    ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(x), d_w, d_c, ab.F16, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=True,
                     tok=ab.to_dev(g["tok"]), ch=ab.to_dev(g["scale"]), group_counts=ab.to_dev(counts), groups=G, act=1))
    ab.sync()
    got = orc.f16_bits_to_f32(d_c.download())
    ok = np.isclose(got, g["golden_gelu"].astype(np.float32), rtol=1e-3, atol=1e-3)
    assert (~ok).mean() <= 1e-4  # the example's acceptance rule (verify_result.py:19-41)


def test_gemm_small_m_uses_the_64_row_instruction_exactly():
    """M <= 64 (decode-sized batches) and ragged last tiles take the M = 64 instruction: int32 results stay exact, for every
    layout of B and with a bias, incl. the rows that sit in lanes 0-15 of each TMEM quadrant."""
    ab = dev()
    for m, n, k, trans_b in [(64, 512, 256, True), (33, 320, 384, False), (192 + 17, 256, 128, True), (1, 64, 128, True)]:
        rng, a, b = _i8_inputs(m, n, k, False, trans_b, m * 3 + n)
        bias = rng.integers(-1000, 1000, n).astype(np.int32)
        d_c = ab.empty((m, n), np.int32)
        d_c.fill(0x5A)
        ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.S32, trans_b=trans_b, bias=ab.to_dev(bias)))
        ab.sync()
        assert (d_c.download().reshape(m, n) == orc.gemm_i8(a, b, bias, trans_b=trans_b)).all(), (m, n, k)


@pytest.mark.parametrize("m,n,k", [(300, 328, 256), (2304, 1376, 384)])   # single-CTA kernel / CTA pairs with a 160-column slab tile
def test_gemm_writes_a_column_slab_of_a_wider_c(m, n, k):
    """N-slab sharding writes C[:, slab] of a wider matrix (ldc > n): bulk stores clip at the slab's width, the columns beside
    it keep their contents.  bf16 (staged), int8 (staged) and int32 (from registers) outputs; lda / ldb padded too."""
    ab = dev()
    rng = np.random.default_rng(m + n)
    lda, ldb, ldc, col0 = k + 32, k + 64, (n + 200 + 15) // 16 * 16, 80   # every row and the slab start stay 16-byte aligned
    a_full = rng.integers(-127, 128, (m, lda), dtype=np.int8)
    b_full = rng.integers(-127, 128, (n, ldb), dtype=np.int8)
    a, b = a_full[:, :k], b_full[:, :k]
    acc = orc.gemm_i8(np.ascontiguousarray(a), np.ascontiguousarray(b), trans_b=True)
    tok = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
    ch = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    d_a, d_b = ab.to_dev(a_full), ab.to_dev(b_full)
    for c_dtype, np_t, fill in ((ab.BF16, np.uint16, 0x5A5A), (ab.S32, np.int32, 0x5A5A5A5A), (ab.S8, np.int8, 0x5A)):
        d_c = ab.empty((m, ldc), np_t)
        d_c.fill(0x5A)
        esz = np.dtype(np_t).itemsize
        view = d_c.ptr + col0 * esz   # the entry points take plain device addresses
        if c_dtype == ab.BF16:
            rc = ab.gemm(ab.KIND_S8, m, n, k, d_a, d_b, view, c_dtype, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=True, lda=lda, ldb=ldb, ldc=ldc,
                         tok=ab.to_dev(tok), ch=ab.to_dev(ch))
            ref = orc.dequant_tok_ch(acc, tok, ch, orc.BF16)
        elif c_dtype == ab.S32:
            rc = ab.gemm(ab.KIND_S8, m, n, k, d_a, d_b, view, c_dtype, trans_b=True, lda=lda, ldb=ldb, ldc=ldc)
            ref = acc
        else:
            q = quant_params(rng.uniform(2e-5, 2e-4, n).astype(np.float32), np.zeros(n, np.int64))
            rc = ab.gemm(ab.KIND_S8, m, n, k, d_a, d_b, view, c_dtype, epilogue=ab.EPI_FIXPIPE_QUANT, trans_b=True, lda=lda, ldb=ldb, ldc=ldc,
                         quant=ab.to_dev(q))
            ref = orc.fixpipe_req8(acc, q)
        ab.check(rc)
        ab.sync()
        got = d_c.download().reshape(m, ldc)
        assert (got[:, col0:col0 + n] == ref).all()
        rest = np.concatenate([got[:, :col0], got[:, col0 + n:]], axis=1)
        assert (rest.view(np.uint8) == 0x5A).all(), "columns outside the slab were written"


def test_gemm_outputs_stay_inside_their_buffers():
    """Exactly sized outputs followed by a guard area, ragged M and N, every output width and both kernels."""
    ab = dev()
    rng = np.random.default_rng(21)

    def guarded(nbytes):
        buf = ab.DevBuf(nbytes + 512)
        buf.fill(0x5A)
        return buf

    def tail_intact(buf, used):
        host = np.zeros(buf.nbytes, np.uint8)
        ab.check(ab.lib().ascb200_memcpy_d2h(host.ctypes.data, buf.ptr, buf.nbytes, None))
        ab.sync()
        return bool((host[used:] == 0x5A).all())

    esz = {ab.F32: 4, ab.F16: 2, ab.BF16: 2, ab.S8: 1, ab.S32: 4, ab.FP8_E4M3: 1}
    for m, n, k in [(200, 328, 128), (2304 + 9, 1000, 256), (61, 72, 64)]:
        a8 = ab.to_dev(rng.integers(-127, 128, (m, k), dtype=np.int8))
        b8 = ab.to_dev(rng.integers(-127, 128, (n, k), dtype=np.int8))
        q = ab.to_dev(quant_params(np.full(n, 1e-4, np.float32), np.zeros(n, np.int64)))
        for c_dtype, kw in [(ab.S32, {}), (ab.S8, dict(epilogue=ab.EPI_FIXPIPE_QUANT, quant=q)), (ab.BF16, dict(epilogue=ab.EPI_FIXPIPE_QUANT, quant=q)),
                            (ab.F16, dict(epilogue=ab.EPI_FIXPIPE_QUANT, quant=q))]:
            c = guarded(m * n * esz[c_dtype])
            ab.check(ab.gemm(ab.KIND_S8, m, n, k, a8, b8, c, c_dtype, trans_b=True, **kw))
            ab.sync()
            assert tail_intact(c, m * n * esz[c_dtype]), ("int8", m, n, c_dtype)
        a16 = ab.to_dev(f16_bits(rng.uniform(-1, 1, (m, k)).astype(np.float32)))
        b16 = ab.to_dev(f16_bits(rng.uniform(-1, 1, (n, k)).astype(np.float32)))
        for c_dtype, c2_dtype in [(ab.F32, ab.BF16), (ab.F16, ab.F32), (ab.BF16, ab.F16)]:
            c, c2 = guarded(m * n * esz[c_dtype]), guarded(m * n * esz[c2_dtype])
            ab.check(ab.gemm(ab.KIND_F16, m, n, k, a16, b16, c, c_dtype, trans_b=True, c2=c2, c2_dtype=c2_dtype))
            ab.sync()
            assert tail_intact(c, m * n * esz[c_dtype]) and tail_intact(c2, m * n * esz[c2_dtype]), ("fp16", m, n, c_dtype)
    for m, n, k in [(100, 200, 192), (2048 + 40, 2600, 256)]:
        _, a, sa, b, sb = _mx_case(m, n, k, m)
        q = ab.to_dev(quant_params(np.full(n, 0.5, np.float32), np.zeros(n, np.int64)))
        c, c2 = guarded(m * n), guarded(m * n * 2)
        ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, ab.to_dev(a), ab.to_dev(b), c, ab.S8, epilogue=ab.EPI_FIXPIPE_QUANT, trans_b=True, scale_a=ab.to_dev(sa),
                         scale_b=ab.to_dev(sb), quant=q, c2=c2, c2_dtype=ab.BF16))
        ab.sync()
        assert tail_intact(c, m * n) and tail_intact(c2, m * n * 2), ("mxfp4", m, n)


def test_gemm_i8_random_shapes_layouts_and_outputs():
    """Seeded random sweep: extents that are multiples of nothing in particular, both B layouts, padded leading dimensions,
    int32 / int8 / bf16 outputs, bit exact against the oracle and with a guard behind every output."""
    ab = dev()
    rng = np.random.default_rng(20251125)
    for case in range(28):
        big = case % 7 == 0
        m = int(rng.integers(1, 2700 if big else 400))
        n = int(rng.integers(1, 1600 if big else 700))
        k = int(rng.integers(1, 40)) * 16
        trans_b = bool(rng.integers(0, 2)) or n % 16 != 0      # [K, N] storage needs 16-byte aligned rows
        ldc = n + int(rng.integers(0, 3)) * 16
        a = rng.integers(-127, 128, (m, k), dtype=np.int8)
        b = rng.integers(-127, 128, (n, k) if trans_b else (k, n), dtype=np.int8)
        acc = orc.gemm_i8(a, b, trans_b=trans_b)
        d_a, d_b = ab.to_dev(a), ab.to_dev(b)
        kind = case % 3
        if kind == 0:
            c_dtype, np_t, kw, ref = ab.S32, np.int32, {}, acc
        elif kind == 1:
            q = quant_params(rng.uniform(2e-5, 3e-4, n).astype(np.float32), rng.integers(-30, 30, n))
            c_dtype, np_t, kw, ref = ab.S8, np.int8, dict(epilogue=ab.EPI_FIXPIPE_QUANT, quant=ab.to_dev(q)), orc.fixpipe_req8(acc, q)
        else:
            tok, ch = rng.uniform(1e-3, 1e-2, m).astype(np.float32), rng.uniform(1e-3, 1e-2, n).astype(np.float32)
            c_dtype, np_t = ab.BF16, np.uint16
            kw, ref = dict(epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, tok=ab.to_dev(tok), ch=ab.to_dev(ch)), orc.dequant_tok_ch(acc, tok, ch, orc.BF16)
        esz = np.dtype(np_t).itemsize
        used = ((m - 1) * ldc + n) * esz
        d_c = ab.DevBuf(used + 256)
        d_c.fill(0x5A)
        ab.check(ab.gemm(ab.KIND_S8, m, n, k, d_a, d_b, d_c, c_dtype, trans_b=trans_b, ldc=ldc, **kw), f"case {case}: {m}x{n}x{k}")
        ab.sync()
        host = np.zeros(used + 256, np.uint8)
        ab.check(ab.lib().ascb200_memcpy_d2h(host.ctypes.data, d_c.ptr, used + 256, None))
        ab.sync()
        assert (host[used:] == 0x5A).all(), f"case {case}: wrote past the end ({m}x{n}x{k}, ldc {ldc})"
        rows = np.zeros((m, ldc * esz), np.uint8).reshape(-1)
        rows[:used] = host[:used]
        got = rows.reshape(m, ldc * esz)[:, :n * esz].copy().view(np_t)
        assert (got == ref).all(), f"case {case}: {m}x{n}x{k} trans_b={trans_b} out={c_dtype}: {(got != ref).sum()} differ"
        pad = rows.reshape(m, ldc * esz)[:-1, n * esz:]
        assert (pad == 0x5A).all(), f"case {case}: padding between rows was written"


def test_gemm_mxfp4_and_f16_random_shapes():
    """Seeded random extents for the fp32-accumulating kinds (K a multiple of 64 for MXFP4), within the north-star tolerance."""
    ab = dev()
    rng = np.random.default_rng(7)
    for case in range(8):
        m, n, k = int(rng.integers(1, 600)), int(rng.integers(1, 900)), int(rng.integers(1, 12)) * 64
        _, a, sa, b, sb = _mx_case(m, n, k, case)
        d_c = ab.empty((m, n), np.float32)
        ab.check(ab.gemm(ab.KIND_MXFP4, m, n, k, ab.to_dev(a), ab.to_dev(b), d_c, ab.F32, trans_b=True, scale_a=ab.to_dev(sa), scale_b=ab.to_dev(sb)),
                 f"mxfp4 {m}x{n}x{k}")
        ab.sync()
        ref = orc.gemm_mxf4(a, sa, b, sb, base_k=256)
        assert np.allclose(d_c.download().reshape(m, n), ref, rtol=RTOL, atol=ATOL), f"mxfp4 {m}x{n}x{k}"
    for case in range(8):
        m, n, k = int(rng.integers(1, 500)), int(rng.integers(1, 90)) * 8, int(rng.integers(1, 60)) * 8
        if case & 1:
            m = (m + 7) // 8 * 8   # A stored [K, M]: rows of 16-byte multiples, the tensor-map rule
        run_f16(m, n, k, bool(case & 1), bool(case & 2), bf16=bool(case & 4), bias=bool(case % 3), c_dtype=case % 3, seed=case)


def test_grouped_random_counts_and_shapes():
    """Seeded random group lists (empty groups, single rows, tails of every length), both weight layouts, bf16 and fp16 outputs."""
    ab = dev()
    rng = np.random.default_rng(99)
    for case in range(12):
        G = int(rng.integers(1, 13))
        counts = rng.integers(0, 400, G).astype(np.int64) * (rng.random(G) > 0.2)
        counts = counts.astype(np.int64)
        m = int(counts.sum())
        if m == 0:
            counts[0], m = 5, 5
        n, k = int(rng.integers(1, 40)) * 16, int(rng.integers(1, 24)) * 16
        trans_b = bool(case & 1)
        x = rng.integers(-127, 128, (m, k), dtype=np.int8)
        w = rng.integers(-127, 128, (G, n, k) if trans_b else (G, k, n), dtype=np.int8)
        tok = rng.uniform(1e-3, 1e-2, m).astype(np.float32)
        ch = rng.uniform(1e-3, 1e-2, (G, n)).astype(np.float32)
        c_dtype = ab.BF16 if case % 3 else ab.F16
        d_c = ab.DevBuf(m * n * 2 + 256)
        d_c.fill(0x5A)
        ab.check(ab.gemm(ab.KIND_S8, m, n, k, ab.to_dev(x), ab.to_dev(w), d_c, c_dtype, epilogue=ab.EPI_DEQUANT_TOKEN_CHANNEL, trans_b=trans_b,
                         tok=ab.to_dev(tok), ch=ab.to_dev(ch), group_counts=ab.to_dev(counts), groups=G), f"case {case}")
        ab.sync()
        host = np.zeros(m * n * 2 + 256, np.uint8)
        ab.check(ab.lib().ascb200_memcpy_d2h(host.ctypes.data, d_c.ptr, host.size, None))
        ab.sync()
        assert (host[m * n * 2:] == 0x5A).all(), f"case {case}: wrote past the end"
        ref = orc.grouped_i8(x, w, counts, tok, ch, orc.BF16 if c_dtype == ab.BF16 else orc.F16, trans_b=trans_b)
        got = host[:m * n * 2].view(np.uint16).reshape(m, n)
        assert (got == ref).all(), f"case {case}: counts {counts.tolist()} n {n} k {k}: {(got != ref).sum()} differ"


def test_bounded_wait_expires_and_reports():
    """Failure detection without a fault: a wait that nothing can satisfy runs into its time limit, the kernel returns
    normally, the status word reports it once (ASCB200_ETIMEOUT), is cleared by the read, and the device keeps working."""
    import ctypes as C
    ab = dev()
    ab.sync()
    res = (C.c_uint32 * 3)()
    ab.check(ab.lib().ascb200_selftest_bounded_wait(res, None), "selftest")
    assert res[0] == 1 and res[1] == 1, list(res)
    assert 150 <= res[2] <= 5000, f"waited {res[2] * 1024} cycles for a limit of 200000"
    st = C.c_uint32(0)
    assert ab.lib().ascb200_device_status(None, C.byref(st)) == ab.ETIMEOUT and st.value & 1
    assert ab.lib().ascb200_device_status(None, C.byref(st)) == 0 and st.value == 0   # cleared by the read above
    # the context is intact: a GEMM right after it is exact
    rng = np.random.default_rng(3)
    a = rng.integers(-127, 128, (128, 256), dtype=np.int8)
    b = rng.integers(-127, 128, (128, 256), dtype=np.int8)
    d_c = ab.empty((128, 128), np.int32)
    ab.check(ab.gemm(ab.KIND_S8, 128, 128, 256, ab.to_dev(a), ab.to_dev(b), d_c, ab.S32, trans_b=True))
    ab.sync()
    assert (d_c.download() == orc.gemm_i8(a, b, trans_b=True)).all()
