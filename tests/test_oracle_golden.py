"""Pins the CPU oracle against fixtures produced by the reference's own Python generators
(tests/golden/make_golden.py).  Runs without a GPU."""
import os

import numpy as np
import pytest

import oracle as orc


def load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_casts(golden_dir):
    g = load(golden_dir, "casts.npz")
    L = orc.lib()
    assert [L.orc_f32_to_f16_sat(float(v)) for v in g["f32_to_f16_in"]] == g["f32_to_f16_out"].tolist()
    assert [L.orc_f32_to_s8(float(v)) for v in g["f32_to_s8_in"]] == g["f32_to_s8_out"].tolist()
    assert [L.orc_f32_to_bf16(float(v)) for v in g["f32_to_bf16_in"]] == g["f32_to_bf16_out"].tolist()


def test_f16_roundtrip_all_bit_patterns():
    L = orc.lib()
    bits = np.arange(0, 0x10000, dtype=np.uint32).astype(np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    for b in list(range(0, 0x10000, 97)) + [0x0001, 0x03FF, 0x0400, 0x7BFF, 0x7C00, 0xFC00, 0x8000]:
        v = L.orc_f16_to_f32(b)
        assert np.float32(v).tobytes() == ref[b].tobytes() or (np.isnan(v) and np.isnan(ref[b]))
        if not np.isnan(ref[b]):
            assert L.orc_f32_to_f16(float(ref[b])) == b
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 300.0, 7e4)])
    got = np.array([L.orc_f32_to_f16(float(v)) for v in x], np.uint16)
    with np.errstate(over="ignore"):
        assert (got == x.astype(np.float16).view(np.uint16)).all()


@pytest.mark.parametrize("relu", [0, 1])
def test_fixpipe_req8_and_qf322b8_match_reference_scripts(golden_dir, relu):
    g = load(golden_dir, "fixpipe.npz")
    assert (orc.fixpipe_req8(g["acc_i"], g["q"], relu) == g[f"req8_relu{relu}"]).all()
    assert (orc.fixpipe_qf322b8(g["acc_f"], g["q"], relu) == g[f"qf322b8_relu{relu}"]).all()
    # scalar (per-tensor) parameter = every channel carrying the same value
    q0 = g["q"][5]
    ref = orc.fixpipe_req8(g["acc_i"], np.full(g["q"].shape, q0, np.uint64), relu)
    assert (orc.fixpipe_req8(g["acc_i"], q0, relu) == ref).all()


def test_fixpipe_deqf16_matches_reference_script(golden_dir):
    g = load(golden_dir, "fixpipe.npz")
    assert (orc.fixpipe_deqf16(g["acc_d"], g["qd"]) == g["deqf16"].view(np.uint16)).all()


def test_matmul_fp16_recipe(golden_dir):
    g = load(golden_dir, "matmul_fp16.npz")
    c = orc.gemm_f16(g["a"].view(np.uint16), g["b"].view(np.uint16), g["bias"])
    # the reference's own acceptance rule: rtol = atol = 1e-3 (matmul/scripts/verify_result.py:19-47)
    assert np.isclose(c, g["golden"], rtol=1e-3, atol=1e-3).all()
    # K chunking (baseK) only reorders fp32 additions
    c64 = orc.gemm_f16(g["a"].view(np.uint16), g["b"].view(np.uint16), g["bias"], base_k=64)
    assert np.isclose(c64, g["golden"], rtol=1e-3, atol=1e-3).all()
    # transposed operand layouts give the same numbers
    ct = orc.gemm_f16(np.ascontiguousarray(g["a"].T).view(np.uint16), np.ascontiguousarray(g["b"].T).view(np.uint16),
                      g["bias"], trans_a=True, trans_b=True)
    assert (ct == c).all()


def test_matmul_quant_recipe(golden_dir):
    g = load(golden_dir, "matmul_quant.npz")
    acc = orc.gemm_i8(g["a"], g["b"], g["bias"])
    assert (acc == g["a"].astype(np.int32) @ g["b"].astype(np.int32) + g["bias"]).all()
    out = orc.fixpipe_deqf16(acc, g["q"]).view(np.float16).astype(np.float32)
    # the example golden multiplies in fp16 after casting the int32 sum to fp16 (matmul_quant/scripts/gen_data.py:27-44),
    # fixpipe multiplies in fp32 and rounds once: equal within half precision
    assert np.isclose(out, g["golden"].astype(np.float32), rtol=2e-3, atol=1e-3).all()


def test_softmax_recipe(golden_dir):
    g = load(golden_dir, "softmax.npz")
    y, mx, sm = orc.softmax(g["x16"].view(np.uint16), orc.F16)
    yf = y.view(np.float16).astype(np.float32)
    assert np.allclose(yf, g["y16"], rtol=1e-3, atol=1e-7)
    assert (mx == g["max16"][:, 0]).all()
    assert np.allclose(sm, g["sum16"][:, 0], rtol=1e-5)
    y32, mx32, sm32 = orc.softmax(g["x32"], orc.F32, brc=True)
    assert mx32.shape == (32, 8) and (mx32 == mx32[:, :1]).all()
    assert np.allclose(y32, g["y32"], rtol=1e-5, atol=1e-9)
    assert (mx32[:, 0] == g["max32"][:, 0]).all()


def test_logsoftmax_recipe(golden_dir):
    """LogSoftMax oracle against the reference example's golden generator (log10 of the softmax)."""
    g = load(golden_dir, "logsoftmax.npz")
    y32, mx32, sm32 = orc.log_softmax(g["x32"], orc.F32, brc=True)
    assert mx32.shape == (128, 8) and (mx32 == g["max32"]).all() and (sm32 == sm32[:, :1]).all()
    assert np.allclose(sm32[:, :1], g["sum32"], rtol=1e-5)
    assert np.allclose(y32, g["y32"], rtol=1e-5, atol=1e-5)
    y16, mx16, sm16 = orc.log_softmax(g["x16"].view(np.uint16), orc.F16)
    assert (mx16.view(np.float16).astype(np.float32) == g["max16"][:, 0]).all()
    assert np.allclose(sm16.view(np.float16).astype(np.float32), g["sum16"][:, 0], rtol=1e-3)
    assert np.allclose(y16.view(np.float16).astype(np.float32), g["y16"], rtol=1e-3, atol=1e-3)


def test_simple_softmax_reproduces_the_softmax_recipe(golden_dir):
    """SimpleSoftMax fed with SoftMax's own max / sum is the same arithmetic: bit-identical y, hence pinned by the softmax golden."""
    g = load(golden_dir, "softmax.npz")
    x16 = g["x16"].view(np.uint16)
    y, mx, sm = orc.softmax(x16, orc.F16)
    assert (orc.simple_softmax(x16, sm, mx, orc.F16, orc.F32) == y).all()
    y32, mx32, sm32 = orc.softmax(g["x32"], orc.F32, brc=True)
    assert (orc.simple_softmax(g["x32"], sm32, mx32, orc.F32, orc.F32) == y32).all()
    ys = orc.simple_softmax(x16, sm, mx, orc.F16, orc.F32).view(np.float16).astype(np.float32)
    assert np.allclose(ys, g["y16"], rtol=1e-3, atol=1e-7)


def test_softmaxgrad_recipe(golden_dir):
    """SoftmaxGrad / SoftmaxGradFront oracle against the reference example's generator."""
    g = load(golden_dir, "softmaxgrad.npz")
    out = orc.softmax_grad(g["grad"], g["src"], orc.F32)
    assert np.allclose(out, g["golden"], rtol=1e-4, atol=1e-5)
    front = orc.softmax_grad(g["grad"], g["src"], orc.F32, front=True)
    assert front.shape == (16, 8) and (front == front[:, :1]).all()
    assert np.allclose(front[:, :1], g["front"], rtol=1e-4, atol=1e-5)
    g16, s16 = g["grad"].astype(np.float16), g["src"].astype(np.float16)
    out16 = orc.softmax_grad(g16.view(np.uint16), s16.view(np.uint16), orc.F16).view(np.float16).astype(np.float32)
    gf, sf = g16.astype(np.float32), s16.astype(np.float32)
    assert np.allclose(out16, (gf - (gf * sf).sum(axis=1, keepdims=True)) * sf, rtol=2e-3, atol=1e-3)


def test_softmax_flash_first_version_on_the_softmax_recipe(golden_dir):
    """SoftmaxFlash without update is SoftMax; two steps over two K tiles rebuild the softmax of the whole row
    (tile 1 rescaled by expMax, tile 2 as returned), checked against the softmax example's golden."""
    g = load(golden_dir, "softmax.npz")
    x16 = g["x16"].view(np.uint16)
    y, mx, sm = orc.softmax(x16, orc.F16)
    y1, s1, m1, _ = orc.softmax_flash(x16, orc.F16, orc.F32, brc=False)
    assert (y1 == y).all() and (m1[:, 0] == mx).all() and (s1[:, 0] == sm).all()
    a, b = np.ascontiguousarray(x16[:, :128]), np.ascontiguousarray(x16[:, 128:])
    ya, sa, ma, _ = orc.softmax_flash(a, orc.F16, orc.F32)
    yb, sb, mb, em = orc.softmax_flash(b, orc.F16, orc.F32, in_sum=sa, in_max=ma)
    f = lambda h: h.view(np.float16).astype(np.float32)
    whole = np.concatenate([f(ya) * f(em)[:, :1], f(yb)], axis=1)
    assert np.allclose(whole, g["y16"], rtol=4e-3, atol=1e-6)
    assert (mb[:, 0] == g["max16"][:, 0]).all() and np.allclose(sb[:, 0], g["sum16"][:, 0], rtol=1e-5)


def test_antiquant_recipe(golden_dir):
    """AscendAntiQuant per channel (int8 -> half) against the reference example's generator: bit exact with its half-arithmetic
    variant (the register code adds and multiplies in half), within one half step of its fp32-arithmetic variant."""
    g = load(golden_dir, "antiquant.npz")
    out = orc.antiquant(g["src"], orc.F16, 1, scale=g["scale"].view(np.uint16), offset=g["offset"].view(np.uint16))
    assert (out == g["golden_f16math"].view(np.uint16)).all()
    a, b = out.view(np.float16).astype(np.float32), g["golden_f32math"].astype(np.float32)
    assert (np.abs(a - b) <= np.abs(b) * 2.0 ** -10).all()
    # transposed form: the same numbers with one pair per row
    out_t = orc.antiquant(np.ascontiguousarray(g["src"].T), orc.F16, 2, scale=g["scale"].view(np.uint16), offset=g["offset"].view(np.uint16))
    assert (out_t == out.T).all()
    # per tensor, bfloat16: fp32 arithmetic and a single rounding
    bf = orc.antiquant(g["src"], orc.BF16, 0, scale_scalar=0.75, offset_scalar=-1.5)
    want = ((g["src"].astype(np.float32) - 1.5) * 0.75)
    assert (orc.bf16_bits_to_f32(bf) == orc.bf16_bits_to_f32(orc.cast_f32(want, orc.BF16))).all()


def test_quant_recipe(golden_dir):
    g = load(golden_dir, "quant.npz")
    # dav-2201 variant: half source; round(src*2+0.9) evaluated by numpy in half precision
    q16 = orc.quant_per_tensor(g["src_f16"].astype(np.float16).view(np.uint16), orc.F16, 2.0, 0.9)
    assert (q16 == g["golden_f16"]).all()
    # dav-3510 variant: fp32 source, numpy golden computed in fp32 while the operator rounds the
    # source, scale and offset to half first (ascend_quant_3510_impl.h:83-100): differ by at most 1 step
    q32 = orc.quant_per_tensor(g["src_f32"], orc.F32, 2.0, 0.9)
    d = np.abs(q32.astype(np.int32) - g["golden_f32"].astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 0.02
    # per-channel with a constant scale tensor reproduces per-tensor
    src = g["src_f16"].astype(np.float16).reshape(32, 32)
    qc = orc.quant_per_channel(src.view(np.uint16), orc.F16, np.full(32, 2.0, np.float16).view(np.uint16), 0.9)
    assert (qc.reshape(-1) == q16).all()


def test_dequant_recipe(golden_dir):
    g = load(golden_dir, "dequant.npz")
    out = orc.dequant(g["src"], g["scale"])
    assert (out == g["golden"]).all()


def test_grouped_recipe(golden_dir):
    g = load(golden_dir, "grouped.npz")
    w_t = np.ascontiguousarray(g["w"].transpose(0, 2, 1))
    for trans_b, w in ((True, w_t), (False, g["w"])):
        lin = orc.grouped_i8(g["x"], w, g["counts"], g["tok"], g["scale"], orc.F32, trans_b=trans_b)
        # reference golden multiplies scale*tok first, then the product (gen_data.py:52); the kernel
        # order is (acc*scale)*tok (quant_group_matmul_custom.asc:433,439): equal to fp32 rounding
        assert np.allclose(lin, g["golden_linear"], rtol=1e-6, atol=1e-9)
    gelu = orc.grouped_i8(g["x"], w_t, g["counts"], g["tok"], g["scale"], orc.F16, act=1).view(np.float16)
    ok = np.isclose(gelu.astype(np.float32), g["golden_gelu"].astype(np.float32), rtol=1e-3, atol=1e-3)
    assert (~ok).mean() <= 1e-4  # quant_group_matmul_high_performance/scripts/verify_result.py:19-41


def test_mxfp4_recipe(golden_dir):
    g = load(golden_dir, "mxfp4.npz")
    c = orc.gemm_mxf4(g["a"], g["sa"], g["b"], g["sb"])
    assert np.allclose(c, g["golden_f64"], rtol=1e-6, atol=1e-6)
    bf = orc.cast_f32(c, orc.BF16)
    assert (bf != g["golden_bf16_bits"]).mean() < 1e-3  # float64 golden rounded straight to bf16
    c64 = orc.gemm_mxf4(g["a"], g["sa"], g["b"], g["sb"], base_k=64)
    assert np.abs(c64 - c).max() <= 1e-6 * np.abs(c).max()  # chunking only reorders fp32 additions


def test_fp8_conversion_matches_ml_dtypes():
    """The oracle's fp32 -> fp8 (round to nearest even) against ml_dtypes for finite in-range values, plus the saturation rule."""
    ml_dtypes = pytest.importorskip("ml_dtypes")
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-3, 1e-2, 0.1, 1, 10, 100)] +
                       [np.array([0, -0.0, 448, -448, 447.9, 1.0, 2.0**-9, 2.0**-10, 2.0**-6, 3 * 2.0**-10, 57344, 61000], np.float32)])
    for e5m2, dt, mx in ((False, ml_dtypes.float8_e4m3fn, 448.0), (True, ml_dtypes.float8_e5m2, 57344.0)):
        xs = x[np.abs(x) <= mx]
        assert (orc.f32_to_fp8(xs, e5m2) == xs.astype(dt).view(np.uint8)).all()
        top = 0x7B if e5m2 else 0x7E
        assert orc.f32_to_fp8(np.array([1e9, -1e9, np.inf], np.float32), e5m2).tolist() == [top, top | 0x80, top]


def test_softmax_flash_v2_recipe(golden_dir):
    """SoftmaxFlashV2 against the golden_max / golden_sum files its example's generator writes ([M, 8] blocks, fp32 rows of 960):
    one step over the whole row, and two steps over two K tiles with the update formulas in between."""
    g = load(golden_dir, "softmaxflashv2.npz")
    x, gmax, gsum = g["x"], g["golden_max"], g["golden_sum"]
    y, s, mx, em = orc.softmax_flash_v2(x, orc.F32, orc.F32, brc=True)
    assert em is None and mx.shape == gmax.shape and s.shape == gsum.shape
    assert (mx == gmax).all()
    assert np.allclose(s, gsum, rtol=1e-6)
    assert np.allclose(y, np.exp(x - gmax[:, :1]), rtol=2e-6, atol=1e-7)
    # online form: tile 1 without update, tile 2 with it; the running maximum and sum end at the whole row's
    a, b = np.ascontiguousarray(x[:, :480]), np.ascontiguousarray(x[:, 480:])
    ya, sa, ma, _ = orc.softmax_flash_v2(a, orc.F32, orc.F32, brc=True)
    yb, sb, mb, emb = orc.softmax_flash_v2(b, orc.F32, orc.F32, in_sum=sa, in_max=ma, brc=True)
    assert (mb == gmax).all()
    assert np.allclose(sb, gsum, rtol=2e-6)
    assert np.allclose(emb[:, :1], np.exp(ma[:, :1] - mb[:, :1]), rtol=2e-6)
    whole = np.concatenate([ya * emb[:, :1], yb], axis=1)
    assert np.allclose(whole, np.exp(x - gmax[:, :1]), rtol=4e-6, atol=1e-7)
    # half data with float statistics: the same step on the rounded input
    xh = x.astype(np.float16)
    _, sh, mh, _ = orc.softmax_flash_v2(xh.view(np.uint16), orc.F16, orc.F32, brc=True)
    xf = xh.astype(np.float32)
    assert (mh[:, 0] == xf.max(axis=1)).all()
    assert np.allclose(sh[:, 0], np.exp(xf - xf.max(axis=1, keepdims=True)).sum(axis=1), rtol=2e-3)


def test_quant_policies_reduce_to_the_pinned_forms(golden_dir):
    """The PER_TOKEN / PER_GROUP policies have no generator in the reference; they are tied to the forms that have one.
    AscendQuant: a PER_TOKEN scale that is the same for every row is the per-tensor form (pinned on the quant example);
    PER_GROUP with one group per row is PER_TOKEN; PER_GROUP along rows (kDim 0) with one group over all rows is the
    per-channel form.  AscendDequant: PER_GROUP along rows with one group is the per-channel form pinned on the dequant
    example; PER_TOKEN is that form on the transposed matrix."""
    rng = np.random.default_rng(77)
    m, n = 24, 128
    src = (rng.standard_normal((m, n)) * 40).astype(np.float16)
    bits = src.view(np.uint16)
    scale, offset = np.float16(1.75), np.float16(-3.5)
    per_tensor = orc.quant_per_tensor(bits, orc.F16, float(scale), float(offset))
    tok_scale = np.full(m, scale, np.float16).view(np.uint16)
    tok_off = np.full(m, offset, np.float16).view(np.uint16)
    per_token = orc.quant_policy(bits, tok_scale, orc.F16, orc.F16, orc.S8, 2, offset=tok_off, has_offset=True)
    assert (per_token.view(np.int8) == per_tensor).all()
    per_token_scalar_off = orc.quant_policy(bits, tok_scale, orc.F16, orc.F16, orc.S8, 2, offset_scalar=float(offset), has_offset=True)
    assert (per_token_scalar_off.view(np.int8) == per_tensor).all()
    # a different scale per row, fp32 scales; one group per row of PER_GROUP must give the same bytes
    s_row = rng.uniform(0.5, 3.0, m).astype(np.float32)
    for dst in (orc.S8, orc.FP8_E4M3, orc.FP8_E5M2):
        a = orc.quant_policy(bits, s_row, orc.F16, orc.F32, dst, 2)
        b = orc.quant_policy(bits, s_row.reshape(m, 1), orc.F16, orc.F32, dst, 3, k_dim=1, group_size=n)
        assert (a == b).all()
    # kDim 0, one group over all rows: a scale per column = the per-channel form
    s_col = rng.uniform(0.5, 3.0, n).astype(np.float16)
    per_channel = orc.quant_per_channel(bits, orc.F16, s_col.view(np.uint16), 0.0)
    per_group0 = orc.quant_policy(bits, s_col.view(np.uint16).reshape(1, n), orc.F16, orc.F16, orc.S8, 3, k_dim=0, group_size=32)
    assert (per_group0[:32].view(np.int8) == per_channel[:32]).all()
    # AscendDequant on the dequant example's data
    g = load(golden_dir, "dequant.npz")
    acc, sc = g["src"], g["scale"]
    rows = acc.shape[0]
    gs = (rows + 31) // 32 * 32
    pinned = orc.dequant(acc, sc, orc.F32, orc.F32)
    assert np.allclose(pinned, g["golden"], rtol=1e-6)
    grp = orc.dequant_policy(acc, sc.reshape(1, -1), orc.F32, orc.F32, 1, k_dim=0, group_size=gs)
    assert (grp.view(np.uint32) == pinned.view(np.uint32)).all()
    tok = orc.dequant_policy(np.ascontiguousarray(acc.T), sc, orc.F32, orc.F32, 0)
    assert (tok.T.view(np.uint32) == pinned.view(np.uint32)).all()
    for dst in (orc.F16, orc.BF16):
        a = orc.dequant_policy(acc, sc.reshape(1, -1), orc.F32, dst, 1, k_dim=0, group_size=gs)
        assert (a == orc.dequant(acc, sc, dst, orc.F32)).all()


def _fp4_codes(packed):
    """packed [R, C/2] (even column in the low nibble) -> codes [R, C]."""
    out = np.empty((packed.shape[0], packed.shape[1] * 2), np.uint8)
    out[:, 0::2], out[:, 1::2] = packed & 15, packed >> 4
    return out


def test_mxfp4_layouts_of_the_untransposed_b_recipe(golden_dir):
    """The reference's layouts for an MX Matmul whose B is not transposed: [K, N] packed two N-neighbours per byte and scaleB
    [sK/2, N, 2].  They are the K-major operands in another order; the oracle on the re-ordered operands meets the float64 golden."""
    g = load(golden_dir, "mxfp4_nd.npz")
    codes_b = _fp4_codes(g["b_nd"])                       # [K, N]
    assert (_fp4_codes(g["b_kmajor"]) == codes_b.T).all()
    assert (_fp4_codes(g["a_t"]) == _fp4_codes(g["a"]).T).all()
    sk2, n, _ = g["sb_paired"].shape
    assert (g["sb_paired"].transpose(1, 0, 2).reshape(n, 2 * sk2) == g["sb"]).all()
    m = g["sa"].shape[0]
    assert (g["sa_paired"].transpose(1, 0, 2).reshape(m, 2 * sk2) == g["sa"]).all()
    ref = orc.gemm_mxf4(g["a"], g["sa"], g["b_kmajor"], g["sb"], base_k=256)
    assert np.allclose(ref, g["golden_f64"], rtol=1e-5, atol=1e-2)


def test_mxfp8_recipe(golden_dir):
    """MX Matmul with fp8 operands on the files the reference's matmul_mx generator writes (e5m2 A [32, 128], B [128, 128] not
    transposed, scaleB in the pair order): the oracle's product equals the generator's golden; the fp8 decoder agrees with
    ml_dtypes on all 256 codes of both formats."""
    import ctypes as C
    import ml_dtypes
    g = load(golden_dir, "mxfp8.npz")
    n = g["b_kn"].shape[1]
    sb = g["sb_paired"].transpose(1, 0, 2).reshape(n, -1)
    got = orc.gemm_mxf8(g["a"], g["sa"], np.ascontiguousarray(g["b_kn"].T), sb, e5m2=True)
    assert np.allclose(got, g["golden"], rtol=1e-6, atol=1e-6)
    fn = orc.lib().orc_fp8_to_f32
    fn.restype = C.c_float
    codes = np.arange(256, dtype=np.uint8)
    for e5m2, t in ((0, ml_dtypes.float8_e4m3fn), (1, ml_dtypes.float8_e5m2)):
        mine = np.array([fn(int(v), e5m2) for v in codes], np.float32)
        want = codes.view(t).astype(np.float32)
        assert ((mine == want) | (np.isnan(mine) & np.isnan(want))).all()


def test_round_modes_follow_the_conversion_rules():
    """float -> int8 under the reference's RoundMode values, on the worked examples of precision_conversion.md and the cases around
    them: 1.5 / 2.5 / -0.5 / -1.5 under nearest-even, floor, ceil, halves-away-from-zero and truncation, with saturation."""
    import ctypes as C
    fn = orc.lib().orc_f32_to_s8_mode
    fn.restype = C.c_int8
    fn.argtypes = [C.c_float, C.c_int]
    x = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 2.4, -2.6, 127.5, 300.0, -128.5, -1e9]
    want = {1: [0, 2, 2, 0, -2, -2, 2, -3, 127, 127, -128, -128],      # CAST_RINT
            2: [0, 1, 2, -1, -2, -3, 2, -3, 127, 127, -128, -128],     # CAST_FLOOR
            3: [1, 2, 3, 0, -1, -2, 3, -2, 127, 127, -128, -128],      # CAST_CEIL
            4: [1, 2, 3, -1, -2, -3, 2, -3, 127, 127, -128, -128],     # CAST_ROUND
            5: [0, 1, 2, 0, -1, -2, 2, -2, 127, 127, -128, -128]}      # CAST_TRUNC
    for mode, w in want.items():
        assert [fn(v, mode) for v in x] == w, mode
    assert fn(float("nan"), 4) == 0
