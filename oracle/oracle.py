"""ctypes binding of the CPU oracle (oracle/asc_oracle.c).  Test infrastructure only.

The shared object is built by oracle/build.py (gcc, OpenMP).  Nothing in the product package may
import this module; it exists for tests, the smoke check and the benchmark's CPU baseline.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
F32, F16, BF16, S8, S32, FP4_E2M1, FP8_E4M3, FP8_E5M2 = 0, 1, 2, 3, 4, 5, 6, 7
_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            from build import build_oracle  # noqa: WPS433  (sibling file)
            build_oracle()
        _lib = C.CDLL(path)
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_f16.restype = C.c_uint16
        _lib.orc_f32_to_f16.argtypes = [C.c_float]
        _lib.orc_f32_to_f16_sat.restype = C.c_uint16
        _lib.orc_f32_to_f16_sat.argtypes = [C.c_float]
        _lib.orc_f32_to_bf16.restype = C.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [C.c_float]
        _lib.orc_f32_to_s8.restype = C.c_int8
        _lib.orc_f32_to_s8.argtypes = [C.c_float]
        _lib.orc_quant_alpha.restype = C.c_float
        _lib.orc_quant_alpha.argtypes = [C.c_uint64]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt=None):
    if a is None:
        return None
    return np.ascontiguousarray(a if dt is None else a.astype(dt, copy=False))


_OUT = {F32: np.float32, F16: np.uint16, BF16: np.uint16}


def gemm_f16(a, b, bias=None, trans_a=False, trans_b=False, is_bf16=False, base_k=0):
    """a, b: uint16 bit patterns. a [M,K] ([K,M] if trans_a); b [K,N] ([N,K] if trans_b). Returns fp32 [M,N]."""
    a, b, bias = _c(a, np.uint16), _c(b, np.uint16), _c(bias, np.float32)
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    N = b.shape[0] if trans_b else b.shape[1]
    c = np.empty((M, N), np.float32)
    lib().orc_gemm_f16(_p(a), _p(b), _p(bias), _p(c), M, N, K, a.shape[1], b.shape[1], int(trans_a), int(trans_b),
                       int(is_bf16), int(base_k))
    return c


def gemm_i8(a, b, bias=None, trans_a=False, trans_b=False):
    a, b, bias = _c(a, np.int8), _c(b, np.int8), _c(bias, np.int32)
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    N = b.shape[0] if trans_b else b.shape[1]
    c = np.empty((M, N), np.int32)
    lib().orc_gemm_i8(_p(a), _p(b), _p(bias), _p(c), M, N, K, a.shape[1], b.shape[1], int(trans_a), int(trans_b))
    return c


def gemm_mxf4(a, sa, b, sb, bias=None, base_k=0):
    """a [M,K/2], b [N,K/2] packed e2m1 bytes; sa [M,K/32], sb [N,K/32] e8m0 bytes. Returns fp32 [M,N]."""
    a, sa, b, sb, bias = _c(a, np.uint8), _c(sa, np.uint8), _c(b, np.uint8), _c(sb, np.uint8), _c(bias, np.float32)
    M, N, K = a.shape[0], b.shape[0], a.shape[1] * 2
    c = np.empty((M, N), np.float32)
    lib().orc_gemm_mxf4(_p(a), _p(sa), _p(b), _p(sb), _p(bias), _p(c), M, N, K, int(base_k))
    return c


def gemm_mxf8(a, sa, b, sb, e5m2, bias=None, base_k=0):
    """a [M,K], b [N,K] fp8 bytes (e4m3fn, or e5m2 when e5m2 is true); sa [M,K/32], sb [N,K/32] e8m0 bytes. Returns fp32 [M,N]."""
    a, sa, b, sb, bias = _c(a, np.uint8), _c(sa, np.uint8), _c(b, np.uint8), _c(sb, np.uint8), _c(bias, np.float32)
    M, N, K = a.shape[0], b.shape[0], a.shape[1]
    c = np.empty((M, N), np.float32)
    lib().orc_gemm_mxf8(_p(a), _p(sa), _p(b), _p(sb), _p(bias), _p(c), M, N, K, int(base_k), int(bool(e5m2)))
    return c


def cast_f32(acc, dtype, relu=False):
    acc = _c(acc, np.float32)
    out = np.empty(acc.shape, _OUT[dtype])
    lib().orc_cast_f32(_p(acc), _p(out), dtype, C.c_size_t(acc.size), int(relu))
    return out


def _fix(fn, acc, acc_dt, out_dt, q, relu):
    acc = _c(acc, acc_dt)
    q = _c(np.atleast_1d(q), np.uint64)
    M, N = acc.shape
    out = np.empty((M, N), out_dt)
    getattr(lib(), fn)(_p(acc), _p(out), M, N, _p(q), int(q.size > 1), int(relu))
    return out


def fixpipe_req8(acc, q, relu=False):
    return _fix("orc_fixpipe_req8", acc, np.int32, np.int8, q, relu)


def fixpipe_qf322b8(acc, q, relu=False):
    return _fix("orc_fixpipe_qf322b8", acc, np.float32, np.int8, q, relu)


def fixpipe_qf322fp8(acc, q, relu=False, e5m2=False):
    acc = _c(acc, np.float32)
    q = _c(np.atleast_1d(q), np.uint64)
    M, N = acc.shape
    out = np.empty((M, N), np.uint8)
    lib().orc_fixpipe_qf322fp8(_p(acc), _p(out), M, N, _p(q), int(q.size > 1), int(relu), int(e5m2))
    return out


def f32_to_fp8(x, e5m2=False):
    fn = lib().orc_f32_to_fp8
    fn.argtypes = [C.c_float, C.c_int]
    fn.restype = C.c_uint8
    return np.array([fn(float(v), int(e5m2)) for v in np.asarray(x, np.float32).ravel()], np.uint8).reshape(np.shape(x))


def nz_pack(w, c0):
    """[G, K, N] -> fractal NZ [G, N/c0, K/16, 16, c0] exactly as the grouped example stores its weights
    (quant_group_matmul_high_performance/scripts/gen_data.py:62)."""
    G, K, N = w.shape
    return np.ascontiguousarray(w.reshape(G, K // 16, 16, N // c0, c0).transpose(0, 3, 1, 2, 4))


def fixpipe_deqf16(acc, q, relu=False):
    return _fix("orc_fixpipe_deqf16", acc, np.int32, np.uint16, q, relu)


def fixpipe_qs322bf16(acc, q, relu=False):
    return _fix("orc_fixpipe_qs322bf16", acc, np.int32, np.uint16, q, relu)


def dequant_tok_ch(acc, tok, ch, dtype=BF16, act=0):
    acc, tok, ch = _c(acc, np.int32), _c(tok, np.float32), _c(ch, np.float32)
    M, N = acc.shape
    out = np.empty((M, N), _OUT[dtype])
    lib().orc_dequant_tok_ch(_p(acc), _p(out), dtype, M, N, _p(tok), _p(ch), int(act))
    return out


def grouped_i8(x, w, counts, tok, ch, dtype=BF16, trans_b=True, act=0):
    """x [sumM,K] int8; w [G,N,K] (trans_b) or [G,K,N]; counts int64 [G]; tok [sumM]; ch [G,N]."""
    x, w, counts, tok, ch = _c(x, np.int8), _c(w, np.int8), _c(counts, np.int64), _c(tok, np.float32), _c(ch, np.float32)
    G = w.shape[0]
    K = x.shape[1]
    N = w.shape[1] if trans_b else w.shape[2]
    out = np.zeros((x.shape[0], N), _OUT[dtype])
    lib().orc_grouped_i8(_p(x), _p(w), _p(counts), G, _p(tok), _p(ch), _p(out), dtype, K, N, int(trans_b), int(act))
    return out


def softmax(x, dtype=F16, brc=False):
    """x: uint16 half bits (dtype F16) or float32 [M,K]. Returns (y, max, sum)."""
    x = _c(x, np.uint16 if dtype == F16 else np.float32)
    M, K = x.shape
    y = np.empty_like(x)
    rep = 8 if brc else 1
    mx = np.empty((M, rep), np.float32)
    sm = np.empty((M, rep), np.float32)
    lib().orc_softmax(_p(x), _p(y), _p(mx), _p(sm), M, K, dtype, int(brc))
    return (y, mx, sm) if brc else (y, mx[:, 0], sm[:, 0])


def log_softmax(x, dtype=F16, brc=False):
    """x: uint16 half bits (dtype F16) or float32 [M,K]. Returns (y, max, sum); max/sum in the source dtype."""
    t = np.uint16 if dtype == F16 else np.float32
    x = _c(x, t)
    M, K = x.shape
    y = np.empty_like(x)
    rep = (16 if dtype == F16 else 8) if brc else 1
    mx = np.empty((M, rep), t)
    sm = np.empty((M, rep), t)
    lib().orc_log_softmax(_p(x), _p(y), _p(mx), _p(sm), M, K, dtype, int(brc))
    return (y, mx, sm) if brc else (y, mx[:, 0], sm[:, 0])


def simple_softmax(x, in_sum, in_max, dtype=F16, stats_dtype=F32):
    """x [M,K] (uint16 half bits or float32); in_sum / in_max [M] or [M, rep] in stats_dtype storage. Returns y."""
    x = _c(x, np.uint16 if dtype == F16 else np.float32)
    st = np.uint16 if stats_dtype == F16 else np.float32
    in_sum, in_max = _c(in_sum, st).reshape(x.shape[0], -1), _c(in_max, st).reshape(x.shape[0], -1)
    y = np.empty_like(x)
    lib().orc_simple_softmax(_p(x), _p(y), _p(in_sum), _p(in_max), x.shape[0], x.shape[1], dtype, stats_dtype, in_sum.shape[1])
    return y


def softmax_grad(grad, src, dtype=F16, front=False):
    """grad, src [M,K] (uint16 half bits or float32). Returns dst [M,K], or [M, 32/sizeof(T)] when front."""
    t = np.uint16 if dtype == F16 else np.float32
    grad, src = _c(grad, t), _c(src, t)
    M, K = grad.shape
    out = np.empty((M, (16 if dtype == F16 else 8)) if front else (M, K), t)
    lib().orc_softmax_grad(_p(grad), _p(src), _p(out), M, K, dtype, int(front))
    return out


def antiquant(src, dtype, mode, scale=None, offset=None, scale_scalar=1.0, offset_scalar=0.0):
    """AscendAntiQuant of int8 src [rows, cols]; scale / offset are uint16 bit patterns of `dtype` (F16 / BF16). Returns uint16 bits."""
    src = _c(src, np.int8)
    out = np.empty(src.shape, np.uint16)
    sc = None if scale is None else _c(scale, np.uint16)
    of = None if offset is None else _c(offset, np.uint16)
    lib().orc_antiquant(_p(src), _p(out), src.shape[0], src.shape[1], dtype, mode, _p(sc) if sc is not None else None,
                        _p(of) if of is not None else None, C.c_float(scale_scalar), C.c_float(offset_scalar))
    return out


def _src(x, dtype):
    return _c(x, np.float32 if dtype == F32 else np.uint16)


def quant_per_tensor(src, dtype, scale, offset):
    src = _src(src, dtype)
    dst = np.empty(src.shape, np.int8)
    lib().orc_quant_per_tensor(_p(src), _p(dst), C.c_size_t(src.size), dtype, C.c_float(scale), C.c_float(offset))
    return dst


def quant_per_channel(src, dtype, scale, offset):
    """scale: [K] of the source dtype; offset: same-shaped array or a python float."""
    src, scale = _src(src, dtype), _src(scale, dtype)
    rows, K = src.shape
    dst = np.empty(src.shape, np.int8)
    off_t = None if np.isscalar(offset) else _src(offset, dtype)
    lib().orc_quant_per_channel(_p(src), _p(dst), rows, K, dtype, _p(scale), _p(off_t),
                                C.c_float(offset if off_t is None else 0.0))
    return dst


def dequant(src, scale, dst_dtype=F32, scale_dtype=F32, cal_count=None, n_dst=None):
    src = _c(src, np.int32)
    m, n = src.shape
    cal_count = n if cal_count is None else cal_count
    n_dst = n if n_dst is None else n_dst
    if np.isscalar(scale):
        sc, sdt = np.array([scale], np.float32), -1
    else:
        sc, sdt = _src(scale, scale_dtype), scale_dtype
    dst = np.zeros((m, n_dst), _OUT[dst_dtype])
    lib().orc_dequant(_p(src), _p(dst), m, n, cal_count, n_dst, dst_dtype, _p(sc), sdt)
    return dst


def num_threads():
    return int(lib().orc_num_threads())


def set_num_threads(n):
    """OpenMP threads of every later call (overrides an OMP_NUM_THREADS the launcher exported)."""
    lib().orc_set_num_threads(int(n))


def f16_bits_to_f32(bits):
    return np.asarray(bits, np.uint16).view(np.float16).astype(np.float32)


def bf16_bits_to_f32(bits):
    return (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)


def quant_policy(src, scale, src_dtype, scale_dtype, dst_dtype, policy, k_dim=1, group_size=0, offset=None, offset_scalar=0.0, has_offset=False,
                 round_mode=1):
    """AscendQuant PER_TOKEN (policy 2) / PER_GROUP (policy 3). src [m, n] as stored (uint16 bits for F16 / BF16, float32 for F32);
    returns uint8 [m, n] (int8 / fp8 bytes) or [m, n/2] packed e2m1."""
    src = np.ascontiguousarray(src)
    scale = np.ascontiguousarray(scale)
    m, n = src.shape
    out = np.zeros((m, n // 2) if dst_dtype == FP4_E2M1 else (m, n), np.uint8)
    off = None if offset is None else np.ascontiguousarray(offset)
    lib().orc_quant_policy_rm(_p(src), _p(out), m, n, src_dtype, scale_dtype, dst_dtype, policy, k_dim, group_size, _p(scale),
                              _p(off) if off is not None else None, C.c_float(offset_scalar), int(has_offset), int(round_mode))
    return out


def dequant_policy(src, scale, scale_dtype, dst_dtype, policy, k_dim=1, group_size=0):
    """AscendDequant PER_TOKEN (policy 0) / PER_GROUP (policy 1); src int32 or float32 [m, n]."""
    src = np.ascontiguousarray(src)
    scale = np.ascontiguousarray(scale)
    m, n = src.shape
    out = np.empty((m, n), _OUT[dst_dtype])
    lib().orc_dequant_policy(_p(src), _p(out), m, n, int(src.dtype == np.float32), scale_dtype, dst_dtype, policy, k_dim, group_size, _p(scale))
    return out


def softmax_flash(x, dtype, stats_dtype, in_sum=None, in_max=None, brc=True):
    """SoftmaxFlash (first version) step: the V2 step plus the normalisation. Same arguments and returns as softmax_flash_v2."""
    return softmax_flash_v2(x, dtype, stats_dtype, in_sum, in_max, brc, _fn="orc_softmax_flash")


def softmax_flash_v2(x, dtype, stats_dtype, in_sum=None, in_max=None, brc=True, _fn="orc_softmax_flash_v2"):
    """SoftmaxFlashV2 step. x [M, K] as stored. Returns (y, sum, max, expmax or None); stats are [M, rep]."""
    x = np.ascontiguousarray(x)
    M, K = x.shape
    update = in_sum is not None
    srep = (32 // (2 if stats_dtype == F16 else 4)) if brc else 1
    erep = (32 // (2 if dtype == F16 else 4)) if brc else 1
    y = np.empty((M, K), _OUT[dtype])
    s = np.empty((M, srep), _OUT[stats_dtype])
    mx = np.empty((M, srep), _OUT[stats_dtype])
    em = np.empty((M, erep), _OUT[dtype])
    getattr(lib(), _fn)(_p(x), _p(y), _p(s), _p(mx), _p(em), _p(np.ascontiguousarray(in_sum)) if update else None,
                        _p(np.ascontiguousarray(in_max)) if update else None, M, K, dtype, stats_dtype, int(update), int(brc))
    return y, s, mx, (em if update else None)
