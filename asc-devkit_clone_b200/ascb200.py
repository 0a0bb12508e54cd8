"""ctypes binding of libascb200.so for tests and the benchmark.

Thin on purpose: numpy arrays in host memory, explicit device buffers, every call goes through the
C ABI declared in include/ascb200.h.  There is no fallback of any kind: if the shared library is
missing or a call fails, an exception is raised.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

F32, F16, BF16, S8, S32, FP4, FP8_E4M3, FP8_E5M2 = 0, 1, 2, 3, 4, 5, 6, 7
KIND_F16, KIND_BF16, KIND_S8, KIND_MXFP4, KIND_MXFP8_E4M3, KIND_MXFP8_E5M2 = 0, 1, 2, 3, 4, 5
EPI_CAST, EPI_FIXPIPE_QUANT, EPI_DEQUANT_TOKEN_CHANNEL = 0, 1, 2
EINVAL, EALIGN, EUNSUPPORTED, ENODEV, ECUDA, ETIMEOUT, ETOOBIG = -1, -2, -3, -4, -5, -6, -7

EXPORTS = [
    "ascb200_init", "ascb200_strerror", "ascb200_last_cuda_error", "ascb200_device_status", "ascb200_sm_count", "ascb200_selftest_bounded_wait",
    "ascb200_malloc", "ascb200_free", "ascb200_malloc_host", "ascb200_free_host", "ascb200_memcpy_h2d", "ascb200_memcpy_d2h",
    "ascb200_memset", "ascb200_stream_create", "ascb200_stream_destroy", "ascb200_stream_sync", "ascb200_event_create",
    "ascb200_event_destroy", "ascb200_event_record", "ascb200_stream_wait_event", "ascb200_event_elapsed_ms", "ascb200_gemm", "ascb200_grouped_gemm",
    "ascb200_gemm_mxfp4_noalloc", "ascb200_noalloc_status", "ascb200_mx_scale_prepacked_bytes", "ascb200_mx_scale_prepack", "ascb200_fp4_transpose", "ascb200_shard_nslab", "ascb200_shard_groups_lpt", "ascb200_comm_unique_id", "ascb200_comm_init", "ascb200_comm_init_all", "ascb200_comm_destroy", "ascb200_group_start", "ascb200_group_end", "ascb200_allgather_slabs", "ascb200_interleave_slabs", "ascb200_graph_begin", "ascb200_graph_end", "ascb200_graph_launch", "ascb200_graph_destroy",
    "ascb200_nz_unpack", "ascb200_quant_policy", "ascb200_quant_policy_rm", "ascb200_dequant_policy", "ascb200_softmax_flash_v2", "ascb200_softmax", "ascb200_log_softmax", "ascb200_antiquant", "ascb200_softmax_flash", "ascb200_softmax_grad", "ascb200_simple_softmax", "ascb200_quant_per_tensor", "ascb200_quant_per_channel", "ascb200_softmax_quant", "ascb200_dequant",
]


class GemmDesc(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
        ("a_dev", C.c_void_p), ("b_dev", C.c_void_p), ("lda", C.c_int64), ("ldb", C.c_int64),
        ("trans_a", C.c_int32), ("trans_b", C.c_int32),
        ("scale_a_dev", C.c_void_p), ("scale_b_dev", C.c_void_p), ("bias_dev", C.c_void_p),
        ("c_dev", C.c_void_p), ("ldc", C.c_int64), ("c_dtype", C.c_int32),
        ("c2_dev", C.c_void_p), ("ldc2", C.c_int64), ("c2_dtype", C.c_int32),
        ("epilogue", C.c_int32), ("quant_dev", C.c_void_p), ("quant_scalar", C.c_uint64),
        ("tok_scale_dev", C.c_void_p), ("ch_scale_dev", C.c_void_p),
        ("relu", C.c_int32), ("act", C.c_int32), ("atomic", C.c_int32), ("scale_flags", C.c_int32), ("c_layout", C.c_int32), ("reserved", C.c_int32 * 1),
    ]


class Ascb200Error(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__(f"{what}: {code} ({lib().ascb200_strerror(code).decode()}; cuda={lib().ascb200_last_cuda_error()})")


_lib = None


def lib_path():
    return os.path.join(_HERE, "libascb200.so")


def lib():
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run `python asc-devkit_clone_b200/build.py` (there is no CPU fallback)")
        _lib = C.CDLL(path)
        _lib.ascb200_init.argtypes = [C.c_int]
        _lib.ascb200_strerror.restype = C.c_char_p
        _lib.ascb200_strerror.argtypes = [C.c_int]
        _lib.ascb200_malloc.argtypes = [C.POINTER(C.c_void_p), C.c_size_t]
        _lib.ascb200_free.argtypes = [C.c_void_p]
        _lib.ascb200_malloc_host.argtypes = [C.POINTER(C.c_void_p), C.c_size_t]
        _lib.ascb200_free_host.argtypes = [C.c_void_p]
        _lib.ascb200_memcpy_h2d.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        _lib.ascb200_memcpy_d2h.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
        _lib.ascb200_memset.argtypes = [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]
        _lib.ascb200_stream_create.argtypes = [C.POINTER(C.c_void_p)]
        _lib.ascb200_stream_destroy.argtypes = [C.c_void_p]
        _lib.ascb200_stream_sync.argtypes = [C.c_void_p]
        _lib.ascb200_event_create.argtypes = [C.POINTER(C.c_void_p)]
        _lib.ascb200_event_destroy.argtypes = [C.c_void_p]
        _lib.ascb200_event_record.argtypes = [C.c_void_p, C.c_void_p]
        _lib.ascb200_stream_wait_event.argtypes = [C.c_void_p, C.c_void_p]
        _lib.ascb200_event_elapsed_ms.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]
        _lib.ascb200_device_status.argtypes = [C.c_void_p, C.POINTER(C.c_uint32)]
        _lib.ascb200_selftest_bounded_wait.argtypes = [C.POINTER(C.c_uint32), C.c_void_p]
        _lib.ascb200_gemm.argtypes = [C.POINTER(GemmDesc), C.c_void_p]
        _lib.ascb200_grouped_gemm.argtypes = [C.POINTER(GemmDesc), C.c_void_p, C.c_int32, C.c_void_p]
        _lib.ascb200_gemm_mxfp4_noalloc.argtypes = [C.POINTER(GemmDesc), C.c_void_p]
        _lib.ascb200_noalloc_status.argtypes = [C.c_void_p, C.POINTER(C.c_uint32)]
        _lib.ascb200_mx_scale_prepacked_bytes.argtypes = [C.c_int32, C.c_int32]
        _lib.ascb200_mx_scale_prepacked_bytes.restype = C.c_size_t
        _lib.ascb200_mx_scale_prepack.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p]
        _lib.ascb200_fp4_transpose.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
        _lib.ascb200_shard_nslab.argtypes = [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        _lib.ascb200_shard_groups_lpt.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
        _lib.ascb200_comm_unique_id.argtypes = [C.c_void_p]
        _lib.ascb200_comm_init.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_void_p]
        _lib.ascb200_comm_init_all.argtypes = [C.POINTER(C.c_void_p), C.c_int32, C.c_void_p]
        _lib.ascb200_comm_destroy.argtypes = [C.c_void_p]
        _lib.ascb200_group_start.argtypes = []
        _lib.ascb200_group_end.argtypes = []
        _lib.ascb200_allgather_slabs.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p,
                                                 C.c_int64, C.c_void_p]
        _lib.ascb200_interleave_slabs.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_void_p]
        _lib.ascb200_graph_begin.argtypes = [C.c_void_p]
        _lib.ascb200_graph_end.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        _lib.ascb200_graph_launch.argtypes = [C.c_void_p, C.c_void_p]
        _lib.ascb200_graph_destroy.argtypes = [C.c_void_p]
        _lib.ascb200_nz_unpack.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
        _lib.ascb200_quant_policy.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                              C.c_int32, C.c_void_p, C.c_void_p, C.c_float, C.c_int32, C.c_void_p]
        _lib.ascb200_quant_policy_rm.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                 C.c_int32, C.c_void_p, C.c_void_p, C.c_float, C.c_int32, C.c_int32, C.c_void_p]
        _lib.ascb200_dequant_policy.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                C.c_int32, C.c_void_p, C.c_void_p]
        _lib.ascb200_softmax_flash_v2.argtypes = [C.c_void_p] * 7 + [C.c_int32] * 6 + [C.c_void_p]
        _lib.ascb200_simple_softmax.argtypes = [C.c_void_p] * 4 + [C.c_int32] * 5 + [C.c_void_p]
        _lib.ascb200_softmax_grad.argtypes = [C.c_void_p] * 3 + [C.c_int32] * 4 + [C.c_void_p]
        _lib.ascb200_softmax_flash.argtypes = [C.c_void_p] * 7 + [C.c_int32] * 6 + [C.c_void_p]
        _lib.ascb200_antiquant.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                           C.c_float, C.c_float, C.c_void_p]
        _lib.ascb200_log_softmax.argtypes = [C.c_void_p] * 4 + [C.c_int32] * 4 + [C.c_void_p]
        _lib.ascb200_softmax.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                         C.c_void_p]
        _lib.ascb200_quant_per_tensor.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_float, C.c_void_p]
        _lib.ascb200_quant_per_channel.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                                   C.c_float, C.c_void_p]
        _lib.ascb200_softmax_quant.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                               C.c_float, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
        _lib.ascb200_dequant.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                         C.c_int32, C.c_float, C.c_void_p]
    return _lib


def check(code, what="ascb200 call"):
    if code != 0:
        raise Ascb200Error(code, what)


def init(device=0):
    check(lib().ascb200_init(device), "ascb200_init")


class DevBuf:
    """A device allocation made through ascb200_malloc; holds shape / dtype of the numpy array it mirrors."""

    def __init__(self, nbytes, shape=None, dtype=None):
        self.nbytes = int(nbytes)
        self.shape, self.dtype = shape, dtype
        p = C.c_void_p()
        check(lib().ascb200_malloc(C.byref(p), max(self.nbytes, 1)), "ascb200_malloc")
        self.ptr = p.value

    def free(self):
        if self.ptr:
            lib().ascb200_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def upload(self, a, stream=None):
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        check(lib().ascb200_memcpy_h2d(self.ptr, a.ctypes.data, a.nbytes, stream), "h2d")
        check(lib().ascb200_stream_sync(stream), "sync")
        return self

    def download(self, stream=None, shape=None, dtype=None):
        out = np.empty(shape or self.shape, dtype or self.dtype)
        check(lib().ascb200_memcpy_d2h(out.ctypes.data, self.ptr, out.nbytes, stream), "d2h")
        check(lib().ascb200_stream_sync(stream), "sync")
        return out

    def fill(self, byte, stream=None):
        check(lib().ascb200_memset(self.ptr, byte, self.nbytes, stream), "memset")


def to_dev(a):
    a = np.ascontiguousarray(a)
    return DevBuf(a.nbytes, a.shape, a.dtype).upload(a)


def empty(shape, dtype):
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    return DevBuf(n, tuple(shape), np.dtype(dtype))


def sync(stream=None):
    check(lib().ascb200_stream_sync(stream), "sync")
    st = C.c_uint32(0)
    check(lib().ascb200_device_status(stream, C.byref(st)), "device status")


def _ptr(b):
    return None if b is None else (b.ptr if isinstance(b, DevBuf) else b)


def gemm(kind, m, n, k, a, b, c, c_dtype, epilogue=EPI_CAST, trans_a=False, trans_b=False, lda=0, ldb=0, ldc=0, bias=None,
         scale_a=None, scale_b=None, c2=None, c2_dtype=0, ldc2=0, quant=None, quant_scalar=0, tok=None, ch=None, relu=False, act=0,
         group_counts=None, groups=0, stream=None, noalloc=False, atomic=0, scale_flags=0, c_layout=0):
    d = GemmDesc()
    d.kind, d.m, d.n, d.k = kind, m, n, k
    d.a_dev, d.b_dev, d.lda, d.ldb = _ptr(a), _ptr(b), lda, ldb
    d.trans_a, d.trans_b = int(trans_a), int(trans_b)
    d.scale_a_dev, d.scale_b_dev, d.bias_dev = _ptr(scale_a), _ptr(scale_b), _ptr(bias)
    d.c_dev, d.ldc, d.c_dtype = _ptr(c), ldc, c_dtype
    d.c2_dev, d.ldc2, d.c2_dtype = _ptr(c2), ldc2, c2_dtype
    d.epilogue, d.quant_dev, d.quant_scalar = epilogue, _ptr(quant), int(quant_scalar)
    d.tok_scale_dev, d.ch_scale_dev, d.relu, d.act = _ptr(tok), _ptr(ch), int(relu), act
    d.atomic = int(atomic)
    d.scale_flags = int(scale_flags)
    d.c_layout = int(c_layout)
    if noalloc:
        return lib().ascb200_gemm_mxfp4_noalloc(C.byref(d), stream)
    if groups:
        return lib().ascb200_grouped_gemm(C.byref(d), _ptr(group_counts), groups, stream)
    return lib().ascb200_gemm(C.byref(d), stream)


SCALE_A_PREPACKED, SCALE_B_PREPACKED = 1, 2
C_ROW_MAJOR, C_COLUMN_MAJOR, C_NZ = 0, 1, 2


SCALE_A_PAIRED, SCALE_B_PAIRED = 4, 8


def mx_scale_prepack(scale, rows, k, stream=None, paired=False):
    """Re-tiles an MX scale tensor [rows, k/32] once; returns the device buffer to pass with the matching SCALE_*_PREPACKED flag."""
    n = lib().ascb200_mx_scale_prepacked_bytes(rows, k)
    out = DevBuf(n, (n,), np.uint8)
    check(lib().ascb200_mx_scale_prepack(_ptr(scale), rows, k, int(paired), out.ptr, n, stream), "mx_scale_prepack")
    return out


def shard_nslab(n, rank, world, align=16):
    lo, hi = C.c_int64(), C.c_int64()
    check(lib().ascb200_shard_nslab(n, rank, world, align, C.byref(lo), C.byref(hi)), "shard_nslab")
    return lo.value, hi.value


def shard_groups_lpt(counts, world):
    """Owner rank of every group (greedy by rows)."""
    counts = np.ascontiguousarray(counts, np.int64)
    owner = np.empty(len(counts), np.int32)
    check(lib().ascb200_shard_groups_lpt(counts.ctypes.data, len(counts), world, owner.ctypes.data), "shard_groups_lpt")
    return owner


def nz_unpack(src_nz, dst, groups, k, n, elem_bytes, to_nk=True, stream=None):
    return lib().ascb200_nz_unpack(_ptr(src_nz), _ptr(dst), groups, k, n, elem_bytes, int(to_nk), stream)


def softmax(src, dst, sum_, max_, m, k, dtype=F16, brc=False, stream=None):
    return lib().ascb200_softmax(_ptr(src), _ptr(dst), _ptr(sum_), _ptr(max_), m, k, dtype, int(brc), stream)


def log_softmax(src, dst, sum_, max_, m, k, dtype=F16, brc=False, stream=None):
    return lib().ascb200_log_softmax(_ptr(src), _ptr(dst), _ptr(sum_), _ptr(max_), m, k, dtype, int(brc), stream)


def simple_softmax(src, dst, in_sum, in_max, m, k, dtype=F16, stats_dtype=F32, brc=True, stream=None):
    return lib().ascb200_simple_softmax(_ptr(src), _ptr(dst), _ptr(in_sum), _ptr(in_max), m, k, dtype, stats_dtype, int(brc), stream)


def softmax_grad(grad, src, dst, m, k, dtype=F16, is_front=False, stream=None):
    return lib().ascb200_softmax_grad(_ptr(grad), _ptr(src), _ptr(dst), m, k, dtype, int(is_front), stream)


def softmax_flash_v2(src, dst, exp_sum, max_, exp_max, in_exp_sum, in_max, m, k, dtype=F16, stats_dtype=F32, update=False, brc=True, stream=None):
    return lib().ascb200_softmax_flash_v2(_ptr(src), _ptr(dst), _ptr(exp_sum), _ptr(max_), _ptr(exp_max), _ptr(in_exp_sum), _ptr(in_max), m, k,
                                          dtype, stats_dtype, int(update), int(brc), stream)


def softmax_flash(src, dst, sum_, max_, exp_max, in_sum, in_max, m, k, dtype=F16, stats_dtype=F32, update=False, brc=True, stream=None):
    return lib().ascb200_softmax_flash(_ptr(src), _ptr(dst), _ptr(sum_), _ptr(max_), _ptr(exp_max), _ptr(in_sum), _ptr(in_max), m, k,
                                       dtype, stats_dtype, int(update), int(brc), stream)


def antiquant(src, dst, rows, cols, dst_dtype, mode, scale=None, offset=None, scale_scalar=1.0, offset_scalar=0.0, stream=None):
    return lib().ascb200_antiquant(_ptr(src), _ptr(dst), rows, cols, dst_dtype, mode, _ptr(scale), _ptr(offset), C.c_float(scale_scalar),
                                   C.c_float(offset_scalar), stream)


def softmax_quant(src, dst, sum_, max_, q, scale, offset_t, offset, m, k, brc=False, stream=None):
    return lib().ascb200_softmax_quant(_ptr(src), _ptr(dst), _ptr(sum_), _ptr(max_), _ptr(q), _ptr(scale), _ptr(offset_t),
                                       C.c_float(offset), m, k, int(brc), stream)


def quant_per_tensor(src, dst, n, dtype, scale, offset, stream=None):
    return lib().ascb200_quant_per_tensor(_ptr(src), _ptr(dst), n, dtype, C.c_float(scale), C.c_float(offset), stream)


def quant_per_channel(src, dst, rows, k, dtype, scale, offset_t=None, offset=0.0, stream=None):
    return lib().ascb200_quant_per_channel(_ptr(src), _ptr(dst), rows, k, dtype, _ptr(scale), _ptr(offset_t), C.c_float(offset), stream)


QUANT_PER_TOKEN, QUANT_PER_GROUP = 2, 3


def quant_policy(src, dst, m, n, src_dtype, scale_dtype, dst_dtype, policy, scale, k_dim=1, group_size=0, offset=None, offset_scalar=0.0,
                 has_offset=False, stream=None, round_mode=None):
    if round_mode is not None:
        return lib().ascb200_quant_policy_rm(_ptr(src), _ptr(dst), m, n, src_dtype, scale_dtype, dst_dtype, policy, k_dim, group_size, _ptr(scale),
                                             _ptr(offset), C.c_float(offset_scalar), int(has_offset), int(round_mode), stream)
    return lib().ascb200_quant_policy(_ptr(src), _ptr(dst), m, n, src_dtype, scale_dtype, dst_dtype, policy, k_dim, group_size, _ptr(scale),
                                      _ptr(offset), C.c_float(offset_scalar), int(has_offset), stream)


DEQUANT_PER_TOKEN, DEQUANT_PER_GROUP = 0, 1


def dequant_policy(src, dst, m, n, src_dtype, scale_dtype, dst_dtype, policy, scale, k_dim=1, group_size=0, stream=None):
    return lib().ascb200_dequant_policy(_ptr(src), _ptr(dst), m, n, src_dtype, scale_dtype, dst_dtype, policy, k_dim, group_size, _ptr(scale),
                                        stream)


def dequant(src, dst, m, n, cal, n_dst, dst_dtype, scale=None, scale_dtype=F32, scale_scalar=0.0, stream=None):
    return lib().ascb200_dequant(_ptr(src), _ptr(dst), m, n, cal, n_dst, dst_dtype, _ptr(scale), scale_dtype, C.c_float(scale_scalar),
                                 stream)


class Graph:
    """Records what `fn()` issues on `stream` into a CUDA graph (through the C ABI) and replays it."""

    def __init__(self, stream, fn):
        self.stream = stream
        check(lib().ascb200_graph_begin(stream), "graph begin")
        try:
            fn()
        finally:
            self.exec = C.c_void_p()
            check(lib().ascb200_graph_end(stream, C.byref(self.exec)), "graph end")

    def launch(self):
        check(lib().ascb200_graph_launch(self.exec, self.stream), "graph launch")

    def destroy(self):
        lib().ascb200_graph_destroy(self.exec)


class Timer:
    """CUDA-event timer on one stream (the stream the kernels are launched on)."""

    def __init__(self, stream=None):
        self.stream = stream
        self.e0, self.e1 = C.c_void_p(), C.c_void_p()
        check(lib().ascb200_event_create(C.byref(self.e0)))
        check(lib().ascb200_event_create(C.byref(self.e1)))

    def start(self):
        check(lib().ascb200_event_record(self.e0, self.stream))

    def stop_ms(self):
        check(lib().ascb200_event_record(self.e1, self.stream))
        ms = C.c_float()
        check(lib().ascb200_event_elapsed_ms(self.e0, self.e1, C.byref(ms)))
        return float(ms.value)
