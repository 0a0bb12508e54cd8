"""Regenerate the golden fixtures in this folder from the reference's own Python code.

Run once, on a machine that has the reference tree (pass its location with --ref):

    python tests/golden/make_golden.py --ref <path of the reference tree>

The reference ships no stored result vectors for this path (its kernel unit tests assert all-zero
outputs); what it does ship are Python golden generators and fixpipe algorithm scripts.  This
script imports / executes exactly those files under a fixed numpy seed and stores small
input+output samples as .npz, so the tests can pin the CPU oracle without the reference tree.

  fixpipe.npz        req8_pre / qf322b8_pre / deqf16 of
                     examples/01_simd_cpp_api/03_basic_api/03_matrix_compute/fixpipe_l0c2gm/scripts/gen_data_{s322s8,f322s8,s322f16}.py
  matmul_fp16.npz    04_advanced_api/00_matmul/matmul/scripts/gen_data.py (rows/cols sampled)
  matmul_quant.npz   04_advanced_api/00_matmul/matmul_quant/scripts/gen_data.py, vector mode (sampled)
  softmax.npz        04_advanced_api/01_activation/softmax/scripts/gen_data.py: softmax_py_float
  logsoftmax.npz     04_advanced_api/01_activation/logsoftmax/scripts/gen_data.py: softmax_2d_py_float(log=True) on the
                     example's 128x128 uniform(-10, 10) input, plus a half input widened to fp32
  softmaxgrad.npz    04_advanced_api/01_activation/softmaxgrad/scripts/gen_data.py: softmax_grad_float, both modes, on the
                     example's uniform(-1, 1) inputs (rows sampled from its 960x960 shape)
  softmaxflashv2.npz 04_advanced_api/01_activation/softmaxflashv2/scripts/gen_data.py run as a script: its 960x960 uniform(-1, 1)
                     fp32 input and the golden_max / golden_sum files it writes ([M, 8]: every row's value repeated over one
                     32-byte block), rows sampled
  antiquant.npz      04_advanced_api/03_quantization/antiquant/scripts/gen_data.py, both arch variants (half arithmetic / fp32 arithmetic)
  quant.npz          04_advanced_api/03_quantization/quant/scripts/gen_data.py (both arch variants)
  dequant.npz        04_advanced_api/03_quantization/dequant/scripts/gen_data.py
  grouped.npz        05_best_practices/03_fusion_compute/quant_group_matmul_high_performance/scripts/gen_data.py
                     (its formulas on a reduced shape; the script's own shape is 8192x1024x8192)
  mxfp4.npz          05_best_practices/01_matrix_compute/matmul_mxfp4_high_performance/scripts/gen_data.py:39-69
                     (needs the absent en_dtypes package; its float64 golden formula is applied here to
                     e2m1 operands made with ml_dtypes.float4_e2m1fn, on a reduced shape)
  mxfp4_nd.npz       the same example's layouts for a B that is not transposed: [K, N] packed by its own pack_two_fp4 (the
                     function is taken out of the file's syntax tree and executed, since importing the file needs en_dtypes),
                     scaleB re-ordered to [sK/2, N, 2] as in gen_data.py:63; A transposed ([K, M]) with scaleA in the same pair
                     order, as 04_advanced_api/00_matmul/matmul_mx/scripts/gen_data.py:71-76 does for is_trans_scalea
  mxfp8.npz          04_advanced_api/00_matmul/matmul_mx/scripts/gen_data.py run as a script: fp8 e5m2 operands A [32, 128] and
                     B [128, 128] (not transposed), e8m0 scales A [32, 4] and B in the pair order [2, 128, 2], fp32 golden from its
                     float64 product
  casts.npz          CAST_RINT rule of docs/zh/api/SIMD-API/basic_api/data_structures/precision_conversion.md:19-23
                     with its worked examples (1.5 -> 2, 2.5 -> 2, 2^6+0.5 -> 2^6, 2^7-0.5 -> 2^7-1 saturated)
                     plus IEEE boundary cases worked out by hand from the same rule
"""
import argparse
import importlib.util
import os
import runpy
import struct
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
EX = "examples/01_simd_cpp_api"


def load_module(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def run_script_in_tmp(path, seed, argv=()):
    """Execute a reference gen_data.py as __main__ in a scratch folder; return {relative file: bytes}."""
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        cwd = os.getcwd()
        old_argv = sys.argv
        os.chdir(tmp)
        try:
            np.random.seed(seed)
            sys.argv = [path, *argv]
            runpy.run_path(path, run_name="__main__")
        finally:
            sys.argv = old_argv
            os.chdir(cwd)
        for root, _, files in os.walk(tmp):
            for f in files:
                p = os.path.join(root, f)
                out[os.path.relpath(p, tmp)] = open(p, "rb").read()
    return out


def f32_bits(x):
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


def fixpipe(ref):
    d = os.path.join(ref, EX, "03_basic_api/03_matrix_compute/fixpipe_l0c2gm/scripts")
    s8 = load_module(os.path.join(d, "gen_data_s322s8.py"), "ref_s322s8")
    f8 = load_module(os.path.join(d, "gen_data_f322s8.py"), "ref_f322s8")
    h16 = load_module(os.path.join(d, "gen_data_s322f16.py"), "ref_s322f16")
    rng = np.random.default_rng(20251)
    M, N = 24, 32
    # per-channel scales with full fp32 mantissas: the scripts keep only bits [31:13]
    scales = rng.uniform(0.001, 0.05, N).astype(np.float32)
    scales[:4] = [2.0, 0.5, 1.0, 0.0078125]
    offsets = rng.integers(0, 20, N)
    offsets[::3] = 0
    q = np.zeros(N, dtype=np.uint64)
    for j in range(N):
        q[j] = f32_bits(scales[j]) | (int(offsets[j]) << 37) | (1 << 46)
    acc_i = rng.integers(-60000, 60000, (M, N)).astype(np.int32)
    acc_i[0, :8] = [0, 1, -1, 2**31 - 1, -(2**31), 127, -128, 255]
    acc_f = (rng.standard_normal((M, N)) * 3000).astype(np.float32)
    acc_f[0, :6] = [0.0, 0.5, -0.5, 1.5, 2.5, -2.5]
    out = {"q": q, "acc_i": acc_i, "acc_f": acc_f}
    for relu in (0, 1):
        req = np.zeros((M, N), np.int8)
        qf = np.zeros((M, N), np.int8)
        for i in range(M):
            for j in range(N):
                relu_pre = 0 if relu else int(q[j])
                req[i, j] = s8.req8_pre(acc_i[i, j], q[j], relu_pre)
                qf[i, j] = f8.qf322b8_pre(acc_f[i, j], q[j], relu_pre)
        out[f"req8_relu{relu}"] = req
        out[f"qf322b8_relu{relu}"] = qf
    # deqf16: the script's saturation() helper rounds to an integer before the half cast, an
    # artefact that is invisible for its own data (integer accumulators, scale 2).  Keep to that
    # domain: power-of-two / small integer scales >= 1 and no offset, so every product is an integer.
    qd = np.zeros(N, dtype=np.uint64)
    dscales = np.array([1.0, 2.0, 4.0, 3.0] * (N // 4), dtype=np.float32)
    for j in range(N):
        qd[j] = f32_bits(dscales[j]) | (1 << 46)
    acc_d = rng.integers(-2000, 2000, (M, N)).astype(np.int32)
    acc_d[1, :4] = [40000, -40000, 70000, -70000]  # exercises half saturation
    deq = np.zeros((M, N), np.float16)
    for i in range(M):
        for j in range(N):
            deq[i, j] = h16.deqf16(acc_d[i, j], qd[j], int(qd[j]))
    out.update(qd=qd, acc_d=acc_d, deqf16=deq)
    np.savez_compressed(os.path.join(HERE, "fixpipe.npz"), **out)


def matmul_fp16(ref):
    files = run_script_in_tmp(os.path.join(ref, EX, "04_advanced_api/00_matmul/matmul/scripts/gen_data.py"), 11)
    m, n, k = 128, 2048, 1024
    a = np.frombuffer(files["input/x1_gm.bin"], np.float16).reshape(m, k)
    b = np.frombuffer(files["input/x2_gm.bin"], np.float16).reshape(k, n)
    bias = np.frombuffer(files["input/bias_gm.bin"], np.float32)
    g = np.frombuffer(files["output/golden.bin"], np.float32).reshape(m, n)
    rows = np.arange(0, m, 8)
    cols = np.arange(0, n, 32)
    np.savez_compressed(os.path.join(HERE, "matmul_fp16.npz"), a=a[rows], b=np.ascontiguousarray(b[:, cols]),
                        bias=bias[cols], golden=g[np.ix_(rows, cols)])


def matmul_quant(ref):
    files = run_script_in_tmp(os.path.join(ref, EX, "04_advanced_api/00_matmul/matmul_quant/scripts/gen_data.py"), 12,
                              ["-m", "1"])
    m = n = k = 1024
    a = np.frombuffer(files["input/x1_gm.bin"], np.int8).reshape(m, k)
    b = np.frombuffer(files["input/x2_gm.bin"], np.int8).reshape(k, n)
    bias = np.frombuffer(files["input/bias_gm.bin"], np.int32)
    qv = np.frombuffer(files["input/quant_vector_gm.bin"], np.uint64)
    g = np.frombuffer(files["output/golden.bin"], np.float16).reshape(m, n)
    rows = np.arange(0, m, 64)
    cols = np.arange(0, n, 16)
    np.savez_compressed(os.path.join(HERE, "matmul_quant.npz"), a=a[rows], b=np.ascontiguousarray(b[:, cols]),
                        bias=bias[cols], q=qv[cols], golden=g[np.ix_(rows, cols)])


def softmax(ref):
    mod = load_module(os.path.join(ref, EX, "04_advanced_api/01_activation/softmax/scripts/gen_data.py"), "ref_softmax")
    rng = np.random.default_rng(13)
    x32 = rng.uniform(-1, 1, (32, 32)).astype(np.float32)
    x32[0, :] = mod.FLOAT32_MIN
    y32, mx32, sm32 = mod.softmax_py_float(x32.copy())
    x16 = (rng.standard_normal((48, 256)) * 3).astype(np.float16)
    y16, mx16, sm16 = mod.softmax_py_float(x16.astype(np.float32))
    np.savez_compressed(os.path.join(HERE, "softmax.npz"), x32=x32, y32=y32, max32=mx32, sum32=sm32, x16=x16,
                        y16=y16.astype(np.float32), max16=mx16, sum16=sm16)


def logsoftmax(ref):
    mod = load_module(os.path.join(ref, EX, "04_advanced_api/01_activation/logsoftmax/scripts/gen_data.py"), "ref_logsoftmax")
    rng = np.random.default_rng(17)
    x32 = rng.uniform(-10, 10, (128, 128)).astype(np.float32)
    y32, mx32, sm32, _ = mod.softmax_2d_py_float(x32.copy(), update=False, log=True)
    x16 = rng.uniform(-10, 10, (40, 512)).astype(np.float16)
    y16, mx16, sm16, _ = mod.softmax_2d_py_float(x16.astype(np.float32), update=False, log=True)
    np.savez_compressed(os.path.join(HERE, "logsoftmax.npz"), x32=x32, y32=y32.astype(np.float32), max32=mx32, sum32=sm32, x16=x16,
                        y16=y16.astype(np.float32), max16=mx16, sum16=sm16)


def softmaxgrad(ref):
    mod = load_module(os.path.join(ref, EX, "04_advanced_api/01_activation/softmaxgrad/scripts/gen_data.py"), "ref_softmaxgrad")
    rng = np.random.default_rng(19)
    grad = rng.uniform(-1, 1, (16, 960)).astype(np.float32)
    src = rng.uniform(-1, 1, (16, 960)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "softmaxgrad.npz"), grad=grad, src=src, golden=mod.softmax_grad_float(grad, src, isFront=False),
                        front=mod.softmax_grad_float(grad, src, isFront=True))


def softmaxflashv2(ref):
    files = run_script_in_tmp(os.path.join(ref, EX, "04_advanced_api/01_activation/softmaxflashv2/scripts/gen_data.py"), 21)
    x = np.frombuffer(files["input/input_x.bin"], np.float32).reshape(960, 960)
    gmax = np.frombuffer(files["output/golden_max.bin"], np.float32).reshape(960, 8)
    gsum = np.frombuffer(files["output/golden_sum.bin"], np.float32).reshape(960, 8)
    rows = np.arange(0, 960, 24)
    np.savez_compressed(os.path.join(HERE, "softmaxflashv2.npz"), x=x[rows], golden_max=gmax[rows], golden_sum=gsum[rows])


def quant(ref):
    p = os.path.join(ref, EX, "04_advanced_api/03_quantization/quant/scripts/gen_data.py")
    out = {}
    for arch, tag in (("dav-2201", "f16"), ("dav-3510", "f32")):
        mod = load_module(p, "ref_quant_" + tag)
        with tempfile.TemporaryDirectory() as tmp:
            cwd = os.getcwd()
            os.chdir(tmp)
            try:
                np.random.seed(14)
                mod.gen_golden_data_simple(arch)
                out["src_" + tag] = np.fromfile("input/input.bin", np.float32)
                out["golden_" + tag] = np.fromfile("output/golden.bin", np.int8)
            finally:
                os.chdir(cwd)
    np.savez_compressed(os.path.join(HERE, "quant.npz"), **out)


def antiquant(ref):
    p = os.path.join(ref, EX, "04_advanced_api/03_quantization/antiquant/scripts/gen_data.py")
    out = {}
    for arch, tag in (("dav-2201", "f16math"), ("dav-3510", "f32math")):
        mod = load_module(p, "ref_antiquant_" + tag)
        with tempfile.TemporaryDirectory() as tmp:
            cwd = os.getcwd()
            os.chdir(tmp)
            try:
                mod.gen_golden_data_simple(arch)   # seeds numpy itself
                out["src"] = np.fromfile("input/input_src.bin", np.int8).reshape(8, 128)
                out["offset"] = np.fromfile("input/input_offset.bin", np.float16)
                out["scale"] = np.fromfile("input/input_scale.bin", np.float16)
                out["golden_" + tag] = np.fromfile("output/golden.bin", np.float16).reshape(8, 128)
            finally:
                os.chdir(cwd)
    np.savez_compressed(os.path.join(HERE, "antiquant.npz"), **out)


def dequant(ref):
    files = run_script_in_tmp(os.path.join(ref, EX, "04_advanced_api/03_quantization/dequant/scripts/gen_data.py"), 15)
    np.savez_compressed(os.path.join(HERE, "dequant.npz"),
                        src=np.frombuffer(files["input/input.bin"], np.int32).reshape(128, 32),
                        scale=np.frombuffer(files["input/scale.bin"], np.float32),
                        golden=np.frombuffer(files["output/golden.bin"], np.float32).reshape(128, 32))


def grouped(ref):
    mod = load_module(os.path.join(ref, EX, "05_best_practices/03_fusion_compute/quant_group_matmul_high_performance/scripts/gen_data.py"),
                      "ref_grouped")
    rng = np.random.default_rng(16)
    G, k, n = 4, 256, 96
    counts = np.array([40, 0, 7, 81], dtype=np.int64)
    m = int(counts.sum())
    x = rng.integers(-10, 10, (m, k)).astype(np.int8)
    w = rng.integers(-10, 10, (G, k, n)).astype(np.int8)
    scale = rng.normal(0, 0.01, (G, n)).astype(np.float32)
    tok = rng.normal(0, 0.01, (m, 1)).astype(np.float32)
    mm = np.empty((m, n), np.float32)
    idx = [0] + np.cumsum(counts).tolist()
    for i in range(G):  # gen_data.py:45-52
        s, e = idx[i], idx[i + 1]
        mm[s:e] = np.dot(x[s:e].astype(np.float32), w[i].astype(np.float32))
        mm[s:e] *= scale[i] * tok[s:e]
    np.savez_compressed(os.path.join(HERE, "grouped.npz"), x=x, w=w, counts=counts, scale=scale, tok=tok[:, 0],
                        golden_linear=mm, golden_gelu=mod.FastGelu(mm).astype(np.float16))


def mxfp4(ref):
    import ml_dtypes
    rng = np.random.default_rng(17)
    m, n, k = 48, 80, 256
    sk = int(np.ceil(k / 64) * 2)
    grid = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    ca = rng.integers(0, 16, (m, k)).astype(np.uint8)
    cb = rng.integers(0, 16, (n, k)).astype(np.uint8)  # K-major B ([N,K]) = the isTransB path
    x1 = grid[ca].astype(ml_dtypes.float4_e2m1fn)
    x2 = grid[cb].astype(ml_dtypes.float4_e2m1fn)
    assert (x1.view(np.uint8) & 15 == ca).all() and (x2.view(np.uint8) & 15 == cb).all()
    s1 = rng.integers(120, 134, (m, sk)).astype(np.uint8)
    s2 = rng.integers(120, 134, (n, sk)).astype(np.uint8)
    x1f = x1.astype(np.float64) * np.repeat(2.0 ** (s1.astype(np.float64) - 127), 32, axis=1)  # gen_data.py:51-57
    x2f = x2.astype(np.float64) * np.repeat(2.0 ** (s2.astype(np.float64) - 127), 32, axis=1)
    golden = np.matmul(x1f, x2f.T)
    pa = (ca[:, 0::2] | (ca[:, 1::2] << 4)).astype(np.uint8)  # pack_two_fp4: even index in the low nibble
    pb = (cb[:, 0::2] | (cb[:, 1::2] << 4)).astype(np.uint8)
    np.savez_compressed(os.path.join(HERE, "mxfp4.npz"), a=pa, b=pb, sa=s1, sb=s2, golden_f64=golden,
                        golden_bf16_bits=golden.astype(ml_dtypes.bfloat16).view(np.uint16))


def function_from_file(path, name):
    """Compiles one top-level function of a Python file without importing the file (whose imports may be unavailable)."""
    import ast
    tree = ast.parse(open(path).read())
    fn = next(node for node in tree.body if isinstance(node, ast.FunctionDef) and node.name == name)
    ns = {"np": np}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), path, "exec"), ns)
    return ns[name]


def mxfp4_nd(ref):
    import ml_dtypes
    path = os.path.join(ref, EX, "05_best_practices/01_matrix_compute/matmul_mxfp4_high_performance/scripts/gen_data.py")
    pack_two_fp4 = function_from_file(path, "pack_two_fp4")
    rng = np.random.default_rng(23)
    m, n, k = 48, 80, 256
    sk = int(np.ceil(k / 64) * 2)
    grid = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    ca = rng.integers(0, 16, (m, k)).astype(np.uint8)      # A [M, K]
    cb = rng.integers(0, 16, (k, n)).astype(np.uint8)      # B [K, N]: not transposed, the example's layout
    x1 = grid[ca].astype(ml_dtypes.float4_e2m1fn)
    x2 = grid[cb].astype(ml_dtypes.float4_e2m1fn)
    s1 = rng.integers(120, 134, (m, sk)).astype(np.uint8)  # scaleA [M, sK]
    s2 = rng.integers(120, 134, (sk, n)).astype(np.uint8)  # scaleB [sK, N]
    x1f = x1.astype(np.float64) * np.repeat(2.0 ** (s1.astype(np.float64) - 127), 32, axis=1)
    x2f = x2.astype(np.float64) * np.repeat(2.0 ** (s2.astype(np.float64) - 127), 32, axis=0)
    golden = np.matmul(x1f, x2f)
    np.savez_compressed(
        os.path.join(HERE, "mxfp4_nd.npz"),
        a=pack_two_fp4(x1), b_nd=pack_two_fp4(x2),                                           # gen_data.py:64-65
        a_t=pack_two_fp4(np.ascontiguousarray(x1.T)),                                        # A stored [K, M]
        sa=s1, sb_paired=np.ascontiguousarray(s2.reshape(sk // 2, 2, n).transpose(0, 2, 1)),  # gen_data.py:63
        sa_paired=np.ascontiguousarray(s1.T.reshape(sk // 2, 2, m).transpose(0, 2, 1)),      # matmul_mx gen_data.py:71-74
        b_kmajor=pack_two_fp4(np.ascontiguousarray(x2.T)), sb=np.ascontiguousarray(s2.T),    # the transposed-B form of the same operands
        golden_f64=golden)


def mxfp8(ref):
    files = run_script_in_tmp(os.path.join(ref, EX, "04_advanced_api/00_matmul/matmul_mx/scripts/gen_data.py"), 29)
    m, n, k = 32, 128, 128
    np.savez_compressed(os.path.join(HERE, "mxfp8.npz"),
                        a=np.frombuffer(files["input/x1_gm.bin"], np.uint8).reshape(m, k),
                        b_kn=np.frombuffer(files["input/x2_gm.bin"], np.uint8).reshape(k, n),
                        sa=np.frombuffer(files["input/x1_mx_gm.bin"], np.uint8).reshape(m, k // 32),
                        sb_paired=np.frombuffer(files["input/x2_mx_gm.bin"], np.uint8).reshape(k // 64, n, 2),
                        golden=np.frombuffer(files["output/golden.bin"], np.float32).reshape(m, n))


def casts(ref):
    # precision_conversion.md: the CAST_RINT rule and its worked examples, plus hand-derived boundary cases
    np.savez_compressed(
        os.path.join(HERE, "casts.npz"),
        # float -> half, CAST_RINT: 2^-24 ties and neighbours, max half, overflow saturates
        f32_to_f16_in=np.array([1.0, 1.00048828125, 1.000732421875, 65504.0, 65520.0, 1e6, -1e6, 2.98e-8, 5.96e-8], np.float32),
        f32_to_f16_out=np.array([0x3C00, 0x3C00, 0x3C01, 0x7BFF, 0x7BFF, 0x7BFF, 0xFBFF, 0x0000, 0x0001], np.uint16),
        # float -> int8, CAST_RINT with saturation
        f32_to_s8_in=np.array([0.5, 1.5, 2.5, -0.5, -1.5, 64.5, 126.5, 127.5, 300.0, -128.5, -129.0, -1e9], np.float32),
        f32_to_s8_out=np.array([0, 2, 2, 0, -2, 64, 126, 127, 127, -128, -128, -128], np.int8),
        # float -> bf16, CAST_RINT
        f32_to_bf16_in=np.array([1.0, 1.00390625, 1.005859375, 1.01171875, 3.3895314e38], np.float32),
        f32_to_bf16_out=np.array([0x3F80, 0x3F80, 0x3F81, 0x3F82, 0x7F7F], np.uint16),
    )


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("ASC_REFERENCE_ROOT", "reference"))
    args = ap.parse_args()
    for fn in (fixpipe, matmul_fp16, matmul_quant, softmax, logsoftmax, softmaxgrad, softmaxflashv2, quant, antiquant, dequant, grouped, mxfp4, mxfp4_nd, mxfp8, casts):
        fn(args.ref)
        print("wrote", fn.__name__)
