/*
 * CPU oracle for the Ascend C high-level operator hot path (TEST INFRASTRUCTURE, not product).
 *
 * This file restates, in plain C, the arithmetic that the reference's adv_api Matmul / SoftMax /
 * AscendQuant / AscendDequant perform.  The reference executes that arithmetic inside the closed
 * CANN CPU twin (tikicpulib: mad, mad_mx, copy_matrix_cc_to_gm, vector ops), which is not part of
 * the reference tree, so every function below follows the reference call site, its documentation
 * and its own golden-data scripts, cited per function (paths relative to the reference project).
 *
 * Parity pin: the fixpipe epilogues are pinned against the reference's algorithm scripts
 * (fixpipe_l0c2gm/scripts/gen_data_{s322s8,f322s8,s322f16}.py), the casts against the worked
 * examples of precision_conversion.md, and the GEMM / softmax / quant / dequant bodies against
 * the example generators' numpy recipes; the fixtures live in tests/golden.  The reference's own
 * kernel unit tests assert only all-zero outputs, so there are no stored result vectors to pin to.
 *
 * Only tests, the smoke check and the benchmark's cpu_baseline / reference arm may link this file.
 * Build: gcc -O3 -march=x86-64-v3 -ffp-contract=off -fopenmp -shared -fPIC.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* dtype codes shared with include/ascb200.h */
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2, ORC_S8 = 3, ORC_S32 = 4, ORC_FP4_E2M1 = 5, ORC_FP8_E4M3 = 6, ORC_FP8_E5M2 = 7 };

/* ---------------------------------------------------------------------------------------------
 * Scalar conversions.  CAST_RINT = round to nearest, ties to even
 * (docs/zh/api/SIMD-API/basic_api/data_structures/precision_conversion.md:19-23).
 * ------------------------------------------------------------------------------------------- */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

ORC_API float orc_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return u2f(sign);
        float v = (float)man * 5.9604644775390625e-08f; /* 2^-24 */
        return sign ? -v : v;
    }
    if (exp == 31) return u2f(sign | 0x7F800000u | (man << 13));
    return u2f(sign | ((exp + 112u) << 23) | (man << 13));
}

/* fp32 -> fp16, RINT.  sat != 0 clamps overflow to +-65504 (the reference's RndR SatS vector cast,
 * impl/adv_api/detail/quantization/quant/ascend_quant_3510_impl.h:96); sat == 0 gives IEEE inf. */
static inline uint16_t f32_to_f16(float f, int sat)
{
    uint32_t u = f2u(f);
    uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);          /* NaN */
    if (a >= 0x477FF000u) {                                          /* rounds to >= 65520 */
        if (a == 0x7F800000u && !sat) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | (sat ? 0x7BFFu : 0x7C00u));
    }
    if (a < 0x33000001u) return sign;                                /* |f| <= 2^-25 -> 0 */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }               /* subnormal half */
    else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7FFFFFu; }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q));                            /* carry into exponent is right */
}
ORC_API uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f, 0); }
ORC_API uint16_t orc_f32_to_f16_sat(float f) { return f32_to_f16(f, 1); }

ORC_API float orc_bf16_to_f32(uint16_t b) { return u2f((uint32_t)b << 16); }
ORC_API uint16_t orc_f32_to_bf16(float f)
{
    uint32_t u = f2u(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}

/* float -> int8, RINT with saturation (precision_conversion.md:379-382). NaN -> 0. */
static inline int8_t f32_to_s8_rint_sat(float f)
{
    if (f != f) return 0;
    if (f >= 127.0f) return 127;
    if (f <= -128.0f) return -128;
    return (int8_t)nearbyintf(f);
}
ORC_API int8_t orc_f32_to_s8(float f) { return f32_to_s8_rint_sat(f); }

/* fp4 e2m1 nibble -> value {0,.5,1,1.5,2,3,4,6} with sign; e8m0 byte -> 2^(b-127)
 * (docs/zh/api/SIMD-API/basic_api/cube_compute_ISASI/mmad_compute/MmadMx.md:71-75). */
static const float k_e2m1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
ORC_API float orc_e2m1_to_f32(uint8_t nib)
{
    float v = k_e2m1[nib & 7u];
    return (nib & 8u) ? -v : v;
}
ORC_API float orc_e8m0_to_f32(uint8_t b)
{
    if (b == 255) return NAN;
    if (b == 0) return u2f(0x00400000u); /* 2^-127 */
    return u2f((uint32_t)b << 23);
}

/* The (1,8,10) scale that fixpipe reads from bits [31:13] of the 64-bit quant parameter
 * (examples/01_simd_cpp_api/03_basic_api/03_matrix_compute/fixpipe_l0c2gm/scripts/gen_data_s322s8.py:35-58;
 *  equivalently float(bits & 0xFFFFE000), 04_advanced_api/00_matmul/matmul_quant/scripts/gen_data.py:37-40). */
ORC_API float orc_quant_alpha(uint64_t q) { return u2f((uint32_t)(q & 0xFFFFE000u)); }
static inline int quant_offset9(uint64_t q)
{
    /* gen_data_s322s8.py:46 reads the 9 bits as an unsigned value; the documentation calls the
     * field a signed 9-bit offset.  Interpret two's complement: the scripts only use offset 0. */
    int o = (int)((q >> 37) & 0x1FFu);
    return (o & 0x100) ? o - 512 : o;
}

/* ---------------------------------------------------------------------------------------------
 * GEMM bodies.  Accumulation follows the adv_api scheduler: one output block accumulates K in
 * sequential baseK chunks, the first chunk initialises (bias first when enabled)
 * (impl/adv_api/detail/matmul/scheduler/base/scheduler_norm.h:193-296,
 *  impl/adv_api/detail/matmul/scheduler/bias/bias_scheduler_v220.h:85-135).
 * Inside a chunk the summation order of the cube unit is not documented; we sum k ascending.
 * ------------------------------------------------------------------------------------------- */

/* C[M,N] fp32 = A*B (+bias).  A is [M,K] (lda) or, transA, [K,M]; B is [K,N] (ldb) or, transB, [N,K].
 * Elements are fp16 (is_bf16 == 0) or bf16.  Mmad.md:186-237 (fp16/bf16 in, fp32 accumulate). */
ORC_API void orc_gemm_f16(const uint16_t* A, const uint16_t* B, const float* bias, float* C, int M, int N, int K,
                          int lda, int ldb, int transA, int transB, int is_bf16, int baseK)
{
    if (baseK <= 0) baseK = K;
    float* Af = (float*)malloc((size_t)M * K * sizeof(float));
    float* Bt = (float*)malloc((size_t)N * K * sizeof(float)); /* [N,K] */
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int k = 0; k < K; ++k) {
            uint16_t v = transA ? A[(size_t)k * lda + m] : A[(size_t)m * lda + k];
            Af[(size_t)m * K + k] = is_bf16 ? orc_bf16_to_f32(v) : orc_f16_to_f32(v);
        }
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k) {
            uint16_t v = transB ? B[(size_t)n * ldb + k] : B[(size_t)k * ldb + n];
            Bt[(size_t)n * K + k] = is_bf16 ? orc_bf16_to_f32(v) : orc_f16_to_f32(v);
        }
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        const float* a = Af + (size_t)m * K;
        for (int n = 0; n < N; ++n) {
            const float* b = Bt + (size_t)n * K;
            float acc = bias ? bias[n] : 0.0f;
            for (int k0 = 0; k0 < K; k0 += baseK) {
                int k1 = k0 + baseK < K ? k0 + baseK : K;
                float part = 0.0f;
                for (int k = k0; k < k1; ++k) part += a[k] * b[k];
                acc += part;
            }
            C[(size_t)m * N + n] = acc;
        }
    }
    free(Af);
    free(Bt);
}

/* int8 x int8 -> int32 (+ int32 bias), exact.  Mmad.md:186-237 (s8 in, s32 accumulate). */
ORC_API void orc_gemm_i8(const int8_t* A, const int8_t* B, const int32_t* bias, int32_t* C, int M, int N, int K,
                         int lda, int ldb, int transA, int transB)
{
    int8_t* Ar = (int8_t*)A;
    int8_t* Bt = (int8_t*)B;
    if (transA) {
        Ar = (int8_t*)malloc((size_t)M * K);
        for (int m = 0; m < M; ++m)
            for (int k = 0; k < K; ++k) Ar[(size_t)m * K + k] = A[(size_t)k * lda + m];
        lda = K;
    }
    if (!transB) {
        Bt = (int8_t*)malloc((size_t)N * K);
#pragma omp parallel for schedule(static)
        for (int n = 0; n < N; ++n)
            for (int k = 0; k < K; ++k) Bt[(size_t)n * K + k] = B[(size_t)k * ldb + n];
        ldb = K;
    }
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        const int8_t* a = Ar + (size_t)m * lda;
        for (int n = 0; n < N; ++n) {
            const int8_t* b = Bt + (size_t)n * ldb;
            int32_t acc = bias ? bias[n] : 0;
            for (int k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            C[(size_t)m * N + n] = acc;
        }
    }
    if (transA) free(Ar);
    if (!transB) free(Bt);
}

/* MX matmul, fp4 e2m1 operands, one e8m0 scale per 32 K elements, fp32 accumulate
 * (MmadMx.md:71-75,160-171).  Both operands K-major: A [M,K/2] bytes, B [N,K/2] bytes, low nibble
 * = even k (05_best_practices/01_matrix_compute/matmul_mxfp4_high_performance/scripts/gen_data.py:25-36);
 * sA [M,K/32], sB [N,K/32].  Every product (value x value x 2^e) is exact in fp32; the sum is taken
 * in double per baseK chunk and rounded to fp32 once per chunk, the chunks added in fp32 - the
 * reference golden sums in float64 (gen_data.py:51-59). */
ORC_API void orc_gemm_mxf4(const uint8_t* A, const uint8_t* sA, const uint8_t* B, const uint8_t* sB, const float* bias,
                           float* C, int M, int N, int K, int baseK)
{
    if (baseK <= 0) baseK = K;
    const int K2 = K / 2, KS = K / 32;
    float* Af = (float*)malloc((size_t)M * K * sizeof(float));
    float* Bf = (float*)malloc((size_t)N * K * sizeof(float));
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int k = 0; k < K; ++k) {
            uint8_t byte = A[(size_t)m * K2 + k / 2];
            Af[(size_t)m * K + k] = orc_e2m1_to_f32((k & 1) ? (byte >> 4) : (byte & 15)) * orc_e8m0_to_f32(sA[(size_t)m * KS + k / 32]);
        }
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k) {
            uint8_t byte = B[(size_t)n * K2 + k / 2];
            Bf[(size_t)n * K + k] = orc_e2m1_to_f32((k & 1) ? (byte >> 4) : (byte & 15)) * orc_e8m0_to_f32(sB[(size_t)n * KS + k / 32]);
        }
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        const float* a = Af + (size_t)m * K;
        for (int n = 0; n < N; ++n) {
            const float* b = Bf + (size_t)n * K;
            float acc = bias ? bias[n] : 0.0f;
            for (int k0 = 0; k0 < K; k0 += baseK) {
                int k1 = k0 + baseK < K ? k0 + baseK : K;
                double part = 0.0;
                for (int k = k0; k < k1; ++k) part += (double)a[k] * (double)b[k];
                acc += (float)part;
            }
            C[(size_t)m * N + n] = acc;
        }
    }
    free(Af);
    free(Bf);
}

/* fp8 -> fp32: e4m3fn (bias 7, no infinities, 0x7F / 0xFF are NaN) or e5m2 (bias 15, IEEE-like infinities and NaNs). */
ORC_API float orc_fp8_to_f32(uint8_t v, int e5m2)
{
    const int mbits = e5m2 ? 2 : 3, bias = e5m2 ? 15 : 7;
    const int sign = v >> 7, exp = (v & 0x7F) >> mbits, man = v & ((1 << mbits) - 1);
    float f;
    if (e5m2 && exp == 31) f = man ? NAN : INFINITY;
    else if (!e5m2 && exp == 15 && man == 7) f = NAN;
    else if (exp == 0) f = ldexpf((float)man, 1 - bias - mbits);
    else f = ldexpf((float)(man | (1 << mbits)), exp - bias - mbits);
    return sign ? -f : f;
}

/* MX matmul with fp8 operands (e4m3fn or e5m2, one byte per element), one e8m0 scale per 32 K elements, fp32 result
 * (MmadMx.md:71-75,160-171; golden recipe examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul_mx/scripts/gen_data.py:60-68:
 * operands times 2^(scale - 127), float64 matmul, cast to fp32).  Both operands K-major: A [M,K], B [N,K], sA [M,K/32], sB [N,K/32].
 * Products are exact in double; summed in double per baseK chunk, the chunks added in fp32. */
ORC_API void orc_gemm_mxf8(const uint8_t* A, const uint8_t* sA, const uint8_t* B, const uint8_t* sB, const float* bias, float* C, int M, int N,
                           int K, int baseK, int e5m2)
{
    if (baseK <= 0) baseK = K;
    const int KS = K / 32;
    float* Af = (float*)malloc((size_t)M * K * sizeof(float));
    float* Bf = (float*)malloc((size_t)N * K * sizeof(float));
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int k = 0; k < K; ++k) Af[(size_t)m * K + k] = orc_fp8_to_f32(A[(size_t)m * K + k], e5m2) * orc_e8m0_to_f32(sA[(size_t)m * KS + k / 32]);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
        for (int k = 0; k < K; ++k) Bf[(size_t)n * K + k] = orc_fp8_to_f32(B[(size_t)n * K + k], e5m2) * orc_e8m0_to_f32(sB[(size_t)n * KS + k / 32]);
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        const float* a = Af + (size_t)m * K;
        for (int n = 0; n < N; ++n) {
            const float* b = Bf + (size_t)n * K;
            float acc = bias ? bias[n] : 0.0f;
            for (int k0 = 0; k0 < K; k0 += baseK) {
                int k1 = k0 + baseK < K ? k0 + baseK : K;
                double part = 0.0;
                for (int k = k0; k < k1; ++k) part += (double)a[k] * (double)b[k];
                acc += (float)part;
            }
            C[(size_t)m * N + n] = acc;
        }
    }
    free(Af);
    free(Bf);
}

/* ---------------------------------------------------------------------------------------------
 * Fixpipe epilogues (L0C -> GM).
 * ------------------------------------------------------------------------------------------- */

/* Plain cast of fp32 accumulators: F322F16 / F322BF16 are RINT
 * (docs/zh/api/SIMD-API/basic_api/cube_compute_ISASI/fixpipe/accompanying_quantization.md:5). */
ORC_API void orc_cast_f32(const float* acc, void* out, int dtype, size_t n, int relu)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        float v = acc[i];
        if (relu && v < 0.0f) v = 0.0f;
        if (dtype == ORC_F32) ((float*)out)[i] = v;
        else if (dtype == ORC_F16) ((uint16_t*)out)[i] = f32_to_f16(v, 1);
        else ((uint16_t*)out)[i] = orc_f32_to_bf16(v);
    }
}

static inline float clipf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* REQ8 / VREQ8: int32 -> int8.  gen_data_s322s8.py:69-89:
 *   f = float(x) * alpha (relu_alpha when x < 0); q = rint(clip(f,-256,255)) + offset9; out = rint(clip(q,-128,127)).
 * q points at one parameter (per_channel == 0) or N of them.  relu_mode: 0 none (relu_alpha = alpha), 1 relu (0). */
ORC_API void orc_fixpipe_req8(const int32_t* acc, int8_t* out, int M, int N, const uint64_t* q, int per_channel, int relu)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            uint64_t p = q[per_channel ? n : 0];
            float f = (float)acc[(size_t)m * N + n];
            f = (f >= 0.0f || !relu) ? f * orc_quant_alpha(p) : 0.0f;
            float t = nearbyintf(clipf(f, -256.0f, 255.0f)) + (float)quant_offset9(p);
            out[(size_t)m * N + n] = (int8_t)nearbyintf(clipf(t, -128.0f, 127.0f));
        }
}

/* QF322B8_PRE / VQF322B8_PRE: fp32 -> int8, same arithmetic on an fp32 accumulator (gen_data_f322s8.py:66-85). */
ORC_API void orc_fixpipe_qf322b8(const float* acc, int8_t* out, int M, int N, const uint64_t* q, int per_channel, int relu)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            uint64_t p = q[per_channel ? n : 0];
            float f = acc[(size_t)m * N + n];
            f = (f >= 0.0f || !relu) ? f * orc_quant_alpha(p) : 0.0f;
            float t = nearbyintf(clipf(f, -256.0f, 255.0f)) + (float)quant_offset9(p);
            out[(size_t)m * N + n] = (f != f) ? 0 : (int8_t)nearbyintf(clipf(t, -128.0f, 127.0f));
        }
}

/* fp32 -> fp8 (e4m3fn: 4 exponent bits, bias 7, no infinities, largest finite 448; e5m2: 5 exponent bits, bias 15, largest
 * finite 57344), round to nearest even, saturating to the largest finite value, NaN -> 0x7F (e4m3) / 0x7F (e5m2 quiet NaN).
 * Format definitions: OCP 8-bit floating point specification; the reference only names the mode (QF322FP8_PRE,
 * impl/adv_api/detail/matmul/stage/copy_cube_out/quant/quant_processor_fixpipe.h:103-104), its arithmetic lives in the closed
 * CPU twin, so saturation instead of overflow-to-NaN is this build's choice (the same as the GPU's cvt.rn.satfinite). */
ORC_API uint8_t orc_f32_to_fp8(float x, int e5m2)
{
    const int mbits = e5m2 ? 2 : 3, bias = e5m2 ? 15 : 7;
    const float maxv = e5m2 ? 57344.0f : 448.0f;
    uint32_t u;
    memcpy(&u, &x, 4);
    const uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    if (x != x) return (uint8_t)(sign | 0x7Fu);
    float a = fabsf(x);
    if (a >= maxv) a = maxv;  /* saturate (also infinities) */
    /* quantum of the binade: 2^(e - mbits), subnormals share the quantum of the smallest normal binade */
    int e;
    frexpf(a, &e);            /* a = f * 2^e, f in [0.5, 1) -> unbiased exponent e - 1 */
    int ue = e - 1;
    if (a == 0.0f || ue < 1 - bias) ue = 1 - bias;
    const float q = ldexpf(1.0f, ue - mbits);
    float r = nearbyintf(a / q) * q;  /* exact: division by a power of two; ties to even */
    if (r > maxv) r = maxv;
    if (r == 0.0f) return sign;
    int re;
    const float rf = frexpf(r, &re);
    int rue = re - 1;
    uint32_t bits;
    if (rue < 1 - bias) {  /* subnormal */
        bits = (uint32_t)nearbyintf(r / ldexpf(1.0f, 1 - bias - mbits));
    } else {
        const uint32_t man = (uint32_t)nearbyintf((rf * 2.0f - 1.0f) * (float)(1 << mbits));
        bits = ((uint32_t)(rue + bias) << mbits) | man;
    }
    return (uint8_t)(sign | bits);
}

/* QF322FP8_PRE / VQF322FP8_PRE (950 only): fp32 -> fp8 = fp8_sat(x * alpha), ReLU first when enabled. */
ORC_API void orc_fixpipe_qf322fp8(const float* acc, uint8_t* out, int M, int N, const uint64_t* q, int per_channel, int relu, int e5m2)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            uint64_t p = q[per_channel ? n : 0];
            float f = acc[(size_t)m * N + n];
            f = (f >= 0.0f || !relu) ? f * orc_quant_alpha(p) : 0.0f;
            out[(size_t)m * N + n] = orc_f32_to_fp8(f, e5m2);
        }
}

/* DEQF16 / VDEQF16: int32 -> half = half_sat(float(x) * alpha) (gen_data_s322f16.py:66-83). */
ORC_API void orc_fixpipe_deqf16(const int32_t* acc, uint16_t* out, int M, int N, const uint64_t* q, int per_channel, int relu)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            uint64_t p = q[per_channel ? n : 0];
            float f = (float)acc[(size_t)m * N + n];
            f = (f >= 0.0f || !relu) ? f * orc_quant_alpha(p) : 0.0f;
            out[(size_t)m * N + n] = f32_to_f16(f, 1);
        }
}

/* QS322BF16_PRE / VQS322BF16_PRE (950 only): int32 -> bf16 = bf16_rint(float(x) * alpha)
 * (impl/adv_api/detail/matmul/stage/copy_cube_out/quant/quant_processor_fixpipe.h:211-235). */
ORC_API void orc_fixpipe_qs322bf16(const int32_t* acc, uint16_t* out, int M, int N, const uint64_t* q, int per_channel, int relu)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            uint64_t p = q[per_channel ? n : 0];
            float f = (float)acc[(size_t)m * N + n];
            f = (f >= 0.0f || !relu) ? f * orc_quant_alpha(p) : 0.0f;
            out[(size_t)m * N + n] = orc_f32_to_bf16(f);
        }
}

/* Per-channel x per-token dequant that the grouped example applies after the int8 matmul:
 * AscendDequant (float(acc) * scale[n]) then Mul by perTokenScale[m], then Cast RINT
 * (examples/01_simd_cpp_api/05_best_practices/03_fusion_compute/quant_group_matmul_high_performance/
 *  quant_group_matmul_custom.asc:433,439,450).  act: 0 identity, 1 FasterGelu x*e^(.851(x-|x|))/(1+e^(-1.702|x|))
 *  (scripts/gen_data.py:19-23). */
ORC_API void orc_dequant_tok_ch(const int32_t* acc, void* out, int dtype, int M, int N, const float* tok, const float* ch, int act)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float v = (float)acc[(size_t)m * N + n] * ch[n];
            if (tok) v = v * tok[m];
            if (act == 1) {
                float ax = fabsf(v);
                v = v * expf(0.851f * (v - ax)) / (1.0f + expf(-1.702f * ax));
            }
            size_t i = (size_t)m * N + n;
            if (dtype == ORC_F32) ((float*)out)[i] = v;
            else if (dtype == ORC_F16) ((uint16_t*)out)[i] = f32_to_f16(v, 1);
            else ((uint16_t*)out)[i] = orc_f32_to_bf16(v);
        }
}

/* Grouped int8 matmul: rows of x are split into consecutive groups by counts[g] (counts, not a
 * cumulative sum; groups with count <= 0 are skipped, quant_group_matmul_custom.asc:263-264);
 * group g multiplies by W[g] ([N,K] when transB else [K,N]) and scale ch[g*N + n]. */
ORC_API void orc_grouped_i8(const int8_t* x, const int8_t* W, const int64_t* counts, int G, const float* tok, const float* ch,
                            void* out, int dtype, int K, int N, int transB, int act)
{
    int64_t row = 0;
    for (int g = 0; g < G; ++g) {
        int64_t mg = counts[g];
        if (mg <= 0) continue;
        int32_t* acc = (int32_t*)malloc((size_t)mg * N * sizeof(int32_t));
        orc_gemm_i8(x + (size_t)row * K, W + (size_t)g * N * K, NULL, acc, (int)mg, N, K, K, transB ? K : N, 0, transB);
        size_t esz = dtype == ORC_F32 ? 4 : 2;
        orc_dequant_tok_ch(acc, (char*)out + (size_t)row * N * esz, dtype, (int)mg, N, tok ? tok + row : NULL, ch + (size_t)g * N, act);
        free(acc);
        row += mg;
    }
}

/* ---------------------------------------------------------------------------------------------
 * SoftMax: per row x32 = float(x); max; e = exp(x32 - max); sum; y = e / sum; cast RINT
 * (impl/adv_api/detail/activation/softmax/membase/common/softmax_impl/softmax_generic_nd_impl.h:92-121,
 *  impl/adv_api/detail/common/common.h:27-28; formula docs SoftMax.md, golden
 *  examples/01_simd_cpp_api/04_advanced_api/01_activation/softmax/scripts/gen_data.py:23-37).
 * max/sum are written once per row (brc == 0) or broadcast over one 32-byte block (brc == 1:
 * 8 floats for fp32 statistics; include/adv_api/activation/softmax.h:92-109).
 * The reduction order of the vector unit is not documented; we sum k ascending in fp32.
 * ------------------------------------------------------------------------------------------- */
ORC_API void orc_softmax(const void* x, void* y, float* max_out, float* sum_out, int M, int K, int dtype, int brc)
{
    const int rep = brc ? 8 : 1;
#pragma omp parallel
    {
        float* row = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            float mx = -INFINITY;
            for (int k = 0; k < K; ++k) {
                float v = dtype == ORC_F16 ? orc_f16_to_f32(((const uint16_t*)x)[(size_t)m * K + k]) : ((const float*)x)[(size_t)m * K + k];
                row[k] = v;
                if (v > mx) mx = v;
            }
            float s = 0.0f;
            for (int k = 0; k < K; ++k) {
                row[k] = expf(row[k] - mx);
                s += row[k];
            }
            for (int k = 0; k < K; ++k) {
                float v = row[k] / s;
                if (dtype == ORC_F16) ((uint16_t*)y)[(size_t)m * K + k] = f32_to_f16(v, 1);
                else ((float*)y)[(size_t)m * K + k] = v;
            }
            for (int r = 0; r < rep; ++r) {
                max_out[(size_t)m * rep + r] = mx;
                sum_out[(size_t)m * rep + r] = s;
            }
        }
        free(row);
    }
}

/* ---------------------------------------------------------------------------------------------
 * LogSoftMax: the SoftMax above followed by y = ln(e / sum) * 0.4342944819 (= log10), all in fp32;
 * for half sources the row is widened to fp32 first and y, max and sum are cast to half RINT at the end
 * (impl/adv_api/detail/activation/softmax/membase/common/logsoftmax_common_impl.h:277-311 log step,
 *  :313-338 fp32, :341-376 half; constant SCALAR_NATURE_LOG_10 at :30; golden
 *  examples/01_simd_cpp_api/04_advanced_api/01_activation/logsoftmax/scripts/gen_data.py:19-33).
 * max/sum have the source dtype (include/adv_api/activation/logsoftmax.h:56-59): once per row (brc == 0)
 * or over one 32-byte block (brc == 1: 16 halves / 8 floats).
 * ------------------------------------------------------------------------------------------- */
ORC_API void orc_log_softmax(const void* x, void* y, void* max_out, void* sum_out, int M, int K, int dtype, int brc)
{
    const int rep = brc ? (dtype == ORC_F16 ? 16 : 8) : 1;
#pragma omp parallel
    {
        float* row = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            float mx = -INFINITY;
            for (int k = 0; k < K; ++k) {
                float v = dtype == ORC_F16 ? orc_f16_to_f32(((const uint16_t*)x)[(size_t)m * K + k]) : ((const float*)x)[(size_t)m * K + k];
                row[k] = v;
                if (v > mx) mx = v;
            }
            float s = 0.0f;
            for (int k = 0; k < K; ++k) {
                row[k] = expf(row[k] - mx);
                s += row[k];
            }
            for (int k = 0; k < K; ++k) {
                float v = logf(row[k] / s) * 0.4342944819f;
                if (dtype == ORC_F16) ((uint16_t*)y)[(size_t)m * K + k] = f32_to_f16(v, 1);
                else ((float*)y)[(size_t)m * K + k] = v;
            }
            for (int r = 0; r < rep; ++r) {
                if (dtype == ORC_F16) {
                    ((uint16_t*)max_out)[(size_t)m * rep + r] = f32_to_f16(mx, 1);
                    ((uint16_t*)sum_out)[(size_t)m * rep + r] = f32_to_f16(s, 1);
                } else {
                    ((float*)max_out)[(size_t)m * rep + r] = mx;
                    ((float*)sum_out)[(size_t)m * rep + r] = s;
                }
            }
        }
        free(row);
    }
}

/* ---------------------------------------------------------------------------------------------
 * SimpleSoftMax: y = exp(float(x) - float(inMax)) / float(inSum), cast RINT; the statistics are given
 * (impl/adv_api/detail/activation/softmax/membase/common/simple_softmax_common_impl.h:320-364 all half,
 *  :367-389 fp32, :466-502 half data with fp32 statistics).  rep = values stored per row.
 * ------------------------------------------------------------------------------------------- */
ORC_API void orc_simple_softmax(const void* x, void* y, const void* in_sum, const void* in_max, int M, int K, int dtype, int stats_dtype,
                                int rep)
{
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        const float mx = stats_dtype == ORC_F16 ? orc_f16_to_f32(((const uint16_t*)in_max)[(size_t)m * rep]) : ((const float*)in_max)[(size_t)m * rep];
        const float sm = stats_dtype == ORC_F16 ? orc_f16_to_f32(((const uint16_t*)in_sum)[(size_t)m * rep]) : ((const float*)in_sum)[(size_t)m * rep];
        for (int k = 0; k < K; ++k) {
            const float v = dtype == ORC_F16 ? orc_f16_to_f32(((const uint16_t*)x)[(size_t)m * K + k]) : ((const float*)x)[(size_t)m * K + k];
            const float r = expf(v - mx) / sm;
            if (dtype == ORC_F16) ((uint16_t*)y)[(size_t)m * K + k] = f32_to_f16(r, 1);
            else ((float*)y)[(size_t)m * K + k] = r;
        }
    }
}

/* ---------------------------------------------------------------------------------------------
 * SoftmaxGrad / SoftmaxGradFront: s = rowsum(float(grad) * float(src)); front: dst[m, rep] = s;
 * else dst = (grad - s) * src; fp32 arithmetic, cast RINT for half
 * (impl/adv_api/detail/activation/softmax/membase/common/softmax_grad_nd_impl.h:27-60; golden
 *  examples/01_simd_cpp_api/04_advanced_api/01_activation/softmaxgrad/scripts/gen_data.py:20-27).
 * rep = 32 / sizeof(T).  Row sums add k ascending.
 * ------------------------------------------------------------------------------------------- */
ORC_API void orc_softmax_grad(const void* grad, const void* src, void* dst, int M, int K, int dtype, int front)
{
    const int rep = dtype == ORC_F16 ? 16 : 8;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        float s = 0.0f;
        for (int k = 0; k < K; ++k) {
            const size_t i = (size_t)m * K + k;
            const float g = dtype == ORC_F16 ? orc_f16_to_f32(((const uint16_t*)grad)[i]) : ((const float*)grad)[i];
            const float y = dtype == ORC_F16 ? orc_f16_to_f32(((const uint16_t*)src)[i]) : ((const float*)src)[i];
            s += g * y;
        }
        if (front) {
            for (int r = 0; r < rep; ++r) {
                if (dtype == ORC_F16) ((uint16_t*)dst)[(size_t)m * rep + r] = f32_to_f16(s, 1);
                else ((float*)dst)[(size_t)m * rep + r] = s;
            }
            continue;
        }
        for (int k = 0; k < K; ++k) {
            const size_t i = (size_t)m * K + k;
            const float g = dtype == ORC_F16 ? orc_f16_to_f32(((const uint16_t*)grad)[i]) : ((const float*)grad)[i];
            const float y = dtype == ORC_F16 ? orc_f16_to_f32(((const uint16_t*)src)[i]) : ((const float*)src)[i];
            const float r = (g - s) * y;
            if (dtype == ORC_F16) ((uint16_t*)dst)[i] = f32_to_f16(r, 1);
            else ((float*)dst)[i] = r;
        }
    }
}

/* ---------------------------------------------------------------------------------------------
 * AscendQuant -> int8.  All arithmetic in fp16: src (and fp32 scale/offset) cast to half RINT with
 * saturation, Mul in half, Add in half, half -> int8 RINT with saturation
 * (impl/adv_api/detail/quantization/quant/ascend_quant_3510_impl.h:34-66 per tensor,
 *  :275-322 per channel half, :335-378 per channel fp32; default round mode CAST_RINT,
 *  include/adv_api/quantization/ascend_quant_utils.h:64,70).
 * ------------------------------------------------------------------------------------------- */
static inline uint16_t half_mul(uint16_t a, uint16_t b) { return f32_to_f16(orc_f16_to_f32(a) * orc_f16_to_f32(b), 0); }
static inline uint16_t half_add(uint16_t a, uint16_t b) { return f32_to_f16(orc_f16_to_f32(a) + orc_f16_to_f32(b), 0); }
static inline uint16_t load_as_half(const void* p, size_t i, int dtype)
{
    if (dtype == ORC_F16) return ((const uint16_t*)p)[i];
    if (dtype == ORC_BF16) return f32_to_f16(orc_bf16_to_f32(((const uint16_t*)p)[i]), 1);
    return f32_to_f16(((const float*)p)[i], 1);
}

ORC_API void orc_quant_per_tensor(const void* src, int8_t* dst, size_t n, int dtype, float scale, float offset)
{
    const uint16_t hs = f32_to_f16(scale, 0), ho = f32_to_f16(offset, 0); /* static_cast<half>(scale) */
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; ++i) {
        uint16_t v = half_add(half_mul(load_as_half(src, i, dtype), hs), ho);
        dst[i] = f32_to_s8_rint_sat(orc_f16_to_f32(v));
    }
}

/* scale has scale_count entries of the source dtype; offset is a tensor of the same kind
 * (offset_is_tensor) or one scalar of the source dtype passed in offset_scalar. */
ORC_API void orc_quant_per_channel(const void* src, int8_t* dst, int rows, int scale_count, int dtype, const void* scale,
                                   const void* offset_tensor, float offset_scalar)
{
    uint16_t hos = dtype == ORC_F32 ? f32_to_f16(offset_scalar, 1)
                 : dtype == ORC_BF16 ? f32_to_f16(orc_bf16_to_f32(orc_f32_to_bf16(offset_scalar)), 1)
                                     : f32_to_f16(offset_scalar, 0);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < scale_count; ++c) {
            size_t i = (size_t)r * scale_count + c;
            uint16_t hs = load_as_half(scale, c, dtype);
            uint16_t ho = offset_tensor ? load_as_half(offset_tensor, c, dtype) : hos;
            uint16_t v = half_add(half_mul(load_as_half(src, i, dtype), hs), ho);
            dst[i] = f32_to_s8_rint_sat(orc_f16_to_f32(v));
        }
}

/* ---------------------------------------------------------------------------------------------
 * AscendDequant: dst[i,j] = dstT(float(src[i,j]) * float(scale[j])) for j < cal_count; src rows
 * have n int32 each; dst rows have n_dst elements (n rounded up to a 32-byte multiple)
 * (impl/adv_api/detail/quantization/dequant/ascend_dequant_common_impl.h:261-365;
 *  golden examples/01_simd_cpp_api/04_advanced_api/03_quantization/dequant/scripts/gen_data.py:19-34).
 * scale_dtype: ORC_F32, ORC_BF16, or -1 for a single fp32 scalar in *scale.
 * ------------------------------------------------------------------------------------------- */
ORC_API void orc_dequant(const int32_t* src, void* dst, int m, int n, int cal_count, int n_dst, int dst_dtype, const void* scale,
                         int scale_dtype)
{
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < cal_count; ++j) {
            float s = scale_dtype == -1 ? ((const float*)scale)[0]
                    : scale_dtype == ORC_BF16 ? orc_bf16_to_f32(((const uint16_t*)scale)[j])
                                              : ((const float*)scale)[j];
            float v = (float)src[(size_t)i * n + j] * s;
            size_t o = (size_t)i * n_dst + j;
            if (dst_dtype == ORC_F32) ((float*)dst)[o] = v;
            else if (dst_dtype == ORC_F16) ((uint16_t*)dst)[o] = f32_to_f16(v, 1);
            else ((uint16_t*)dst)[o] = orc_f32_to_bf16(v);
        }
}

/* Sets the number of OpenMP threads of every later call (launchers such as torchrun export OMP_NUM_THREADS=1,
 * which would silently turn the timed CPU baseline into a single-core run). */
ORC_API void orc_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}


/* fp32 -> e2m1 code (sign, values 0, .5, 1, 1.5, 2, 3, 4, 6), round to nearest even code, saturating. */
ORC_API uint8_t orc_f32_to_e2m1(float x)
{
    const uint8_t sign = (x < 0.0f || (x == 0.0f && signbit(x))) ? 8u : 0u;
    const float a = fabsf(x);
    uint8_t c;
    if (a <= 0.25f) c = 0;          /* tie 0.25 -> 0 (even) */
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;     /* ties 0.75 and 1.25 -> 1.0 (even) */
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;      /* ties 1.75 and 2.5 -> 2.0 */
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;      /* ties 3.5 and 5.0 -> 4.0 */
    else c = 7;
    return (uint8_t)(sign | c);
}

/* AscendQuant with the PER_TOKEN (policy 2) and PER_GROUP (policy 3) policies, following the register code of
 * impl/adv_api/detail/quantization/quant/ascend_quant_per_group_3510_impl.h:34-80 (fp8: fp32 arithmetic), :143-178 and :499-538
 * (int8: arithmetic in the scale's type, then TransRegForS8 = round to nearest even, saturate,
 * impl/adv_api/detail/quantization/quant/ascend_quant_3510_impl.h:935-990), :347-381 (fp4: scale's type -> bfloat16 -> e2m1,
 * ascend_quant_3510_impl.h:992-1030; no offset).  Scale shapes: [m] | [m, ceil(n/group)] (k_dim 1) | [ceil(m/group), n] (k_dim 0). */
static float load_f32(const void* p, size_t i, int dtype)
{
    if (dtype == ORC_F16) return orc_f16_to_f32(((const uint16_t*)p)[i]);
    if (dtype == ORC_BF16) return orc_bf16_to_f32(((const uint16_t*)p)[i]);
    return ((const float*)p)[i];
}
static float round_to(float v, int dtype)
{
    if (dtype == ORC_F16) return orc_f16_to_f32(f32_to_f16(v, 0));
    if (dtype == ORC_BF16) return orc_bf16_to_f32(orc_f32_to_bf16(v));
    return v;
}
ORC_API void orc_quant_policy_rm(const void* src, uint8_t* dst, int m, int n, int src_dtype, int scale_dtype, int dst_dtype, int policy, int k_dim,
                                 int group_size, const void* scale, const void* offset_t, float offset_scalar, int has_offset, int round_mode);

/* fp32 -> int8 under a RoundMode of the reference (impl/basic_api/utils/kernel_utils_mode.h:103-120; the rules and worked examples of
 * docs/zh/api/SIMD-API/basic_api/data_structures/precision_conversion.md): 1 RINT nearest even, 2 FLOOR, 3 CEIL, 4 ROUND halves away
 * from zero, 5 TRUNC; saturating, NaN -> 0. */
ORC_API int8_t orc_f32_to_s8_mode(float f, int round_mode)
{
    if (f != f) return 0;
    float r;
    switch (round_mode) {
        case 2: r = floorf(f); break;
        case 3: r = ceilf(f); break;
        case 4: r = roundf(f); break;
        case 5: r = truncf(f); break;
        default: return f32_to_s8_rint_sat(f);
    }
    return (int8_t)(r < -128.0f ? -128.0f : r > 127.0f ? 127.0f : r);
}

ORC_API void orc_quant_policy(const void* src, uint8_t* dst, int m, int n, int src_dtype, int scale_dtype, int dst_dtype, int policy, int k_dim,
                              int group_size, const void* scale, const void* offset_t, float offset_scalar, int has_offset)
{
    orc_quant_policy_rm(src, dst, m, n, src_dtype, scale_dtype, dst_dtype, policy, k_dim, group_size, scale, offset_t, offset_scalar, has_offset, 1);
}

/* AscendQuant PER_TOKEN / PER_GROUP with config.roundMode applied to the final conversion of int8 destinations
 * (include/adv_api/quantization/ascend_quant_utils.h:55-64). */
ORC_API void orc_quant_policy_rm(const void* src, uint8_t* dst, int m, int n, int src_dtype, int scale_dtype, int dst_dtype, int policy, int k_dim,
                                 int group_size, const void* scale, const void* offset_t, float offset_scalar, int has_offset, int round_mode)
{
    const int scale_cols = policy == 3 ? (n + group_size - 1) / group_size : 1;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            const size_t si = policy == 2 ? (size_t)i : (k_dim == 1 ? (size_t)i * scale_cols + j / group_size : (size_t)(i / group_size) * n + j);
            const float x = load_f32(src, (size_t)i * n + j, src_dtype);
            const float s = load_f32(scale, si, scale_dtype);
            const float o = offset_t ? load_f32(offset_t, si, scale_dtype) : round_to(offset_scalar, scale_dtype);
            float v;
            if (dst_dtype == ORC_FP8_E4M3 || dst_dtype == ORC_FP8_E5M2) {
                v = x * s;
                if (has_offset) v = v + o;
                dst[(size_t)i * n + j] = orc_f32_to_fp8(v, dst_dtype == ORC_FP8_E5M2);
                continue;
            }
            /* products and sums of 16-bit floats are computed in fp32 and rounded once to the 16-bit type */
            v = round_to(x * s, scale_dtype);
            if (has_offset && dst_dtype != ORC_FP4_E2M1) v = round_to(v + o, scale_dtype);
            if (dst_dtype == ORC_S8) {
                dst[(size_t)i * n + j] = (uint8_t)orc_f32_to_s8_mode(v, round_mode);
            } else {
                const uint8_t c = orc_f32_to_e2m1(orc_bf16_to_f32(orc_f32_to_bf16(v)));
                uint8_t* b = dst + ((size_t)i * n + j) / 2;
                const int hi = (int)(((size_t)i * n + j) & 1);
                /* n is even: a byte is written by one thread only */
                *b = hi ? (uint8_t)((*b & 0x0F) | (c << 4)) : (uint8_t)((*b & 0xF0) | c);
            }
        }
}


/* AscendDequant PER_TOKEN (policy 0) / PER_GROUP (policy 1): dst = cast(float(src) * float(scale))
 * (impl/adv_api/detail/quantization/dequant/ascend_dequant_3510_impl.h:253-286, 345-600). */
ORC_API void orc_dequant_policy(const void* src, void* dst, int m, int n, int src_is_f32, int scale_dtype, int dst_dtype, int policy, int k_dim,
                                int group_size, const void* scale)
{
    const int scale_cols = policy == 1 ? (n + group_size - 1) / group_size : 1;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            const size_t e = (size_t)i * n + j;
            const size_t si = policy == 0 ? (size_t)i : (k_dim == 1 ? (size_t)i * scale_cols + j / group_size : (size_t)(i / group_size) * n + j);
            const float x = src_is_f32 ? ((const float*)src)[e] : (float)((const int32_t*)src)[e];
            const float v = x * load_f32(scale, si, scale_dtype);
            if (dst_dtype == ORC_F32) ((float*)dst)[e] = v;
            else if (dst_dtype == ORC_F16) ((uint16_t*)dst)[e] = f32_to_f16(v, 1);
            else ((uint16_t*)dst)[e] = orc_f32_to_bf16(v);
        }
}


/* SoftmaxFlashV2 (docs/zh/api/SIMD-API/adv_api/activation_functions/SoftMax_interface/SoftmaxFlashV2.md:49-63):
 *   update 0: max = rowmax(x); y = exp(x - max); sum = rowsum(y)
 *   update 1: max = max(inmax, rowmax(x)); y = exp(x - max); expmax = exp(inmax - max); sum = expmax * insum + rowsum(y)
 * fp32 arithmetic; x / y / expmax in `dtype`, max / sum tensors in `stats_dtype`; per-row values repeated over one 32-byte block
 * when brc is set. */
static void stat_put(void* p, size_t i, float v, int dtype)
{
    if (dtype == ORC_F16) ((uint16_t*)p)[i] = f32_to_f16(v, 1);
    else ((float*)p)[i] = v;
}
static void softmax_flash_rows(const void* x, void* y, void* sum_out, void* max_out, void* expmax_out, const void* in_sum, const void* in_max,
                               int M, int K, int dtype, int stats_dtype, int update, int brc, int normalise)
{
    const int srep = brc ? 32 / (stats_dtype == ORC_F16 ? 2 : 4) : 1, erep = brc ? 32 / (dtype == ORC_F16 ? 2 : 4) : 1;
#pragma omp parallel
    {
        float* row = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (int m = 0; m < M; ++m) {
            float mx = -INFINITY;
            for (int k = 0; k < K; ++k) {
                row[k] = load_f32(x, (size_t)m * K + k, dtype);
                if (row[k] > mx) mx = row[k];
            }
            float em = 1.0f, old_sum = 0.0f;
            if (update) {
                const float old_max = load_f32(in_max, (size_t)m * srep, stats_dtype);
                old_sum = load_f32(in_sum, (size_t)m * srep, stats_dtype);
                if (old_max > mx) mx = old_max;
                em = expf(old_max - mx);
            }
            float s = 0.0f;
            for (int k = 0; k < K; ++k) {
                row[k] = expf(row[k] - mx);
                s += row[k];
            }
            if (update) s = em * old_sum + s;
            if (normalise && update) em = em * old_sum / s;
            for (int k = 0; k < K; ++k) stat_put(y, (size_t)m * K + k, normalise ? row[k] / s : row[k], dtype);
            for (int r = 0; r < srep; ++r) {
                stat_put(sum_out, (size_t)m * srep + r, s, stats_dtype);
                stat_put(max_out, (size_t)m * srep + r, mx, stats_dtype);
            }
            if (update)
                for (int r = 0; r < erep; ++r) stat_put(expmax_out, (size_t)m * erep + r, em, dtype);
        }
        free(row);
    }
}

ORC_API void orc_softmax_flash_v2(const void* x, void* y, void* sum_out, void* max_out, void* expmax_out, const void* in_sum, const void* in_max,
                                  int M, int K, int dtype, int stats_dtype, int update, int brc)
{
    softmax_flash_rows(x, y, sum_out, max_out, expmax_out, in_sum, in_max, M, K, dtype, stats_dtype, update, brc, 0);
}

/* SoftmaxFlash, the first version (docs/zh/api/SIMD-API/adv_api/activation_functions/SoftMax_interface/SoftmaxFlash.md:43-62):
 * the V2 step followed by the normalisation: sum as above, expmax = exp(inmax - max) * insum / sum, y = exp(x - max) / sum;
 * without update it is SoftMax. */
ORC_API void orc_softmax_flash(const void* x, void* y, void* sum_out, void* max_out, void* expmax_out, const void* in_sum, const void* in_max,
                               int M, int K, int dtype, int stats_dtype, int update, int brc)
{
    softmax_flash_rows(x, y, sum_out, max_out, expmax_out, in_sum, in_max, M, K, dtype, stats_dtype, update, brc, 1);
}

/* ---------------------------------------------------------------------------------------------
 * AscendAntiQuant, int8 source: dst = scale * (src + offset)
 * (impl/adv_api/detail/quantization/antiquant/ascend_antiquant_3510_impl.h: per tensor half :336-358 (half add, half mul),
 *  per tensor bfloat16 :360-392 (fp32 add, fp32 mul, one cast), per channel along the row :461-495 (add and mul in the output
 *  type), per channel transposed :615-645 half / :647-690 bfloat16 in fp32; golden
 *  examples/01_simd_cpp_api/04_advanced_api/03_quantization/antiquant/scripts/gen_data.py:21-44).
 * mode 0 scalar pair, 1 one pair per column, 2 one pair per row; scale / offset in the output type (offset may be NULL).
 * ------------------------------------------------------------------------------------------- */
static inline uint16_t round16(float v, int dtype, int sat) { return dtype == ORC_F16 ? f32_to_f16(v, sat) : orc_f32_to_bf16(v); }
static inline float widen16(uint16_t v, int dtype) { return dtype == ORC_F16 ? orc_f16_to_f32(v) : orc_bf16_to_f32(v); }
ORC_API void orc_antiquant(const int8_t* src, uint16_t* dst, int rows, int cols, int dtype, int mode, const uint16_t* scale, const uint16_t* offset,
                           float scale_scalar, float offset_scalar)
{
    const uint16_t ss = round16(scale_scalar, dtype, 0), os = round16(offset_scalar, dtype, 0);
    const int f32_math = dtype == ORC_BF16 && mode != 1;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) {
            const int p = mode == 1 ? c : r;
            const float s = widen16(mode == 0 ? ss : scale[p], dtype);
            const float o = widen16((mode == 0 || !offset) ? os : offset[p], dtype);
            const float x = (float)src[(size_t)r * cols + c];
            uint16_t out;
            if (f32_math) out = round16((x + o) * s, dtype, 1);
            else out = round16(widen16(round16(x + o, dtype, 0), dtype) * s, dtype, 0);
            dst[(size_t)r * cols + c] = out;
        }
}
