// AscendQuant with the PER_TOKEN and PER_GROUP policies (include/adv_api/quantization/ascend_quant.h:682-790,
// impl/adv_api/detail/quantization/quant/ascend_quant_per_group_3510_impl.h): y = cast(x * scale [+ offset]) with one
// scale per row (PER_TOKEN), per group of `group_size` columns of a row (PER_GROUP, kDim = 1) or per group of rows and
// column (PER_GROUP, kDim = 0).  Destinations: int8, fp8 e4m3 / e5m2, and fp4 e2m1 (PER_GROUP only, no offset) - the
// producer of block-scaled operands.  Arithmetic follows the reference's register code:
//   fp8:  always fp32 (scale and offset widened), one rounding to fp8 (saturating);
//   int8: in the scale's type (fp32 when the scale is fp32, else half / bfloat16 multiply and add), then round to
//         nearest even and saturate (the reference goes fp32 -> int16 -> half -> int8, which is the same function);
//   fp4:  in the scale's type, then to bfloat16 (nearest even) and from there to e2m1 (nearest even, saturating).
// Element-wise and HBM bound: eight elements per thread, 16-byte loads, 8-byte (4-byte for fp4) stores.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdint>
#include <type_traits>

#include "ascb200.h"
#include "common.cuh"

namespace ascb200 {
namespace {

enum : int { POL_TOKEN = ASCB200_QUANT_PER_TOKEN, POL_GROUP = ASCB200_QUANT_PER_GROUP };

struct QuantPolicyArgs {
    const void* src;
    void* dst;
    const void* scale;
    const void* offset;  // tensor of the scale's shape, or nullptr
    float offset_scalar;
    int has_offset;
    int m, n;
    int policy, k_dim, group_size;
    int scale_cols;  // columns of the scale tensor for PER_GROUP
    int round_mode;  // RoundMode of the final conversion (int8 destinations): 1 RINT, 2 FLOOR, 3 CEIL, 4 ROUND (half away from zero), 5 TRUNC
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// x * s (+ o) in the scale's type ST, result widened to fp32 (exact).
template <typename ST>
__device__ __forceinline__ float mul_add_in(float x, ST s, ST o, bool has_offset)
{
    if constexpr (sizeof(ST) == 4) {
        float v = __fmul_rn(x, s);
        return has_offset ? __fadd_rn(v, o) : v;
    } else if constexpr (std::is_same<ST, __half>::value) {
        // the _rn forms are never contracted into a fused multiply-add: the reference multiplies, rounds, then adds
        __half v = __hmul_rn(__float2half_rn(x), s);  // x is a half widened exactly
        if (has_offset) v = __hadd_rn(v, o);
        return __half2float(v);
    } else {
        __nv_bfloat16 v = __hmul_rn(__float2bfloat16_rn(x), s);
        if (has_offset) v = __hadd_rn(v, o);
        return __bfloat162float(v);
    }
}

template <int DST>
__device__ __forceinline__ uint32_t to_byte(float v, int round_mode = 1)
{
    if constexpr (DST == ASCB200_S8) {
        int r;
        if (round_mode == 1) asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));  // NaN -> 0
        else if (round_mode == 2) asm("cvt.rmi.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
        else if (round_mode == 3) asm("cvt.rpi.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
        else if (round_mode == 5) asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
        else asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(roundf(v)));   // CAST_ROUND: halves away from zero, then exact
        return static_cast<uint32_t>(r) & 0xFFu;
    } else {
        uint16_t pair;
        if constexpr (DST == ASCB200_FP8_E4M3) asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.0f), "f"(v));
        else asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(0.0f), "f"(v));
        return pair & 0xFFu;
    }
}
// two values -> one byte of packed e2m1, first value in the low nibble; via bfloat16 like the reference
__device__ __forceinline__ uint32_t to_fp4_pair(float lo, float hi)
{
    lo = __bfloat162float(__float2bfloat16_rn(lo));
    hi = __bfloat162float(__float2bfloat16_rn(hi));
    uint16_t out;
    asm("{\n\t.reg .b8 b;\n\tcvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\n\tcvt.u16.u8 %0, b;\n\t}" : "=h"(out) : "f"(hi), "f"(lo));
    return out & 0xFFu;
}

template <typename T, typename ST, int DST>
__device__ __forceinline__ ST pick(const QuantPolicyArgs& a, const void* base, int row, int col)
{
    const ST* p = static_cast<const ST*>(base);
    if (a.policy == POL_TOKEN) return p[row];
    if (a.k_dim == 1) return p[static_cast<size_t>(row) * a.scale_cols + col / a.group_size];
    return p[static_cast<size_t>(row / a.group_size) * a.n + col];
}

// Row and column of element i, and the scale / offset of that element.
template <typename T, typename ST, int DST>
__device__ __forceinline__ void quant_policy_params(const QuantPolicyArgs& a, size_t i, ST off_scalar, int& row, int& col, ST& s, ST& o)
{
    // 32-bit division where the element index allows it (a 64-bit division costs more than the conversion of the eight values)
    row = i < 0xFFFFFFFFull ? static_cast<int>(static_cast<uint32_t>(i) / static_cast<uint32_t>(a.n)) : static_cast<int>(i / a.n);
    col = static_cast<int>(i - static_cast<size_t>(row) * a.n);
    s = pick<T, ST, DST>(a, a.scale, row, col);
    o = off_scalar;
    if (a.has_offset && a.offset) o = pick<T, ST, DST>(a, a.offset, row, col);
}

// Converts STEP consecutive elements of one row starting at element index i (values already widened to fp32 in v);
// s / o: scale and offset of the first element.
template <typename T, typename ST, int DST, int STEP>
__device__ __forceinline__ void quant_policy_store(const QuantPolicyArgs& a, size_t i, int row, int col, ST s, ST o, float (&v)[STEP])
{
    // groups are multiples of 32 columns: eight aligned columns share the scale unless it varies per column (kDim = 0)
    const bool per_col = a.policy == POL_GROUP && a.k_dim == 0;
#pragma unroll
    for (int j = 0; j < STEP; ++j) {
        if (per_col && j > 0) {
            s = pick<T, ST, DST>(a, a.scale, row, col + j);
            if (a.has_offset && a.offset) o = pick<T, ST, DST>(a, a.offset, row, col + j);
        }
        if constexpr (DST == ASCB200_FP8_E4M3 || DST == ASCB200_FP8_E5M2) {
            // fp8: fp32 arithmetic whatever the scale's type
            float r = __fmul_rn(v[j], to_f32<ST>(s));
            v[j] = a.has_offset ? __fadd_rn(r, to_f32<ST>(o)) : r;
        } else {
            v[j] = mul_add_in<ST>(v[j], s, o, a.has_offset && DST != ASCB200_FP4_E2M1);
        }
    }
    if constexpr (DST == ASCB200_FP4_E2M1) {
        uint8_t* out = static_cast<uint8_t*>(a.dst) + i / 2;
        if constexpr (STEP == 8) {
            const uint32_t w = to_fp4_pair(v[0], v[1]) | (to_fp4_pair(v[2], v[3]) << 8) | (to_fp4_pair(v[4], v[5]) << 16) | (to_fp4_pair(v[6], v[7]) << 24);
            *reinterpret_cast<uint32_t*>(out) = w;
        } else {
            *out = static_cast<uint8_t>(to_fp4_pair(v[0], v[1]));
        }
    } else {
        uint8_t* out = static_cast<uint8_t*>(a.dst) + i;
        if constexpr (STEP == 8) {
            uint32_t w0 = 0, w1 = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w0 |= to_byte<DST>(v[j], a.round_mode) << (8 * j);
                w1 |= to_byte<DST>(v[4 + j], a.round_mode) << (8 * j);
            }
            *reinterpret_cast<uint2*>(out) = make_uint2(w0, w1);
        } else {
            *out = static_cast<uint8_t>(to_byte<DST>(v[0], a.round_mode));
        }
    }
}

template <typename ST>
__device__ __forceinline__ ST offset_as(float v)
{
    if constexpr (sizeof(ST) == 4) return v;
    else if constexpr (std::is_same<ST, __half>::value) return __float2half_rn(v);
    else return __float2bfloat16_rn(v);
}

// Vector form (n % 8 == 0): a block covers 256 x 4 groups of eight consecutive elements; every thread issues its four
// 16-byte loads before it converts anything, so that enough bytes are in flight per SM to cover the HBM latency.
// SHARED (n a multiple of 32, scale constant over 32 aligned columns): the four lanes that hold one aligned run of 32 columns
// share its scale, so one load instruction per warp fetches the parameters of all 32 runs the warp converts (lane u*8 + j holds
// those of lanes 4j .. 4j+3 in round u) and shuffles hand them out: three quarters fewer parameter loads per data load.
template <typename T, typename ST, int DST, bool SHARED>
__global__ void __launch_bounds__(256) quant_policy_vec_kernel(const QuantPolicyArgs a)
{
    constexpr int VPT = 4;
    const size_t vecs = static_cast<size_t>(a.m) * a.n / 8;
    const T* src = static_cast<const T*>(a.src);
    const ST off_scalar = offset_as<ST>(a.offset_scalar);
    const size_t base = static_cast<size_t>(blockIdx.x) * (256 * VPT) + threadIdx.x;
    uint4 raw[VPT][sizeof(T) == 2 ? 1 : 2];
    int row[VPT], col[VPT];
    ST sc[VPT], of[VPT];
    int my_row = 0, my_col = 0;
    ST my_sc = off_scalar, my_of = off_scalar;
    if constexpr (SHARED) {
        const int lane = threadIdx.x & 31;
        const size_t mine = base - lane + static_cast<size_t>(lane >> 3) * 256 + (lane & 7) * 4;
        if (mine < vecs) quant_policy_params<T, ST, DST>(a, mine * 8, off_scalar, my_row, my_col, my_sc, my_of);
    }
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const size_t vi = base + static_cast<size_t>(u) * 256;
        if (vi < vecs) {
            raw[u][0] = __ldg(reinterpret_cast<const uint4*>(src + vi * 8));
            if constexpr (sizeof(T) == 4) raw[u][1] = __ldg(reinterpret_cast<const uint4*>(src + vi * 8) + 1);
            if constexpr (!SHARED) quant_policy_params<T, ST, DST>(a, vi * 8, off_scalar, row[u], col[u], sc[u], of[u]);  // with the data loads
        }
    }
    if constexpr (SHARED) {
        const int lane = threadIdx.x & 31;
#pragma unroll
        for (int u = 0; u < VPT; ++u) {
            const int from = u * 8 + (lane >> 2);
            row[u] = __shfl_sync(0xFFFFFFFFu, my_row, from);
            col[u] = __shfl_sync(0xFFFFFFFFu, my_col, from) + (lane & 3) * 8;
            if constexpr (sizeof(ST) == 4) {
                sc[u] = __shfl_sync(0xFFFFFFFFu, my_sc, from);
                of[u] = __shfl_sync(0xFFFFFFFFu, my_of, from);
            } else {
                const unsigned short sb = __shfl_sync(0xFFFFFFFFu, *reinterpret_cast<const unsigned short*>(&my_sc), from);
                const unsigned short ob = __shfl_sync(0xFFFFFFFFu, *reinterpret_cast<const unsigned short*>(&my_of), from);
                sc[u] = *reinterpret_cast<const ST*>(&sb);
                of[u] = *reinterpret_cast<const ST*>(&ob);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const size_t vi = base + static_cast<size_t>(u) * 256;
        if (vi >= vecs) break;
        float v[8];
        if constexpr (sizeof(T) == 2) {
            const T* e = reinterpret_cast<const T*>(&raw[u][0]);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = to_f32<T>(e[j]);
        } else {
            const float* e = reinterpret_cast<const float*>(&raw[u][0]);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = e[j];
        }
        quant_policy_store<T, ST, DST, 8>(a, vi * 8, row[u], col[u], sc[u], of[u], v);
    }
}

// Generic form: one element (two for fp4) per thread, grid-stride.
template <typename T, typename ST, int DST>
__global__ void __launch_bounds__(256) quant_policy_kernel(const QuantPolicyArgs a)
{
    const size_t total = static_cast<size_t>(a.m) * a.n;
    const T* src = static_cast<const T*>(a.src);
    const ST off_scalar = offset_as<ST>(a.offset_scalar);
    constexpr int STEP = DST == ASCB200_FP4_E2M1 ? 2 : 1;
    for (size_t i = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * STEP; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x * STEP) {
        float v[STEP];
#pragma unroll
        for (int j = 0; j < STEP; ++j) v[j] = to_f32<T>(src[i + j]);
        int row, col;
        ST sc, of;
        quant_policy_params<T, ST, DST>(a, i, off_scalar, row, col, sc, of);
        quant_policy_store<T, ST, DST, STEP>(a, i, row, col, sc, of, v);
    }
}

template <typename T, typename ST, int DST>
int launch_policy(const QuantPolicyArgs& a, bool vec8, int sms, cudaStream_t s)
{
    const size_t total = static_cast<size_t>(a.m) * a.n;
    if (vec8) {
        const size_t blocks = (total / 8 + 256 * 4 - 1) / (256 * 4);
        if (blocks > 0x7FFFFFFFull) return ASCB200_ETOOBIG;
        const bool shared = a.n % 32 == 0 && !(a.policy == POL_GROUP && a.k_dim == 0);
        if (shared) quant_policy_vec_kernel<T, ST, DST, true><<<static_cast<unsigned>(blocks), 256, 0, s>>>(a);
        else quant_policy_vec_kernel<T, ST, DST, false><<<static_cast<unsigned>(blocks), 256, 0, s>>>(a);
    } else {
        const size_t step = DST == ASCB200_FP4_E2M1 ? 2 : 1;
        const size_t threads = (total + step - 1) / step;
        const unsigned grid = static_cast<unsigned>(std::min<size_t>((threads + 255) / 256, static_cast<size_t>(sms) * 16));
        quant_policy_kernel<T, ST, DST><<<grid, 256, 0, s>>>(a);
    }
    ASCB200_CUDA(cudaGetLastError());
    return ASCB200_OK;
}

template <typename T, typename ST>
int dispatch_dst(const QuantPolicyArgs& a, int dst_dtype, bool vec8, int sms, cudaStream_t s)
{
    switch (dst_dtype) {
        case ASCB200_S8: return launch_policy<T, ST, ASCB200_S8>(a, vec8, sms, s);
        case ASCB200_FP8_E4M3: return launch_policy<T, ST, ASCB200_FP8_E4M3>(a, vec8, sms, s);
        case ASCB200_FP8_E5M2: return launch_policy<T, ST, ASCB200_FP8_E5M2>(a, vec8, sms, s);
        case ASCB200_FP4_E2M1: return launch_policy<T, ST, ASCB200_FP4_E2M1>(a, vec8, sms, s);
        default: return ASCB200_EUNSUPPORTED;
    }
}

// ---- AscendDequant with the PER_TOKEN / PER_GROUP policies ---------------------------------------------------------------
// dst = cast(float(src) * float(scale)) (impl/adv_api/detail/quantization/dequant/ascend_dequant_3510_impl.h:253-286 per token,
// :345-600 per group); src int32 or fp32, scale fp32 / half / bfloat16 (widened), dst fp32 / half / bfloat16 (round to nearest
// even, fp16 saturating).  The offset tensor of the interface takes no part in the reference's arithmetic.
struct DequantPolicyArgs {
    const void* src;
    void* dst;
    const void* scale;
    int m, n;
    int per_group, k_dim, group_size, scale_cols;
};

template <typename ST>
__device__ __forceinline__ float dequant_scale_at(const DequantPolicyArgs& a, int row, int col)
{
    const ST* scale = static_cast<const ST*>(a.scale);
    const size_t si = !a.per_group ? static_cast<size_t>(row)
                      : a.k_dim == 1 ? static_cast<size_t>(row) * a.scale_cols + col / a.group_size
                                     : static_cast<size_t>(row / a.group_size) * a.n + col;
    return to_f32<ST>(scale[si]);
}
template <typename DT>
__device__ __forceinline__ void dequant_store8(DT* out, const float (&v)[8])
{
    if constexpr (std::is_same<DT, float>::value) {
        reinterpret_cast<float4*>(out)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(out)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if constexpr (std::is_same<DT, __half>::value) {
                const __half2 h = __halves2half2(f32_to_f16_sat(v[2 * j]), f32_to_f16_sat(v[2 * j + 1]));
                w[j] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        *reinterpret_cast<uint4*>(out) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// Vector form (n % 8 == 0): eight elements per thread, two vectors per thread in flight; with SHARED (n % 32 == 0, scale
// constant over 32 aligned columns) one lane in four fetches the scale and shuffles hand it to its neighbours.
template <typename SRC, typename ST, typename DT, bool SHARED>
__global__ void __launch_bounds__(256) dequant_policy_vec_kernel(const DequantPolicyArgs a)
{
    constexpr int VPT = 2;
    const size_t vecs = static_cast<size_t>(a.m) * a.n / 8;
    const SRC* src = static_cast<const SRC*>(a.src);
    DT* dst = static_cast<DT*>(a.dst);
    const size_t base = static_cast<size_t>(blockIdx.x) * (256 * VPT) + threadIdx.x;
    const int lane = threadIdx.x & 31;
    uint4 raw[VPT][2];
    float sc[VPT] = {};
    int row[VPT] = {}, col[VPT] = {};
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const size_t vi = base + static_cast<size_t>(u) * 256;
        if (vi < vecs) {
            const size_t e = vi * 8;
            raw[u][0] = __ldg(reinterpret_cast<const uint4*>(src + e));
            raw[u][1] = __ldg(reinterpret_cast<const uint4*>(src + e) + 1);
            row[u] = e < 0xFFFFFFFFull ? static_cast<int>(static_cast<uint32_t>(e) / static_cast<uint32_t>(a.n)) : static_cast<int>(e / a.n);
            col[u] = static_cast<int>(e - static_cast<size_t>(row[u]) * a.n);
            if (!SHARED || (lane & 3) == 0) sc[u] = dequant_scale_at<ST>(a, row[u], col[u]);
        }
    }
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        const size_t vi = base + static_cast<size_t>(u) * 256;
        if constexpr (SHARED) sc[u] = __shfl_sync(0xFFFFFFFFu, sc[u], lane & ~3);  // lanes 4j .. 4j+3 are valid together
        if (vi >= vecs) continue;
        float v[8];
        const bool per_col = a.per_group && a.k_dim == 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t w = j < 4 ? (&raw[u][0].x)[j] : (&raw[u][1].x)[j - 4];
            const float x = std::is_same<SRC, float>::value ? __uint_as_float(w) : __int2float_rn(static_cast<int>(w));
            const float s = (per_col && j > 0) ? dequant_scale_at<ST>(a, row[u], col[u] + j) : sc[u];
            v[j] = __fmul_rn(x, s);
        }
        dequant_store8<DT>(dst + vi * 8, v);
    }
}

// Generic form: one element per thread, grid-stride.
template <typename SRC, typename ST, typename DT>
__global__ void __launch_bounds__(256) dequant_policy_kernel(const DequantPolicyArgs a)
{
    const size_t total = static_cast<size_t>(a.m) * a.n;
    const SRC* src = static_cast<const SRC*>(a.src);
    DT* dst = static_cast<DT*>(a.dst);
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int row = static_cast<int>(i / a.n), col = static_cast<int>(i % a.n);
        const float v = __fmul_rn(static_cast<float>(src[i]), dequant_scale_at<ST>(a, row, col));
        if constexpr (std::is_same<DT, float>::value) dst[i] = v;
        else if constexpr (std::is_same<DT, __half>::value) dst[i] = f32_to_f16_sat(v);
        else dst[i] = __float2bfloat16_rn(v);
    }
}

template <typename SRC, typename ST, typename DT>
int dequant_policy_launch(const DequantPolicyArgs& a, bool vec, unsigned grid, cudaStream_t s)
{
    if (vec) {
        const size_t blocks = (static_cast<size_t>(a.m) * a.n / 8 + 511) / 512;
        if (blocks > 0x7FFFFFFFull) return ASCB200_ETOOBIG;
        const bool shared = a.n % 32 == 0 && !(a.per_group && a.k_dim == 0);
        if (shared) dequant_policy_vec_kernel<SRC, ST, DT, true><<<static_cast<unsigned>(blocks), 256, 0, s>>>(a);
        else dequant_policy_vec_kernel<SRC, ST, DT, false><<<static_cast<unsigned>(blocks), 256, 0, s>>>(a);
    } else {
        dequant_policy_kernel<SRC, ST, DT><<<grid, 256, 0, s>>>(a);
    }
    return ASCB200_OK;
}

template <typename SRC, typename ST>
int dequant_policy_dst(const DequantPolicyArgs& a, int dst_dtype, bool vec, unsigned grid, cudaStream_t s)
{
    int rc;
    switch (dst_dtype) {
        case ASCB200_F32: rc = dequant_policy_launch<SRC, ST, float>(a, vec, grid, s); break;
        case ASCB200_F16: rc = dequant_policy_launch<SRC, ST, __half>(a, vec, grid, s); break;
        case ASCB200_BF16: rc = dequant_policy_launch<SRC, ST, __nv_bfloat16>(a, vec, grid, s); break;
        default: return ASCB200_EUNSUPPORTED;
    }
    if (rc != ASCB200_OK) return rc;
    ASCB200_CUDA(cudaGetLastError());
    return ASCB200_OK;
}
template <typename SRC>
int dequant_policy_scale(const DequantPolicyArgs& a, int scale_dtype, int dst_dtype, bool vec, unsigned grid, cudaStream_t s)
{
    switch (scale_dtype) {
        case ASCB200_F32: return dequant_policy_dst<SRC, float>(a, dst_dtype, vec, grid, s);
        case ASCB200_F16: return dequant_policy_dst<SRC, __half>(a, dst_dtype, vec, grid, s);
        case ASCB200_BF16: return dequant_policy_dst<SRC, __nv_bfloat16>(a, dst_dtype, vec, grid, s);
        default: return ASCB200_EUNSUPPORTED;
    }
}


// ---- AscendAntiQuant, int8 source (include/adv_api/quantization/ascend_antiquant.h:47-200) ---------------------------------
// dst = scale * (src + offset) with the arithmetic of the reference's register code
// (impl/adv_api/detail/quantization/antiquant/ascend_antiquant_3510_impl.h): half outputs add and multiply in half (two
// roundings, :336-358 per tensor, :461-495 and :615-645 per channel); bfloat16 outputs add and multiply in bfloat16 for
// per-channel parameters along the row (:461-495) and in fp32 with one rounding for a per-tensor pair (:360-392) or
// per-row parameters (the transposed form, :647-690).  int8 -> half / bfloat16 is exact.
// MODE 0: one (scale, offset) pair; 1: one pair per column (no transpose: src [K, N], parameters [N]); 2: one pair per row
// (isTranspose: src [N, K], parameters [N]).  A thread converts 16 consecutive elements of one row.
template <typename DT, int MODE, bool F32_MATH>
__global__ void __launch_bounds__(256)
antiquant_i8_kernel(const int8_t* __restrict__ src, DT* __restrict__ dst, const DT* __restrict__ scale, const DT* __restrict__ offset, DT scale_s,
                    DT offset_s, size_t nvec, int vec_per_row)
{
    const size_t v = static_cast<size_t>(blockIdx.x) * 256 + threadIdx.x;
    if (v >= nvec) return;
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + v * 16));
    const size_t row = v / static_cast<size_t>(vec_per_row);
    const int col0 = static_cast<int>(v - row * vec_per_row) * 16;
    DT sc[16], of[16];
    if constexpr (MODE == 1) {
        *reinterpret_cast<uint4*>(sc) = __ldg(reinterpret_cast<const uint4*>(scale + col0));
        *reinterpret_cast<uint4*>(sc + 8) = __ldg(reinterpret_cast<const uint4*>(scale + col0 + 8));
        if (offset) {
            *reinterpret_cast<uint4*>(of) = __ldg(reinterpret_cast<const uint4*>(offset + col0));
            *reinterpret_cast<uint4*>(of + 8) = __ldg(reinterpret_cast<const uint4*>(offset + col0 + 8));
        }
    }
    DT s1 = scale_s, o1 = offset_s;
    if constexpr (MODE == 2) {
        s1 = scale[row];
        if (offset) o1 = offset[row];
    }
    const int8_t* b = reinterpret_cast<const int8_t*>(&raw);
    DT out[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const DT s = MODE == 1 ? sc[j] : s1;
        const DT o = MODE == 1 ? (offset ? of[j] : offset_s) : o1;
        if constexpr (F32_MATH) {
            const float r = __fmul_rn(__fadd_rn(static_cast<float>(b[j]), static_cast<float>(o)), static_cast<float>(s));
            if constexpr (std::is_same<DT, __half>::value) out[j] = __float2half_rn(fminf(fmaxf(r, -65504.0f), 65504.0f));
            else out[j] = __float2bfloat16_rn(r);
        } else {
            DT x;
            if constexpr (std::is_same<DT, __half>::value) x = __short2half_rn(b[j]);
            else x = __float2bfloat16_rn(static_cast<float>(b[j]));
            out[j] = __hmul_rn(__hadd_rn(x, o), s);
        }
    }
    *reinterpret_cast<uint4*>(dst + v * 16) = *reinterpret_cast<const uint4*>(out);
    *reinterpret_cast<uint4*>(dst + v * 16 + 8) = *reinterpret_cast<const uint4*>(out + 8);
}

// Per-column parameters: a thread keeps the 16 (scale, offset) pairs of its columns in registers and walks kAntiRows rows,
// so that the parameters are loaded once per eight vectors instead of once per vector.
constexpr int kAntiRows = 8;
template <typename DT>
__global__ void __launch_bounds__(128)
antiquant_i8_columns_kernel(const int8_t* __restrict__ src, DT* __restrict__ dst, const DT* __restrict__ scale, const DT* __restrict__ offset,
                            DT offset_s, int rows, int vec_per_row)
{
    const int cv = blockIdx.x * 128 + threadIdx.x;
    if (cv >= vec_per_row) return;
    const int r0 = blockIdx.y * kAntiRows;
    const size_t cols = static_cast<size_t>(vec_per_row) * 16;
    uint4 raw[kAntiRows];
#pragma unroll
    for (int r = 0; r < kAntiRows; ++r)
        if (r0 + r < rows) raw[r] = __ldg(reinterpret_cast<const uint4*>(src + (r0 + r) * cols + cv * 16));
    DT sc[16], of[16];
    *reinterpret_cast<uint4*>(sc) = __ldg(reinterpret_cast<const uint4*>(scale + cv * 16));
    *reinterpret_cast<uint4*>(sc + 8) = __ldg(reinterpret_cast<const uint4*>(scale + cv * 16 + 8));
    if (offset) {
        *reinterpret_cast<uint4*>(of) = __ldg(reinterpret_cast<const uint4*>(offset + cv * 16));
        *reinterpret_cast<uint4*>(of + 8) = __ldg(reinterpret_cast<const uint4*>(offset + cv * 16 + 8));
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) of[j] = offset_s;
    }
#pragma unroll
    for (int r = 0; r < kAntiRows; ++r) {
        if (r0 + r >= rows) break;
        const int8_t* b = reinterpret_cast<const int8_t*>(&raw[r]);
        DT out[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            DT x;
            if constexpr (std::is_same<DT, __half>::value) x = __short2half_rn(b[j]);
            else x = __float2bfloat16_rn(static_cast<float>(b[j]));
            out[j] = __hmul_rn(__hadd_rn(x, of[j]), sc[j]);
        }
        DT* d = dst + (r0 + r) * cols + cv * 16;
        *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(out);
        *reinterpret_cast<uint4*>(d + 8) = *reinterpret_cast<const uint4*>(out + 8);
    }
}

template <typename DT>
int launch_antiquant(const int8_t* src, DT* dst, int rows, int cols, int mode, const DT* scale, const DT* offset, float scale_f, float offset_f,
                     cudaStream_t st)
{
    const size_t nvec = static_cast<size_t>(rows) * (cols / 16);
    const size_t blocks = (nvec + 255) / 256;
    if (blocks > 0x7FFFFFFFull) return ASCB200_ETOOBIG;
    const DT ss = static_cast<DT>(scale_f), os = static_cast<DT>(offset_f);  // the scalars arrive in the output type
    constexpr bool BF = std::is_same<DT, __nv_bfloat16>::value;
    const unsigned g = static_cast<unsigned>(blocks);
    if (mode == 0) antiquant_i8_kernel<DT, 0, BF><<<g, 256, 0, st>>>(src, dst, scale, offset, ss, os, nvec, cols / 16);
    else if (mode == 1) {
        const int row_blocks = (rows + kAntiRows - 1) / kAntiRows;
        if (row_blocks > 65535) antiquant_i8_kernel<DT, 1, false><<<g, 256, 0, st>>>(src, dst, scale, offset, ss, os, nvec, cols / 16);
        else antiquant_i8_columns_kernel<DT><<<dim3((cols / 16 + 127) / 128, row_blocks), 128, 0, st>>>(src, dst, scale, offset, os, rows, cols / 16);
    }
    else antiquant_i8_kernel<DT, 2, BF><<<g, 256, 0, st>>>(src, dst, scale, offset, ss, os, nvec, cols / 16);
    ASCB200_CUDA(cudaGetLastError());
    return ASCB200_OK;
}
}  // namespace
}  // namespace ascb200

extern "C" int ascb200_dequant_policy(const void* src, void* dst, int32_t m, int32_t n, int32_t src_dtype, int32_t scale_dtype, int32_t dst_dtype,
                                      int32_t policy, int32_t k_dim, int32_t group_size, const void* scale, void* stream)
{
    using namespace ascb200;
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!src || !dst || !scale || m < 0 || n < 0) return ASCB200_EINVAL;
    if (policy != ASCB200_DEQUANT_PER_TOKEN && policy != ASCB200_DEQUANT_PER_GROUP) return ASCB200_EUNSUPPORTED;
    if (policy == ASCB200_DEQUANT_PER_GROUP && (group_size <= 0 || group_size % 32 != 0 || (k_dim != 0 && k_dim != 1))) return ASCB200_EINVAL;
    if (src_dtype != ASCB200_S32 && src_dtype != ASCB200_F32) return ASCB200_EUNSUPPORTED;
    if (!aligned_to(src, 16) || !aligned_to(dst, 4)) return ASCB200_EALIGN;
    if (m == 0 || n == 0) return ASCB200_OK;
    DequantPolicyArgs a;
    a.src = src;
    a.dst = dst;
    a.scale = scale;
    a.m = m;
    a.n = n;
    a.per_group = policy == ASCB200_DEQUANT_PER_GROUP;
    a.k_dim = k_dim;
    a.group_size = a.per_group ? group_size : 1;
    a.scale_cols = a.per_group ? (n + group_size - 1) / group_size : 1;
    const size_t threads = static_cast<size_t>(m) * n;
    const unsigned grid = static_cast<unsigned>(std::min<size_t>((threads + 255) / 256, static_cast<size_t>(st->sm_count) * 16));
    const bool vec = n % 8 == 0 && aligned_to(dst, 16);  // src is 16-byte aligned (checked above)
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (src_dtype == ASCB200_S32) return dequant_policy_scale<int32_t>(a, scale_dtype, dst_dtype, vec, grid, s);
    return dequant_policy_scale<float>(a, scale_dtype, dst_dtype, vec, grid, s);
}

extern "C" int ascb200_quant_policy(const void* src, void* dst, int32_t m, int32_t n, int32_t src_dtype, int32_t scale_dtype, int32_t dst_dtype,
                                    int32_t policy, int32_t k_dim, int32_t group_size, const void* scale, const void* offset_tensor,
                                    float offset_scalar, int32_t has_offset, void* stream)
{
    return ascb200_quant_policy_rm(src, dst, m, n, src_dtype, scale_dtype, dst_dtype, policy, k_dim, group_size, scale, offset_tensor, offset_scalar,
                                   has_offset, /*CAST_RINT*/ 1, stream);
}

extern "C" int ascb200_quant_policy_rm(const void* src, void* dst, int32_t m, int32_t n, int32_t src_dtype, int32_t scale_dtype, int32_t dst_dtype,
                                       int32_t policy, int32_t k_dim, int32_t group_size, const void* scale, const void* offset_tensor,
                                       float offset_scalar, int32_t has_offset, int32_t round_mode, void* stream)
{
    using namespace ascb200;
    if (round_mode == 0) round_mode = 1;                                                  // CAST_NONE: the default rounding
    if (round_mode < 1 || round_mode > 5) return ASCB200_EUNSUPPORTED;                    // CAST_ODD, CAST_HYBRID, ... are not built
    if (round_mode != 1 && dst_dtype != ASCB200_S8) return ASCB200_EUNSUPPORTED;          // fp8 / fp4 destinations round to nearest even only
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!src || !dst || !scale || m < 0 || n < 0) return ASCB200_EINVAL;
    if (policy != ASCB200_QUANT_PER_TOKEN && policy != ASCB200_QUANT_PER_GROUP) return ASCB200_EUNSUPPORTED;
    if (policy == ASCB200_QUANT_PER_GROUP && (group_size <= 0 || group_size % 32 != 0 || (k_dim != 0 && k_dim != 1))) return ASCB200_EINVAL;
    if (dst_dtype == ASCB200_FP4_E2M1 && (policy != ASCB200_QUANT_PER_GROUP || n % 2 != 0)) return ASCB200_EUNSUPPORTED;  // like the reference
    // the scale is fp32, or has the source's 16-bit type (the reference loads the source into registers of the scale's type)
    if (!(scale_dtype == ASCB200_F32 || (scale_dtype == src_dtype && (src_dtype == ASCB200_F16 || src_dtype == ASCB200_BF16)))) return ASCB200_EUNSUPPORTED;
    if (m == 0 || n == 0) return ASCB200_OK;
    QuantPolicyArgs a;
    a.src = src;
    a.dst = dst;
    a.scale = scale;
    a.offset = offset_tensor;
    a.offset_scalar = offset_scalar;
    a.has_offset = has_offset ? 1 : 0;
    a.m = m;
    a.n = n;
    a.policy = policy;
    a.k_dim = k_dim;
    a.group_size = policy == ASCB200_QUANT_PER_GROUP ? group_size : 1;
    a.scale_cols = policy == ASCB200_QUANT_PER_GROUP ? (n + group_size - 1) / group_size : 1;
    a.round_mode = round_mode;
    const int esz = src_dtype == ASCB200_F32 ? 4 : 2;
    const bool vec8 = n % 8 == 0 && aligned_to(src, 16) && aligned_to(dst, 8) && (src_dtype == ASCB200_F32 || esz == 2);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int sms = st->sm_count;
    if (src_dtype == ASCB200_F16) {
        if (scale_dtype == ASCB200_F32) return dispatch_dst<__half, float>(a, dst_dtype, vec8, sms, s);
        return dispatch_dst<__half, __half>(a, dst_dtype, vec8, sms, s);
    }
    if (src_dtype == ASCB200_BF16) {
        if (scale_dtype == ASCB200_F32) return dispatch_dst<__nv_bfloat16, float>(a, dst_dtype, vec8, sms, s);
        return dispatch_dst<__nv_bfloat16, __nv_bfloat16>(a, dst_dtype, vec8, sms, s);
    }
    if (src_dtype == ASCB200_F32) return dispatch_dst<float, float>(a, dst_dtype, vec8, sms, s);
    return ASCB200_EUNSUPPORTED;
}

extern "C" int ascb200_antiquant(const int8_t* src, void* dst, int32_t rows, int32_t cols, int32_t dst_dtype, int32_t mode, const void* scale,
                                 const void* offset, float scale_scalar, float offset_scalar, void* stream)
{
    using namespace ascb200;
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!src || !dst || rows < 0 || cols < 0 || mode < 0 || mode > 2) return ASCB200_EINVAL;
    if (mode != 0 && !scale) return ASCB200_EINVAL;
    if (dst_dtype != ASCB200_F16 && dst_dtype != ASCB200_BF16) return ASCB200_EUNSUPPORTED;
    if (cols % 32 != 0) return ASCB200_EALIGN;  // rows of whole 32-byte blocks, like the reference's tensors
    if (!aligned_to(src, 16) || !aligned_to(dst, 16)) return ASCB200_EALIGN;
    if (mode == 1 && (!aligned_to(scale, 16) || (offset && !aligned_to(offset, 16)))) return ASCB200_EALIGN;
    if (rows == 0 || cols == 0) return ASCB200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dst_dtype == ASCB200_F16)
        return launch_antiquant<__half>(src, static_cast<__half*>(dst), rows, cols, mode, static_cast<const __half*>(scale),
                                        static_cast<const __half*>(offset), scale_scalar, offset_scalar, s);
    return launch_antiquant<__nv_bfloat16>(src, static_cast<__nv_bfloat16*>(dst), rows, cols, mode, static_cast<const __nv_bfloat16*>(scale),
                                           static_cast<const __nv_bfloat16*>(offset), scale_scalar, offset_scalar, s);
}
