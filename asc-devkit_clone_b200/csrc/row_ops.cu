// Memory-bound row operators: SoftMax, AscendQuant, AscendDequant and the fused SoftMax+AscendQuant.
// Every kernel reads its input once with 128-bit loads, keeps the row in registers, reduces with
// warp shuffles and writes each output once with vector stores.
#include "common.cuh"

namespace ascb200 {
namespace {

constexpr float kNegInf = -__builtin_huge_valf();

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p)
{
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ float exp2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// AscendQuant on two values at a time: half(x) * half(scale) + half(offset), each step rounded to
// half (no fused multiply-add), then round-to-nearest-even to int8 with saturation, NaN -> 0.
// The rounding uses the fp16 grid itself: after clamping to [-128, 127], adding 1536 lands in
// [1024, 2048) where consecutive halves are 1 apart, so the sum is rint(v) + 1536 exactly and the
// low byte of its bit pattern is the two's-complement int8.
__device__ __forceinline__ uint32_t quant_half2_bits(__half2 x, __half2 s, __half2 o)
{
    __half2 v = __hadd2_rn(__hmul2_rn(x, s), o);
    uint32_t bits = *reinterpret_cast<uint32_t*>(&v) & __heq2_mask(v, v);  // NaN lanes -> +0
    v = *reinterpret_cast<__half2*>(&bits);
    v = __hmax2(__hmin2(v, __float2half2_rn(127.0f)), __float2half2_rn(-128.0f));
    v = __hadd2_rn(v, __float2half2_rn(1536.0f));
    return *reinterpret_cast<uint32_t*>(&v);  // bytes 0 and 2 hold the two int8 results
}
// Packs the int8 results of two quant_half2_bits() words into the low / high halves of 4 bytes.
__device__ __forceinline__ uint32_t pack_s8x4(uint32_t ab, uint32_t cd) { return __byte_perm(ab, cd, 0x6420); }

__device__ __forceinline__ float clamp_half_range(float v) { return (v != v) ? v : fminf(fmaxf(v, -65504.0f), 65504.0f); }
// Two source elements -> half2 the way the operator converts its input (RINT, saturating).
__device__ __forceinline__ __half2 to_half2_src(__half a, __half b) { return __halves2half2(a, b); }
__device__ __forceinline__ __half2 to_half2_src(__nv_bfloat16 a, __nv_bfloat16 b)
{
    return __floats2half2_rn(clamp_half_range(__bfloat162float(a)), clamp_half_range(__bfloat162float(b)));
}
__device__ __forceinline__ __half2 to_half2_src(float a, float b) { return __floats2half2_rn(clamp_half_range(a), clamp_half_range(b)); }
__device__ __forceinline__ int quant_half(__half x, __half s, __half o)
{
    const uint32_t b = quant_half2_bits(__halves2half2(x, x), __halves2half2(s, s), __halves2half2(o, o));
    return static_cast<int>(static_cast<int8_t>(b & 0xFFu));
}
__device__ __forceinline__ __half to_half_src(__half v) { return v; }
__device__ __forceinline__ __half to_half_src(__nv_bfloat16 v) { return __float2half_rn(clamp_half_range(__bfloat162float(v))); }
__device__ __forceinline__ __half to_half_src(float v) { return __float2half_rn(clamp_half_range(v)); }

template <int TPR>
__device__ __forceinline__ float row_reduce_max(float v, float* red)
{
    v = warp_max(v);
    if constexpr (TPR > 32) {
        const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
        __syncthreads();
        if (l == 0) red[w] = v;
        __syncthreads();
        v = (l < TPR / 32) ? red[l] : kNegInf;
        v = warp_max(v);
    }
    return v;
}
template <int TPR>
__device__ __forceinline__ float row_reduce_sum(float v, float* red)
{
    v = warp_sum(v);
    if constexpr (TPR > 32) {
        const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
        __syncthreads();
        if (l == 0) red[w] = v;
        __syncthreads();
        v = (l < TPR / 32) ? red[l] : 0.0f;
        v = warp_sum(v);
    }
    return v;
}

// One row per group of TPR threads (a warp, or the whole block).  Thread t of the group owns the
// 16-byte chunks t, t+TPR, ... (NCHUNK of them).  T = __half (8 per chunk) or float (4 per chunk).
// Warp rows (TPR == 32) are persistent: the grid is sized to the machine, every warp walks rows
// row, row + #warps, ... and issues the loads of its next row before it works on the current one,
// so that no wave of blocks ends with a mostly idle machine and HBM requests stay in flight.
template <typename T, int TPR, int NCHUNK>
__device__ __forceinline__ void softmax_load_row(const T* __restrict__ srow, int t, int nchunks, uint4 (&raw)[NCHUNK])
{
    constexpr int VEC = 16 / sizeof(T);
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        const int c = t + i * TPR;
        if (c < nchunks) raw[i] = ldg_nc_v4(srow + c * VEC);
    }
}

// One statistic of a row.  Volatile: the compiler keeps the load where it is written (ahead of the first use of the row's
// data) instead of sinking it to its first use, where it would add a memory latency to the row's critical path.
template <typename ST> __device__ __forceinline__ float stat_load(const ST* p, size_t i);
template <> __device__ __forceinline__ float stat_load<float>(const float* p, size_t i)
{
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p + i));
    return v;
}
template <> __device__ __forceinline__ float stat_load<__half>(const __half* p, size_t i)
{
    unsigned short b;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(b) : "l"(p + i));
    return __half2float(__ushort_as_half(b));
}
// MODE: kSoftmaxPlain, kSoftmaxQuant (also writes the int8 AscendQuant of the result) or kSoftmaxLog
// (LogSoftMax: y = ln(e / sum) * log10(e) computed in fp32, statistics stored in T;
// impl/adv_api/detail/activation/softmax/membase/common/logsoftmax_common_impl.h:277-376).
// kSoftmaxSimpleF32 / kSoftmaxSimpleF16: SimpleSoftMax, y = exp(x - inMax) / inSum with the statistics READ from
// max_out / sum_out (fp32, or half behind the same pointers) instead of reduced from the row
// (impl/adv_api/detail/activation/softmax/membase/common/simple_softmax_common_impl.h:320-502).
constexpr int kSoftmaxPlain = 0, kSoftmaxQuant = 1, kSoftmaxLog = 2, kSoftmaxSimpleF32 = 3, kSoftmaxSimpleF16 = 4;

template <typename T, int TPR, int NCHUNK, int MODE>
__device__ __forceinline__ void softmax_one_row(const uint4 (&raw)[NCHUNK], int row, int t, int nchunks, T* __restrict__ dst,
                                                float* __restrict__ sum_out, float* __restrict__ max_out, int8_t* __restrict__ q_out,
                                                const __half* __restrict__ q_scale, const __half* __restrict__ q_offset, __half q_offset_scalar,
                                                int k, int stats_rep, float* red)
{
    constexpr int VEC = 16 / sizeof(T);
    constexpr bool SIMPLE = MODE == kSoftmaxSimpleF32 || MODE == kSoftmaxSimpleF16;
    float v[NCHUNK * VEC];
    float mx = kNegInf, given_sum = 1.0f;
    if constexpr (MODE == kSoftmaxSimpleF32) {
        mx = stat_load<float>(max_out, static_cast<size_t>(row) * stats_rep);
        given_sum = stat_load<float>(sum_out, static_cast<size_t>(row) * stats_rep);
    } else if constexpr (MODE == kSoftmaxSimpleF16) {
        mx = stat_load<__half>(reinterpret_cast<const __half*>(max_out), static_cast<size_t>(row) * stats_rep);
        given_sum = stat_load<__half>(reinterpret_cast<const __half*>(sum_out), static_cast<size_t>(row) * stats_rep);
    }
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        const int c = t + i * TPR;
        if (c < nchunks) {
            if constexpr (sizeof(T) == 2) {
                const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float2 f = __half22float2(h[j]);
                    v[i * 8 + 2 * j] = f.x;
                    v[i * 8 + 2 * j + 1] = f.y;
                }
            } else {
                v[i * 4 + 0] = __uint_as_float(raw[i].x);
                v[i * 4 + 1] = __uint_as_float(raw[i].y);
                v[i * 4 + 2] = __uint_as_float(raw[i].z);
                v[i * 4 + 3] = __uint_as_float(raw[i].w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[i * VEC + j] = kNegInf;
        }
        if constexpr (!SIMPLE) {
#pragma unroll
            for (int j = 0; j < VEC; ++j) mx = fmaxf(mx, v[i * VEC + j]);
        }
    }
    if constexpr (!SIMPLE) mx = row_reduce_max<TPR>(mx, red);

    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NCHUNK * VEC; ++i) {
        v[i] = exp2_approx((v[i] - mx) * 1.4426950408889634f);  // exp(x - max); -inf padding gives 0
        s += v[i];
    }
    if constexpr (SIMPLE) s = given_sum;
    else s = row_reduce_sum<TPR>(s, red);
    const float inv = __frcp_rn(s);
    if constexpr (SIMPLE && sizeof(T) == 2) {  // foreign statistics can push y past the half range: saturate like the reference's cast
#pragma unroll
        for (int i = 0; i < NCHUNK * VEC; ++i) v[i] = clamp_half_range(v[i] * inv);
    }
    if constexpr (MODE == kSoftmaxLog) {
#pragma unroll
        for (int i = 0; i < NCHUNK * VEC; ++i) v[i] = __log2f(v[i] * inv) * (0.6931471805599453f * 0.4342944819f);  // ln(.) * SCALAR_NATURE_LOG_10
    }
    const float outmul = (MODE == kSoftmaxLog || (SIMPLE && sizeof(T) == 2)) ? 1.0f : inv;

    T* drow = dst + static_cast<size_t>(row) * k;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        const int c = t + i * TPR;
        if (c < nchunks) {
            if constexpr (sizeof(T) == 2) {
                uint4 o;  // softmax values lie in [0, 1] and their log10 above -46: the half cast cannot overflow
                __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(v[i * 8 + 2 * j] * outmul, v[i * 8 + 2 * j + 1] * outmul);
                *reinterpret_cast<uint4*>(drow + c * 8) = o;
                if constexpr (MODE == kSoftmaxQuant) {
                    const uint4 sc = __ldg(reinterpret_cast<const uint4*>(q_scale + c * 8));
                    uint4 of = make_uint4(0u, 0u, 0u, 0u);
                    if (q_offset) of = __ldg(reinterpret_cast<const uint4*>(q_offset + c * 8));
                    const __half2* hs = reinterpret_cast<const __half2*>(&sc);
                    const __half2* ho = reinterpret_cast<const __half2*>(&of);
                    const __half2 os = __half2half2(q_offset_scalar);
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) w[j] = quant_half2_bits(h[j], hs[j], q_offset ? ho[j] : os);
                    *reinterpret_cast<uint2*>(q_out + static_cast<size_t>(row) * k + c * 8) = make_uint2(pack_s8x4(w[0], w[1]), pack_s8x4(w[2], w[3]));
                }
            } else {
                float4 o = make_float4(v[i * 4] * outmul, v[i * 4 + 1] * outmul, v[i * 4 + 2] * outmul, v[i * 4 + 3] * outmul);
                *reinterpret_cast<float4*>(drow + c * 4) = o;
            }
        }
    }
    if constexpr (SIMPLE) return;
    if (t < stats_rep) {
        if constexpr (MODE == kSoftmaxLog && sizeof(T) == 2) {  // LogSoftMax keeps its statistics in T
            reinterpret_cast<__half*>(sum_out)[static_cast<size_t>(row) * stats_rep + t] = __float2half_rn(s);
            reinterpret_cast<__half*>(max_out)[static_cast<size_t>(row) * stats_rep + t] = __float2half_rn(mx);
        } else {
            sum_out[static_cast<size_t>(row) * stats_rep + t] = s;
            max_out[static_cast<size_t>(row) * stats_rep + t] = mx;
        }
    }
}

constexpr int kSoftmaxWarpBlock = 224;  // 7 warps; two such blocks per SM
#ifndef ASCB200_SOFTMAX_PREFETCH_ROWS
#define ASCB200_SOFTMAX_PREFETCH_ROWS 1
#endif
// Rows per warp requested from L2 before the dependency wait.  Measured on 4096 x 2048 halves with the fused quantisation,
// cold inputs, consecutive launches of one stream: 8.93 us without, 8.06 us with one row, 8.96 us with two or four.
constexpr int kSoftmaxPrefetchRows = ASCB200_SOFTMAX_PREFETCH_ROWS;

// PERSIST (warp rows only): few rows per warp -> machine-sized grid with next-row prefetch; many rows ->
// one row per warp and small blocks, where 20 resident warps per SM keep more requests in flight.
template <typename T, int TPR, int NCHUNK, int MODE, bool PERSIST>
__global__ void __launch_bounds__(TPR > 32 ? TPR : (PERSIST ? kSoftmaxWarpBlock : 128), TPR > 32 ? 1 : (PERSIST ? 2 : 5))
softmax_rows_kernel(const T* __restrict__ src, T* __restrict__ dst, float* __restrict__ sum_out, float* __restrict__ max_out,
                    int8_t* __restrict__ q_out, const __half* __restrict__ q_scale, const __half* __restrict__ q_offset,
                    __half q_offset_scalar, int m, int k, int stats_rep)
{
    constexpr int VEC = 16 / sizeof(T);
    __shared__ float red[32];
    const int nchunks = k / VEC;
    if constexpr (TPR <= 32) {
        // While the kernel before this one in the stream drains, ask L2 for the warp's first row (a hint: nothing is read into
        // the program before the dependency wait, and L2 stays coherent if that kernel still writes the row).
        const int first = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
        const int line = (threadIdx.x & 31) * 128;
        const int ahead_rows = PERSIST ? kSoftmaxPrefetchRows : 1;
        for (int i = 0, row = first; i < ahead_rows && row < m; ++i, row += gridDim.x * (blockDim.x >> 5))
            if (line < k * static_cast<int>(sizeof(T)))
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(src + static_cast<size_t>(row) * k) + line));
    }
    grid_dependency_wait();
    if constexpr (TPR > 32) {
        const int row = blockIdx.x;
        uint4 raw[NCHUNK];
        softmax_load_row<T, TPR, NCHUNK>(src + static_cast<size_t>(row) * k, threadIdx.x, nchunks, raw);
        softmax_one_row<T, TPR, NCHUNK, MODE>(raw, row, threadIdx.x, nchunks, dst, sum_out, max_out, q_out, q_scale, q_offset, q_offset_scalar, k,
                                               stats_rep, red);
    } else {
        const int t = threadIdx.x & 31;
        const int warps_per_block = blockDim.x >> 5;
        const int stride = gridDim.x * warps_per_block;
        int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
        if (row >= m) return;  // whole warp leaves together
        uint4 raw[NCHUNK];
        softmax_load_row<T, TPR, NCHUNK>(src + static_cast<size_t>(row) * k, t, nchunks, raw);
        if constexpr (!PERSIST) {
            softmax_one_row<T, TPR, NCHUNK, MODE>(raw, row, t, nchunks, dst, sum_out, max_out, q_out, q_scale, q_offset, q_offset_scalar, k,
                                                   stats_rep, red);
        } else {
            while (true) {
                const int next = row + stride;
                uint4 ahead[NCHUNK];
                if (next < m) softmax_load_row<T, TPR, NCHUNK>(src + static_cast<size_t>(next) * k, t, nchunks, ahead);
                softmax_one_row<T, TPR, NCHUNK, MODE>(raw, row, t, nchunks, dst, sum_out, max_out, q_out, q_scale, q_offset, q_offset_scalar,
                                                       k, stats_rep, red);
                if (next >= m) break;
#pragma unroll
                for (int i = 0; i < NCHUNK; ++i) raw[i] = ahead[i];
                row = next;
            }
        }
    }
}

template <typename T, int MODE>
int launch_softmax(const T* src, T* dst, float* sum, float* mx, int8_t* q, const __half* qs, const __half* qo, __half qos, int m,
                   int k, int rep, int sms, cudaStream_t st)
{
    constexpr int wpb = kSoftmaxWarpBlock / 32;
    const int warp_grid = std::min((m + wpb - 1) / wpb, 2 * sms);  // persistent: at most two blocks per SM
    const bool persist = m <= 4 * 2 * sms * wpb;                    // up to four rows per warp
    constexpr int VEC = 16 / sizeof(T);
    const int nchunks = k / VEC;
#define ASCB200_SM_WARP(NC)                                                                                              \
    do {                                                                                                                  \
        if (persist) ASCB200_CUDA(launch_pdl(softmax_rows_kernel<T, 32, NC, MODE, true>, warp_grid, kSoftmaxWarpBlock, 0, st, src, dst, sum, mx, q, qs, qo, qos, m, k, rep)); \
        else ASCB200_CUDA(launch_pdl(softmax_rows_kernel<T, 32, NC, MODE, false>, (m + 3) / 4, 128, 0, st, src, dst, sum, mx, q, qs, qo, qos, m, k, rep));                \
    } while (0)
#define ASCB200_SM_BLOCK(TPR, NC) softmax_rows_kernel<T, TPR, NC, MODE, false><<<m, TPR, 0, st>>>(src, dst, sum, mx, q, qs, qo, qos, m, k, rep)
    if (nchunks <= 32) ASCB200_SM_WARP(1);
    else if (nchunks <= 64) ASCB200_SM_WARP(2);
    else if (nchunks <= 128) ASCB200_SM_WARP(4);
    else if (nchunks <= 256) ASCB200_SM_WARP(8);
    else if (nchunks <= 1024) ASCB200_SM_BLOCK(256, 4);
    else if (nchunks <= 2048) ASCB200_SM_BLOCK(256, 8);
    else if (nchunks <= 8192) ASCB200_SM_BLOCK(1024, 8);
    else return ASCB200_ETOOBIG;
#undef ASCB200_SM_WARP
#undef ASCB200_SM_BLOCK
    ASCB200_CUDA(cudaGetLastError());
    return ASCB200_OK;
}

// ---- AscendQuant ------------------------------------------------------------------------------
// 8 elements per thread.  PER_CHANNEL: scale/offset indexed by (element index % scale_count).
template <typename T, bool PER_CHANNEL>
__global__ void __launch_bounds__(256)
quant_vec8_kernel(const T* __restrict__ src, int8_t* __restrict__ dst, size_t n8, int scale_count, const T* __restrict__ scale,
                  const T* __restrict__ offset, __half scale_h, __half offset_h)
{
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n8; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        T x[8], s[8], o[8];
        const size_t e = i * 8;
        if constexpr (sizeof(T) == 2) {
            *reinterpret_cast<uint4*>(x) = ldg_nc_v4(src + e);
        } else {
            *reinterpret_cast<uint4*>(x) = ldg_nc_v4(src + e);
            *reinterpret_cast<uint4*>(x + 4) = ldg_nc_v4(src + e + 4);
        }
        if constexpr (PER_CHANNEL) {
            const int c = static_cast<int>(e % static_cast<size_t>(scale_count));
#pragma unroll
            for (int j = 0; j < 8; ++j) s[j] = scale[c + j];
            if (offset) {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = offset[c + j];
            }
        }
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            __half2 hs = __half2half2(scale_h), ho = __half2half2(offset_h);
            if constexpr (PER_CHANNEL) {
                hs = to_half2_src(s[2 * j], s[2 * j + 1]);
                if (offset) ho = to_half2_src(o[2 * j], o[2 * j + 1]);
            }
            w[j] = quant_half2_bits(to_half2_src(x[2 * j], x[2 * j + 1]), hs, ho);
        }
        const uint32_t pk[2] = {pack_s8x4(w[0], w[1]), pack_s8x4(w[2], w[3])};
        *reinterpret_cast<uint2*>(dst + e) = make_uint2(pk[0], pk[1]);
    }
}
// Per-channel fast path (scale_count a multiple of 8): a thread owns one 8-column vector, converts its scale / offset once
// and walks eight rows with all eight 16-byte loads issued up front, so parameter loads are one per eight data loads
// (one per data load held this kernel at 4.4 TB/s).
template <typename T>
__global__ void __launch_bounds__(256)
quant_channel_rows_kernel(const T* __restrict__ src, int8_t* __restrict__ dst, size_t rows, int nvec, const T* __restrict__ scale,
                          const T* __restrict__ offset, __half offset_h)
{
    constexpr int R = 8;
    const size_t r0 = static_cast<size_t>(blockIdx.x) * R;
    for (int cv = threadIdx.x; cv < nvec; cv += 256) {
        T s[8], o[8];
        *reinterpret_cast<uint4*>(s) = __ldg(reinterpret_cast<const uint4*>(scale + cv * 8));
        if constexpr (sizeof(T) == 4) *reinterpret_cast<uint4*>(s + 4) = __ldg(reinterpret_cast<const uint4*>(scale + cv * 8) + 1);
        if (offset) {
            *reinterpret_cast<uint4*>(o) = __ldg(reinterpret_cast<const uint4*>(offset + cv * 8));
            if constexpr (sizeof(T) == 4) *reinterpret_cast<uint4*>(o + 4) = __ldg(reinterpret_cast<const uint4*>(offset + cv * 8) + 1);
        }
        T x[R][8];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r0 + r < rows) {
                const T* p = src + ((r0 + r) * nvec + cv) * 8;
                *reinterpret_cast<uint4*>(x[r]) = ldg_nc_v4(p);
                if constexpr (sizeof(T) == 4) *reinterpret_cast<uint4*>(x[r] + 4) = ldg_nc_v4(p + 4);
            }
        }
        __half2 hs[4], ho[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            hs[j] = to_half2_src(s[2 * j], s[2 * j + 1]);
            ho[j] = offset ? to_half2_src(o[2 * j], o[2 * j + 1]) : __half2half2(offset_h);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r0 + r < rows) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) w[j] = quant_half2_bits(to_half2_src(x[r][2 * j], x[r][2 * j + 1]), hs[j], ho[j]);
                *reinterpret_cast<uint2*>(dst + ((r0 + r) * nvec + cv) * 8) = make_uint2(pack_s8x4(w[0], w[1]), pack_s8x4(w[2], w[3]));
            }
        }
    }
}
// Scalar path for extents or pointers that do not allow the 8-wide path.
template <typename T, bool PER_CHANNEL>
__global__ void __launch_bounds__(256)
quant_scalar_kernel(const T* __restrict__ src, int8_t* __restrict__ dst, size_t n, int scale_count, const T* __restrict__ scale,
                    const T* __restrict__ offset, __half scale_h, __half offset_h)
{
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        __half hs = scale_h, ho = offset_h;
        if constexpr (PER_CHANNEL) {
            const int c = static_cast<int>(i % static_cast<size_t>(scale_count));
            hs = to_half_src(scale[c]);
            if (offset) ho = to_half_src(offset[c]);
        }
        dst[i] = static_cast<int8_t>(quant_half(to_half_src(src[i]), hs, ho));
    }
}

template <typename T>
int launch_quant(const void* src, int8_t* dst, size_t n, int scale_count, const void* scale, const void* offset, __half scale_h,
                 __half offset_h, int sms, cudaStream_t st)
{
    const bool per_channel = scale != nullptr;
    const bool vec = (n % 8 == 0) && aligned_to(src, 16) && aligned_to(dst, 8) && (!per_channel || scale_count % 8 == 0);
    const size_t work = vec ? n / 8 : n;
    if (work == 0) return ASCB200_OK;
    const int grid = static_cast<int>(std::min<size_t>((work + 255) / 256, static_cast<size_t>(sms) * 16));
    const T* s = static_cast<const T*>(src);
    const T* sc = static_cast<const T*>(scale);
    const T* of = static_cast<const T*>(offset);
    if (vec && per_channel && n % scale_count == 0 && aligned_to(scale, 16) && (!offset || aligned_to(offset, 16)) && n / scale_count <= 0x7FFFFFFFull * 8) {
        const size_t rows = n / scale_count;
        quant_channel_rows_kernel<T><<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(s, dst, rows, scale_count / 8, sc, of, offset_h);
    } else if (vec) {
        if (per_channel) quant_vec8_kernel<T, true><<<grid, 256, 0, st>>>(s, dst, work, scale_count, sc, of, scale_h, offset_h);
        else quant_vec8_kernel<T, false><<<grid, 256, 0, st>>>(s, dst, work, 1, nullptr, nullptr, scale_h, offset_h);
    } else {
        if (per_channel) quant_scalar_kernel<T, true><<<grid, 256, 0, st>>>(s, dst, work, scale_count, sc, of, scale_h, offset_h);
        else quant_scalar_kernel<T, false><<<grid, 256, 0, st>>>(s, dst, work, 1, nullptr, nullptr, scale_h, offset_h);
    }
    ASCB200_CUDA(cudaGetLastError());
    return ASCB200_OK;
}

// ---- AscendDequant ----------------------------------------------------------------------------
template <typename D>
__device__ __forceinline__ D dequant_cast(float v);
template <>
__device__ __forceinline__ float dequant_cast<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half dequant_cast<__half>(float v) { return f32_to_f16_sat(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 dequant_cast<__nv_bfloat16>(float v) { return f32_to_bf16(v); }

// SCALE: 0 scalar, 1 fp32 tensor, 2 bf16 tensor.  VEC = 4 (vector path) or 1.
template <typename D, int SCALE, int VEC>
__global__ void __launch_bounds__(256)
dequant_kernel(const int32_t* __restrict__ src, D* __restrict__ dst, int m, int n, int cal_count, int n_dst, const void* __restrict__ scale,
               float scale_scalar)
{
    const int per_row = cal_count / VEC;
    const size_t total = static_cast<size_t>(m) * per_row;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int r = static_cast<int>(i / per_row);
        const int c = static_cast<int>(i % per_row) * VEC;
        int32_t x[VEC];
        D y[VEC];
        if constexpr (VEC == 4) *reinterpret_cast<uint4*>(x) = ldg_nc_v4(src + static_cast<size_t>(r) * n + c);
        else x[0] = src[static_cast<size_t>(r) * n + c];
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            float s = scale_scalar;
            if constexpr (SCALE == 1) s = static_cast<const float*>(scale)[c + j];
            if constexpr (SCALE == 2) s = __bfloat162float(static_cast<const __nv_bfloat16*>(scale)[c + j]);
            y[j] = dequant_cast<D>(__fmul_rn(static_cast<float>(x[j]), s));
        }
        D* out = dst + static_cast<size_t>(r) * n_dst + c;
        if constexpr (VEC == 4 && sizeof(D) == 4) *reinterpret_cast<uint4*>(out) = *reinterpret_cast<uint4*>(y);
        else if constexpr (VEC == 4) *reinterpret_cast<uint2*>(out) = *reinterpret_cast<uint2*>(y);
        else out[0] = y[0];
    }
}

template <typename D, int SCALE>
int launch_dequant(const int32_t* src, void* dst, int m, int n, int cal, int n_dst, const void* scale, float ss, int sms, cudaStream_t st)
{
    const bool vec = n % 4 == 0 && cal % 4 == 0 && n_dst % 4 == 0 && aligned_to(src, 16) && aligned_to(dst, 16);
    const size_t work = static_cast<size_t>(m) * (vec ? cal / 4 : cal);
    if (work == 0) return ASCB200_OK;
    const int grid = static_cast<int>(std::min<size_t>((work + 255) / 256, static_cast<size_t>(sms) * 16));
    if (vec) dequant_kernel<D, SCALE, 4><<<grid, 256, 0, st>>>(src, static_cast<D*>(dst), m, n, cal, n_dst, scale, ss);
    else dequant_kernel<D, SCALE, 1><<<grid, 256, 0, st>>>(src, static_cast<D*>(dst), m, n, cal, n_dst, scale, ss);
    ASCB200_CUDA(cudaGetLastError());
    return ASCB200_OK;
}

// ---- SoftmaxFlashV2 (include/adv_api/activation/softmaxflashv2.h:93-300) -------------------------------------------------
// One step of the online softmax of FlashAttention-2 over rows [m, k]:
//   update == 0:  max = rowmax(x);                 y = exp(x - max); expSum = rowsum(y)
//   update == 1:  max = max(inMax, rowmax(x));     y = exp(x - max); expMax = exp(inMax - max); expSum = expMax * inExpSum + rowsum(y)
// (formulas of docs/zh/api/SIMD-API/adv_api/activation_functions/SoftMax_interface/SoftmaxFlashV2.md:49-63).  y is not normalised.
// T: element type of x, y and expMax; ST: type of the max / sum tensors (T, or float with half data).  Arithmetic is fp32
// inside, like the reference's half path.  Same row mapping as softmax_rows_kernel (row in registers, read once).
// Volatile loads: the compiler keeps them where they are written (ahead of the row loads) instead of sinking them to
// their first use after the row maximum, where each would add a memory latency to the row's critical path.
template <typename ST> __device__ __forceinline__ void stat_store(ST* p, size_t i, float v);
template <> __device__ __forceinline__ void stat_store<float>(float* p, size_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void stat_store<__half>(__half* p, size_t i, float v) { p[i] = __float2half_rn(clamp_half_range(v)); }

constexpr int kFlashSimple = 2;  // the kernel's `normalise` argument: 0 SoftmaxFlashV2, 1 SoftmaxFlash (normalised y), 2 SimpleSoftMax

template <typename T, typename ST, int TPR, int NCHUNK, bool UPDATE>
__global__ void __launch_bounds__(TPR > 32 ? TPR : 128, TPR > 32 ? 1 : 5)
softmax_flash_rows_kernel(const T* __restrict__ src, T* __restrict__ dst, ST* __restrict__ sum_out, ST* __restrict__ max_out, T* __restrict__ expmax_out,
                          const ST* __restrict__ in_sum, const ST* __restrict__ in_max, int m, int k, int stats_rep, int expmax_rep,
                          int normalise)
{
    constexpr int VEC = 16 / sizeof(T);
    __shared__ float red[32];
    const int nchunks = k / VEC;
    const int t = TPR > 32 ? threadIdx.x : (threadIdx.x & 31);
    const int row = TPR > 32 ? blockIdx.x : blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    // The previous statistics are requested ahead of the row loads (asked for after the row maximum they would put a second
    // memory latency on every row's critical path) and by as few load instructions as possible: every extra load
    // instruction per row measurably costs bandwidth here (two loads per warp: 4.6 TB/s, one: 5.4, one per four rows: see
    // the benchmark).  Warp rows: eight threads of the block fetch the values of its four rows and pass them through shared
    // memory; block rows: threads 0 and 1.
    __shared__ float prev[2][4];
    const bool valid = row < m;
    float old_max = 0.0f, old_sum = 0.0f, exp_max = 1.0f;
    if constexpr (UPDATE) {
        if constexpr (TPR == 32) {
            const int r = blockIdx.x * 4 + (threadIdx.x >> 1);
            if (threadIdx.x < 8 && r < m) old_max = stat_load<ST>((threadIdx.x & 1) ? in_sum : in_max, static_cast<size_t>(r) * stats_rep);
        } else {
            if (threadIdx.x < 2) old_max = stat_load<ST>((threadIdx.x & 1) ? in_sum : in_max, static_cast<size_t>(row) * stats_rep);
        }
    }
    uint4 raw[NCHUNK];
    if (valid) softmax_load_row<T, TPR, NCHUNK>(src + static_cast<size_t>(row) * k, t, nchunks, raw);
    if constexpr (UPDATE) {
        if (threadIdx.x < (TPR == 32 ? 8 : 2)) prev[threadIdx.x & 1][TPR == 32 ? (threadIdx.x >> 1) : 0] = old_max;
        __syncthreads();  // reached by every thread of the block; the row loads stay in flight meanwhile
        old_max = prev[0][TPR == 32 ? (threadIdx.x >> 5) : 0];
        old_sum = prev[1][TPR == 32 ? (threadIdx.x >> 5) : 0];
    }
    if (!valid) return;  // whole warp / block leaves together
    float v[NCHUNK * VEC];
    float mx = kNegInf;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        const int c = t + i * TPR;
        if (c < nchunks) {
            if constexpr (sizeof(T) == 2) {
                const __half2* h = reinterpret_cast<const __half2*>(&raw[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __half22float2(h[j]);
                    v[i * 8 + 2 * j] = f.x;
                    v[i * 8 + 2 * j + 1] = f.y;
                }
            } else {
                v[i * 4 + 0] = __uint_as_float(raw[i].x);
                v[i * 4 + 1] = __uint_as_float(raw[i].y);
                v[i * 4 + 2] = __uint_as_float(raw[i].z);
                v[i * 4 + 3] = __uint_as_float(raw[i].w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[i * VEC + j] = kNegInf;
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) mx = fmaxf(mx, v[i * VEC + j]);
    }
    // normalise == kFlashSimple (UPDATE instantiations only): SimpleSoftMax, the given statistics ARE the maximum and the sum
    // (impl/adv_api/detail/activation/softmax/membase/common/simple_softmax_common_impl.h:320-502); nothing is reduced or stored.
    const bool simple = UPDATE && normalise == kFlashSimple;
    if (simple) {
        mx = old_max;
    } else {
        mx = row_reduce_max<TPR>(mx, red);
        if constexpr (UPDATE) {
            mx = fmaxf(mx, old_max);
            exp_max = exp2_approx((old_max - mx) * 1.4426950408889634f);
        }
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NCHUNK * VEC; ++i) {
        v[i] = exp2_approx((v[i] - mx) * 1.4426950408889634f);
        s += v[i];
    }
    if (simple) {
        s = old_sum;
    } else {
        s = row_reduce_sum<TPR>(s, red);
        if constexpr (UPDATE) s = __fadd_rn(__fmul_rn(exp_max, old_sum), s);
    }
    if (normalise) {  // SoftmaxFlash (the first version): y = exp(x - max) / sum, expMax = exp(inMax - max) * inSum / sum
        const float inv = __frcp_rn(s);
#pragma unroll
        for (int i = 0; i < NCHUNK * VEC; ++i) {
            v[i] *= inv;
            if constexpr (sizeof(T) == 2) v[i] = fminf(v[i], 65504.0f);  // statistics of another tile can push y past the half range
        }
        if constexpr (UPDATE) exp_max = __fmul_rn(exp_max, old_sum) * inv;
    }

    T* drow = dst + static_cast<size_t>(row) * k;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        const int c = t + i * TPR;
        if (c < nchunks) {
            if constexpr (sizeof(T) == 2) {
                uint4 o;  // values lie in [0, 1]
                __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(v[i * 8 + 2 * j], v[i * 8 + 2 * j + 1]);
                *reinterpret_cast<uint4*>(drow + c * 8) = o;
            } else {
                *reinterpret_cast<float4*>(drow + c * 4) = make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
            }
        }
    }
    if (simple) return;
    if (t < stats_rep) {
        stat_store<ST>(sum_out, static_cast<size_t>(row) * stats_rep + t, s);
        stat_store<ST>(max_out, static_cast<size_t>(row) * stats_rep + t, mx);
    }
    if (UPDATE && t < expmax_rep) {
        if constexpr (sizeof(T) == 2) expmax_out[static_cast<size_t>(row) * expmax_rep + t] = __float2half_rn(exp_max);
        else expmax_out[static_cast<size_t>(row) * expmax_rep + t] = exp_max;
    }
}

template <typename T, typename ST, bool UPDATE>
int launch_softmax_flash(const T* src, T* dst, ST* sum, ST* mx, T* expmax, const ST* in_sum, const ST* in_max, int m, int k, int stats_rep,
                         int expmax_rep, int normalise, cudaStream_t st)
{
    constexpr int VEC = 16 / sizeof(T);
    const int nchunks = k / VEC;
#define ASCB200_SF_WARP(NC) softmax_flash_rows_kernel<T, ST, 32, NC, UPDATE><<<(m + 3) / 4, 128, 0, st>>>(src, dst, sum, mx, expmax, in_sum, in_max, m, k, stats_rep, expmax_rep, normalise)
#define ASCB200_SF_BLOCK(TPR, NC) softmax_flash_rows_kernel<T, ST, TPR, NC, UPDATE><<<m, TPR, 0, st>>>(src, dst, sum, mx, expmax, in_sum, in_max, m, k, stats_rep, expmax_rep, normalise)
    if (nchunks <= 32) ASCB200_SF_WARP(1);
    else if (nchunks <= 64) ASCB200_SF_WARP(2);
    else if (nchunks <= 128) ASCB200_SF_WARP(4);
    else if (nchunks <= 256) ASCB200_SF_WARP(8);
    else if (nchunks <= 1024) ASCB200_SF_BLOCK(256, 4);
    else if (nchunks <= 2048) ASCB200_SF_BLOCK(256, 8);
    else return ASCB200_ETOOBIG;
#undef ASCB200_SF_WARP
#undef ASCB200_SF_BLOCK
    ASCB200_CUDA(cudaGetLastError());
    return ASCB200_OK;
}

// ---- SoftmaxGrad / SoftmaxGradFront (include/adv_api/activation/softmaxgrad.h:57-175) ------------------------------------
// Per row of grad and src (the softmax output y): s = rowsum(grad * src) in fp32;
//   FRONT:  dst[m, rep] = s (one 32-byte block per row);      else: dst[m, k] = (grad - s) * src, cast RINT
// (impl/adv_api/detail/activation/softmax/membase/common/softmax_grad_nd_impl.h:27-60).  Both rows stay in registers between
// the reduction and the output pass: 6 bytes of traffic per half element (4 in FRONT mode), each byte moved once.
template <typename T>
__device__ __forceinline__ void unpack_chunk(const uint4& raw, float (&f)[16 / sizeof(T)])
{
    if constexpr (sizeof(T) == 2) {
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 v = __half22float2(h[j]);
            f[2 * j] = v.x;
            f[2 * j + 1] = v.y;
        }
    } else {
        f[0] = __uint_as_float(raw.x);
        f[1] = __uint_as_float(raw.y);
        f[2] = __uint_as_float(raw.z);
        f[3] = __uint_as_float(raw.w);
    }
}

template <typename T, int TPR, int NCHUNK, bool FRONT>
__global__ void __launch_bounds__(TPR > 32 ? TPR : 128, TPR > 32 ? 1 : 4)
softmax_grad_rows_kernel(const T* __restrict__ grad, const T* __restrict__ src, T* __restrict__ dst, int m, int k, int front_rep)
{
    constexpr int VEC = 16 / sizeof(T);
    __shared__ float red[32];
    const int nchunks = k / VEC;
    const int t = TPR > 32 ? threadIdx.x : (threadIdx.x & 31);
    const int row = TPR > 32 ? blockIdx.x : blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= m) return;  // a whole warp (or block) leaves together
    uint4 rg[NCHUNK], rs[NCHUNK];
    softmax_load_row<T, TPR, NCHUNK>(grad + static_cast<size_t>(row) * k, t, nchunks, rg);
    softmax_load_row<T, TPR, NCHUNK>(src + static_cast<size_t>(row) * k, t, nchunks, rs);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        if (t + i * TPR < nchunks) {
            float g[VEC], y[VEC];
            unpack_chunk<T>(rg[i], g);
            unpack_chunk<T>(rs[i], y);
#pragma unroll
            for (int j = 0; j < VEC; ++j) s += __fmul_rn(g[j], y[j]);  // Mul then ReduceSum: the product is rounded before it is added
        }
    }
    s = row_reduce_sum<TPR>(s, red);
    if constexpr (FRONT) {
        if (t < front_rep) {
            if constexpr (sizeof(T) == 2) dst[static_cast<size_t>(row) * front_rep + t] = __float2half_rn(clamp_half_range(s));
            else dst[static_cast<size_t>(row) * front_rep + t] = s;
        }
    } else {
        T* drow = dst + static_cast<size_t>(row) * k;
#pragma unroll
        for (int i = 0; i < NCHUNK; ++i) {
            const int c = t + i * TPR;
            if (c < nchunks) {
                float g[VEC], y[VEC];
                unpack_chunk<T>(rg[i], g);
                unpack_chunk<T>(rs[i], y);
#pragma unroll
                for (int j = 0; j < VEC; ++j) g[j] = __fmul_rn(__fsub_rn(g[j], s), y[j]);
                if constexpr (sizeof(T) == 2) {
                    uint4 o;
                    __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
                    for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(clamp_half_range(g[2 * j]), clamp_half_range(g[2 * j + 1]));
                    *reinterpret_cast<uint4*>(drow + c * 8) = o;
                } else {
                    *reinterpret_cast<float4*>(drow + c * 4) = make_float4(g[0], g[1], g[2], g[3]);
                }
            }
        }
    }
}

template <typename T, bool FRONT>
int launch_softmax_grad(const T* grad, const T* src, T* dst, int m, int k, int front_rep, cudaStream_t st)
{
    constexpr int VEC = 16 / sizeof(T);
    const int nchunks = k / VEC;
#define ASCB200_SG_WARP(NC) softmax_grad_rows_kernel<T, 32, NC, FRONT><<<(m + 3) / 4, 128, 0, st>>>(grad, src, dst, m, k, front_rep)
#define ASCB200_SG_BLOCK(TPR, NC) softmax_grad_rows_kernel<T, TPR, NC, FRONT><<<m, TPR, 0, st>>>(grad, src, dst, m, k, front_rep)
    if (nchunks <= 32) ASCB200_SG_WARP(1);
    else if (nchunks <= 64) ASCB200_SG_WARP(2);
    else if (nchunks <= 128) ASCB200_SG_WARP(4);
    else if (nchunks <= 256) ASCB200_SG_WARP(8);
    else if (nchunks <= 1024) ASCB200_SG_BLOCK(256, 4);
    else if (nchunks <= 2048) ASCB200_SG_BLOCK(256, 8);
    else if (nchunks <= 8192) ASCB200_SG_BLOCK(1024, 8);
    else return ASCB200_ETOOBIG;
#undef ASCB200_SG_WARP
#undef ASCB200_SG_BLOCK
    ASCB200_CUDA(cudaGetLastError());
    return ASCB200_OK;
}

int check_softmax_args(const void* src, void* dst, float* sum, float* mx, int m, int k, int dtype)
{
    if (!src || !dst || !sum || !mx || m < 0 || k <= 0) return ASCB200_EINVAL;
    if (dtype != ASCB200_F16 && dtype != ASCB200_F32) return ASCB200_EUNSUPPORTED;
    const int esz = dtype == ASCB200_F16 ? 2 : 4;
    if ((static_cast<size_t>(k) * esz) % 32 != 0) return ASCB200_EALIGN;  // the reference's last-axis rule
    if (!aligned_to(src, 16) || !aligned_to(dst, 16)) return ASCB200_EALIGN;
    return ASCB200_OK;
}

__half scalar_as_src_half(float v, int dtype)
{
    // The per-channel overload takes the scalar offset in the source type T; the operator then
    // converts T to half exactly like the tensor elements.
    if (dtype == ASCB200_F16) return __float2half_rn(v);
    if (dtype == ASCB200_BF16) v = __bfloat162float(__float2bfloat16_rn(v));
    unsigned short b = __half_as_ushort(__float2half_rn(v));
    if ((b & 0x7FFFu) == 0x7C00u) b = (b & 0x8000u) | 0x7BFFu;
    return __ushort_as_half(b);
}

}  // namespace
}  // namespace ascb200

using namespace ascb200;

extern "C" {

int ascb200_softmax(const void* src, void* dst, float* sum, float* mx, int32_t m, int32_t k, int32_t dtype, int32_t stats_brc,
                    void* stream)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    int rc = check_softmax_args(src, dst, sum, mx, m, k, dtype);
    if (rc != ASCB200_OK) return rc;
    if (m == 0) return ASCB200_OK;
    const int rep = stats_brc ? 8 : 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == ASCB200_F16)
        return launch_softmax<__half, kSoftmaxPlain>(static_cast<const __half*>(src), static_cast<__half*>(dst), sum, mx, nullptr, nullptr,
                                             nullptr, __half(), m, k, rep, st->sm_count, s);
    return launch_softmax<float, kSoftmaxPlain>(static_cast<const float*>(src), static_cast<float*>(dst), sum, mx, nullptr, nullptr, nullptr,
                                        __half(), m, k, rep, st->sm_count, s);
}

int ascb200_log_softmax(const void* src, void* dst, void* sum, void* mx, int32_t m, int32_t k, int32_t dtype, int32_t stats_brc,
                        void* stream)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    int rc = check_softmax_args(src, dst, static_cast<float*>(sum), static_cast<float*>(mx), m, k, dtype);
    if (rc != ASCB200_OK) return rc;
    if (m == 0) return ASCB200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == ASCB200_F16)  // statistics in half: one 32-byte block holds 16 of them
        return launch_softmax<__half, kSoftmaxLog>(static_cast<const __half*>(src), static_cast<__half*>(dst), static_cast<float*>(sum),
                                                   static_cast<float*>(mx), nullptr, nullptr, nullptr, __half(), m, k, stats_brc ? 16 : 1,
                                                   st->sm_count, s);
    return launch_softmax<float, kSoftmaxLog>(static_cast<const float*>(src), static_cast<float*>(dst), static_cast<float*>(sum),
                                              static_cast<float*>(mx), nullptr, nullptr, nullptr, __half(), m, k, stats_brc ? 8 : 1,
                                              st->sm_count, s);
}

int ascb200_simple_softmax(const void* src, void* dst, const void* in_sum, const void* in_max, int32_t m, int32_t k, int32_t dtype,
                           int32_t stats_dtype, int32_t stats_brc, void* stream)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!src || !dst || !in_sum || !in_max || m < 0 || k <= 0) return ASCB200_EINVAL;
    if (dtype != ASCB200_F16 && dtype != ASCB200_F32) return ASCB200_EUNSUPPORTED;
    // statistics have the data type, or fp32 beside half data (the two overload families of the reference)
    if (stats_dtype != dtype && !(dtype == ASCB200_F16 && stats_dtype == ASCB200_F32)) return ASCB200_EUNSUPPORTED;
    const int esz = dtype == ASCB200_F16 ? 2 : 4;
    if ((static_cast<size_t>(k) * esz) % 32 != 0) return ASCB200_EALIGN;
    if (!aligned_to(src, 16) || !aligned_to(dst, 16)) return ASCB200_EALIGN;
    if (m == 0) return ASCB200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int rep = stats_brc ? (stats_dtype == ASCB200_F16 ? 16 : 8) : 1;
    // Rows that fit the flash kernel (16384 halves / 8192 floats) go there: its statistics arrive through shared memory from one
    // load instruction per four rows, which measures 6 - 15 % faster than one per warp.
    if (k / (16 / esz) <= 2048) {
        if (dtype == ASCB200_F32)
            return launch_softmax_flash<float, float, true>(static_cast<const float*>(src), static_cast<float*>(dst), nullptr, nullptr, nullptr,
                                                            static_cast<const float*>(in_sum), static_cast<const float*>(in_max), m, k, rep, 1,
                                                            kFlashSimple, s);
        if (stats_dtype == ASCB200_F32)
            return launch_softmax_flash<__half, float, true>(static_cast<const __half*>(src), static_cast<__half*>(dst), nullptr, nullptr, nullptr,
                                                             static_cast<const float*>(in_sum), static_cast<const float*>(in_max), m, k, rep, 1,
                                                             kFlashSimple, s);
        return launch_softmax_flash<__half, __half, true>(static_cast<const __half*>(src), static_cast<__half*>(dst), nullptr, nullptr, nullptr,
                                                          static_cast<const __half*>(in_sum), static_cast<const __half*>(in_max), m, k, rep, 1,
                                                          kFlashSimple, s);
    }
    // longer rows: the row kernel reads the statistics through its (otherwise output) statistics pointers
    float* sum = static_cast<float*>(const_cast<void*>(in_sum));
    float* mx = static_cast<float*>(const_cast<void*>(in_max));
    if (dtype == ASCB200_F32)
        return launch_softmax<float, kSoftmaxSimpleF32>(static_cast<const float*>(src), static_cast<float*>(dst), sum, mx, nullptr, nullptr,
                                                        nullptr, __half(), m, k, rep, st->sm_count, s);
    if (stats_dtype == ASCB200_F32)
        return launch_softmax<__half, kSoftmaxSimpleF32>(static_cast<const __half*>(src), static_cast<__half*>(dst), sum, mx, nullptr, nullptr,
                                                         nullptr, __half(), m, k, rep, st->sm_count, s);
    return launch_softmax<__half, kSoftmaxSimpleF16>(static_cast<const __half*>(src), static_cast<__half*>(dst), sum, mx, nullptr, nullptr,
                                                     nullptr, __half(), m, k, rep, st->sm_count, s);
}

int ascb200_softmax_grad(const void* grad, const void* src, void* dst, int32_t m, int32_t k, int32_t dtype, int32_t is_front, void* stream)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!grad || !src || !dst || m < 0 || k <= 0) return ASCB200_EINVAL;
    if (dtype != ASCB200_F16 && dtype != ASCB200_F32) return ASCB200_EUNSUPPORTED;
    const int esz = dtype == ASCB200_F16 ? 2 : 4;
    if ((static_cast<size_t>(k) * esz) % 32 != 0) return ASCB200_EALIGN;
    if (!aligned_to(grad, 16) || !aligned_to(src, 16) || !aligned_to(dst, is_front ? esz : 16)) return ASCB200_EALIGN;
    if (m == 0) return ASCB200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int rep = 32 / esz;
    if (dtype == ASCB200_F16) {
        const __half *g = static_cast<const __half*>(grad), *y = static_cast<const __half*>(src);
        return is_front ? launch_softmax_grad<__half, true>(g, y, static_cast<__half*>(dst), m, k, rep, s)
                        : launch_softmax_grad<__half, false>(g, y, static_cast<__half*>(dst), m, k, rep, s);
    }
    const float *g = static_cast<const float*>(grad), *y = static_cast<const float*>(src);
    return is_front ? launch_softmax_grad<float, true>(g, y, static_cast<float*>(dst), m, k, rep, s)
                    : launch_softmax_grad<float, false>(g, y, static_cast<float*>(dst), m, k, rep, s);
}

static int softmax_flash_entry(const void* src, void* dst, void* exp_sum, void* max, void* exp_max, const void* in_exp_sum, const void* in_max,
                        int32_t m, int32_t k, int32_t dtype, int32_t stats_dtype, int32_t update, int32_t stats_brc, int normalise, void* stream)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!src || !dst || !exp_sum || !max || m < 0 || k <= 0) return ASCB200_EINVAL;
    if (update && (!exp_max || !in_exp_sum || !in_max)) return ASCB200_EINVAL;
    if (dtype != ASCB200_F16 && dtype != ASCB200_F32) return ASCB200_EUNSUPPORTED;
    if (!(stats_dtype == dtype || (dtype == ASCB200_F16 && stats_dtype == ASCB200_F32))) return ASCB200_EUNSUPPORTED;  // the reference's overloads
    const int esz = dtype == ASCB200_F16 ? 2 : 4;
    if ((static_cast<size_t>(k) * esz) % 32 != 0) return ASCB200_EALIGN;
    if (!aligned_to(src, 16) || !aligned_to(dst, 16)) return ASCB200_EALIGN;
    if (m == 0) return ASCB200_OK;
    const int stats_rep = stats_brc ? 32 / (stats_dtype == ASCB200_F16 ? 2 : 4) : 1;  // one 32-byte block per row
    const int expmax_rep = stats_brc ? 32 / esz : 1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define ASCB200_SF_CALL(T, ST, UPD)                                                                                                      \
    return launch_softmax_flash<T, ST, UPD>(static_cast<const T*>(src), static_cast<T*>(dst), static_cast<ST*>(exp_sum), static_cast<ST*>(max), \
                                            static_cast<T*>(exp_max), static_cast<const ST*>(in_exp_sum), static_cast<const ST*>(in_max), m, k, \
                                            stats_rep, expmax_rep, normalise, s)
    if (dtype == ASCB200_F32) {
        if (update) ASCB200_SF_CALL(float, float, true);
        ASCB200_SF_CALL(float, float, false);
    }
    if (stats_dtype == ASCB200_F32) {
        if (update) ASCB200_SF_CALL(__half, float, true);
        ASCB200_SF_CALL(__half, float, false);
    }
    if (update) ASCB200_SF_CALL(__half, __half, true);
    ASCB200_SF_CALL(__half, __half, false);
#undef ASCB200_SF_CALL
}

int ascb200_softmax_flash_v2(const void* src, void* dst, void* exp_sum, void* max, void* exp_max, const void* in_exp_sum, const void* in_max,
                             int32_t m, int32_t k, int32_t dtype, int32_t stats_dtype, int32_t update, int32_t stats_brc, void* stream)
{
    return softmax_flash_entry(src, dst, exp_sum, max, exp_max, in_exp_sum, in_max, m, k, dtype, stats_dtype, update, stats_brc, 0, stream);
}

int ascb200_softmax_flash(const void* src, void* dst, void* sum, void* max, void* exp_max, const void* in_sum, const void* in_max, int32_t m,
                          int32_t k, int32_t dtype, int32_t stats_dtype, int32_t update, int32_t stats_brc, void* stream)
{
    return softmax_flash_entry(src, dst, sum, max, exp_max, in_sum, in_max, m, k, dtype, stats_dtype, update, stats_brc, 1, stream);
}

int ascb200_softmax_quant(const void* src, void* dst, float* sum, float* mx, int8_t* q, const void* scale, const void* offset_t,
                          float offset, int32_t m, int32_t k, int32_t stats_brc, void* stream)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    int rc = check_softmax_args(src, dst, sum, mx, m, k, ASCB200_F16);
    if (rc != ASCB200_OK) return rc;
    if (!q || !scale) return ASCB200_EINVAL;
    if (!aligned_to(q, 8) || !aligned_to(scale, 16) || (offset_t && !aligned_to(offset_t, 16))) return ASCB200_EALIGN;
    if (m == 0) return ASCB200_OK;
    return launch_softmax<__half, kSoftmaxQuant>(static_cast<const __half*>(src), static_cast<__half*>(dst), sum, mx, q,
                                        static_cast<const __half*>(scale), static_cast<const __half*>(offset_t),
                                        __float2half_rn(offset), m, k, stats_brc ? 8 : 1, st->sm_count, static_cast<cudaStream_t>(stream));
}

int ascb200_quant_per_tensor(const void* src, int8_t* dst, int64_t cal_count, int32_t dtype, float scale, float offset, void* stream)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!src || !dst || cal_count < 0) return ASCB200_EINVAL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const __half hs = __float2half_rn(scale), ho = __float2half_rn(offset);  // static_cast<half>(scale)
    const size_t n = static_cast<size_t>(cal_count);
    switch (dtype) {
        case ASCB200_F16: return launch_quant<__half>(src, dst, n, 1, nullptr, nullptr, hs, ho, st->sm_count, s);
        case ASCB200_BF16: return launch_quant<__nv_bfloat16>(src, dst, n, 1, nullptr, nullptr, hs, ho, st->sm_count, s);
        case ASCB200_F32: return launch_quant<float>(src, dst, n, 1, nullptr, nullptr, hs, ho, st->sm_count, s);
        default: return ASCB200_EUNSUPPORTED;
    }
}

int ascb200_quant_per_channel(const void* src, int8_t* dst, int32_t rows, int32_t scale_count, int32_t dtype, const void* scale,
                              const void* offset_t, float offset, void* stream)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!src || !dst || !scale || rows < 0 || scale_count <= 0) return ASCB200_EINVAL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t n = static_cast<size_t>(rows) * scale_count;
    const __half ho = scalar_as_src_half(offset, dtype);
    switch (dtype) {
        case ASCB200_F16: return launch_quant<__half>(src, dst, n, scale_count, scale, offset_t, __half(), ho, st->sm_count, s);
        case ASCB200_BF16: return launch_quant<__nv_bfloat16>(src, dst, n, scale_count, scale, offset_t, __half(), ho, st->sm_count, s);
        case ASCB200_F32: return launch_quant<float>(src, dst, n, scale_count, scale, offset_t, __half(), ho, st->sm_count, s);
        default: return ASCB200_EUNSUPPORTED;
    }
}

int ascb200_dequant(const int32_t* src, void* dst, int32_t m, int32_t n, int32_t cal_count, int32_t n_dst, int32_t dst_dtype,
                    const void* scale, int32_t scale_dtype, float scale_scalar, void* stream)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!src || !dst || m < 0 || n <= 0 || cal_count < 0 || cal_count > n || n_dst < cal_count) return ASCB200_EINVAL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int sms = st->sm_count;
#define ASCB200_DEQ(D)                                                                                                     \
    do {                                                                                                                   \
        if (!scale) return launch_dequant<D, 0>(src, dst, m, n, cal_count, n_dst, nullptr, scale_scalar, sms, s);          \
        if (scale_dtype == ASCB200_F32) return launch_dequant<D, 1>(src, dst, m, n, cal_count, n_dst, scale, 0.f, sms, s);  \
        if (scale_dtype == ASCB200_BF16) return launch_dequant<D, 2>(src, dst, m, n, cal_count, n_dst, scale, 0.f, sms, s); \
        return ASCB200_EUNSUPPORTED;                                                                                       \
    } while (0)
    switch (dst_dtype) {
        case ASCB200_F32: ASCB200_DEQ(float);
        case ASCB200_F16: ASCB200_DEQ(__half);
        case ASCB200_BF16: ASCB200_DEQ(__nv_bfloat16);
        default: return ASCB200_EUNSUPPORTED;
    }
#undef ASCB200_DEQ
}

}  // extern "C"
