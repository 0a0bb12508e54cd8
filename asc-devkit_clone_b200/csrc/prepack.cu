// Layout conversion of fractal ("NZ") matrices into the row-major layouts the GEMM kernels read.
//
// The reference stores a [K, N] weight in NZ format as [N/C0][K/16][16][C0] with C0 = 32 bytes / element size
// (int8: 32, fp16/bf16: 16), i.e. 512-byte blocks of 16 K-rows x C0 columns, all K of one column block
// contiguous (the grouped matmul example writes its int8 weights as
// weight.reshape([g, k/16, 16, n/32, 32]).transpose([0, 3, 1, 2, 4]),
// quant_group_matmul_high_performance/scripts/gen_data.py:62).  On Ascend this is the layout the cube unit
// consumes; tcgen05 reads 128-byte-swizzled row-major tiles placed by TMA, so an NZ weight is unpacked once
// (weights are static) into [N, K] (K contiguous, the layout of the timed configs) or [K, N].
#include <cstdint>

#include "ascb200.h"
#include "common.cuh"

namespace ascb200 {
namespace {

constexpr int TILE_K = 512;  // K rows per block: 16 KB of source, contiguous in NZ

// 4 x 4 byte transpose: in r[j] byte b = element (row j, column b); out c[b] byte j = the same element.
__device__ __forceinline__ void transpose4x4_bytes(const uint32_t (&r)[4], uint32_t (&c)[4])
{
    const uint32_t t0 = __byte_perm(r[0], r[1], 0x5140), t1 = __byte_perm(r[2], r[3], 0x5140);  // columns 0,1 of rows (0,1) / (2,3)
    const uint32_t t2 = __byte_perm(r[0], r[1], 0x7362), t3 = __byte_perm(r[2], r[3], 0x7362);  // columns 2,3
    c[0] = __byte_perm(t0, t1, 0x5410);
    c[1] = __byte_perm(t0, t1, 0x7632);
    c[2] = __byte_perm(t2, t3, 0x5410);
    c[3] = __byte_perm(t2, t3, 0x7632);
}

// grid = groups * (n / C0) * k_tiles blocks of 256 threads
template <int ESZ, bool TO_NK>
__global__ void __launch_bounds__(256) nz_unpack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int k, int n, int k_tiles)
{
    constexpr int C0 = 32 / ESZ;
    // K row r sits at word r * 8 + (r / 16) * 4: 16 bytes of padding after every 16 rows, so that the lanes of a warp, which
    // read the same column word of rows 16 apart, hit 32 different banks, and every row stays 16-byte aligned
    __shared__ __align__(16) uint32_t tile[TILE_K * 8 + (TILE_K / 16) * 4];
    const int n_blocks = n / C0;
    const int kt = blockIdx.x % k_tiles;
    const int nb = (blockIdx.x / k_tiles) % n_blocks;
    const size_t g = blockIdx.x / (static_cast<size_t>(k_tiles) * n_blocks);
    const int k0 = kt * TILE_K;
    const int rows = min(TILE_K, k - k0);  // a multiple of 16
    const uint4* s16 = reinterpret_cast<const uint4*>(src + ((g * n_blocks + nb) * static_cast<size_t>(k) + k0) * 32);
    if constexpr (!TO_NK) {
        // [K, N]: every K row of the block is 32 contiguous bytes of the output row
        for (int i = threadIdx.x; i < rows * 2; i += 256) {
            const uint4 v = __ldg(s16 + i);
            uint8_t* out = dst + ((g * k + k0 + (i >> 1)) * static_cast<size_t>(n) + static_cast<size_t>(nb) * C0) * ESZ + (i & 1) * 16;
            *reinterpret_cast<uint4*>(out) = v;
        }
    } else {
    for (int i = threadIdx.x; i < rows * 2; i += 256) {
        const int r = i >> 1;
        *reinterpret_cast<uint4*>(tile + r * 8 + (r >> 4) * 4 + (i & 1) * 4) = __ldg(s16 + i);
    }
    __syncthreads();
    const auto word_at = [&](int r, int w) { return tile[r * 8 + (r >> 4) * 4 + w]; };
    if constexpr (ESZ == 1) {
        // A thread owns 4 columns x 16 K: sixteen words in, four 4x4 byte transposes, one 16-byte vector out per column.
        // Eight neighbouring lanes take eight consecutive K groups of the same columns: a store instruction of the warp
        // then writes 128 contiguous bytes to each of four output rows.
        static_assert(TILE_K / 16 * 8 == 256, "one task per thread");
        for (int task = threadIdx.x; task < 256; task += 256) {
            const int kg = (task & 7) + (task >> 6) * 8, nw = (task >> 3) & 7;
            if (kg >= rows / 16) continue;
            uint32_t col[4][4];  // [column][quarter of the 16 K]
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t r[4], c[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) r[j] = word_at(kg * 16 + q * 4 + j, nw);
                transpose4x4_bytes(r, c);
#pragma unroll
                for (int b = 0; b < 4; ++b) col[b][q] = c[b];
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                uint8_t* out = dst + (g * n + static_cast<size_t>(nb) * C0 + nw * 4 + b) * k + k0 + kg * 16;
                *reinterpret_cast<uint4*>(out) = make_uint4(col[b][0], col[b][1], col[b][2], col[b][3]);
            }
        }
    } else {
        // 2-byte elements: a thread owns 2 columns x 8 K: eight words in, halves regrouped, one 16-byte vector per column.
        for (int task = threadIdx.x; task < 8 * (rows / 8); task += 256) {
            const int nw = task & 7, kg = task >> 3;
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t a = word_at(kg * 8 + 2 * j, nw), b = word_at(kg * 8 + 2 * j + 1, nw);
                lo[j] = __byte_perm(a, b, 0x5410);  // column 2 nw of rows (2j, 2j+1)
                hi[j] = __byte_perm(a, b, 0x7632);  // column 2 nw + 1
            }
            uint8_t* out = dst + ((g * n + static_cast<size_t>(nb) * C0 + nw * 2) * k + k0 + kg * 8) * 2;
            *reinterpret_cast<uint4*>(out) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            *reinterpret_cast<uint4*>(out + static_cast<size_t>(k) * 2) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        }
    }
    }
}

}  // namespace
}  // namespace ascb200

extern "C" int ascb200_nz_unpack(const void* src_nz, void* dst, int32_t groups, int32_t k, int32_t n, int32_t elem_bytes, int32_t to_nk, void* stream)
{
    using namespace ascb200;
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!src_nz || !dst || groups < 0 || k < 0 || n < 0) return ASCB200_EINVAL;
    if (elem_bytes != 1 && elem_bytes != 2) return ASCB200_EUNSUPPORTED;
    const int c0 = 32 / elem_bytes;
    if (k % 16 != 0 || n % c0 != 0) return ASCB200_EINVAL;  // whole fractal blocks only, like the reference's NZ shapes
    if (!aligned_to(src_nz, 16) || !aligned_to(dst, 16)) return ASCB200_EALIGN;
    if (groups == 0 || k == 0 || n == 0) return ASCB200_OK;
    const int k_tiles = (k + TILE_K - 1) / TILE_K;
    const long long blocks = static_cast<long long>(groups) * (n / c0) * k_tiles;
    if (blocks > 0x7FFFFFFFll) return ASCB200_ETOOBIG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t* src = static_cast<const uint8_t*>(src_nz);
    uint8_t* out = static_cast<uint8_t*>(dst);
    const unsigned grid = static_cast<unsigned>(blocks);
    if (elem_bytes == 1) {
        if (to_nk) nz_unpack_kernel<1, true><<<grid, 256, 0, s>>>(src, out, k, n, k_tiles);
        else nz_unpack_kernel<1, false><<<grid, 256, 0, s>>>(src, out, k, n, k_tiles);
    } else {
        if (to_nk) nz_unpack_kernel<2, true><<<grid, 256, 0, s>>>(src, out, k, n, k_tiles);
        else nz_unpack_kernel<2, false><<<grid, 256, 0, s>>>(src, out, k, n, k_tiles);
    }
    ASCB200_CUDA(cudaGetLastError());
    return ASCB200_OK;
}
