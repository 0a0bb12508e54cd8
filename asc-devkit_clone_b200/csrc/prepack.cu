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

// Transposition of a packed fp4 matrix: src [rows][cols / 2] (column pairs per byte, even column low) -> dst [cols][rows / 2]
// (row pairs per byte, even row low).  A block moves a tile of 256 rows x 64 columns through shared memory (rows read as 32
// contiguous bytes; 36-byte row pitch keeps the word writes off each other's banks); a thread then builds, for one column, the 32
// output bytes of 64 consecutive rows and stores them as two 16-byte vectors when the destination allows.
constexpr int FP4_T_ROWS = 256, FP4_T_COLS = 64, FP4_T_PITCH = 36;

__global__ void __launch_bounds__(256)
fp4_transpose_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int rows, int cols, int src_pitch, int dst_pitch)
{
    __shared__ __align__(16) uint8_t tile[FP4_T_ROWS * FP4_T_PITCH];
    grid_dependency_wait();
    const int r0 = blockIdx.y * FP4_T_ROWS, c0 = blockIdx.x * FP4_T_COLS;
    {
        // thread t loads row r0 + t: 32 bytes = columns c0 .. c0 + 63
        const int r = r0 + threadIdx.x;
        uint32_t w[8];
        const uint8_t* p = src + static_cast<size_t>(r) * src_pitch + c0 / 2;
        const bool full = r < rows && c0 + FP4_T_COLS <= cols && (reinterpret_cast<uintptr_t>(p) & 3) == 0;
        if (full) {
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = __ldg(reinterpret_cast<const uint32_t*>(p) + j);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                w[j] = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    if (r < rows && c0 + (4 * j + b) * 2 < cols) w[j] |= static_cast<uint32_t>(p[4 * j + b]) << (8 * b);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) *reinterpret_cast<uint32_t*>(tile + threadIdx.x * FP4_T_PITCH + 4 * j) = w[j];
    }
    __syncthreads();
    // thread (c, q): column c0 + c, rows r0 + 64 q .. + 63 -> 32 output bytes
    const int c = threadIdx.x & 63, q = threadIdx.x >> 6;
    if (c0 + c >= cols) return;
    const int shift = 4 * (c & 1);
    uint32_t out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int rp = 64 * q + 2 * (4 * j + b);   // even row of the pair, inside the tile
            const uint32_t lo = (tile[rp * FP4_T_PITCH + (c >> 1)] >> shift) & 0xFu;
            const uint32_t hi = (tile[(rp + 1) * FP4_T_PITCH + (c >> 1)] >> shift) & 0xFu;
            word |= (lo | (hi << 4)) << (8 * b);
        }
        out[j] = word;
    }
    uint8_t* o = dst + static_cast<size_t>(c0 + c) * dst_pitch + (r0 + 64 * q) / 2;
    const int valid = min(32, (rows - (r0 + 64 * q) + 1) / 2);   // output bytes that lie inside the matrix
    if (valid <= 0) return;
    if (valid == 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
        *reinterpret_cast<uint4*>(o) = make_uint4(out[0], out[1], out[2], out[3]);
        *reinterpret_cast<uint4*>(o + 16) = make_uint4(out[4], out[5], out[6], out[7]);
    } else {
        for (int b = 0; b < valid; ++b) o[b] = static_cast<uint8_t>(out[b >> 2] >> (8 * (b & 3)));
    }
}

}  // namespace

int fp4_transpose(const void* src, void* dst, int rows, int cols, cudaStream_t stream)
{
    if (!src || !dst || rows < 0 || cols < 0 || (rows & 1) || (cols & 1)) return ASCB200_EINVAL;
    if (rows == 0 || cols == 0) return ASCB200_OK;
    dim3 grid((cols + FP4_T_COLS - 1) / FP4_T_COLS, (rows + FP4_T_ROWS - 1) / FP4_T_ROWS);
    if (grid.y > 65535u) return ASCB200_ETOOBIG;
    ASCB200_CUDA(launch_pdl(fp4_transpose_kernel, grid, dim3(256), 0, stream, static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, cols,
                            cols / 2, rows / 2));
    return ASCB200_OK;
}

}  // namespace ascb200

extern "C" int ascb200_fp4_transpose(const void* src_dev, void* dst_dev, int32_t rows, int32_t cols, void* stream)
{
    if (!ascb200::current_state()) return ASCB200_ENODEV;
    return ascb200::fp4_transpose(src_dev, dst_dev, rows, cols, static_cast<cudaStream_t>(stream));
}

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
