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

constexpr int TILE_K = 256;  // K rows per block: 8 KB of source, contiguous in NZ

// grid = groups * (n / C0) * k_tiles blocks of 256 threads
template <int ESZ, bool TO_NK>
__global__ void __launch_bounds__(256) nz_unpack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int k, int n, int k_tiles)
{
    constexpr int C0 = 32 / ESZ;
    constexpr int ROW_WORDS = 9;  // 32 data bytes + 4 of padding per K row: column gathers spread over the banks
    __shared__ uint32_t tile[TILE_K * ROW_WORDS];
    const int n_blocks = n / C0;
    const int kt = blockIdx.x % k_tiles;
    const int nb = (blockIdx.x / k_tiles) % n_blocks;
    const size_t g = blockIdx.x / (static_cast<size_t>(k_tiles) * n_blocks);
    const int k0 = kt * TILE_K;
    const int rows = min(TILE_K, k - k0);
    const uint4* s16 = reinterpret_cast<const uint4*>(src + ((g * n_blocks + nb) * static_cast<size_t>(k) + k0) * 32);
    for (int i = threadIdx.x; i < rows * 2; i += 256) {
        const uint4 v = __ldg(s16 + i);
        uint32_t* t = tile + (i >> 1) * ROW_WORDS + (i & 1) * 4;
        t[0] = v.x;
        t[1] = v.y;
        t[2] = v.z;
        t[3] = v.w;
    }
    __syncthreads();
    if constexpr (TO_NK) {
        // output row = one column of the block: 16-byte vectors of 16 / ESZ consecutive K
        constexpr int KV = 16 / ESZ;
        const int vec_per_row = rows / KV;  // rows is a multiple of 16
        const uint8_t* tb = reinterpret_cast<const uint8_t*>(tile);
        for (int v = threadIdx.x; v < C0 * vec_per_row; v += 256) {
            const int nl = v % C0, kv = v / C0;
            uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < KV; ++j) {
                const uint8_t* e = tb + (kv * KV + j) * (ROW_WORDS * 4) + nl * ESZ;
                if constexpr (ESZ == 1) w[j >> 2] |= static_cast<uint32_t>(e[0]) << (8 * (j & 3));
                else w[j >> 1] |= static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(e)) << (16 * (j & 1));
            }
            uint8_t* out = dst + ((g * n + static_cast<size_t>(nb) * C0 + nl) * k + k0 + kv * KV) * ESZ;
            *reinterpret_cast<uint4*>(out) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
        for (int i = threadIdx.x; i < rows * 2; i += 256) {
            const uint32_t* t = tile + (i >> 1) * ROW_WORDS + (i & 1) * 4;
            uint8_t* out = dst + ((g * k + k0 + (i >> 1)) * static_cast<size_t>(n) + static_cast<size_t>(nb) * C0) * ESZ + (i & 1) * 16;
            *reinterpret_cast<uint4*>(out) = make_uint4(t[0], t[1], t[2], t[3]);
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
