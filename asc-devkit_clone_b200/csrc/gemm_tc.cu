// Tensor-core GEMM for sm_100a: the contraction behind Matmul::IterateAll and the grouped quantized
// matmul.  One persistent, warp-specialised kernel template:
//
//   warp 0    TMA producer: global -> shared memory tiles (128-byte swizzle), NUM_STAGES deep ring
//   warp 1    MMA issuer: one thread issues tcgen05.mma (kind::f16 / kind::i8 / kind::mxf4.block_scale),
//             accumulators live in TMEM
//   warp 2    TMEM allocation / release
//   warps 4-11 epilogue: tcgen05.ld TMEM -> registers, fused fixpipe stage (bias, cast, dequant,
//             requant, per-token x per-channel scaling), vector stores to global memory; two warps
//             per TMEM lane quadrant, each draining half of the tile's columns
//
// A CTA computes 128 x BLOCK_N output tiles; with two accumulator stages in TMEM the epilogue of
// tile i overlaps the main loop of tile i+1.  Tiles are visited M-fastest so that concurrently
// running CTAs share B columns in L2.  No load uses cluster multicast.
#include <algorithm>
#include <cstring>
#include <mutex>

#include "tc_common.cuh"

namespace ascb200 {
namespace {

using namespace tc;

constexpr int BLOCK_M = 128;
constexpr int ROW_BYTES = 128;          // one swizzle row: 64 x 16-bit, 128 x 8-bit, 256 x 4-bit along the contiguous axis
constexpr int A_TILE_BYTES = BLOCK_M * ROW_BYTES;
constexpr int NUM_THREADS = 384;        // 4 control warps + 8 epilogue warps
constexpr int NUM_EPI_WARPS = 8;
constexpr int MAX_GROUPS = 1024;
constexpr int SF_CHUNK_BYTES = 512;     // scale factors of 128 rows x 4 K-blocks (of 32 elements)
constexpr int kSfPadBlocks = 2;         // re-tiled scale tensors carry two 128-row blocks of padding: a tile may start in the last block and read two more

enum : int {
    OUT_F32 = ASCB200_F32, OUT_F16 = ASCB200_F16, OUT_BF16 = ASCB200_BF16, OUT_S8 = ASCB200_S8, OUT_S32 = ASCB200_S32,
    OUT_E4M3 = ASCB200_FP8_E4M3, OUT_E5M2 = ASCB200_FP8_E5M2
};

struct EpiParams {
    void* c;
    void* c2;
    long long ldc, ldc2;
    int c_dtype, c2_dtype;
    int mode;
    int relu, act;
    int vec_c, vec_c2;       // rows of c / c2 are 16-byte aligned at every 32-column boundary
    int tma_c, tma_c2;       // c / c2 (1- or 2-byte elements) may be written with bulk tensor stores
    int atomic;              // 1 add / 2 max / 3 min into c instead of overwriting it (fp32 / int32 / fp16 / bf16 outputs)
    int layout;              // ASCB200_C_*: row-major, column-major or fractal NZ (the last two are stored from registers)
    const void* bias;        // float (fp32 accumulators) or int32 (int32 accumulators)
    const float* tok;
    const float* ch;
    const unsigned long long* quant;
    unsigned long long quant_scalar;
};

struct GemmParams {
    int m, n, k;
    int num_k_blocks;
    int a_mn, b_mn;          // operand is MN-major (contiguous along M / N) instead of K-major
    int groups;              // > 0: grouped mode
    const long long* group_counts;
    const uint8_t* sfa;      // MXFP4: re-tiled scale factors (see retile_scales_kernel)
    const uint8_t* sfb;
    int sf_kc;               // 512-byte chunks per 128-row block in sfa / sfb
    int pair_n;              // CTA-pair kernels for fp16 / bf16 / int8: columns per tile (multiple of 16, at most 256)
    int allow_m64;           // fp16 / bf16 / int8, single-CTA kernel: tiles of at most 64 rows use the 64-row instruction
    int band_m;              // not grouped: tiles are walked in bands of band_m row blocks (all columns of a band before the next band)
    int split_k;             // single-CTA kernel: > 1 = that many CTAs of a cluster share every tile, each multiplying its own range of K
                             // blocks; the leader adds the others' accumulators, which they write into its shared memory (one tile per cluster)
    int ring_stages;         // CTA-pair kernels, fp16 / bf16 / int8 with K-major B: the shared-memory ring is cut for the call's tile width,
    int ring_stage_bytes;    // so that narrower tiles get more stages in flight (0: the kernel's compile-time geometry)
    int group_swap;          // grouped int8 on CTA pairs: a group's last, partial 256-row block is multiplied with the operand roles swapped
    uint32_t idesc;
    uint32_t idesc_swap;     // instruction descriptor of such a block without its N field (the weights are then the 256-row operand)
    uint32_t* status;
    EpiParams epi;
};

template <int KIND, int BLOCK_N>
struct Cfg {
    static constexpr int B_TILE_BYTES = BLOCK_N * ROW_BYTES;
    static constexpr int SF_B_BLOCKS = (BLOCK_N + 127) / 128;  // 128-row scale blocks that one B tile touches
    static constexpr bool IS_MX = KIND == KIND_MXF4 || KIND == KIND_MXF8;
    static constexpr int SF_CHUNKS = KIND == KIND_MXF4 ? 2 : 1;  // 512-byte scale chunks (4 scales per row) per 128 rows and K block
    static constexpr int SF_BYTES = IS_MX ? (1 + SF_B_BLOCKS) * SF_CHUNKS * SF_CHUNK_BYTES : 0;
    static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES + SF_BYTES;
    // per epilogue warp: 2 KB stage a 2-byte output chunk for its bulk tensor store; the third KB stages a 1-byte chunk beside it
    // (two outputs) or, for the per-token x per-channel dequant, holds the per-channel scales of the warp's columns
    static constexpr int EPI_BYTES_PER_WARP = (IS_MX && BLOCK_N == 256) ? 0 : 3072;
    static constexpr int EPI_BYTES = NUM_EPI_WARPS * EPI_BYTES_PER_WARP;
    static constexpr int FIXED_BYTES = 1024 /*alignment slack*/ + 256 /*barriers*/ + 2 * (MAX_GROUPS + 1) * static_cast<int>(sizeof(int)) + EPI_BYTES;
    static constexpr int NUM_STAGES = std::min(8, (227 * 1024 - FIXED_BYTES) / STAGE_BYTES);
    static constexpr int ACC_STAGES = (IS_MX && BLOCK_N == 256) ? 1 : 2;  // 2 x 256 accumulator columns would leave no TMEM for scales
    static constexpr int ACC_COLS = ACC_STAGES * BLOCK_N;
    static constexpr int SF_COLS_PER_STAGE = 24;  // 8 for A + 16 for B
    static constexpr int SF_COL0 = ACC_COLS;
    static constexpr int TMEM_NEED = ACC_COLS + (IS_MX ? NUM_STAGES * SF_COLS_PER_STAGE : 0);
    static constexpr int TMEM_COLS = TMEM_NEED <= 32 ? 32 : TMEM_NEED <= 64 ? 64 : TMEM_NEED <= 128 ? 128 : TMEM_NEED <= 256 ? 256 : 512;
    static_assert(TMEM_NEED <= 512, "TMEM budget");
    // bytes of one K step of the instruction (32 in every kind) -> elements along K per tile row
    static constexpr int BLOCK_K = KIND == KIND_F16 ? 64 : KIND == KIND_MXF4 ? 256 : 128;
    static constexpr int UMMA_K = BLOCK_K / 4;
    static constexpr int SMEM_BYTES = NUM_STAGES * STAGE_BYTES + FIXED_BYTES;
};

struct TileInfo {
    int row0, row_end, n0, n_end, group;  // n_end: first column after the tile
    int m64;  // the tile holds at most 64 rows (of its group, or of the matrix) and is multiplied with the 64-row instruction
    int swap_n;  // CTA pairs, grouped: > 0 for a group's partial last block: its rows rounded up to 16, the N of the swapped instruction
};

// Tensor maps of the outputs (rank 2, box 32 x 32, swizzle = bytes of one box row).
struct OutMaps {
    CUtensorMap c, c2;
};

// Where one epilogue warp stages a 32 x 32 output chunk for a bulk tensor store.  A map pointer of
// nullptr selects direct stores from registers (4-byte outputs, unaligned tensors, rows of a group
// that end inside the warp's 32 rows).
struct EpiStage {
    const CUtensorMap* map_c;
    const CUtensorMap* map_c2;
    uint32_t smem_c, smem_c2;
    int row_base;  // first output row of the warp
    bool dual;     // both outputs staged: two bulk groups are in flight per chunk
};

// Grouped mode: prefix sums of rows and of tiles per group, built once per CTA by warp 0.
__device__ void build_group_tables(const long long* counts, int groups, int num_n, int tile_rows, int* row_start, int* tile_start)
{
    const int lane = threadIdx.x & 31;
    int rows_carry = 0, tiles_carry = 0;
    for (int base = 0; base < groups; base += 32) {
        const int g = base + lane;
        long long c = g < groups ? counts[g] : 0;
        int rows = c > 0 ? static_cast<int>(c) : 0;
        int tiles = ((rows + tile_rows - 1) / tile_rows) * num_n;
        int rs = rows, ts = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int r2 = __shfl_up_sync(0xFFFFFFFFu, rs, o);
            int t2 = __shfl_up_sync(0xFFFFFFFFu, ts, o);
            if (lane >= o) {
                rs += r2;
                ts += t2;
            }
        }
        if (g < groups) {
            row_start[g + 1] = rows_carry + rs;
            tile_start[g + 1] = tiles_carry + ts;
        }
        rows_carry += __shfl_sync(0xFFFFFFFFu, rs, 31);
        tiles_carry += __shfl_sync(0xFFFFFFFFu, ts, 31);
    }
    if (lane == 0) {
        row_start[0] = 0;
        tile_start[0] = 0;
    }
}

// Tile order of a plain (not grouped) GEMM.  Tiles that run at the same time should share operands: with num_m row blocks
// walked first (band_m >= num_m) a wave of tiles touches every row block of A and few column tiles of B, and once A is
// larger than L2 every wave streams it from HBM again.  In bands of band_m row blocks (a band's column tiles one after the
// other, row blocks fastest inside) a wave covers about band_m row blocks x (wave / band_m) column tiles, so what it reads
// of A and of B is of similar size and stays in L2 from one wave to the next.
__device__ __forceinline__ void raster_tile(int tile, int num_m, int num_n, int band_m, int& m_idx, int& n_idx)
{
    if (band_m <= 0 || band_m >= num_m) {
        m_idx = tile % num_m;
        n_idx = tile / num_m;
        return;
    }
    const int per_band = band_m * num_n;
    const int band = tile / per_band, r = tile - band * per_band;
    const int rows = min(band_m, num_m - band * band_m);  // the last band may be narrower
    n_idx = r / rows;
    m_idx = band * band_m + (r - n_idx * rows);
}

template <int BLOCK_N>
__device__ __forceinline__ bool locate_tile(const GemmParams& p, int tile, int num_m, int total_tiles, const int* row_start,
                                            const int* tile_start, int& cursor, TileInfo& t)
{
    if (tile >= total_tiles) return false;
    if (p.groups > 0) {
        while (tile >= tile_start[cursor + 1]) ++cursor;
        const int local = tile - tile_start[cursor];
        const int rows = row_start[cursor + 1] - row_start[cursor];
        const int m_tiles = (rows + BLOCK_M - 1) / BLOCK_M;
        t.group = cursor;
        t.row0 = row_start[cursor] + (local % m_tiles) * BLOCK_M;
        t.row_end = row_start[cursor + 1];
        t.n0 = (local / m_tiles) * BLOCK_N;
        t.n_end = t.n0 + BLOCK_N;
        t.m64 = p.allow_m64 && t.row_end - t.row0 <= 64;
        t.swap_n = 0;
    } else {
        t.swap_n = 0;
        t.group = 0;
        int m_idx, n_idx;
        raster_tile(tile, num_m, total_tiles / num_m, p.band_m, m_idx, n_idx);
        t.row0 = m_idx * BLOCK_M;
        t.row_end = p.m;
        t.n0 = n_idx * BLOCK_N;
        t.n_end = t.n0 + BLOCK_N;
        t.m64 = p.allow_m64 && t.row_end - t.row0 <= 64;
    }
    return true;
}

// Same for the CTA-pair kernel: tiles of 256 rows and `bn` columns; row0 is the first row of the pair's tile.
__device__ __forceinline__ bool locate_pair_tile(const GemmParams& p, int tile, int num_m, int total_tiles, int bn, const int* row_start, const int* tile_start,
                                                 int& cursor, TileInfo& t)
{
    if (tile >= total_tiles) return false;
    if (p.groups > 0) {
        while (tile >= tile_start[cursor + 1]) ++cursor;
        const int local = tile - tile_start[cursor];
        const int m_tiles = (row_start[cursor + 1] - row_start[cursor] + 2 * BLOCK_M - 1) / (2 * BLOCK_M);
        t.group = cursor;
        t.row0 = row_start[cursor] + (local % m_tiles) * 2 * BLOCK_M;
        t.row_end = row_start[cursor + 1];
        t.n0 = (local / m_tiles) * bn;
        const int rows = t.row_end - t.row0;
        t.swap_n = (p.group_swap && rows < 2 * BLOCK_M) ? (rows + 15) & ~15 : 0;
    } else {
        t.group = 0;
        int m_idx, n_idx;
        raster_tile(tile, num_m, total_tiles / num_m, p.band_m, m_idx, n_idx);
        t.row0 = m_idx * 2 * BLOCK_M;
        t.row_end = p.m;
        t.n0 = n_idx * bn;
        t.swap_n = 0;
    }
    t.n_end = t.n0 + bn;
    t.m64 = 0;
    return true;
}

// ---- epilogue helpers -------------------------------------------------------------------------
// FasterGelu of the grouped example: x * e^(0.851 (x - |x|)) / (1 + e^(-1.702 |x|))
// (quant_group_matmul_high_performance/scripts/gen_data.py:19-23), which is x / (1 + e^(-1.702 x)) written
// so that no exponential overflows.  Evaluated in the short form with one ex2 and one fast division:
// for x << 0 the exponential overflows to +inf and the quotient is -0, the limit of the long form.
// Five instructions per value: the flush-to-zero forms of ex2 and rcp need none of the range handling that the compiler
// wraps around __expf and __fdividef (about forty instructions per value, which made the epilogue issue bound).
__device__ __forceinline__ float faster_gelu(float x)
{
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -2.4554669595930156f));  // e^(-1.702 x) = 2^(-1.702 log2(e) x)
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return x * r;
}

// fp32 -> int8 value, round to nearest even, saturating, NaN -> 0 (one conversion instruction).
__device__ __forceinline__ int cvt_rni_sat_s8(float v)
{
    int r;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}
// Two independent fp32 products in one instruction (round to nearest, no fusion with anything else).
__device__ __forceinline__ float2 mul_f32x2(float2 a, float2 b)
{
    unsigned long long x, y, z;
    asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(y) : "f"(b.x), "f"(b.y));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(z) : "l"(x), "l"(y));
    float2 r;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(z));
    return r;
}
__device__ __forceinline__ void st_v4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    *reinterpret_cast<uint4*>(p) = make_uint4(a, b, c, d);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack_f16x2_sat(float lo, float hi)
{
    // round to nearest even; overflow and infinities saturate to +-65504, NaN is kept: one instruction for both values
    uint32_t v;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(v) : "f"(hi), "f"(lo));
    return v;
}

// Stores 32 consecutive outputs of one row; DT is the element type of the destination.
// f: values for F32/F16/BF16, qi: values for S8/S32.
// Reduces 32 consecutive outputs of one row into the destination (enAtomic of GetTensorC / IterateAll: 1 add, 2 max,
// 3 min; impl/adv_api/detail/matmul/utils/matmul_config_utils.h:53-55): one reduction per element.  Sums of 16-bit types go
// through the half / bfloat16 atomics (rounded to the destination type); max / min of floats through the integer order of
// their bit patterns (ascending for positive, descending for negative values), of 16-bit types through a
// compare-and-swap on the element.
constexpr int kAtomicAdd = 1, kAtomicMax = 2;  // 3: minimum (the remaining value of enAtomic)

__device__ __forceinline__ void atomic_maxmin_f32(float* p, float v, bool is_max)
{
    // max with v >= 0 or min with v < 0 can only move the stored bits up in signed / unsigned integer order respectively
    if (is_max == !signbit(v)) {
        if (is_max) atomicMax(reinterpret_cast<int*>(p), __float_as_int(v));
        else atomicMax(reinterpret_cast<unsigned*>(p), __float_as_uint(v));
    } else {
        if (is_max) atomicMin(reinterpret_cast<unsigned*>(p), __float_as_uint(v));
        else atomicMin(reinterpret_cast<int*>(p), __float_as_int(v));
    }
}
template <typename H>
__device__ __forceinline__ void atomic_maxmin_16(H* p, H v, bool is_max)
{
    unsigned short* u = reinterpret_cast<unsigned short*>(p);
    unsigned short old = *u;
    for (int guard = 0; guard < 4096; ++guard) {  // every failed exchange means another thread made progress
        const H cur = *reinterpret_cast<const H*>(&old);
        const float c = static_cast<float>(cur), w = static_cast<float>(v);
        if (is_max ? !(w > c) : !(w < c)) return;
        const unsigned short seen = atomicCAS(u, old, *reinterpret_cast<const unsigned short*>(&v));
        if (seen == old) return;
        old = seen;
    }
}

template <int DT>
__device__ __forceinline__ void atomic_row32(void* base, long long ld, int row, int col0, int ncols, const float (&f)[32], const int (&qi)[32],
                                             int op)
{
    const size_t off = static_cast<size_t>(row) * static_cast<size_t>(ld) + col0;
    if (op == kAtomicAdd) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (j >= ncols) break;
            if constexpr (DT == OUT_F32) atomicAdd(static_cast<float*>(base) + off + j, f[j]);
            else if constexpr (DT == OUT_S32) atomicAdd(static_cast<int*>(base) + off + j, qi[j]);
            else if constexpr (DT == OUT_F16) atomicAdd(static_cast<__half*>(base) + off + j, __float2half_rn(fminf(fmaxf(f[j], -65504.0f), 65504.0f)));
            else if constexpr (DT == OUT_BF16) atomicAdd(static_cast<__nv_bfloat16*>(base) + off + j, __float2bfloat16_rn(f[j]));
        }
        return;
    }
    const bool is_max = op == kAtomicMax;
#pragma unroll  // full: a partial unroll would index f / qi dynamically and push them into local memory
    for (int j = 0; j < 32; ++j) {
        if (j >= ncols) break;
        if constexpr (DT == OUT_F32) atomic_maxmin_f32(static_cast<float*>(base) + off + j, f[j], is_max);
        else if constexpr (DT == OUT_S32) {
            if (is_max) atomicMax(static_cast<int*>(base) + off + j, qi[j]);
            else atomicMin(static_cast<int*>(base) + off + j, qi[j]);
        } else if constexpr (DT == OUT_F16)
            atomic_maxmin_16(static_cast<__half*>(base) + off + j, __float2half_rn(fminf(fmaxf(f[j], -65504.0f), 65504.0f)), is_max);
        else if constexpr (DT == OUT_BF16) atomic_maxmin_16(static_cast<__nv_bfloat16*>(base) + off + j, __float2bfloat16_rn(f[j]), is_max);
    }
}

template <int DT>
__device__ __forceinline__ void store_row32(void* base, long long ld, int vec, int row, int col0, int ncols, const float (&f)[32],
                                            const int (&qi)[32])
{
    const size_t off = static_cast<size_t>(row) * static_cast<size_t>(ld) + col0;
    if constexpr (DT == OUT_F32 || DT == OUT_S32) {
        uint32_t w[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) w[j] = DT == OUT_F32 ? __float_as_uint(f[j]) : static_cast<uint32_t>(qi[j]);
        uint32_t* out = static_cast<uint32_t*>(base) + off;
        if (vec && ncols == 32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) st_v4(out + 4 * j, w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        } else if (vec && ncols == 16) {
#pragma unroll
            for (int j = 0; j < 4; ++j) st_v4(out + 4 * j, w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols) out[j] = w[j];
        }
    } else if constexpr (DT == OUT_F16 || DT == OUT_BF16) {
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) w[j] = DT == OUT_F16 ? pack_f16x2_sat(f[2 * j], f[2 * j + 1]) : pack_bf16x2(f[2 * j], f[2 * j + 1]);
        uint16_t* out = static_cast<uint16_t*>(base) + off;
        if (vec && ncols == 32) {
#pragma unroll
            for (int j = 0; j < 4; ++j) st_v4(out + 8 * j, w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        } else if (vec && ncols == 16) {
#pragma unroll
            for (int j = 0; j < 2; ++j) st_v4(out + 8 * j, w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols) out[j] = static_cast<uint16_t>(w[j >> 1] >> (16 * (j & 1)));
        }
    } else {  // OUT_S8
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            w[j] = (qi[4 * j] & 0xFF) | ((qi[4 * j + 1] & 0xFF) << 8) | ((qi[4 * j + 2] & 0xFF) << 16) | (static_cast<uint32_t>(qi[4 * j + 3]) << 24);
        int8_t* out = static_cast<int8_t*>(base) + off;
        if (vec && ncols == 32) {
            st_v4(out, w[0], w[1], w[2], w[3]);
            st_v4(out + 16, w[4], w[5], w[6], w[7]);
        } else if (vec && ncols == 16) {
            st_v4(out, w[0], w[1], w[2], w[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols) out[j] = static_cast<int8_t>(w[j >> 2] >> (8 * (j & 3)));
        }
    }
}

// 32 consecutive outputs of one row into a column-major or fractal (NZ) C.  Column-major: element (row, n) at n * ld + row,
// so for every column the 32 lanes of a warp (32 consecutive rows) write one contiguous run.  NZ: blocks of C0 columns
// (16, or 32 for 1-byte types), row-major inside a block: element at ((n / C0) * ld + row) * C0 + n % C0; a lane writes
// whole C0-element pieces of its row with 16-byte stores when the chunk is complete and the base is aligned.
template <int DT>
__device__ __forceinline__ void store_row32_layout(void* base, long long ld, int layout, int row, int col0, int ncols, const float (&f)[32],
                                                   const int (&qi)[32])
{
    constexpr int ESZ = (DT == OUT_F32 || DT == OUT_S32) ? 4 : (DT == OUT_F16 || DT == OUT_BF16) ? 2 : 1;
    uint32_t v[32];   // one element per entry, already in the output type's bit pattern
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        if constexpr (DT == OUT_F32) v[j] = __float_as_uint(f[j]);
        else if constexpr (DT == OUT_S32) v[j] = static_cast<uint32_t>(qi[j]);
        else if constexpr (DT == OUT_F16) v[j] = pack_f16x2_sat(f[j], 0.0f) & 0xFFFFu;
        else if constexpr (DT == OUT_BF16) v[j] = pack_bf16x2(f[j], 0.0f) & 0xFFFFu;
        else v[j] = static_cast<uint32_t>(qi[j]) & 0xFFu;
    }
    if (layout == ASCB200_C_COLUMN_MAJOR) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            if (j >= ncols) break;
            const size_t off = static_cast<size_t>(col0 + j) * static_cast<size_t>(ld) + row;
            if constexpr (ESZ == 4) static_cast<uint32_t*>(base)[off] = v[j];
            else if constexpr (ESZ == 2) static_cast<uint16_t*>(base)[off] = static_cast<uint16_t>(v[j]);
            else static_cast<uint8_t*>(base)[off] = static_cast<uint8_t>(v[j]);
        }
        return;
    }
    constexpr int C0 = ESZ == 1 ? 32 : 16;
    const bool vec = ncols == 32 && (col0 % C0) == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0;
    if (vec) {
#pragma unroll
        for (int g = 0; g < 32 / C0; ++g) {
            uint8_t* out = static_cast<uint8_t*>(base) + ((static_cast<size_t>((col0 + g * C0) / C0) * ld + row) * C0) * ESZ;
            if constexpr (ESZ == 4) {
#pragma unroll
                for (int q = 0; q < 4; ++q) st_v4(out + 16 * q, v[g * 16 + 4 * q], v[g * 16 + 4 * q + 1], v[g * 16 + 4 * q + 2], v[g * 16 + 4 * q + 3]);
            } else if constexpr (ESZ == 2) {
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int b = g * 16 + 8 * q;
                    st_v4(out + 16 * q, v[b] | (v[b + 1] << 16), v[b + 2] | (v[b + 3] << 16), v[b + 4] | (v[b + 5] << 16), v[b + 6] | (v[b + 7] << 16));
                }
            } else {
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int b = 16 * q;
                    st_v4(out + 16 * q, v[b] | (v[b + 1] << 8) | (v[b + 2] << 16) | (v[b + 3] << 24), v[b + 4] | (v[b + 5] << 8) | (v[b + 6] << 16) | (v[b + 7] << 24),
                          v[b + 8] | (v[b + 9] << 8) | (v[b + 10] << 16) | (v[b + 11] << 24), v[b + 12] | (v[b + 13] << 8) | (v[b + 14] << 16) | (v[b + 15] << 24));
                }
            }
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        if (j >= ncols) break;
        const int n = col0 + j;
        const size_t off = (static_cast<size_t>(n / C0) * static_cast<size_t>(ld) + row) * C0 + n % C0;
        if constexpr (ESZ == 4) static_cast<uint32_t*>(base)[off] = v[j];
        else if constexpr (ESZ == 2) static_cast<uint16_t*>(base)[off] = static_cast<uint16_t>(v[j]);
        else static_cast<uint8_t*>(base)[off] = static_cast<uint8_t>(v[j]);
    }
}

// Same values as store_row32 for a 1- or 2-byte type, but through shared memory and one bulk tensor
// store per warp: lane i writes row i of the 32 x 32 chunk (16-byte pieces XOR-swizzled like the tensor
// map, so the writes do not collide on banks), lane 0 hands the chunk to the TMA unit, which writes
// whole rows and clips at the edges of the matrix.  PENDING bulk groups of lane 0 may still be reading
// other buffers; this buffer's previous group is older than those and has finished.
template <int DT>
__device__ __forceinline__ void stage_store32(const CUtensorMap* map, uint32_t smem, bool dual, int lane, int row_base, int col0,
                                              const float (&f)[32], const int (&qi)[32], int atomic = 0)
{
    static_assert(DT == OUT_F16 || DT == OUT_BF16 || DT == OUT_S8, "staged stores carry 1- and 2-byte outputs");
    // (bulk groups belong to the thread that committed them: the wait, the store and the final wait before the CTA exits all
    // run on the lane that elect.sync picks, which is the same one every time for a full warp; the compiler then keeps the
    // tensor map address and the coordinates in uniform registers, which shortens the issue of the store)
    if (elect_one()) {
        if (dual) bulk_wait_group_read<1>();
        else bulk_wait_group_read<0>();
    }
    __syncwarp();
    if constexpr (DT == OUT_S8) {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            w[j] = (qi[4 * j] & 0xFF) | ((qi[4 * j + 1] & 0xFF) << 8) | ((qi[4 * j + 2] & 0xFF) << 16) | (static_cast<uint32_t>(qi[4 * j + 3]) << 24);
        const uint32_t row = smem + lane * 32, sw = (lane >> 2) & 1;  // 32-byte swizzle: piece ^= bit 2 of the row
        st_shared_v4(row + ((0 ^ sw) << 4), w[0], w[1], w[2], w[3]);
        st_shared_v4(row + ((1 ^ sw) << 4), w[4], w[5], w[6], w[7]);
    } else {
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) w[j] = DT == OUT_F16 ? pack_f16x2_sat(f[2 * j], f[2 * j + 1]) : pack_bf16x2(f[2 * j], f[2 * j + 1]);
        const uint32_t row = smem + lane * 64, sw = (lane >> 1) & 3;  // 64-byte swizzle: piece ^= bits 1-2 of the row
#pragma unroll
        for (int j = 0; j < 4; ++j) st_shared_v4(row + ((j ^ sw) << 4), w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (elect_one()) {
        if (atomic == 0) tma_store_2d(map, smem, col0, row_base);
        else if (atomic == kAtomicAdd) tma_reduce_add_2d(map, smem, col0, row_base);  // the tensor map then carries the real element type
        else if (atomic == kAtomicMax) tma_reduce_max_2d(map, smem, col0, row_base);
        else tma_reduce_min_2d(map, smem, col0, row_base);
        bulk_commit_group();
    }
}

// 32 per-channel fp32 parameters starting at p[0]: eight 128-bit loads when aligned.
__device__ __forceinline__ void load_params32(const float* p, int ncols, float (&out)[32])
{
    if (ncols == 32 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(p) + j);
            out[4 * j] = v.x;
            out[4 * j + 1] = v.y;
            out[4 * j + 2] = v.z;
            out[4 * j + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) out[j] = j < ncols ? __ldg(p + j) : 0.0f;
    }
}

// The fixpipe stage for 32 accumulators r[] of output row `row`, columns col0 .. col0+ncols.
// MODE / DT are compile-time so that each combination is a short straight-line sequence.
// chan0: index of column col0 in bias / quant; ch_off: index in the per-channel scale array.
// ch_smem: per-token x per-channel dequant only: shared-memory address of the chunk's 32 per-channel scales (0 beyond the
// tile or the matrix), which the caller put there before the tile's first chunk.
template <bool ACC_INT, int MODE, int DT>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&r)[32], const EpiParams& e, const EpiStage& st, int row, bool row_ok, int col0, int ncols,
                                               size_t chan0, uint32_t ch_smem, float tok)
{
    // Runs on all 32 lanes (the quantising path exchanges per-column parameters with shuffles); lanes whose
    // row lies outside the matrix compute on whatever their TMEM lane holds and store nothing.
    float f[32];
    int qi[32];
    if constexpr (ACC_INT) {
        if (e.bias) {
            const int* bias = static_cast<const int*>(e.bias) + chan0;
#pragma unroll
            for (int j = 0; j < 32; ++j) qi[j] = static_cast<int>(r[j]) + (j < ncols ? __ldg(bias + j) : 0);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) qi[j] = static_cast<int>(r[j]);
        }
        if constexpr (MODE != ASCB200_EPI_CAST) {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = static_cast<float>(qi[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
        if (e.bias) {
            float b[32];
            load_params32(static_cast<const float*>(e.bias) + chan0, ncols, b);
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __fadd_rn(f[j], b[j]);
        }
        if (st.map_c2) {
            const int lane = threadIdx.x & 31;
            if (e.c2_dtype == OUT_BF16) stage_store32<OUT_BF16>(st.map_c2, st.smem_c2, st.dual, lane, st.row_base, col0, f, qi);
            else stage_store32<OUT_F16>(st.map_c2, st.smem_c2, st.dual, lane, st.row_base, col0, f, qi);
        } else if (e.c2 && row_ok) {
            if (e.c2_dtype == OUT_BF16) store_row32<OUT_BF16>(e.c2, e.ldc2, e.vec_c2, row, col0, ncols, f, qi);
            else if (e.c2_dtype == OUT_F16) store_row32<OUT_F16>(e.c2, e.ldc2, e.vec_c2, row, col0, ncols, f, qi);
            else store_row32<OUT_F32>(e.c2, e.ldc2, e.vec_c2, row, col0, ncols, f, qi);
        }
    }
    if constexpr (MODE == ASCB200_EPI_CAST) {
        if (e.relu) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if constexpr (ACC_INT) qi[j] = max(qi[j], 0);
                else f[j] = fmaxf(f[j], 0.0f);
            }
        }
    } else if constexpr (MODE == ASCB200_EPI_FIXPIPE_QUANT) {
        // Lane j decodes the parameter of column j once (scale = bits [31:13], 9-bit offset); every lane then
        // fetches the 32 decoded values with shuffles instead of loading and decoding them itself.
        const int lane = threadIdx.x & 31;
        const unsigned long long q = (e.quant && lane < ncols) ? __ldg(e.quant + chan0 + lane) : e.quant_scalar;
        const float my_alpha = quant_alpha(q), my_off = quant_offset(q);
        const bool any_off = __any_sync(0xFFFFFFFFu, my_off != 0.0f);
        if (DT == OUT_S8 && !any_off && !e.relu) {
            // no offsets in this chunk: rint(clip(rint(clip(v, -256, 255)), -128, 127)) == rint-and-saturate of v; NaN -> 0
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                const float2 v = mul_f32x2(make_float2(f[j], f[j + 1]),
                                           make_float2(__shfl_sync(0xFFFFFFFFu, my_alpha, j), __shfl_sync(0xFFFFFFFFu, my_alpha, j + 1)));
                qi[j] = cvt_rni_sat_s8(v.x);
                qi[j + 1] = cvt_rni_sat_s8(v.y);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float alpha = __shfl_sync(0xFFFFFFFFu, my_alpha, j);
                const float v = (f[j] >= 0.0f || !e.relu) ? __fmul_rn(f[j], alpha) : 0.0f;
                if constexpr (DT == OUT_S8) {
                    // REQ8 / QF322B8_PRE: clip to 9 bits, round, add the offset, clip to int8
                    const float t = rintf(fminf(fmaxf(v, -256.0f), 255.0f)) + __shfl_sync(0xFFFFFFFFu, my_off, j);
                    qi[j] = (v != v) ? 0 : __float2int_rn(fminf(fmaxf(t, -128.0f), 127.0f));
                }
                f[j] = v;
            }
        }
    } else {  // ASCB200_EPI_DEQUANT_TOKEN_CHANNEL
        float s[32];  // every lane reads the same 16 bytes: one broadcast per load
#pragma unroll
        for (int j = 0; j < 32; j += 4) ld_shared_v4(ch_smem + 4 * j, s[j], s[j + 1], s[j + 2], s[j + 3]);
        if (e.act == 0) {  // without activation: two packed multiplies per column pair
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
                // (acc * ch[n]) * tok[m], each product rounded to nearest like the separate Mul steps of the reference
                float2 v = mul_f32x2(mul_f32x2(make_float2(f[j], f[j + 1]), make_float2(s[j], s[j + 1])), make_float2(tok, tok));
                f[j] = v.x;
                f[j + 1] = v.y;
            }
        } else {  // FasterGelu
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = faster_gelu(__fmul_rn(__fmul_rn(f[j], s[j]), tok));
        }
    }
    if constexpr (DT == OUT_E4M3 || DT == OUT_E5M2) {
        // QF322FP8_PRE: the scaled value rounded to nearest even, saturating to the largest finite fp8; stored as bytes
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            uint16_t pair;
            if constexpr (DT == OUT_E4M3) asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(f[j + 1]), "f"(f[j]));
            else asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(pair) : "f"(f[j + 1]), "f"(f[j]));
            qi[j] = pair & 0xFF;
            qi[j + 1] = pair >> 8;
        }
        if (st.map_c) stage_store32<OUT_S8>(st.map_c, st.smem_c, st.dual, threadIdx.x & 31, st.row_base, col0, f, qi);
        else if (row_ok && e.layout != ASCB200_C_ROW_MAJOR) store_row32_layout<OUT_S8>(e.c, e.ldc, e.layout, row, col0, ncols, f, qi);
        else if (row_ok) store_row32<OUT_S8>(e.c, e.ldc, e.vec_c, row, col0, ncols, f, qi);
        return;
    } else {
        if constexpr (DT == OUT_F16 || DT == OUT_BF16 || DT == OUT_S8) {
            if (st.map_c) {
                stage_store32<DT>(st.map_c, st.smem_c, st.dual, threadIdx.x & 31, st.row_base, col0, f, qi, e.atomic);
                return;
            }
        }
        if (!row_ok) return;
        if (e.layout != ASCB200_C_ROW_MAJOR) {
            store_row32_layout<DT>(e.c, e.ldc, e.layout, row, col0, ncols, f, qi);
            return;
        }
        if constexpr (DT != OUT_S8) {
            if (e.atomic) {
                atomic_row32<DT>(e.c, e.ldc, row, col0, ncols, f, qi, e.atomic);
                return;
            }
        }
        store_row32<DT>(e.c, e.ldc, e.vec_c, row, col0, ncols, f, qi);
    }
}

// Drains this warp's share of one accumulator tile: TMEM lanes of `quad`, chunks [chunk0, chunk1).
// What an epilogue warp loads for its next tile before it waits for that tile's accumulators (per-token x per-channel dequant):
// the per-token scale of the lane's row and four of the per-channel scales of the warp's columns (the warp owns at most four
// chunks = 128 columns; lane l loads columns 4 l .. 4 l + 3 of them).  Their latency then falls into the wait instead of in
// front of the first chunk, which matters for a CTA's last tile, whose epilogue nothing overlaps.
struct EpiPre {
    float tok;
    float4 ch;
};
constexpr int kEpiChOffset = 2048;  // where in a warp's staging area the per-channel scales live (behind the 2-byte output chunk)
__device__ __forceinline__ EpiPre epilogue_preload(const GemmParams& p, const TileInfo& t, int quad, int lane, int chunk0)
{
    EpiPre r = {1.0f, make_float4(0.0f, 0.0f, 0.0f, 0.0f)};
    if (p.epi.mode != ASCB200_EPI_DEQUANT_TOKEN_CHANNEL) return r;
    const int row = t.m64 ? t.row0 + quad * 16 + lane : t.row0 + quad * 32 + lane;
    if (row < t.row_end && !(t.m64 && lane >= 16) && p.epi.tok) r.tok = __ldg(p.epi.tok + row);
    const int col = t.n0 + chunk0 * 32 + lane * 4, end = min(p.n, t.n_end);
    const float* src = p.epi.ch + static_cast<size_t>(t.group) * p.n + col;
    if (col + 4 <= end && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        r.ch = __ldg(reinterpret_cast<const float4*>(src));
    } else {
        if (col < end) r.ch.x = __ldg(src);
        if (col + 1 < end) r.ch.y = __ldg(src + 1);
        if (col + 2 < end) r.ch.z = __ldg(src + 2);
        if (col + 3 < end) r.ch.w = __ldg(src + 3);
    }
    return r;
}

template <bool ACC_INT, int MODE, int DT, int BLOCK_N>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, const TileInfo& t, const OutMaps& outs, uint32_t stage_smem, int stage_bytes,
                                              uint32_t t_addr, int quad, int lane, int chunk0, int chunk1, const EpiPre& pre, uint32_t sk_base,
                                              int sk_parts)
{
    // 128-row tiles: lane l of quadrant q holds row 32 q + l; 64-row tiles: lanes 0-15 hold rows 16 q + l
    const int row = t.m64 ? t.row0 + quad * 16 + lane : t.row0 + quad * 32 + lane;
    const bool row_ok = row < t.row_end && !(t.m64 && lane >= 16);
    const float tok = MODE == ASCB200_EPI_DEQUANT_TOKEN_CHANNEL ? pre.tok : 1.0f;
    if constexpr (MODE == ASCB200_EPI_DEQUANT_TOKEN_CHANNEL) {
        __syncwarp();  // every lane has finished reading the previous tile's scales
        st_shared_v4(stage_smem + kEpiChOffset + lane * 16, __float_as_uint(pre.ch.x), __float_as_uint(pre.ch.y), __float_as_uint(pre.ch.z),
                     __float_as_uint(pre.ch.w));
        __syncwarp();
    }
    EpiStage st;
    st.row_base = t.row0 + quad * 32;
    // bulk stores clip at the matrix edge only: a group that ends inside this warp's rows is stored from registers
    const bool rows_mine = !t.m64 && (p.groups == 0 || st.row_base + 32 <= t.row_end);
    constexpr bool BYTE_OUT = DT == OUT_S8 || DT == OUT_E4M3 || DT == OUT_E5M2;
    constexpr int C_BYTES = BYTE_OUT ? 1024 : 2048;
    const bool stage_c = (DT == OUT_F16 || DT == OUT_BF16 || BYTE_OUT) && p.epi.tma_c && rows_mine && C_BYTES <= stage_bytes;
    const int c_used = stage_c ? C_BYTES : 0;
    const bool stage_c2 = !ACC_INT && p.epi.c2 && p.epi.tma_c2 && rows_mine && c_used + 2048 <= stage_bytes;
    st.map_c = stage_c ? &outs.c : nullptr;
    st.map_c2 = stage_c2 ? &outs.c2 : nullptr;
    st.smem_c = stage_smem;
    st.smem_c2 = stage_smem + c_used;
    st.dual = stage_c && stage_c2;
    const EpiStage direct = {nullptr, nullptr, 0u, 0u, st.row_base, false};
#pragma unroll 1
    for (int c = chunk0; c < chunk1; ++c) {
        const int col0 = t.n0 + c * 32;
        if (col0 >= p.n || col0 >= t.n_end) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        // split K: add what the other CTAs of the cluster accumulated over their K ranges, in rank order (see splitk_send_tile)
        for (int s = 0; s < sk_parts; ++s) {
            const uint32_t part = sk_base + static_cast<uint32_t>(s) * (BLOCK_N * 512) + ((c * 8) * 128 + quad * 32 + lane) * 16;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                float x0, x1, x2, x3;
                ld_shared_v4(part + (j / 4) * 2048, x0, x1, x2, x3);
                if constexpr (ACC_INT) {
                    r[j] += __float_as_uint(x0), r[j + 1] += __float_as_uint(x1), r[j + 2] += __float_as_uint(x2), r[j + 3] += __float_as_uint(x3);
                } else {
                    r[j] = __float_as_uint(__uint_as_float(r[j]) + x0), r[j + 1] = __float_as_uint(__uint_as_float(r[j + 1]) + x1);
                    r[j + 2] = __float_as_uint(__uint_as_float(r[j + 2]) + x2), r[j + 3] = __float_as_uint(__uint_as_float(r[j + 3]) + x3);
                }
            }
        }
        // a chunk that the tile only half owns (tile widths are multiples of 16) is stored from registers: the
        // bulk store's 32-column box would reach into the neighbouring tile.  So is a chunk that crosses the right edge of
        // the matrix: the TMA unit clips columns in 16-byte pieces, not per element (an int8 matrix of 328 columns got 8
        // bytes past its edge written), so only whole rows are left to its clipping.
        const bool whole = col0 + 32 <= t.n_end && col0 + 32 <= p.n;
        epilogue_chunk<ACC_INT, MODE, DT>(r, p.epi, whole ? st : direct, row, row_ok, col0, min(whole ? 32 : t.n_end - col0, p.n - col0),
                                          static_cast<size_t>(col0), stage_smem + kEpiChOffset + (c - chunk0) * 128, tok);
    }
}

template <bool ACC_INT, int BLOCK_N>
__device__ __forceinline__ void epilogue_dispatch(const GemmParams& p, const TileInfo& t, const OutMaps& outs, uint32_t stage_smem, int stage_bytes,
                                                  uint32_t t_addr, int quad, int lane, int chunk0, int chunk1, const EpiPre& pre, uint32_t sk_base = 0,
                                                  int sk_parts = 0)
{
#define ASCB200_EPI_CASE(MODE, DT)                                                                          \
    if (p.epi.mode == MODE && p.epi.c_dtype == DT) {                                                          \
        epilogue_tile<ACC_INT, MODE, DT, BLOCK_N>(p, t, outs, stage_smem, stage_bytes, t_addr, quad, lane, chunk0, chunk1, pre, sk_base, sk_parts); \
        return;                                                                                               \
    }
    if constexpr (ACC_INT) {
        ASCB200_EPI_CASE(ASCB200_EPI_DEQUANT_TOKEN_CHANNEL, OUT_BF16)
        ASCB200_EPI_CASE(ASCB200_EPI_DEQUANT_TOKEN_CHANNEL, OUT_F16)
        ASCB200_EPI_CASE(ASCB200_EPI_DEQUANT_TOKEN_CHANNEL, OUT_F32)
        ASCB200_EPI_CASE(ASCB200_EPI_CAST, OUT_S32)
        ASCB200_EPI_CASE(ASCB200_EPI_FIXPIPE_QUANT, OUT_S8)
        ASCB200_EPI_CASE(ASCB200_EPI_FIXPIPE_QUANT, OUT_F16)
        ASCB200_EPI_CASE(ASCB200_EPI_FIXPIPE_QUANT, OUT_BF16)
    } else {
        ASCB200_EPI_CASE(ASCB200_EPI_CAST, OUT_F32)
        ASCB200_EPI_CASE(ASCB200_EPI_CAST, OUT_F16)
        ASCB200_EPI_CASE(ASCB200_EPI_CAST, OUT_BF16)
        ASCB200_EPI_CASE(ASCB200_EPI_FIXPIPE_QUANT, OUT_S8)
        ASCB200_EPI_CASE(ASCB200_EPI_FIXPIPE_QUANT, OUT_F16)
        ASCB200_EPI_CASE(ASCB200_EPI_FIXPIPE_QUANT, OUT_BF16)
        ASCB200_EPI_CASE(ASCB200_EPI_FIXPIPE_QUANT, OUT_F32)
        ASCB200_EPI_CASE(ASCB200_EPI_FIXPIPE_QUANT, OUT_E4M3)
        ASCB200_EPI_CASE(ASCB200_EPI_FIXPIPE_QUANT, OUT_E5M2)
    }
#undef ASCB200_EPI_CASE
}

// Epilogue of a block that was multiplied with the operand roles swapped (grouped int8 on CTA pairs: the last, partial
// 256-row block of a group).  The accumulator is the transpose of the output tile: TMEM lane = weight column, TMEM
// column j = row t.row0 + j of the group, so a thread owns one output column and walks down the rows; the 32 lanes of a
// warp write 32 consecutive elements of one output row per step.  Same arithmetic and rounding as the row-major path:
// (float(acc) * ch[n]) * tok[m], each product rounded, optional FasterGelu, one conversion to the output type.
template <int DT>
__device__ __forceinline__ void epilogue_tile_swapped(const GemmParams& p, const TileInfo& t, uint32_t t_addr, int n_lane, int lane, int chunk0,
                                                      int chunk1)
{
    static_assert(DT == OUT_F32 || DT == OUT_F16 || DT == OUT_BF16, "token x channel dequant writes floating-point outputs");
    const bool n_ok = n_lane < p.n;
    const float ch = n_ok ? __ldg(p.epi.ch + static_cast<size_t>(t.group) * p.n + n_lane) : 0.0f;
    const int act = p.epi.act;
#pragma unroll 1
    for (int c = chunk0; c < chunk1; ++c) {
        const int row_c = t.row0 + c * 32;
        if (row_c >= t.row_end) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int my_row = row_c + lane;
        const float my_tok = (p.epi.tok && my_row < t.row_end) ? __ldg(p.epi.tok + my_row) : 1.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float tok = __shfl_sync(0xFFFFFFFFu, my_tok, j);
            float v = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int>(r[j])), ch), tok);
            if (act == 1) v = faster_gelu(v);
            const int row = row_c + j;
            if (row < t.row_end && n_ok) {
                const size_t off = static_cast<size_t>(row) * static_cast<size_t>(p.epi.ldc) + n_lane;
                if constexpr (DT == OUT_F32) static_cast<float*>(p.epi.c)[off] = v;
                else if constexpr (DT == OUT_F16) static_cast<uint16_t*>(p.epi.c)[off] = static_cast<uint16_t>(pack_f16x2_sat(v, 0.0f));
                else static_cast<uint16_t*>(p.epi.c)[off] = static_cast<uint16_t>(pack_bf16x2(v, 0.0f));
            }
        }
    }
}

// ---- MMA issue (one thread) -------------------------------------------------------------------
// State of the issuing thread for the shared-memory ring: low descriptor words of the current
// stage's A / B / scale tiles and the addresses of its barriers, advanced by one add per stage.
template <int STAGE_BYTES, int NUM_STAGES, int B_OFFSET, int SF_OFFSET, int SF_COLS_PER_STAGE, int SF_SLOTS = NUM_STAGES>
struct IssueCursor {
    uint32_t a_lo, b_lo, sf_lo, full_bar, empty_bar, sf_tmem;
    uint32_t a_lo0, b_lo0, sf_lo0, full_bar0, empty_bar0, sf_tmem0;
    int stage, sf_slot;  // the TMEM columns of the scales rotate on their own (fewer slots than shared-memory stages fit TMEM)
    uint32_t phase;
    uint32_t step16;     // bytes between stages / 16 and the number of stages: the template's, unless the ring was cut at run time
    int nstages;
    __device__ __forceinline__ void init(uint32_t tiles_addr, uint32_t a_lbo_enc, uint32_t b_lbo_enc, uint32_t full0, uint32_t empty0, uint32_t sf_tmem_base,
                                         int stages = NUM_STAGES, int stage_bytes = STAGE_BYTES)
    {
        nstages = stages;
        step16 = static_cast<uint32_t>(stage_bytes) >> 4;
        // A shared-memory descriptor holds the offset inside the issuing CTA's own shared memory (14 bits of address / 16).  In a
        // cluster the shared-window address of every CTA but the first carries its rank above those bits, which would spill
        // into the descriptor's leading-offset field (seen as MN-major boxes read 256 bytes off in the second CTA of a cluster).
        tiles_addr &= 0x3FFFFu;
        a_lo0 = (a_lbo_enc << 16) | (tiles_addr >> 4);
        b_lo0 = (b_lbo_enc << 16) | ((tiles_addr + B_OFFSET) >> 4);
        sf_lo0 = (1u << 16) | ((tiles_addr + SF_OFFSET) >> 4);   // no-swizzle descriptor, leading offset 16 bytes
        full_bar0 = full0;
        empty_bar0 = empty0;
        sf_tmem0 = sf_tmem_base;
        rewind();
        sf_tmem = sf_tmem0;
        sf_slot = 0;
        phase = 0;
    }
    __device__ __forceinline__ void rewind()
    {
        a_lo = a_lo0;
        b_lo = b_lo0;
        sf_lo = sf_lo0;
        full_bar = full_bar0;
        empty_bar = empty_bar0;
        stage = 0;
    }
    __device__ __forceinline__ void advance()
    {
        if (++stage == nstages) {
            rewind();
            phase ^= 1u;
        } else {
            a_lo += step16;
            b_lo += step16;
            sf_lo += step16;
            full_bar += 8;
            empty_bar += 8;
        }
        if (++sf_slot == SF_SLOTS) {
            sf_slot = 0;
            sf_tmem = sf_tmem0;
        } else {
            sf_tmem += SF_COLS_PER_STAGE;
        }
    }
};

// Scale-factor copies of one K block (MXFP4 only): shared memory -> the stage's TMEM columns.
template <int KIND, bool PAIR, int SF_B_BLOCKS, class Cursor>
__device__ __forceinline__ void issue_sf_copies(const Cursor& c)
{
    if constexpr (KIND == KIND_MXF4) {
        // Each copy broadcasts one 512-byte chunk (128 rows x 4 K-blocks of 32) to the four 32-lane quadrants of
        // four TMEM columns; in a pair both CTAs copy from their own shared memory into their own TMEM.
        constexpr uint32_t sf_hi = (128u >> 4) | (1u << 14);  // stride 128 bytes between 8-row groups, descriptor version 1
        // chunk order in shared memory: A kc0, A kc1, then per 128-row block of B: kc0, kc1 (512 bytes each)
        sf_copy_issue<PAIR>(c.sf_tmem + 0, c.sf_lo, sf_hi);
        sf_copy_issue<PAIR>(c.sf_tmem + 4, c.sf_lo + 32, sf_hi);
#pragma unroll
        for (int rb = 0; rb < SF_B_BLOCKS; ++rb) {
            sf_copy_issue<PAIR>(c.sf_tmem + 8 + rb * 4, c.sf_lo + 64 + rb * 64, sf_hi);
            sf_copy_issue<PAIR>(c.sf_tmem + 16 + rb * 4, c.sf_lo + 96 + rb * 64, sf_hi);
        }
    } else if constexpr (KIND == KIND_MXF8) {
        // one chunk per 128 rows and K block (128 elements = four scales per row): A, then the blocks of B
        constexpr uint32_t sf_hi = (128u >> 4) | (1u << 14);
        sf_copy_issue<PAIR>(c.sf_tmem + 0, c.sf_lo, sf_hi);
#pragma unroll
        for (int rb = 0; rb < SF_B_BLOCKS; ++rb) sf_copy_issue<PAIR>(c.sf_tmem + 8 + rb * 4, c.sf_lo + 32 + rb * 32, sf_hi);
    }
}

// The four MMAs of one K block and the commit that releases the shared-memory stage.
template <int KIND, bool PAIR, class Cursor>
__device__ __forceinline__ void issue_mmas(const Cursor& c, uint32_t d_tmem, uint32_t hi_word, uint32_t a_kstep16, uint32_t b_kstep16,
                                           uint32_t idesc, uint32_t idesc_hi_sf, uint32_t sfb_col_offset, bool first)
{
    if constexpr (KIND == KIND_MXF4) {
        const uint32_t sfb = c.sf_tmem + 8 + sfb_col_offset;
        mma_issue_mxf4<PAIR>(d_tmem, c.a_lo, hi_word, c.b_lo, hi_word, idesc, c.sf_tmem, sfb, first ? 0u : 1u);
        mma_issue_mxf4<PAIR>(d_tmem, c.a_lo + 2, hi_word, c.b_lo + 2, hi_word, idesc_hi_sf, c.sf_tmem, sfb, 1u);
        mma_issue_mxf4<PAIR>(d_tmem, c.a_lo + 4, hi_word, c.b_lo + 4, hi_word, idesc, c.sf_tmem + 4, sfb + 8, 1u);
        mma_issue_mxf4<PAIR>(d_tmem, c.a_lo + 6, hi_word, c.b_lo + 6, hi_word, idesc_hi_sf, c.sf_tmem + 4, sfb + 8, 1u);
    } else if constexpr (KIND == KIND_MXF8) {
        // instruction i of the K block takes byte i of the scale columns (selectors in bits 4-5 and 29-30 of the descriptor)
        const uint32_t sfb = c.sf_tmem + 8 + sfb_col_offset;
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i)
            mma_issue_mxf8(d_tmem, c.a_lo + i * a_kstep16, hi_word, c.b_lo + i * b_kstep16, hi_word, idesc | (i << 4) | (i << 29), c.sf_tmem, sfb,
                           (first && i == 0) ? 0u : 1u);
    } else {
        mma_issue<KIND, PAIR>(d_tmem, c.a_lo, hi_word, c.b_lo, hi_word, idesc, first ? 0u : 1u);
        mma_issue<KIND, PAIR>(d_tmem, c.a_lo + a_kstep16, hi_word, c.b_lo + b_kstep16, hi_word, idesc, 1u);
        mma_issue<KIND, PAIR>(d_tmem, c.a_lo + 2 * a_kstep16, hi_word, c.b_lo + 2 * b_kstep16, hi_word, idesc, 1u);
        mma_issue<KIND, PAIR>(d_tmem, c.a_lo + 3 * a_kstep16, hi_word, c.b_lo + 3 * b_kstep16, hi_word, idesc, 1u);
    }
    commit_issue<PAIR>(c.empty_bar);
}

// Issues the tensor-core work of one K block (four MMAs, preceded by the scale-factor copies for
// MXFP4) and the commit that releases the shared-memory stage.
template <int KIND, bool PAIR, int SF_B_BLOCKS, class Cursor>
__device__ __forceinline__ void issue_k_block(const Cursor& c, uint32_t d_tmem, uint32_t hi_word, uint32_t a_kstep16, uint32_t b_kstep16,
                                              uint32_t idesc, uint32_t idesc_hi_sf, uint32_t sfb_col_offset, bool first)
{
    issue_sf_copies<KIND, PAIR, SF_B_BLOCKS>(c);
    issue_mmas<KIND, PAIR>(c, d_tmem, hi_word, a_kstep16, b_kstep16, idesc, idesc_hi_sf, sfb_col_offset, first);
}

// Split K over a cluster (single-CTA kernel): a CTA that is not the leader hands its accumulator to the leader.  Each epilogue
// thread writes the 32 values of its row and chunk into the leader's shared memory (the leader's operand ring, idle by then) as
// eight 16-byte pieces laid out [chunk][piece][row], so that the 32 lanes of a warp write and later read consecutive
// addresses, and then arrives on the leader's barrier with release at cluster scope.  The values travel as raw accumulator
// bits: int32 sums stay exact, fp32 sums are added in rank order (one more rounding per rank than a single chain).
template <int BLOCK_N>
__device__ __forceinline__ void splitk_send_tile(uint32_t leader_part, uint32_t leader_bar, uint32_t t_addr, int quad, int lane, int chunk0, int chunk1)
{
#pragma unroll 1
    for (int c = chunk0; c < chunk1; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const uint32_t dst = leader_part + ((c * 8) * 128 + quad * 32 + lane) * 16;
#pragma unroll
        for (int j = 0; j < 32; j += 4) st_cluster_v4(dst + (j / 4) * 2048, r[j], r[j + 1], r[j + 2], r[j + 3]);
    }
    mbar_arrive_cluster(leader_bar);
}

// ---- the kernel --------------------------------------------------------------------------------
// GROUPED = false compiles the group tables, the per-group tile search and the swapped blocks out of the kernel: a plain
// launch through the grouped build took 0.3 to 0.8 us longer (one rank's slab of the 8-GPU A8W8 split: 21.0 against 20.2 us).
template <int KIND, int BLOCK_N, bool GROUPED>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ OutMaps outs,
               const GemmParams p_in)
{
    GemmParams p = p_in;
    if constexpr (!GROUPED) p.groups = 0, p.group_swap = 0;
    using C = Cfg<KIND, BLOCK_N>;
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzled tiles need 1024-byte aligned bases
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* tiles = smem;
    static_assert(KIND != KIND_I8 || C::EPI_BYTES_PER_WARP >= kEpiChOffset + 512, "room for the per-channel scales of four chunks");
    uint8_t* epi_stage = smem + C::NUM_STAGES * C::STAGE_BYTES;  // [NUM_EPI_WARPS][EPI_BYTES_PER_WARP], 1024-byte aligned
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + C::EPI_BYTES);
    uint64_t* full_bar = bars;                         // [NUM_STAGES]
    uint64_t* empty_bar = bars + C::NUM_STAGES;        // [NUM_STAGES]
    uint64_t* acc_full_bar = bars + 2 * C::NUM_STAGES; // [2]
    uint64_t* acc_empty_bar = acc_full_bar + 2;        // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;
    uint64_t* parts_full_bar = reinterpret_cast<uint64_t*>(tmem_slot + 2);  // split K, leader: every other CTA's accumulator has arrived
    uint64_t* ring_free_bar = parts_full_bar + 1;                          // split K, others: the leader's ring may be overwritten
    static_assert((2 * 8 + 4 + 2) * 8 + 8 <= 256, "barrier area");
    int* row_start = reinterpret_cast<int*>(epi_stage + C::EPI_BYTES + 256);
    int* tile_start = row_start + (MAX_GROUPS + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_n = (p.n + BLOCK_N - 1) / BLOCK_N;
    const int num_m = (p.m + BLOCK_M - 1) / BLOCK_M;
    // Split K: the sk CTAs of a cluster take the same tile (one per cluster, the host sees to that) and consecutive ranges of
    // its K blocks, none of them empty.
    const int sk = p.split_k > 1 ? p.split_k : 1;
    const int sk_rank = sk > 1 ? static_cast<int>(cluster_ctarank()) : 0;
    const int kb_per = (p.num_k_blocks + sk - 1) / sk;
    const int kb0 = sk_rank * kb_per, kb1 = min(p.num_k_blocks, kb0 + kb_per);
    const int first_tile = static_cast<int>(blockIdx.x) / sk, tile_stride = static_cast<int>(gridDim.x) / sk;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::NUM_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&acc_full_bar[s]), 1);
            mbar_init(smem_u32(&acc_empty_bar[s]), NUM_EPI_WARPS);
        }
        mbar_init(smem_u32(parts_full_bar), (sk - 1) * NUM_EPI_WARPS * 32 + (sk == 1));  // every epilogue thread of every other CTA
        mbar_init(smem_u32(ring_free_bar), 1);
        *abort_word = 0u;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    // Launched with programmatic stream serialisation: everything above overlaps the tail of the previous kernel in the
    // stream; from here on global memory is read and written, so that kernel must have completed.
    grid_dependency_wait();
    if (warp == 0 && p.groups > 0) build_group_tables(p.group_counts, p.groups, num_n, BLOCK_M, row_start, tile_start);
    if (warp == 2) {
        tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    if (sk > 1) cluster_sync_all();  // the other CTAs' barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = p.groups > 0 ? tile_start[p.groups] : num_m * num_n;

    if (warp == 0) {
        // ===== TMA producer =====
        int stage = 0, cursor = 0;
        uint32_t phase = 0;
        TileInfo t;
        bool ok = true;
        for (int tile = first_tile; ok && locate_tile<BLOCK_N>(p, tile, num_m, total_tiles, row_start, tile_start, cursor, t); tile += tile_stride) {
            for (int kb = kb0; kb < kb1; ++kb) {
                ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_word, p.status);
                if (!ok) break;
                if (elect_one()) {
                    const uint32_t bar = smem_u32(&full_bar[stage]);
                    const uint32_t sa = smem_u32(tiles + stage * C::STAGE_BYTES);
                    const uint32_t sb = sa + A_TILE_BYTES;
                    mbar_expect_tx(bar, C::STAGE_BYTES);
                    const int k0 = kb * C::BLOCK_K;
                    // x coordinates are counted in tensor-map elements (bytes for int8 and packed fp4)
                    const int kx = KIND == KIND_MXF4 ? k0 / 2 : k0;
                    if (!p.a_mn) {
                        tma_load_3d(sa, &tmap_a, kx, t.row0, 0, bar);  // every map is rank 3
                    } else {
                        constexpr int MN_PER_BOX = KIND == KIND_F16 ? 64 : 128;
                        constexpr int BOX_BYTES = C::BLOCK_K * ROW_BYTES;
#pragma unroll
                        for (int j = 0; j < BLOCK_M / MN_PER_BOX; ++j) tma_load_3d(sa + j * BOX_BYTES, &tmap_a, t.row0 + j * MN_PER_BOX, k0, 0, bar);
                    }
                    if (!p.b_mn) {
                        tma_load_3d(sb, &tmap_b, kx, t.n0, t.group, bar);
                    } else {
                        constexpr int MN_PER_BOX = KIND == KIND_F16 ? 64 : 128;
                        constexpr int BOX_BYTES = C::BLOCK_K * ROW_BYTES;
#pragma unroll
                        for (int j = 0; j < BLOCK_N / MN_PER_BOX; ++j) tma_load_3d(sb + j * BOX_BYTES, &tmap_b, t.n0 + j * MN_PER_BOX, k0, t.group, bar);
                    }
                    if constexpr (C::IS_MX) {
                        const uint32_t ssf = sb + C::B_TILE_BYTES;
                        constexpr uint32_t SF_LOAD = C::SF_CHUNKS * SF_CHUNK_BYTES;   // the chunks of this K block of one 128-row block
                        const size_t kc = static_cast<size_t>(kb) * C::SF_CHUNKS;
                        bulk_load(ssf, p.sfa + (static_cast<size_t>(t.row0 / 128) * p.sf_kc + kc) * SF_CHUNK_BYTES, SF_LOAD, bar);
#pragma unroll
                        for (int rb = 0; rb < C::SF_B_BLOCKS; ++rb)
                            bulk_load(ssf + (1 + rb) * SF_LOAD, p.sfb + (static_cast<size_t>(t.n0 / 128 + rb) * p.sf_kc + kc) * SF_CHUNK_BYTES, SF_LOAD, bar);
                    }
                }
                __syncwarp();
                if (++stage == C::NUM_STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        int cursor = 0, acc_iter = 0;
        TileInfo t;
        bool ok = true;
        // Shared-memory descriptors, 128-byte swizzle (high word: 1024 bytes between 8-row groups, version 1,
        // layout type 2).  K-major operands: leading offset unused (16), one MMA advances 32 bytes.
        // MN-major: one TMA box per 128 bytes of M/N, BLOCK_K k-rows each, boxes BLOCK_K*128 bytes apart,
        // one MMA advances UMMA_K k-rows.
        constexpr uint32_t hi_word = static_cast<uint32_t>(smem_desc_sw128(0, 1024) >> 32);
        const uint32_t a_lbo = p.a_mn ? (C::BLOCK_K * ROW_BYTES) >> 4 : 1u, b_lbo = p.b_mn ? (C::BLOCK_K * ROW_BYTES) >> 4 : 1u;
        const uint32_t a_k16 = (p.a_mn ? C::UMMA_K * ROW_BYTES : 32) >> 4, b_k16 = (p.b_mn ? C::UMMA_K * ROW_BYTES : 32) >> 4;
        const uint32_t idesc_hi_sf = p.idesc | (2u << 4) | (2u << 29);  // MXFP4: scale bytes 2..3 of the TMEM column
        IssueCursor<C::STAGE_BYTES, C::NUM_STAGES, A_TILE_BYTES, A_TILE_BYTES + C::B_TILE_BYTES, C::SF_COLS_PER_STAGE> cur;
        cur.init(smem_u32(tiles), a_lbo, b_lbo, smem_u32(&full_bar[0]), smem_u32(&empty_bar[0]), tmem_base + C::SF_COL0);
        for (int tile = first_tile; ok && locate_tile<BLOCK_N>(p, tile, num_m, total_tiles, row_start, tile_start, cursor, t); tile += tile_stride, ++acc_iter) {
            const int acc_stage = acc_iter % C::ACC_STAGES;
            const uint32_t acc_phase = (acc_iter / C::ACC_STAGES) & 1u;
            ok = mbar_wait(smem_u32(&acc_empty_bar[acc_stage]), acc_phase ^ 1u, abort_word, p.status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc_stage * BLOCK_N;
            const uint32_t acc_full = smem_u32(&acc_full_bar[acc_stage]);
            const uint32_t sfb_off = static_cast<uint32_t>(t.n0 % 128) / 32;  // a 192-wide tile may start mid-way in a 128-row scale block
            // A tile that holds at most 64 rows (the tail of a group or of the matrix) runs the M = 64 form of the instruction (M / 16 in
            // bits 24-28 of the descriptor): half the multiplications, and under the power cap half the energy, of rows
            // that would be thrown away.  Its accumulator rows 16 q .. 16 q + 15 land in lanes 0-15 of TMEM quadrant q.
            const uint32_t idesc = t.m64 ? ((p.idesc & ~(0x1Fu << 24)) | (4u << 24)) : p.idesc;
            const int last = kb1 - 1;
            for (int kb = kb0; kb <= last; ++kb) {
                ok = mbar_wait(cur.full_bar, cur.phase, abort_word, p.status);
                if (!ok) break;
                tc_fence_after();
                if (elect_one()) {
                    issue_k_block<KIND, false, C::SF_B_BLOCKS>(cur, d_tmem, hi_word, a_k16, b_k16, idesc, idesc_hi_sf, sfb_off, kb == kb0);
                    if (kb == last) tc_commit(acc_full);
                }
                __syncwarp();
                cur.advance();
            }
        }
    } else if (warp >= 4) {
        // ===== epilogue: warps 4-7 drain the first half of the tile's columns, warps 8-11 the second =====
        const int quad = warp & 3;  // TMEM lanes 32*quad .. 32*quad+31 are the ones this warp may read
        const int half = (warp - 4) >> 2;
        constexpr int CHUNKS = BLOCK_N / 32;
        const int chunk0 = half * (CHUNKS / 2), chunk1 = chunk0 + CHUNKS / 2;
        int cursor = 0, acc_iter = 0;
        TileInfo t;
        bool ok = true;
        for (int tile = first_tile; ok && locate_tile<BLOCK_N>(p, tile, num_m, total_tiles, row_start, tile_start, cursor, t); tile += tile_stride, ++acc_iter) {
            const int acc_stage = acc_iter % C::ACC_STAGES;
            const uint32_t acc_phase = (acc_iter / C::ACC_STAGES) & 1u;
            const EpiPre pre = epilogue_preload(p, t, quad, lane, chunk0);
            ok = mbar_wait_relaxed(smem_u32(&acc_full_bar[acc_stage]), acc_phase, abort_word, p.status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc_stage * BLOCK_N;
            if (sk > 1 && sk_rank != 0) {
                // wait until the leader's MMAs have read the last of its ring, then write this CTA's accumulator over it
                ok = mbar_wait_cluster(smem_u32(ring_free_bar), 0u, true, abort_word, p.status);
                if (!ok) break;
                splitk_send_tile<BLOCK_N>(map_to_cta(smem_u32(tiles), 0) + static_cast<uint32_t>(sk_rank - 1) * (BLOCK_N * 512),
                                          map_to_cta(smem_u32(parts_full_bar), 0), t_addr, quad, lane, chunk0, chunk1);
                continue;  // one tile per cluster: nothing follows
            }
            if (sk > 1) {
                // this CTA's MMAs are done (the accumulator is complete), so its ring is free: tell the others, then wait for them
                if (warp == 4 && elect_one())
                    for (int r = 1; r < sk; ++r) mbar_arrive_cluster_tmem(map_to_cta(smem_u32(ring_free_bar), static_cast<uint32_t>(r)));
                ok = mbar_wait_cluster(smem_u32(parts_full_bar), 0u, true, abort_word, p.status);
                if (!ok) break;
            }
            epilogue_dispatch<KIND == KIND_I8, BLOCK_N>(p, t, outs, smem_u32(epi_stage) + (warp - 4) * C::EPI_BYTES_PER_WARP, C::EPI_BYTES_PER_WARP, t_addr,
                                                        quad, lane, chunk0, chunk1, pre, smem_u32(tiles), sk - 1);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[acc_stage]));
        }
        if (elect_one()) bulk_wait_group_read<0>();  // staged chunks have left shared memory before the CTA may exit
    }

    // ===== teardown =====
    tc_fence_before();
    __syncthreads();
    if (*abort_word) {
        // give copies that may still be in flight time to land before the CTA's shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 400000ll) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---- the CTA-pair kernel -----------------------------------------------------------------------
// Same roles and pipeline as gemm_tc_kernel, but two CTAs of a cluster share every MMA
// (tcgen05.mma.cta_group::2): the pair computes a 256 x BLOCK_N tile, each CTA loads its own 128
// rows of A and BLOCK_N/2 rows of B, so every SM reads a third less shared memory per instruction
// and fetches half of B from L2.  The even CTA issues the MMAs; completion is signalled to both
// CTAs with multicast commits; epilogue warps of both CTAs release the accumulator stage on the
// leader's barrier.  Plain (non-grouped) problems only.

constexpr int kMaxRingStages = 8;  // barrier storage of the CTA-pair kernel's operand ring
// Tiles of a CTA pair: cluster c takes tiles c, c + clusters, ...  (Handing tiles out at run time from a counter was measured on
// the grouped configuration, whose tiles differ widely in cost: 554 k against 557 k cycles, and is not kept.)
struct TileFeed {
    int next, stride;
    __device__ __forceinline__ void init(int cluster_id, int num_clusters)
    {
        next = cluster_id;
        stride = num_clusters;
    }
    __device__ __forceinline__ bool take(int total_tiles, int& tile)
    {
        tile = next;
        next += stride;
        return tile < total_tiles;
    }
};

template <int KIND, int BLOCK_N>
struct Cfg2 {
    static constexpr int B_TILE_BYTES = (BLOCK_N / 2) * ROW_BYTES;
    static constexpr int SF_B_BLOCKS = (BLOCK_N + 127) / 128;   // every CTA needs the scales of all BLOCK_N columns
    static constexpr int SF_BLOCK_BYTES = 2 * SF_CHUNK_BYTES;   // scales of one 128-row block and K block (two chunks)
    static constexpr int SF_BYTES = KIND == KIND_MXF4 ? (1 + SF_B_BLOCKS) * SF_BLOCK_BYTES : 0;
    static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES + SF_BYTES;
    static constexpr int ACC_STAGES = 2;
    static constexpr int SF_COLS_PER_STAGE = 24;
    static constexpr int SF_COL0 = ACC_STAGES * BLOCK_N;
    static constexpr int MAX_SF_STAGES = KIND == KIND_MXF4 ? (512 - SF_COL0) / SF_COLS_PER_STAGE : 8;
    static constexpr int EPI_BYTES_PER_WARP = 3072;  // staged output chunks and per-channel scales (see Cfg)
    static constexpr int EPI_BYTES = NUM_EPI_WARPS * EPI_BYTES_PER_WARP;
    static constexpr int TABLE_BYTES = 2 * (MAX_GROUPS + 1) * static_cast<int>(sizeof(int));  // grouped mode: row and tile prefix sums
    static constexpr int NUM_STAGES = std::min(8, (227 * 1024 - 1024 - 256 - EPI_BYTES - TABLE_BYTES) / STAGE_BYTES);
    static constexpr int SF_SLOTS = std::min(NUM_STAGES, MAX_SF_STAGES);  // scale-factor slots in TMEM
    static constexpr int TMEM_COLS = 512;
    static_assert(ACC_STAGES * BLOCK_N + (KIND == KIND_MXF4 ? SF_SLOTS * SF_COLS_PER_STAGE : 0) <= 512, "TMEM budget");
    static constexpr int BLOCK_K = KIND == KIND_F16 ? 64 : KIND == KIND_I8 ? 128 : 256;
    static constexpr int UMMA_K = BLOCK_K / 4;
    static constexpr int SMEM_BYTES = NUM_STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256 + TABLE_BYTES;
};

// KMAJOR = true: both operands are K-major (the usual case, and the only one for MXFP4), which fixes the box walk of the
// producer and the descriptor steps of the issuer at compile time: 5 to 7 % per K block where tiles are narrow (one rank's slab
// of the 8-GPU A8W8 split: 20.4 -> 19.4 us).
template <int KIND, int BLOCK_N, bool GROUPED, bool KMAJOR>   // GROUPED: see gemm_tc_kernel
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb, const __grid_constant__ OutMaps outs,
                    const GemmParams p_in)
{
    GemmParams p = p_in;
    if constexpr (!GROUPED) p.groups = 0, p.group_swap = 0;
    if constexpr (KMAJOR) p.a_mn = 0, p.b_mn = 0;
    using C = Cfg2<KIND, BLOCK_N>;
    constexpr int PAIR_M = 2 * BLOCK_M;
    extern __shared__ uint8_t smem_raw[];
    // both CTAs must use identical offsets: the dynamic shared memory window starts at the same offset in each
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* tiles = smem;
    static_assert(KIND != KIND_I8 || C::EPI_BYTES_PER_WARP >= kEpiChOffset + 512, "room for the per-channel scales of four chunks");
    uint8_t* epi_stage = smem + C::NUM_STAGES * C::STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + C::EPI_BYTES);
    uint64_t* full_bar = bars;                 // [kMaxRingStages]
    uint64_t* empty_bar = bars + kMaxRingStages;
    uint64_t* acc_full_bar = bars + 2 * kMaxRingStages;
    uint64_t* acc_empty_bar = acc_full_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
    volatile uint32_t* abort_word = tmem_slot + 1;
    static_assert((2 * kMaxRingStages + 4) * 8 + 8 <= 256, "barrier area");
    static_assert(C::NUM_STAGES <= kMaxRingStages, "barrier area");
    // The ring of operand stages: the compile-time geometry, or (narrower tiles of a call) more and smaller stages in the same bytes.
    const bool cut_ring = KIND != KIND_MXF4 && p.ring_stages > 0;
    const int num_stages = cut_ring ? p.ring_stages : C::NUM_STAGES;
    const int stage_bytes = cut_ring ? p.ring_stage_bytes : C::STAGE_BYTES;
    int* row_start = reinterpret_cast<int*>(epi_stage + C::EPI_BYTES + 256);  // both CTAs build identical tables
    int* tile_start = row_start + (MAX_GROUPS + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();   // 0 = leader
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;
    // tile width: fixed for MXFP4 (scale blocks), chosen per call otherwise (BLOCK_N is then the upper bound that sizes
    // shared memory and the accumulator stages in TMEM)
    const int bn = KIND == KIND_MXF4 ? BLOCK_N : p.pair_n;
    const int num_n = (p.n + bn - 1) / bn;
    const int num_m = (p.m + PAIR_M - 1) / PAIR_M;

    if (threadIdx.x == 0) {
        for (int s = 0; s < num_stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&acc_full_bar[s]), 1);
            mbar_init(smem_u32(&acc_empty_bar[s]), 2 * NUM_EPI_WARPS);  // epilogue warps of both CTAs
        }
        *abort_word = 0u;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    grid_dependency_wait();  // see gemm_tc_kernel
    if (warp == 3 && p.groups > 0) build_group_tables(p.group_counts, p.groups, num_n, PAIR_M, row_start, tile_start);
    if (warp == 2) {
        tmem_alloc_pair(smem_u32(tmem_slot), C::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything can arrive on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int total_tiles = p.groups > 0 ? tile_start[p.groups] : num_m * num_n;

    if (warp == 0) {
        // ===== TMA producer (both CTAs) =====
        int stage = 0, cursor = 0;
        uint32_t phase = 0;
        bool ok = true;
        TileInfo t;
        TileFeed feed;
        feed.init(cluster_id, num_clusters);
        for (int tile; ok && feed.take(total_tiles, tile) && locate_pair_tile(p, tile, num_m, total_tiles, bn, row_start, tile_start, cursor, t);) {
            // rows past the end of a group belong to the next group (or lie outside the matrix and read as zero): they are
            // multiplied like the others and never stored
            // A swapped block (see GemmParams::group_swap) takes its swap_n rows as the narrow operand: each CTA loads half of
            // them, in boxes of 32 rows (or one box of 128), into the start of its A buffer; the weights are loaded as always.
            const int swap_half = t.swap_n / 2;
            const int row0 = t.swap_n ? t.row0 + static_cast<int>(rank) * swap_half : t.row0 + static_cast<int>(rank) * BLOCK_M;
            const int n0 = t.n0 + static_cast<int>(rank) * (bn / 2);
            const int x_boxes = (swap_half + 31) / 32;  // 1 .. 4
            const uint32_t a_bytes = t.swap_n ? static_cast<uint32_t>(x_boxes) * 32 * ROW_BYTES : A_TILE_BYTES;
            for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_word, p.status);
                if (!ok) break;
                if (elect_one()) {
                    const uint32_t own_bar = smem_u32(&full_bar[stage]);
                    const uint32_t bar = own_bar & kPeerBitMask;  // the leader's barrier counts both CTAs' bytes
                    const uint32_t sa = smem_u32(tiles) + stage * stage_bytes;
                    const uint32_t sb = sa + A_TILE_BYTES;
                    if (rank == 0) mbar_expect_tx(own_bar, 2 * (a_bytes + (bn / 2) * ROW_BYTES + C::SF_BYTES));
                    const int k0 = kb * C::BLOCK_K;
                    const int kx = KIND == KIND_MXF4 ? k0 / 2 : k0;  // packed fp4: two values per tensor-map element
                    constexpr int MN_PER_BOX = KIND == KIND_F16 ? 64 : 128;
                    constexpr int BOX_BYTES = C::BLOCK_K * ROW_BYTES;
                    if constexpr (KIND == KIND_MXF4) {
                        // re-tiled scales as a [chunk, 128 x u32] tensor: the two chunks of this K block per 128-row block
                        const uint32_t ssf = sb + C::B_TILE_BYTES;
                        const int tile_n0 = n0 - static_cast<int>(rank) * (bn / 2);
                        tma_load_2d_pair(ssf, &tmap_sfa, 0, (row0 / 128) * p.sf_kc + 2 * kb, bar);
#pragma unroll
                        for (int rb = 0; rb < C::SF_B_BLOCKS; ++rb)
                            tma_load_2d_pair(ssf + (1 + rb) * C::SF_BLOCK_BYTES, &tmap_sfb, 0, (tile_n0 / 128 + rb) * p.sf_kc + 2 * kb, bar);
                    }
                    if (KIND == KIND_I8 && t.swap_n && x_boxes < 4) {
                        // tmap_sfa is here the map of A with boxes of 32 rows
                        for (int j = 0; j < x_boxes; ++j) tma_load_3d_pair(sa + j * 32 * ROW_BYTES, &tmap_sfa, kx, row0 + 32 * j, 0, bar);
                    } else if (!p.a_mn) {
                        tma_load_3d_pair(sa, &tmap_a, kx, row0, 0, bar);
                    } else {
#pragma unroll
                        for (int j = 0; j < BLOCK_M / MN_PER_BOX; ++j) tma_load_3d_pair(sa + j * BOX_BYTES, &tmap_a, row0 + j * MN_PER_BOX, k0, 0, bar);
                    }
                    if (!p.b_mn) {
                        tma_load_3d_pair(sb, &tmap_b, kx, n0, t.group, bar);
                    } else {
#pragma unroll
                        for (int j = 0; j < (BLOCK_N / 2) / MN_PER_BOX; ++j) tma_load_3d_pair(sb + j * BOX_BYTES, &tmap_b, n0 + j * MN_PER_BOX, k0, t.group, bar);
                    }
                }
                __syncwarp();
                if (++stage == num_stages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
        // drain: every stage's last release (a multicast commit from the leader) must have landed in
        // this CTA's shared memory before the CTA may exit
        for (int i = 0; ok && i < num_stages; ++i) {
            ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_word, p.status);
            if (++stage == num_stages) {
                stage = 0;
                phase ^= 1u;
            }
        }
    } else if (warp == 1 && rank == 0) {
        // ===== MMA issuer (leader CTA only) =====
        int acc_iter = 0;
        bool ok = true;
        constexpr uint32_t hi_word = static_cast<uint32_t>(smem_desc_sw128(0, 1024) >> 32);
        const uint32_t a_lbo = p.a_mn ? (C::BLOCK_K * ROW_BYTES) >> 4 : 1u, b_lbo = p.b_mn ? (C::BLOCK_K * ROW_BYTES) >> 4 : 1u;
        const uint32_t a_k16 = (p.a_mn ? C::UMMA_K * ROW_BYTES : 32) >> 4, b_k16 = (p.b_mn ? C::UMMA_K * ROW_BYTES : 32) >> 4;
        const uint32_t idesc_hi_sf = p.idesc | (2u << 4) | (2u << 29);
        IssueCursor<C::STAGE_BYTES, C::NUM_STAGES, A_TILE_BYTES, A_TILE_BYTES + C::B_TILE_BYTES, C::SF_COLS_PER_STAGE, C::SF_SLOTS> cur;
        cur.init(smem_u32(tiles), a_lbo, b_lbo, smem_u32(&full_bar[0]), smem_u32(&empty_bar[0]), tmem_base + C::SF_COL0, num_stages, stage_bytes);
        int cursor = 0;
        TileInfo t;
        TileFeed feed;
        feed.init(cluster_id, num_clusters);
        for (int tile; ok && feed.take(total_tiles, tile) && locate_pair_tile(p, tile, num_m, total_tiles, bn, row_start, tile_start, cursor, t); ++acc_iter) {
            const int acc_stage = acc_iter & 1;
            const uint32_t acc_phase = (acc_iter >> 1) & 1u;
            ok = mbar_wait(smem_u32(&acc_empty_bar[acc_stage]), acc_phase ^ 1u, abort_word, p.status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc_stage * BLOCK_N;
            const uint32_t acc_full = smem_u32(&acc_full_bar[acc_stage]);
            const uint32_t sfb_off = static_cast<uint32_t>(t.n0 % 128) / 32;
            const int last = p.num_k_blocks - 1;
            int kb = 0;
            if (KIND == KIND_I8 && t.swap_n) {
                // Swapped block: the pair's 256 weight rows (B buffers) are the wide operand, the block's swap_n rows of A the
                // narrow one; the accumulator holds the transpose of the output tile in swap_n columns.
                const uint32_t idesc = p.idesc_swap | (static_cast<uint32_t>(t.swap_n >> 3) << 17);
                for (; kb <= last; ++kb) {
                    ok = mbar_wait(cur.full_bar, cur.phase, abort_word, p.status);
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one()) {
                        mma_issue<KIND_I8, true>(d_tmem, cur.b_lo, hi_word, cur.a_lo, hi_word, idesc, kb == 0 ? 0u : 1u);
                        mma_issue<KIND_I8, true>(d_tmem, cur.b_lo + b_k16, hi_word, cur.a_lo + a_k16, hi_word, idesc, 1u);
                        mma_issue<KIND_I8, true>(d_tmem, cur.b_lo + 2 * b_k16, hi_word, cur.a_lo + 2 * a_k16, hi_word, idesc, 1u);
                        mma_issue<KIND_I8, true>(d_tmem, cur.b_lo + 3 * b_k16, hi_word, cur.a_lo + 3 * a_k16, hi_word, idesc, 1u);
                        commit_issue<true>(cur.empty_bar);
                        if (kb == last) tc_commit_pair(acc_full);
                    }
                    __syncwarp();
                    cur.advance();
                }
                continue;
            }
            if constexpr (KIND == KIND_MXF4) {
                // Copies and MMAs run through one in-order pipe; issuing the scale copies of two K blocks together and then
                // eight MMAs back to back measured 3 % faster than alternating per K block.
                for (; kb < last; kb += 2) {
                    auto nxt = cur;
                    nxt.advance();
                    ok = mbar_wait(cur.full_bar, cur.phase, abort_word, p.status) && mbar_wait(nxt.full_bar, nxt.phase, abort_word, p.status);
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one()) {
                        issue_sf_copies<KIND, true, C::SF_B_BLOCKS>(cur);
                        issue_sf_copies<KIND, true, C::SF_B_BLOCKS>(nxt);
                        issue_mmas<KIND, true>(cur, d_tmem, hi_word, a_k16, b_k16, p.idesc, idesc_hi_sf, sfb_off, kb == 0);
                        issue_mmas<KIND, true>(nxt, d_tmem, hi_word, a_k16, b_k16, p.idesc, idesc_hi_sf, sfb_off, false);
                        if (kb + 1 == last) tc_commit_pair(acc_full);
                    }
                    __syncwarp();
                    cur = nxt;
                    cur.advance();
                }
            }
            for (; ok && kb <= last; ++kb) {
                ok = mbar_wait(cur.full_bar, cur.phase, abort_word, p.status);
                if (!ok) break;
                tc_fence_after();
                if (elect_one()) {
                    issue_k_block<KIND, true, C::SF_B_BLOCKS>(cur, d_tmem, hi_word, a_k16, b_k16, p.idesc, idesc_hi_sf, sfb_off, kb == 0);
                    if (kb == last) tc_commit_pair(acc_full);
                }
                __syncwarp();
                cur.advance();
            }
        }
    } else if (warp >= 4) {
        // ===== epilogue (both CTAs, each for its own 128 rows) =====
        const int quad = warp & 3;
        const int half = (warp - 4) >> 2;
        const int chunks = (bn + 31) / 32, split = (chunks + 1) / 2;
        const int chunk0 = half * split, chunk1 = half ? chunks : split;
        int acc_iter = 0, cursor = 0;
        bool ok = true;
        TileInfo t;
        TileFeed feed;
        feed.init(cluster_id, num_clusters);
        for (int tile; ok && feed.take(total_tiles, tile) && locate_pair_tile(p, tile, num_m, total_tiles, bn, row_start, tile_start, cursor, t); ++acc_iter) {
            const int acc_stage = acc_iter & 1;
            const uint32_t acc_phase = (acc_iter >> 1) & 1u;
            if (!t.swap_n) t.row0 += static_cast<int>(rank) * BLOCK_M;  // this CTA's half of the pair tile
            const EpiPre pre = t.swap_n ? EpiPre{1.0f, 0.0f} : epilogue_preload(p, t, quad, lane, chunk0);
            ok = mbar_wait_relaxed(smem_u32(&acc_full_bar[acc_stage]), acc_phase, abort_word, p.status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc_stage * BLOCK_N;
            if (KIND == KIND_I8 && t.swap_n) {
                // transposed accumulator: this lane owns output column n_lane, the warps of a quadrant split the rows
                const int n_lane = t.n0 + static_cast<int>(rank) * BLOCK_M + quad * 32 + lane;
                const int sw_chunks = (t.swap_n + 31) / 32, sw_split = (sw_chunks + 1) / 2;
                const int c0 = half * sw_split, c1 = half ? sw_chunks : sw_split;
                if (p.epi.c_dtype == OUT_BF16) epilogue_tile_swapped<OUT_BF16>(p, t, t_addr, n_lane, lane, c0, c1);
                else if (p.epi.c_dtype == OUT_F16) epilogue_tile_swapped<OUT_F16>(p, t, t_addr, n_lane, lane, c0, c1);
                else epilogue_tile_swapped<OUT_F32>(p, t, t_addr, n_lane, lane, c0, c1);
            } else {
                epilogue_dispatch<KIND == KIND_I8, BLOCK_N>(p, t, outs, smem_u32(epi_stage) + (warp - 4) * C::EPI_BYTES_PER_WARP, C::EPI_BYTES_PER_WARP,
                                                            t_addr, quad, lane, chunk0, chunk1, pre);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_tmem(smem_u32(&acc_empty_bar[acc_stage]) & kPeerBitMask);
        }
        if (elect_one()) bulk_wait_group_read<0>();
    }

    // ===== teardown =====
    tc_fence_before();
    __syncthreads();
    if (*abort_word) {
        const long long t0 = clock64();
        while (clock64() - t0 < 400000ll) __nanosleep(1000);
        __syncthreads();
    }
    cluster_sync_all();  // neither CTA leaves while the other may still signal into its shared memory
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
    }
}

// Re-tiles MX scale factors [rows, ks] (row-major bytes) into 512-byte chunks: chunk (rb, kc) holds
// the scales of rows rb*128 .. +127 and K-blocks kc*4 .. +3 at byte (r%32)*16 + (r/32)*4 + (ks%4),
// the order tcgen05.cp (32x128b, warpx4) expects.  Missing rows / K-blocks are filled with 127 (1.0).
// One launch covers both operands: blocks [0, rb_a * kc_tiles) re-tile A, the rest B.  A block moves
// 128 rows x 8 chunks through shared memory so that rows are read as whole sectors and chunks written as whole lines.
// `paired` bit 0 / 1: the source of A / B is stored [ks / 2][rows][2] instead (the two scales of a 64-element K step side
// by side, rows next): the order the reference keeps a transposed scaleA and a non-transposed scaleB in
// (examples/.../00_matmul/matmul_mx/scripts/gen_data.py: reshape(sk / 2, 2, n).transpose(0, 2, 1)).
__global__ void __launch_bounds__(256)
retile_scales_kernel(const uint8_t* __restrict__ src_a, uint32_t* __restrict__ dst_a, int rows_a, int rb_a, const uint8_t* __restrict__ src_b,
                     uint32_t* __restrict__ dst_b, int rows_b, int ks, int kc_count, int kc_tiles, int paired)
{
    constexpr int CH = 8;  // chunks per block: 32 bytes of every row, four words per thread, all loads issued before any is used
    __shared__ uint32_t tile[128][CH + 1];  // [position inside a chunk][chunk]
    grid_dependency_wait();
    int blk = blockIdx.x;
    const bool is_a = blk < rb_a * kc_tiles;
    if (!is_a) blk -= rb_a * kc_tiles;
    const uint8_t* src = is_a ? src_a : src_b;
    uint32_t* dst = is_a ? dst_a : dst_b;
    const int rows = is_a ? rows_a : rows_b;
    const int rb = blk / kc_tiles, kc0 = (blk % kc_tiles) * CH;
    const bool pair_src = ((paired >> (is_a ? 0 : 1)) & 1) != 0;
    const bool words = !pair_src && (ks & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 3) == 0;
    uint32_t w[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int idx = threadIdx.x + u * 256;
        // plain source: consecutive threads read along a row; paired source: consecutive threads read consecutive rows
        const int rl = pair_src ? idx % 128 : idx / CH, j = pair_src ? idx / 128 : idx % CH;
        const int r = rb * 128 + rl, k = (kc0 + j) * 4;
        if (pair_src) {
            w[u] = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b)
                w[u] |= ((r < rows && k + b < ks) ? static_cast<uint32_t>(src[(static_cast<size_t>((k + b) >> 1) * rows + r) * 2 + ((k + b) & 1)]) : 127u)
                        << (8 * b);
        } else if (r < rows && k + 3 < ks && words) {
            w[u] = __ldg(reinterpret_cast<const uint32_t*>(src + static_cast<size_t>(r) * ks + k));
        } else {
            w[u] = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) w[u] |= ((r < rows && k + b < ks) ? static_cast<uint32_t>(src[static_cast<size_t>(r) * ks + k + b]) : 127u) << (8 * b);
        }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int idx = threadIdx.x + u * 256;
        const int rl = pair_src ? idx % 128 : idx / CH, j = pair_src ? idx / 128 : idx % CH;
        tile[(rl & 31) * 4 + (rl >> 5)][j] = w[u];
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int idx = threadIdx.x + u * 256;
        const int j = idx >> 7, pos = idx & 127;
        if (kc0 + j < kc_count) dst[(static_cast<size_t>(rb) * kc_count + kc0 + j) * 128 + pos] = tile[pos][j];
    }
}

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
        else
            (void)cudaGetLastError();
    });
    return fn;
}

// rank-3 map over [d2][d1][d0] (d0 contiguous), box {b0, b1, 1}, 128-byte swizzle, zero fill out of bounds.
int make_map(CUtensorMap* map, CUtensorMapDataType dt, int esz, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
             uint64_t stride2_elems, uint32_t b0, uint32_t b1)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return ASCB200_ECUDA;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1_elems * esz, stride2_elems * esz};
    cuuint32_t box[3] = {b0, b1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (!aligned_to(base, 16) || strides[0] % 16 != 0 || strides[1] % 16 != 0) return ASCB200_EALIGN;
    CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? ASCB200_OK : ASCB200_ECUDA;
}

// rank-2 map over re-tiled scales: `chunks` rows of 128 x u32 (512 bytes), box = box_rows rows, no swizzle.
int make_sf_map(CUtensorMap* map, const void* base, uint64_t chunks, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return ASCB200_ECUDA;
    cuuint64_t dims[2] = {128, chunks};
    cuuint64_t strides[1] = {SF_CHUNK_BYTES};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? ASCB200_OK : ASCB200_ECUDA;
}

int out_bytes(int dt) { return (dt == OUT_S8 || dt == OUT_E4M3 || dt == OUT_E5M2) ? 1 : (dt == OUT_F16 || dt == OUT_BF16) ? 2 : 4; }

// rank-2 map over an output [rows][cols] of 1- or 2-byte elements, box 32 x 32, swizzle = bytes of one box row.
// Returns false when the tensor cannot be described (alignment): the kernel then stores from registers.
bool make_out_map(CUtensorMap* map, int dtype, const void* base, uint64_t cols, uint64_t rows, uint64_t ld_elems)
{
    const int esz = out_bytes(dtype);
    // plain stores move bits; a reducing store (atomic add) needs the arithmetic type
    const CUtensorMapDataType mdt = dtype == OUT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : dtype == OUT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                                                           : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    EncodeTiledFn fn = encode_fn();
    if (!fn || (esz != 1 && esz != 2) || !aligned_to(base, 16) || (ld_elems * esz) % 16 != 0 || cols == 0 || rows == 0) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld_elems * esz};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, mdt, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, esz == 1 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int KIND, int BLOCK_N, bool GROUPED>
int launch_gemm_as(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& outs, const GemmParams& p, int grid, cudaStream_t stream)
{
    using C = Cfg<KIND, BLOCK_N>;
    static bool configured[16] = {};
    int dev = 0;
    ASCB200_CUDA(cudaGetDevice(&dev));
    if (!configured[dev & 15]) {
        ASCB200_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<KIND, BLOCK_N, GROUPED>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        configured[dev & 15] = true;
    }
    // Split K over a cluster: only while every cluster gets at most one tile, every CTA at least one K block, and the other
    // CTAs' accumulators (BLOCK_N x 512 bytes each) fit the leader's operand ring.
    GemmParams q = p;
    int sk = p.split_k;
    while (sk > 1 && ((sk - 1) * BLOCK_N * 512 > C::NUM_STAGES * C::STAGE_BYTES || p.num_k_blocks <= (sk - 1) * ((p.num_k_blocks + sk - 1) / sk))) sk >>= 1;
    q.split_k = sk > 1 ? sk : 0;
    if (q.split_k > 1) {
        ASCB200_CUDA(launch_pdl_cluster(gemm_tc_kernel<KIND, BLOCK_N, GROUPED>, grid * q.split_k, NUM_THREADS, C::SMEM_BYTES, stream, static_cast<unsigned>(q.split_k), ta, tb,
                                        outs, q));
        return ASCB200_OK;
    }
    ASCB200_CUDA(launch_pdl(gemm_tc_kernel<KIND, BLOCK_N, GROUPED>, grid, NUM_THREADS, C::SMEM_BYTES, stream, ta, tb, outs, q));
    return ASCB200_OK;
}

// Grouped calls exist for int8 only; every other call takes the build without the group code.
template <int KIND, int BLOCK_N>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& outs, const GemmParams& p, int grid, cudaStream_t stream)
{
    if constexpr (KIND == KIND_I8)
        if (p.groups > 0) return launch_gemm_as<KIND, BLOCK_N, true>(ta, tb, outs, p, grid, stream);
    return launch_gemm_as<KIND, BLOCK_N, false>(ta, tb, outs, p, grid, stream);
}

template <int KIND, int BLOCK_N, bool GROUPED, bool KMAJOR>
int launch_gemm_pair_as(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsfa, const CUtensorMap& tsfb, const OutMaps& outs,
                     const GemmParams& p, int clusters, cudaStream_t stream)
{
    using C = Cfg2<KIND, BLOCK_N>;
    static bool configured[16] = {};
    int dev = 0;
    ASCB200_CUDA(cudaGetDevice(&dev));
    if (!configured[dev & 15]) {
        ASCB200_CUDA(cudaFuncSetAttribute(gemm_tc_pair_kernel<KIND, BLOCK_N, GROUPED, KMAJOR>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        configured[dev & 15] = true;
    }
    GemmParams q = p;
    if (KIND != KIND_MXF4 && !p.b_mn && !(getenv("ASCB200_NO_RING_CUT") && getenv("ASCB200_NO_RING_CUT")[0] == '1')) {
        // K-major B: a stage holds 128 rows of A and pair_n / 2 rows of B, so narrower tiles get the ring's bytes as more
        // stages (worth 1 to 2 % on a 160-column slab tile; what limits those tiles is the duration of a narrow MMA).
        q.ring_stage_bytes = A_TILE_BYTES + (p.pair_n / 2) * ROW_BYTES;
        q.ring_stages = std::min(kMaxRingStages, C::NUM_STAGES * C::STAGE_BYTES / q.ring_stage_bytes);
    }
    ASCB200_CUDA(launch_pdl(gemm_tc_pair_kernel<KIND, BLOCK_N, GROUPED, KMAJOR>, 2 * clusters, NUM_THREADS, C::SMEM_BYTES, stream, ta, tb, tsfa, tsfb, outs, q));
    return ASCB200_OK;
}
template <int KIND, int BLOCK_N>
int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsfa, const CUtensorMap& tsfb, const OutMaps& outs,
                     const GemmParams& p, int clusters, cudaStream_t stream)
{
    if constexpr (KIND == KIND_MXF4) {  // block-scaled operands reach the kernels K-major (transposed once before, if need be)
        return launch_gemm_pair_as<KIND, BLOCK_N, false, true>(ta, tb, tsfa, tsfb, outs, p, clusters, stream);
    } else {
        const bool kmajor = !p.a_mn && !p.b_mn;
        if constexpr (KIND == KIND_I8) {
            if (p.groups > 0)
                return kmajor ? launch_gemm_pair_as<KIND, BLOCK_N, true, true>(ta, tb, tsfa, tsfb, outs, p, clusters, stream)
                              : launch_gemm_pair_as<KIND, BLOCK_N, true, false>(ta, tb, tsfa, tsfb, outs, p, clusters, stream);
        }
        return kmajor ? launch_gemm_pair_as<KIND, BLOCK_N, false, true>(ta, tb, tsfa, tsfb, outs, p, clusters, stream)
                      : launch_gemm_pair_as<KIND, BLOCK_N, false, false>(ta, tb, tsfa, tsfb, outs, p, clusters, stream);
    }
}

// Split K over a cluster (single-CTA kernel): 4 or 2 CTAs per tile, or 0.  Time of a small problem ~ 5 us fixed + 0.21 us per K
// block of the longest CTA + 1.5 / 2.8 us for the exchange with 2 / 4 CTAs (fitted to fp16 512 x 512 x K: K = 1024, 16 blocks,
// 8.3 -> 8.6 / 9.1 us with 2 / 4 CTAs; K = 2048: 11.9 -> 10.4 / 10.2; K = 4096: 19.5 -> 14.5 / 12.5; and 128 x 1024 x 8192: 33.8 ->
// 21.7 / 15.7).  Every cluster needs a tile of its own, every CTA a K block, and the other CTAs' accumulators (block_n x 512 bytes
// each) must fit the leader's operand ring (about 192 KB).  `gain`: estimated time relative to no split.
int pick_split_k(long long tiles, int num_k_blocks, int block_n, int sm_count, double* gain = nullptr)
{
    const double fixed = 5.0, per_block = 0.21, exchange[5] = {0.0, 0.0, 1.5, 0.0, 2.8};
    const double base = fixed + per_block * num_k_blocks;
    int best = 0;
    double best_t = base;
    for (int sk = 2; sk <= 4; sk <<= 1) {
        if (tiles * sk > sm_count || num_k_blocks < 2 * sk) continue;
        if (static_cast<long long>(sk - 1) * block_n * 512 > 192 * 1024) continue;
        const double t = fixed + per_block * ((num_k_blocks + sk - 1) / sk) + exchange[sk];
        if (t < 0.97 * best_t) {
            best_t = t;
            best = sk;
        }
    }
    if (gain) *gain = best_t / base;
    return best;
}

bool is_mxfp8(int kind) { return kind == ASCB200_KIND_MXFP8_E4M3 || kind == ASCB200_KIND_MXFP8_E5M2; }
bool is_mx(int kind) { return kind == ASCB200_KIND_MXFP4 || is_mxfp8(kind); }
int elem_bits(int kind) { return kind == ASCB200_KIND_MXFP4 ? 4 : (kind == ASCB200_KIND_S8 || is_mxfp8(kind)) ? 8 : 16; }

// Device resources of one call when they do not come from the per-device state of ascb200_init.
struct FixedResources {
    uint32_t* status_dev;
    uint8_t* scale_scratch_dev;
    size_t scale_scratch_bytes;
    int sm_count;
    long long l2_bytes;  // 0: unknown, tiles keep the plain order
};

int run_gemm(const ascb200_gemm_desc* d, const int64_t* group_counts, int groups, cudaStream_t stream, const FixedResources* fixed = nullptr)
{
    DeviceState* st = fixed ? nullptr : current_state();
    if (!fixed && !st) return ASCB200_ENODEV;
    const int sm_count = fixed ? fixed->sm_count : st->sm_count;
    if (!d) return ASCB200_EINVAL;
    if (d->m < 0 || d->n < 0 || d->k < 0) return ASCB200_EINVAL;
    if (d->m == 0 || d->n == 0) return ASCB200_OK;
    if (!d->a_dev || !d->b_dev || !d->c_dev || d->k == 0) return ASCB200_EINVAL;
    if (d->reserved[0] != 0) return ASCB200_EINVAL;
    if (d->c_layout < ASCB200_C_ROW_MAJOR || d->c_layout > ASCB200_C_NZ) return ASCB200_EINVAL;
    if (d->c_layout != ASCB200_C_ROW_MAJOR && (d->atomic || d->c2_dev || groups > 0)) return ASCB200_EUNSUPPORTED;
    if (d->scale_flags & ~(ASCB200_SCALE_A_PREPACKED | ASCB200_SCALE_B_PREPACKED | ASCB200_SCALE_A_PAIRED | ASCB200_SCALE_B_PAIRED)) return ASCB200_EINVAL;
    const int kind = d->kind;
    if (kind < ASCB200_KIND_F16 || kind > ASCB200_KIND_MXFP8_E5M2) return ASCB200_EINVAL;
    const bool acc_int = kind == ASCB200_KIND_S8;
    const bool grouped = groups > 0;
    if (grouped && (groups > MAX_GROUPS)) return ASCB200_ETOOBIG;
    if (grouped && (!group_counts || kind != ASCB200_KIND_S8 || d->epilogue != ASCB200_EPI_DEQUANT_TOKEN_CHANNEL || d->trans_a)) return ASCB200_EUNSUPPORTED;

    // ---- epilogue validation ----
    EpiParams e = {};
    e.c = d->c_dev;
    e.layout = d->c_layout;
    e.ldc = d->ldc ? d->ldc : (d->c_layout == ASCB200_C_ROW_MAJOR ? d->n : d->m);
    e.c_dtype = d->c_dtype;
    e.mode = d->epilogue;
    e.relu = d->relu;
    e.act = d->act;
    e.bias = d->bias_dev;
    e.tok = d->tok_scale_dev;
    e.ch = d->ch_scale_dev;
    e.quant = reinterpret_cast<const unsigned long long*>(d->quant_dev);
    e.quant_scalar = d->quant_scalar;
    if (e.ldc < (e.layout == ASCB200_C_ROW_MAJOR ? d->n : d->m)) return ASCB200_EINVAL;
    switch (d->epilogue) {
        case ASCB200_EPI_CAST:
            if (acc_int ? d->c_dtype != OUT_S32 : !(d->c_dtype == OUT_F32 || d->c_dtype == OUT_F16 || d->c_dtype == OUT_BF16)) return ASCB200_EUNSUPPORTED;
            break;
        case ASCB200_EPI_FIXPIPE_QUANT:
            if (acc_int ? !(d->c_dtype == OUT_F16 || d->c_dtype == OUT_S8 || d->c_dtype == OUT_BF16)
                        : !(d->c_dtype == OUT_S8 || d->c_dtype == OUT_F16 || d->c_dtype == OUT_BF16 || d->c_dtype == OUT_F32 || d->c_dtype == OUT_E4M3 ||
                            d->c_dtype == OUT_E5M2))
                return ASCB200_EUNSUPPORTED;
            break;
        case ASCB200_EPI_DEQUANT_TOKEN_CHANNEL:
            if (!acc_int || !d->ch_scale_dev) return ASCB200_EINVAL;
            if (!(d->c_dtype == OUT_F32 || d->c_dtype == OUT_F16 || d->c_dtype == OUT_BF16)) return ASCB200_EUNSUPPORTED;
            break;
        default: return ASCB200_EINVAL;
    }
    if (d->act != 0 && !(d->act == 1 && d->epilogue == ASCB200_EPI_DEQUANT_TOKEN_CHANNEL)) return ASCB200_EUNSUPPORTED;
    if (d->c2_dev) {
        if (acc_int || !(d->c2_dtype == OUT_F32 || d->c2_dtype == OUT_F16 || d->c2_dtype == OUT_BF16)) return ASCB200_EUNSUPPORTED;
        e.c2 = d->c2_dev;
        e.ldc2 = d->ldc2 ? d->ldc2 : d->n;
        e.c2_dtype = d->c2_dtype;
        if (e.ldc2 < d->n) return ASCB200_EINVAL;
        e.vec_c2 = aligned_to(e.c2, 16) && (e.ldc2 * out_bytes(e.c2_dtype)) % 16 == 0;
    }
    e.vec_c = aligned_to(e.c, 16) && (e.ldc * out_bytes(e.c_dtype)) % 16 == 0;
    // 1- and 2-byte outputs leave through shared memory and bulk tensor stores when their layout allows a tensor map
    OutMaps outs;
    std::memset(&outs, 0, sizeof(outs));
    const bool no_tma_store = getenv("ASCB200_NO_TMA_STORE") && getenv("ASCB200_NO_TMA_STORE")[0] == '1';
    e.tma_c = !no_tma_store && e.layout == ASCB200_C_ROW_MAJOR && make_out_map(&outs.c, e.c_dtype, e.c, d->n, d->m, e.ldc);
    e.tma_c2 = !no_tma_store && e.c2 && make_out_map(&outs.c2, e.c2_dtype, e.c2, d->n, d->m, e.ldc2);
    e.atomic = d->atomic;
    if (d->atomic < 0 || d->atomic > 3) return ASCB200_EUNSUPPORTED;                         // enAtomic: 0 off, 1 add, 2 max, 3 min
    if (d->atomic && out_bytes(e.c_dtype) == 1) return ASCB200_EUNSUPPORTED;                 // no 8-bit atomics
    if (d->atomic && out_bytes(e.c_dtype) == 2 && (reinterpret_cast<uintptr_t>(e.c) & 1)) return ASCB200_EALIGN;

    // ---- operands ----
    const int bits = elem_bits(kind);
    const int k = d->k, m = d->m, n = d->n;
    if (is_mx(kind)) {
        // K a multiple of 64 like the reference's MmadMx
        if (k % 64 != 0) return ASCB200_EINVAL;
        if (!d->scale_a_dev || !d->scale_b_dev) return ASCB200_EINVAL;
    }
    if (kind == ASCB200_KIND_MXFP4) {
        if (d->trans_a || !d->trans_b) {
            // The tensor core takes fp4 operands K-major only.  An operand stored the other way round ([K, M] / the reference's
            // ND [K, N], two M- / N-neighbours per byte) is transposed into this stream's scratch first, then the call
            // proceeds on the copies; the scale scratch follows them in the same block.
            if (fixed) return ASCB200_EUNSUPPORTED;   // the allocation-free entry point has no room for operand copies
            if ((d->trans_a && ((m & 1) || (d->lda && d->lda != m))) || (!d->trans_b && ((n & 1) || (d->ldb && d->ldb != n)))) return ASCB200_EUNSUPPORTED;
            auto round256 = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
            const size_t bytes_ta = d->trans_a ? round256(static_cast<size_t>(m) * k / 2) : 0;
            const size_t bytes_tb = !d->trans_b ? round256(static_cast<size_t>(n) * k / 2) : 0;
            const size_t kc2 = 2 * static_cast<size_t>((k + 255) / 256);
            const size_t bytes_sf = (static_cast<size_t>((m + 127) / 128) + (n + 127) / 128 + kSfPadBlocks) * kc2 * SF_CHUNK_BYTES;
            void* ptr = nullptr;
            int rc0 = stream_scratch(st, bytes_ta + bytes_tb + bytes_sf, stream, &ptr);
            if (rc0 != ASCB200_OK) return rc0;
            uint8_t* base = static_cast<uint8_t*>(ptr);
            ascb200_gemm_desc d2 = *d;
            if (d->trans_a) {
                rc0 = fp4_transpose(d->a_dev, base, k, m, stream);
                if (rc0 != ASCB200_OK) return rc0;
                d2.a_dev = base;
                d2.trans_a = 0;
                d2.lda = 0;
            }
            if (!d->trans_b) {
                rc0 = fp4_transpose(d->b_dev, base + bytes_ta, k, n, stream);
                if (rc0 != ASCB200_OK) return rc0;
                d2.b_dev = base + bytes_ta;
                d2.trans_b = 1;
                d2.ldb = 0;
            }
            FixedResources sub = {st->status_dev, base + bytes_ta + bytes_tb, bytes_sf, st->sm_count, st->l2_bytes};
            return run_gemm(&d2, nullptr, 0, stream, &sub);
        }
    }
    const int64_t lda = d->lda ? d->lda : (d->trans_a ? m : k);
    const int64_t ldb = d->ldb ? d->ldb : (d->trans_b ? k : n);
    const int esz = bits == 16 ? 2 : 1;                // bytes per tensor-map element
    const int epb = bits == 4 ? 2 : 1;                 // logical elements per tensor-map element
    const CUtensorMapDataType dt = kind == ASCB200_KIND_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : kind == ASCB200_KIND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const uint32_t row_elems = ROW_BYTES / esz;        // tensor-map elements per 128-byte row
    const int block_k = bits == 16 ? 64 : bits == 8 ? 128 : 256;

    // Tile choice: estimated time = waves x tile work / efficiency of that tile shape (wider tiles read less shared
    // memory and L2 per MAC; measured on 4096 x 4096 x 11008 int8: pair 256x256 1.0, single 128x256 0.88, 128x128 0.75,
    // 128x64 0.5).  Small problems and thin N-slabs get narrower tiles so that the last wave is not mostly idle.
    const int pair_clusters = sm_count / 2;
    const bool pair_possible = !(getenv("ASCB200_NO_PAIR") && getenv("ASCB200_NO_PAIR")[0] == '1');
    // Grouped problems on CTA pairs: full 256-row blocks of a group run like a plain GEMM; the group's last, partial block
    // is multiplied with the operand roles swapped (the pair's 256 weight rows become the M side of the instruction, the
    // block's rows, rounded up to 16, its N side), so that at most 15 rows per group are multiplied in vain.  Without the
    // swap a group's last 256-row tile is half empty on average, and under the board's power cap the wasted MMAs cost as
    // much time as useful ones (64 groups of 512 rows on average: masked pairs 490 us, single-CTA tiles 406-475 us).
    const bool group_swap_ok = grouped && !(getenv("ASCB200_NO_GROUP_SWAP") && getenv("ASCB200_NO_GROUP_SWAP")[0] == '1');
    const bool pair_allowed = pair_possible && (!grouped || group_swap_ok || m / groups >= 16 * BLOCK_M);
    const int wide = is_mx(kind) ? 192 : 256;   // block-scaled kinds at 256 columns cannot double-buffer their accumulators in TMEM
    int block_n = 64;
    bool use_pair = false;
    {
        const long long m_tiles = grouped ? (m + BLOCK_M - 1) / BLOCK_M + groups : (m + BLOCK_M - 1) / BLOCK_M;
        double best = -1.0;
        struct Cand { int bn; bool pair; double eff; };
        Cand cands[20];
        int num_cands = 0;
        cands[num_cands++] = {wide, true, 1.0};
        if (!is_mx(kind) && d->trans_b && !(grouped && group_swap_ok)) {
            // CTA-pair tiles of any width that is a multiple of 16: a narrower tile re-reads A more often per column
            // (128 columns measured at 0.75 of the full width's rate), but may fill the last wave far better
            for (int bn = 240; bn >= 64; bn -= 16) cands[num_cands++] = {bn, true, 1.0 / (1.0 + 0.33 * (256.0 / bn - 1.0))};
        }
        cands[num_cands++] = {wide, false, 0.88};
        cands[num_cands++] = {128, false, 0.75};
        cands[num_cands++] = {64, false, 0.5};
        for (int ci = 0; ci < num_cands; ++ci) {
            const Cand& c = cands[ci];
            if (c.pair && !pair_allowed) continue;
            if (c.bn == 64 && is_mx(kind)) continue;                                         // scale blocks span 128 rows
            if (c.pair && is_mxfp8(kind)) continue;                                          // block-scaled fp8 runs on single CTAs
            if (c.bn == 64 && !c.pair && kind == ASCB200_KIND_S8 && !d->trans_b) continue;   // N-contiguous int8 B comes in boxes of 128 columns
            if (c.bn > 64 && n <= c.bn / 2 && (c.pair || c.bn != 128)) continue;             // do not pad N by more than 2x
            const long long n_tiles = (n + c.bn - 1) / c.bn;
            // grouped: the host does not see the counts; a group ends on average half a tile past its last full one
            // (a swapped block costs its share of rows: half a tile on average, like the masked tail it replaces costs in tiles)
            const long long pair_m_tiles = grouped ? (m + 2 * BLOCK_M - 1) / (2 * BLOCK_M) + (groups + 1) / 2 : (m + 2 * BLOCK_M - 1) / (2 * BLOCK_M);
            const long long tiles = c.pair ? pair_m_tiles * n_tiles : m_tiles * n_tiles;
            const long long slots = c.pair ? pair_clusters : sm_count;
            const long long waves = (tiles + slots - 1) / slots;
            double cost = static_cast<double>(waves) * (c.pair ? 2 : 1) * BLOCK_M * c.bn / c.eff / (c.pair ? 2 : 1);
            if (!c.pair && !grouped && !fixed) {  // single-CTA tiles may split K over a cluster (measured speed-ups, see pick_split_k)
                double gain = 1.0;
                pick_split_k(tiles, (k + block_k - 1) / block_k, c.bn, sm_count, &gain);
                cost *= gain;
            }
            if (best < 0 || cost < best) {
                best = cost;
                block_n = c.bn;
                use_pair = c.pair;
            }
        }
    }
    if (const char* force = getenv("ASCB200_PAIR_N")) {
        // testing / tuning override: CTA-pair kernel with this tile width where the kernel supports it
        const int bn = atoi(force);
        if (pair_possible && !is_mx(kind) && (d->trans_b || bn == 256) && bn >= 16 && bn <= 256 && bn % 16 == 0) {
            block_n = bn;
            use_pair = true;
        }
    }
    const long long pair_tiles = (static_cast<long long>((m + 2 * BLOCK_M - 1) / (2 * BLOCK_M)) + (grouped ? groups : 0)) * ((n + block_n - 1) / block_n);

    const int b_box_rows = use_pair ? block_n / 2 : block_n;

    CUtensorMap ta, tb;
    int rc;
    if (!d->trans_a) rc = make_map(&ta, dt, esz, d->a_dev, k / epb, m, 1, lda / epb, static_cast<uint64_t>(lda / epb) * m, row_elems, BLOCK_M);
    else rc = make_map(&ta, dt, esz, d->a_dev, m, k, 1, lda, static_cast<uint64_t>(lda) * k, row_elems, block_k);
    if (rc != ASCB200_OK) return rc;
    const uint64_t g3 = grouped ? groups : 1;
    if (d->trans_b) rc = make_map(&tb, dt, esz, d->b_dev, k / epb, n, g3, ldb / epb, static_cast<uint64_t>(ldb / epb) * n, row_elems, b_box_rows);
    else rc = make_map(&tb, dt, esz, d->b_dev, n, k, g3, ldb, static_cast<uint64_t>(ldb) * k, row_elems, block_k);
    if (rc != ASCB200_OK) return rc;

    GemmParams p = {};
    p.m = m;
    p.n = n;
    p.k = k;
    p.num_k_blocks = (k + block_k - 1) / block_k;
    p.a_mn = d->trans_a ? 1 : 0;
    p.b_mn = d->trans_b ? 0 : 1;
    p.groups = grouped ? groups : 0;
    p.pair_n = block_n;
    p.allow_m64 = !is_mx(kind) && !(getenv("ASCB200_NO_M64") && getenv("ASCB200_NO_M64")[0] == '1');
    // Banded tile order once A alone takes more than half of L2 (measured in the sustained loop: fp16 8192^3, A = 128 MB, 9 %
    // faster; with operands that fit L2 the plain order was 2 to 4 % faster).
    const long long a_bytes = static_cast<long long>(d->m) * d->k * elem_bits(kind) / 8;
    const long long l2_bytes = fixed ? fixed->l2_bytes : st->l2_bytes;
    p.band_m = (!grouped && l2_bytes > 0 && a_bytes > l2_bytes / 2) ? 8 : 0;
    if (const char* band = getenv("ASCB200_BAND_M")) p.band_m = atoi(band);
    p.group_swap = (grouped && use_pair && block_n == 256 && group_swap_ok) ? 1 : 0;
    p.group_counts = reinterpret_cast<const long long*>(group_counts);
    p.status = fixed ? fixed->status_dev : st->status_dev;
    p.epi = e;

    if (is_mx(kind)) {
        // Scale factors in the 512-byte chunk order the kernels copy into TMEM (layout documented at retile_scales_kernel):
        // taken as they are when the caller prepacked them (ascb200_mx_scale_prepack: static weights), else re-tiled here
        // into scratch that belongs to `stream`, so that calls on different streams do not overwrite each other's scales.
        const int ks = k / 32;
        const int kc = 2 * ((k + 255) / 256);   // chunks (4 scales each) per 128-row block: the same pitch for every MX kind and for prepacked tensors
        const bool pre_a = (d->scale_flags & ASCB200_SCALE_A_PREPACKED) != 0, pre_b = (d->scale_flags & ASCB200_SCALE_B_PREPACKED) != 0;
        const int rba = (m + 127) / 128, rbb = (n + 127) / 128 + kSfPadBlocks;  // B tiles may read up to two blocks past the last row
        const size_t bytes_a = pre_a ? 0 : static_cast<size_t>(rba) * kc * SF_CHUNK_BYTES, bytes_b = pre_b ? 0 : static_cast<size_t>(rbb) * kc * SF_CHUNK_BYTES;
        uint8_t* scratch = nullptr;
        if (bytes_a + bytes_b > 0) {
            if (fixed) {
                if (bytes_a + bytes_b > fixed->scale_scratch_bytes) return ASCB200_ETOOBIG;
                scratch = fixed->scale_scratch_dev;
            } else {
                void* ptr = nullptr;
                rc = stream_scratch(st, bytes_a + bytes_b, stream, &ptr);
                if (rc != ASCB200_OK) return rc;
                scratch = static_cast<uint8_t*>(ptr);
            }
        }
        const uint8_t* sfa = pre_a ? static_cast<const uint8_t*>(d->scale_a_dev) : scratch;
        const uint8_t* sfb = pre_b ? static_cast<const uint8_t*>(d->scale_b_dev) : scratch + bytes_a;
        if (!aligned_to(sfa, 16) || !aligned_to(sfb, 16)) return ASCB200_EALIGN;
        if (scratch) {
            const int kc_tiles = (kc + 7) / 8;
            const int blocks_a = pre_a ? 0 : rba * kc_tiles, blocks_b = pre_b ? 0 : rbb * kc_tiles;
            ASCB200_CUDA(launch_pdl(retile_scales_kernel, dim3(blocks_a + blocks_b), dim3(256), 0, stream, static_cast<const uint8_t*>(d->scale_a_dev),
                                    reinterpret_cast<uint32_t*>(scratch), m, pre_a ? 0 : rba, static_cast<const uint8_t*>(d->scale_b_dev),
                                    reinterpret_cast<uint32_t*>(scratch + bytes_a), n, ks, kc, kc_tiles,
                                    ((d->scale_flags & ASCB200_SCALE_A_PAIRED) ? 1 : 0) | ((d->scale_flags & ASCB200_SCALE_B_PAIRED) ? 2 : 0)));
        }
        p.sfa = sfa;
        p.sfb = sfb;
        p.sf_kc = kc;
    }

    const long long max_tiles = grouped ? (static_cast<long long>((m + BLOCK_M - 1) / BLOCK_M) + groups) * ((n + block_n - 1) / block_n)
                                        : static_cast<long long>((m + BLOCK_M - 1) / BLOCK_M) * ((n + block_n - 1) / block_n);
    const int grid = static_cast<int>(std::min<long long>(max_tiles, sm_count));
    // Few tiles and a long K: clusters of 2 or 4 CTAs share each tile and split its K blocks (a K block cannot take less than
    // about 370 cycles whatever the tile's width, so a small problem's time is its number of K blocks); the leader adds the
    // others' accumulators in rank order.  Never for grouped calls or calls that bring their own device resources.
    if (!use_pair && !grouped && !fixed) {
        int sk = pick_split_k(max_tiles, p.num_k_blocks, block_n, sm_count);
        if (const char* force = getenv("ASCB200_SPLIT_K")) {
            const int v = atoi(force);
            sk = (v == 2 || v == 4 || v == 8) && max_tiles * v <= sm_count ? v : 0;
        }
        p.split_k = sk;
    }

    const uint32_t a_mn = p.a_mn, b_mn = p.b_mn;
    if (use_pair) {
        const int clusters = static_cast<int>(std::min<long long>(pair_tiles, pair_clusters));
        if (kind == ASCB200_KIND_MXFP4) {
            // the re-tiled scales as rank-2 tensors [chunk][128 x u32] for tile loads
            CUtensorMap tsfa, tsfb;
            rc = make_sf_map(&tsfa, p.sfa, static_cast<uint64_t>((m + 127) / 128) * p.sf_kc, 2);
            if (rc == ASCB200_OK) rc = make_sf_map(&tsfb, p.sfb, static_cast<uint64_t>((n + 127) / 128 + kSfPadBlocks) * p.sf_kc, 2);
            if (rc != ASCB200_OK) return rc;
            p.idesc = make_idesc_mxf4(2 * BLOCK_M, 192);
            return launch_gemm_pair<KIND_MXF4, 192>(ta, tb, tsfa, tsfb, outs, p, clusters, stream);
        }
        if (kind == ASCB200_KIND_S8) {
            p.idesc = make_idesc(2, 1, 1, a_mn, b_mn, 2 * BLOCK_M, block_n);
            CUtensorMap tx32 = ta;
            if (p.group_swap) {
                // the weights as the 256-row operand, rows of A as the narrow one (its N field is filled in per block);
                // A once more with boxes of 32 rows, for blocks that hold fewer than 97 rows per CTA
                p.idesc_swap = make_idesc(2, 1, 1, b_mn, a_mn, 2 * BLOCK_M, 0);
                rc = make_map(&tx32, dt, esz, d->a_dev, k, m, 1, lda, static_cast<uint64_t>(lda) * m, row_elems, 32);
                if (rc != ASCB200_OK) return rc;
            }
            return launch_gemm_pair<KIND_I8, 256>(ta, tb, tx32, tb, outs, p, clusters, stream);
        }
        const uint32_t fmt = kind == ASCB200_KIND_BF16 ? 1u : 0u;
        p.idesc = make_idesc(1, fmt, fmt, a_mn, b_mn, 2 * BLOCK_M, block_n);
        return launch_gemm_pair<KIND_F16, 256>(ta, tb, ta, tb, outs, p, clusters, stream);
    }
    if (is_mxfp8(kind)) {
        const uint32_t fmt = kind == ASCB200_KIND_MXFP8_E5M2 ? 1u : 0u;
        p.idesc = make_idesc_mxf8(fmt, fmt, a_mn, b_mn, BLOCK_M, block_n);
        if (block_n == 256) return launch_gemm<KIND_MXF8, 256>(ta, tb, outs, p, grid, stream);
        if (block_n == 192) return launch_gemm<KIND_MXF8, 192>(ta, tb, outs, p, grid, stream);
        return launch_gemm<KIND_MXF8, 128>(ta, tb, outs, p, grid, stream);
    }
    switch (kind) {
        case ASCB200_KIND_F16:
        case ASCB200_KIND_BF16: {
            const uint32_t fmt = kind == ASCB200_KIND_BF16 ? 1u : 0u;
            p.idesc = make_idesc(1, fmt, fmt, a_mn, b_mn, BLOCK_M, block_n);
            if (block_n == 256) return launch_gemm<KIND_F16, 256>(ta, tb, outs, p, grid, stream);
            if (block_n == 128) return launch_gemm<KIND_F16, 128>(ta, tb, outs, p, grid, stream);
            return launch_gemm<KIND_F16, 64>(ta, tb, outs, p, grid, stream);
        }
        case ASCB200_KIND_S8:
            p.idesc = make_idesc(2, 1, 1, a_mn, b_mn, BLOCK_M, block_n);
            if (block_n == 256) return launch_gemm<KIND_I8, 256>(ta, tb, outs, p, grid, stream);
            if (block_n == 128) return launch_gemm<KIND_I8, 128>(ta, tb, outs, p, grid, stream);
            return launch_gemm<KIND_I8, 64>(ta, tb, outs, p, grid, stream);
        default:
            p.idesc = make_idesc_mxf4(BLOCK_M, block_n);
            if (block_n == 256) return launch_gemm<KIND_MXF4, 256>(ta, tb, outs, p, grid, stream);
            if (block_n == 192) return launch_gemm<KIND_MXF4, 192>(ta, tb, outs, p, grid, stream);
            return launch_gemm<KIND_MXF4, 128>(ta, tb, outs, p, grid, stream);
    }
}

// ---- allocation-free MXFP4 variant ------------------------------------------------------------------
// Scratch of ascb200_gemm_mxfp4_noalloc: 256 bytes for the status word of the bounded waits, then the
// re-tiled scale factors.  The array lives in the library image: every GPU that loads the library
// holds these bytes until the process exits.
constexpr size_t NOALLOC_HEAD_BYTES = 256;
constexpr size_t NOALLOC_SCALE_BYTES = ASCB200_NOALLOC_MAX_SCALE_BYTES;
static __device__ __align__(256) uint8_t g_noalloc_scratch[NOALLOC_HEAD_BYTES + NOALLOC_SCALE_BYTES];

struct NoAllocDevice {
    bool ready = false;
    uint8_t* base = nullptr;  // device address of g_noalloc_scratch on this device
    int sm_count = 0;
};
NoAllocDevice g_noalloc_dev[16];
std::mutex g_noalloc_mu;

// Once per device, with that device current: resolve the device address of the array.  In host code
// the symbol itself is only a stand-in and must never be handed to a kernel.
int noalloc_setup(NoAllocDevice** out)
{
    int dev = -1;
    ASCB200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16) return ASCB200_EINVAL;
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    NoAllocDevice* nd = &g_noalloc_dev[dev];
    if (!nd->ready) {
        int major = 0, sms = 0;
        ASCB200_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        if (major != 10) return ASCB200_ENODEV;
        ASCB200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        void* ptr = nullptr;
        ASCB200_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        if (!ptr) return ASCB200_ECUDA;
        nd->base = static_cast<uint8_t*>(ptr);
        nd->sm_count = sms;
        nd->ready = true;
    }
    *out = nd;
    return ASCB200_OK;
}

int run_gemm_mxfp4_noalloc(const ascb200_gemm_desc* d, cudaStream_t stream)
{
    if (!d) return ASCB200_EINVAL;
    if (d->kind != ASCB200_KIND_MXFP4) return ASCB200_EUNSUPPORTED;
    NoAllocDevice* nd = nullptr;
    int rc = noalloc_setup(&nd);
    if (rc != ASCB200_OK) return rc;
    FixedResources fixed;
    fixed.status_dev = reinterpret_cast<uint32_t*>(nd->base);
    fixed.scale_scratch_dev = nd->base + NOALLOC_HEAD_BYTES;
    fixed.scale_scratch_bytes = NOALLOC_SCALE_BYTES;
    fixed.sm_count = nd->sm_count;
    fixed.l2_bytes = 0;
    // The array keeps whatever the previous call left.  Nothing in it has to start at zero: the re-tiling kernel rewrites
    // every scale byte the GEMM reads, and the status word is a latch (zero when the library image is loaded, set by an
    // expired wait, read and cleared by ascb200_noalloc_status).
    return run_gemm(d, nullptr, 0, stream, &fixed);
}

int noalloc_status(cudaStream_t stream, uint32_t* status_host)
{
    NoAllocDevice* nd = nullptr;
    int rc = noalloc_setup(&nd);
    if (rc != ASCB200_OK) return rc;
    uint32_t v = 0;
    ASCB200_CUDA(cudaMemcpyAsync(&v, nd->base, sizeof(v), cudaMemcpyDeviceToHost, stream));
    ASCB200_CUDA(cudaStreamSynchronize(stream));
    if (status_host) *status_host = v;
    if (v != 0) {
        ASCB200_CUDA(cudaMemsetAsync(nd->base, 0, sizeof(v), stream));
        return ASCB200_ETIMEOUT;
    }
    return ASCB200_OK;
}

// Re-tiles one scale tensor [rows, k / 32] into the chunk order of the kernels, padding blocks included.
int mx_scale_prepack(const void* scale_dev, int rows, int k, int paired, void* out_dev, size_t out_bytes, cudaStream_t stream)
{
    if (!scale_dev || !out_dev || rows <= 0 || k <= 0 || k % 64 != 0) return ASCB200_EINVAL;
    if (!aligned_to(out_dev, 16)) return ASCB200_EALIGN;
    const int block_k = 256;
    const int kc = 2 * ((k + block_k - 1) / block_k);
    const int rb = (rows + 127) / 128 + kSfPadBlocks;
    if (out_bytes < static_cast<size_t>(rb) * kc * SF_CHUNK_BYTES) return ASCB200_EINVAL;
    const int kc_tiles = (kc + 7) / 8;
    ASCB200_CUDA(launch_pdl(retile_scales_kernel, dim3(rb * kc_tiles), dim3(256), 0, stream, static_cast<const uint8_t*>(scale_dev),
                            static_cast<uint32_t*>(out_dev), rows, rb, static_cast<const uint8_t*>(nullptr), static_cast<uint32_t*>(nullptr), 0, k / 32,
                            kc, kc_tiles, paired ? 1 : 0));
    return ASCB200_OK;
}

}  // namespace
}  // namespace ascb200

extern "C" {

int ascb200_noalloc_status(void* stream, uint32_t* status_host) { return ascb200::noalloc_status(static_cast<cudaStream_t>(stream), status_host); }

size_t ascb200_mx_scale_prepacked_bytes(int32_t rows, int32_t k)
{
    if (rows <= 0 || k <= 0) return 0;
    return static_cast<size_t>((rows + 127) / 128 + ascb200::kSfPadBlocks) * (2 * ((k + 255) / 256)) * ascb200::SF_CHUNK_BYTES;
}

int ascb200_mx_scale_prepack(const void* scale_dev, int32_t rows, int32_t k, int32_t paired, void* out_dev, size_t out_bytes, void* stream)
{
    if (!ascb200::current_state()) return ASCB200_ENODEV;
    return ascb200::mx_scale_prepack(scale_dev, rows, k, paired, out_dev, out_bytes, static_cast<cudaStream_t>(stream));
}

int ascb200_gemm_mxfp4_noalloc(const ascb200_gemm_desc* desc, void* stream)
{
    return ascb200::run_gemm_mxfp4_noalloc(desc, static_cast<cudaStream_t>(stream));
}

int ascb200_gemm(const ascb200_gemm_desc* desc, void* stream)
{
    return ascb200::run_gemm(desc, nullptr, 0, static_cast<cudaStream_t>(stream));
}

int ascb200_grouped_gemm(const ascb200_gemm_desc* desc, const int64_t* group_counts_dev, int32_t groups, void* stream)
{
    if (groups <= 0) return groups == 0 ? ASCB200_OK : ASCB200_EINVAL;
    return ascb200::run_gemm(desc, group_counts_dev, groups, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

