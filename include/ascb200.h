/*
 * ascb200 - C ABI of the B200 (sm_100a) implementation of the Ascend C high-level operator hot
 * path: adv_api Matmul (IterateAll + fixpipe quant/dequant epilogue), grouped quantized matmul,
 * SoftMax, AscendQuant, AscendDequant.
 *
 * The reference is a header-only C++ template library instantiated inside the user's NPU kernel;
 * it has no FFI of its own.  This header is the boundary a port binds instead: each entry point
 * names the reference interface it replaces (paths relative to the reference project).  The C++
 * mirror of the reference classes (AscendC::Matmul<>, AscendC::SoftMax, ...) in
 * asc-devkit_clone_b200/hostapi calls only these functions.
 *
 * Conventions
 *  - every pointer named *_dev is CUDA device memory owned by the caller; the library never frees it;
 *  - `stream` is a cudaStream_t passed as void* (NULL = the default stream); calls are asynchronous;
 *  - return value: 0 on success, a negative ASCB200_E* code otherwise; nothing throws, aborts or traps;
 *  - there is no CPU fallback: without a usable sm_100 device every compute call returns ASCB200_ENODEV.
 */
#ifndef ASCB200_H
#define ASCB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ASCB200_API __attribute__((visibility("default")))

/* ---- error codes ------------------------------------------------------------------------- */
enum {
    ASCB200_OK = 0,
    ASCB200_EINVAL = -1,      /* bad argument (null pointer, non-positive extent, unknown enum)   */
    ASCB200_EALIGN = -2,      /* pointer or leading dimension violates an alignment rule          */
    ASCB200_EUNSUPPORTED = -3,/* valid in the reference, not implemented here                     */
    ASCB200_ENODEV = -4,      /* no CUDA device of compute capability 10.x                        */
    ASCB200_ECUDA = -5,       /* a CUDA runtime / driver call failed (see ascb200_last_cuda_error) */
    ASCB200_ETIMEOUT = -6,    /* a device-side bounded wait expired (reported by ascb200_device_status) */
    ASCB200_ETOOBIG = -7      /* extent beyond a documented limit                                 */
};

/* ---- element types ----------------------------------------------------------------------- */
enum {
    ASCB200_F32 = 0,
    ASCB200_F16 = 1,
    ASCB200_BF16 = 2,
    ASCB200_S8 = 3,
    ASCB200_S32 = 4,
    ASCB200_FP4_E2M1 = 5,     /* two values per byte, even index in the low nibble */
    ASCB200_FP8_E4M3 = 6,     /* e4m3fn: no infinities, largest finite 448 (output of the QF322FP8_PRE fixpipe mode) */
    ASCB200_FP8_E5M2 = 7      /* e5m2: largest finite 57344 */
};

/* ---- library / device ---------------------------------------------------------------------- */

/* Selects `device`, checks it is sm_100, creates the per-device state (status word, scratch).
 * Replaces the examples' aclInit/aclrtSetDevice
 * (examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul/matmul.asc:212-217). */
ASCB200_API int ascb200_init(int device);
ASCB200_API const char* ascb200_strerror(int code);
/* cudaError_t of the most recent failing CUDA call on this thread (0 if none). */
ASCB200_API int ascb200_last_cuda_error(void);
/* Copies the device status word to *status_host (synchronises `stream`). Bit 0: a bounded wait
 * inside a GEMM kernel expired. Non-zero status makes the call return ASCB200_ETIMEOUT and clears it. */
ASCB200_API int ascb200_device_status(void* stream, uint32_t* status_host);
ASCB200_API int ascb200_sm_count(void);
/* Self-test of the bounded waits (the failure-detection path of the GEMM kernels: every mbarrier wait gives up after a time
 * limit, sets the status bit and lets the kernel return normally).  Launches a one-CTA kernel that waits, with the kernels'
 * own wait routine and a limit of about 0.1 ms, on a barrier that nothing completes.  Nothing hangs or traps.  On return
 * result_host3 = {1 if the wait was abandoned, 1 if the CTA-wide abort word was set, cycles waited / 1024}, and the device
 * status word has bit 0 set: the next ascb200_device_status returns ASCB200_ETIMEOUT and clears it. */
ASCB200_API int ascb200_selftest_bounded_wait(uint32_t* result_host3, void* stream);

/* Memory and stream shims for aclrtMalloc / aclrtMallocHost / aclrtMemcpy(Async) /
 * aclrtSynchronizeStream as used by the examples (matmul.asc:219-260). */
ASCB200_API int ascb200_malloc(void** dev_ptr, size_t bytes);
ASCB200_API int ascb200_free(void* dev_ptr);
ASCB200_API int ascb200_malloc_host(void** host_ptr, size_t bytes);     /* pinned */
ASCB200_API int ascb200_free_host(void* host_ptr);
ASCB200_API int ascb200_memcpy_h2d(void* dst_dev, const void* src_host, size_t bytes, void* stream);
ASCB200_API int ascb200_memcpy_d2h(void* dst_host, const void* src_dev, size_t bytes, void* stream);
ASCB200_API int ascb200_memset(void* dst_dev, int value, size_t bytes, void* stream);
ASCB200_API int ascb200_stream_create(void** stream);
ASCB200_API int ascb200_stream_destroy(void* stream);
ASCB200_API int ascb200_stream_sync(void* stream);
/* Timing helpers (CUDA events on `stream`) so that C hosts can measure without the runtime API. */
ASCB200_API int ascb200_event_create(void** event);
ASCB200_API int ascb200_event_destroy(void* event);
ASCB200_API int ascb200_event_record(void* event, void* stream);
ASCB200_API int ascb200_stream_wait_event(void* stream, void* event);          /* later work on stream waits for event */
ASCB200_API int ascb200_event_elapsed_ms(void* start, void* stop, float* ms); /* synchronises on stop */

/* CUDA-graph shims: record the calls issued on `stream` between begin and end into one graph and
 * replay it with a single launch.  For launch-bound sequences of small operators (the role the
 * reference gives to a single kernel that calls several adv_api operators back to back).  A call
 * that may allocate (the first MXFP4 ascb200_gemm of a larger size on that stream) must be made once before capture. */
ASCB200_API int ascb200_graph_begin(void* stream);
ASCB200_API int ascb200_graph_end(void* stream, void** graph_exec);
ASCB200_API int ascb200_graph_launch(void* graph_exec, void* stream);
ASCB200_API int ascb200_graph_destroy(void* graph_exec);

/* ---- Matmul ---------------------------------------------------------------------------------- */

/* Output stage applied to the accumulator tile, the job of Fixpipe in the reference
 * (impl/adv_api/detail/matmul/stage/copy_cube_out/copy_cube_out_fixpipe.h:339-358). */
enum {
    /* cast only: fp32 acc -> F32 / F16 / BF16 (RINT, F322F16 / F322BF16); int32 acc -> S32 */
    ASCB200_EPI_CAST = 0,
    /* quantising fixpipe modes selected by (accumulator, c_dtype), parameter = `quant`:
     *   int32 -> F16 (V)DEQF16, int32 -> S8 (V)REQ8, int32 -> BF16 (V)QS322BF16_PRE,
     *   fp32 -> S8 (V)QF322B8_PRE, fp32 -> F16/BF16/F32 (V)QF322{F16,BF16,F32}_PRE
     * (impl/adv_api/detail/matmul/stage/copy_cube_out/quant/quant_processor_fixpipe.h:89-116,209-236) */
    ASCB200_EPI_FIXPIPE_QUANT = 1,
    /* int32 acc -> (float(acc) * ch_scale[n]) * tok_scale[m] -> F32 / F16 / BF16: AscendDequant + Mul + Cast
     * of the grouped example (quant_group_matmul_custom.asc:433-450); optional FasterGelu (act = 1) */
    ASCB200_EPI_DEQUANT_TOKEN_CHANNEL = 2
};

enum { ASCB200_KIND_F16 = 0, ASCB200_KIND_BF16 = 1, ASCB200_KIND_S8 = 2, ASCB200_KIND_MXFP4 = 3,
       /* MX Matmul with fp8 operands (one byte per element, e4m3fn or e5m2) and e8m0 block scales, the other operand kinds of
        * MmadMx (docs/zh/api/SIMD-API/basic_api/cube_compute_ISASI/mmad_compute/MmadMx.md:160-171; example
        * examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul_mx): tcgen05.mma.kind::mxf8f6f4.block_scale.  Either operand
        * may be stored K-major or the other way round (trans_a / trans_b as for int8); scales and scale_flags as for MXFP4. */
       ASCB200_KIND_MXFP8_E4M3 = 4, ASCB200_KIND_MXFP8_E5M2 = 5 };

typedef struct ascb200_gemm_desc {
    int32_t kind;            /* ASCB200_KIND_*: operand type; accumulator is fp32 (F16/BF16/MXFP4/MXFP8) or int32 (S8) */
    int32_t m, n, k;         /* C[m,n] = A[m,k] * B[k,n]; k counts elements (fp4 values for MXFP4) */
    const void* a_dev;       /* trans_a == 0: [m,k] row-major (ND); trans_a == 1: [k,m] row-major */
    const void* b_dev;       /* trans_b == 0: [k,n] row-major (ND); trans_b == 1: [n,k] row-major */
    int64_t lda, ldb;        /* leading dimensions in elements (0 = packed) */
    int32_t trans_a, trans_b;
    const void* scale_a_dev; /* MXFP4 / MXFP8: e8m0 bytes [m, k/32] row-major (or see scale_flags) */
    const void* scale_b_dev; /* MXFP4 / MXFP8: e8m0 bytes [n, k/32] row-major (or see scale_flags) */
    const void* bias_dev;    /* NULL or [n]: fp32 for fp32 accumulators, int32 for int32 accumulators */
    void* c_dev;             /* [m,n] row-major, leading dimension ldc (0 = n) */
    int64_t ldc;
    int32_t c_dtype;         /* ASCB200_F32 / F16 / BF16 / S8 / S32; FP8_E4M3 / FP8_E5M2 with FIXPIPE_QUANT on fp32 accumulators */
    void* c2_dev;            /* optional second output: the fp32 accumulator cast to c2_dtype (F16/BF16/F32) */
    int64_t ldc2;
    int32_t c2_dtype;
    int32_t epilogue;        /* ASCB200_EPI_* */
    const uint64_t* quant_dev; /* FIXPIPE_QUANT per channel: [n] parameters (SetQuantVector) or NULL */
    uint64_t quant_scalar;   /* FIXPIPE_QUANT per tensor (SetQuantScalar), used when quant_dev == NULL */
    const float* tok_scale_dev; /* DEQUANT_TOKEN_CHANNEL: [m] or NULL */
    const float* ch_scale_dev;  /* DEQUANT_TOKEN_CHANNEL: [n] */
    int32_t relu;            /* enableRelu of the fixpipe stage */
    int32_t act;             /* 0 none, 1 FasterGelu (DEQUANT_TOKEN_CHANNEL only) */
    int32_t atomic;          /* enAtomic of IterateAll / GetTensorC: 0 C is overwritten, 1 C += result, 2 C = max(C, result), 3 C = min(C, result); F32, S32, F16, BF16 outputs */
    int32_t scale_flags;     /* MXFP4: ASCB200_SCALE_*_PREPACKED bits; 0 = scale_a_dev / scale_b_dev are plain [rows, k/32] tensors */
    int32_t c_layout;        /* ASCB200_C_*: how c_dev is laid out (CubeFormat of C_TYPE); ROW_MAJOR = 0 */
    int32_t reserved[1];     /* must be zero */
} ascb200_gemm_desc;

/* Layouts of C, the formats the reference's copy-out stage writes (CopyOutNZ2ND / CopyOutNZ2NZ / CopyOutNZ2DN,
 * impl/adv_api/detail/matmul/stage/copy_cube_out/copy_cube_out_fixpipe.h:109-127; CubeFormat, include/adv_api/matmul/matmul_config.h:26-37):
 *   ROW_MAJOR     ND: element (i, j) at i * ldc + j;
 *   COLUMN_MAJOR  element (i, j) at j * ldc + i, ldc >= m (0 = m);
 *   NZ            fractal: element (i, j) at ((j / C0) * ldc + i) * C0 + j % C0 with C0 = 16 elements (32 for 1-byte outputs) and
 *                 ldc >= m the row count of the whole matrix (0 = m): blocks of C0 columns, row-major inside a block
 *                 (dstOffset / stride of CopyOutNZ2NZ, copy_cube_out_fixpipe.h:272-290); the buffer holds ceil(n / C0) blocks.
 * The other layouts take every epilogue and output type; `atomic` and the second output (c2_dev) go with ROW_MAJOR only. */
enum { ASCB200_C_ROW_MAJOR = 0, ASCB200_C_COLUMN_MAJOR = 1, ASCB200_C_NZ = 2 };

/* scale_flags: the scale tensor was re-tiled once with ascb200_mx_scale_prepack (static weights); the call then skips its
 * own re-tiling of that tensor and reads the prepacked copy in place. */
enum { ASCB200_SCALE_A_PREPACKED = 1, ASCB200_SCALE_B_PREPACKED = 2,
       /* the (not prepacked) scale tensor is stored [k/64][rows][2] - the two scales of a 64-element K step side by side, rows
        * next - instead of [rows][k/32]: the order the reference keeps a transposed scaleA ([K/32, M] -> isTransposeScaleA) and a
        * non-transposed scaleB ([K/32, N]) in, for LoadData2DMx's 32-byte scale fractals
        * (examples/01_simd_cpp_api/04_advanced_api/00_matmul/matmul_mx/scripts/gen_data.py:73-76;
        *  05_best_practices/01_matrix_compute/matmul_mxfp4_high_performance/scripts/gen_data.py:63) */
       ASCB200_SCALE_A_PAIRED = 4, ASCB200_SCALE_B_PAIRED = 8 };

/* One whole Matmul: what Matmul<...>::IterateAll produces for the object state set by
 * SetTensorA / SetTensorB / SetBias / SetQuantScalar / SetQuantVector
 * (include/adv_api/matmul/matmul.h:79-399; impl/adv_api/detail/matmul/matmul_impl.h:119-139),
 * MX variant with SetTensorScaleA/B (impl/adv_api/detail/matmul/mx_matmul_impl.h:136-173).
 *
 * Integer results do not depend on how the library tiles the problem.  fp32 accumulation follows the tile plan (a tile's K blocks
 * in ascending order; with few tiles and a long K, two or four CTAs of a cluster each sum a consecutive range of K blocks and
 * the ranges are added in ascending order), so a floating-point result is reproducible for a given shape and device, and equal to
 * any other plan's within the rounding of fp32 sums. */
ASCB200_API int ascb200_gemm(const ascb200_gemm_desc* desc, void* stream);
/* MXFP4 and scratch memory.  The tensor core reads MX scale factors in tiles of 128 rows x 4 K-blocks, so ascb200_gemm re-tiles
 * every scale tensor that is not prepacked into device scratch before the GEMM (one extra, small launch).  The scratch belongs
 * to `stream`: calls on different streams use different blocks and may overlap freely; calls on one stream are ordered by it.
 * The first MXFP4 call on a stream, and a call that needs more scratch than any before it on that stream, allocates (and, when it
 * grows, synchronises that stream first): make such a call once before capturing the stream into a graph.  Up to 64 streams per
 * device keep their own block; beyond that the oldest blocks are released after a device-wide synchronisation.  A stream that was
 * destroyed and whose handle value the runtime hands out again simply inherits the block. */

/* The step the reference performs when it moves MX scales GM -> L1 -> L0A_MX / L0B_MX in its pair-interleaved fractal order
 * (LoadData with LoadData2DMxParams: include/basic_api/kernel_struct_mm.h:132-153; examples/.../load_data_2dmx_l12l0), done once
 * for a tensor that does not change between calls (the weights' scales): re-tiles scale_dev, e8m0 bytes [rows, k/32] row-major,
 * into out_dev in the order ascb200_gemm reads (512-byte chunks of 128 rows x 4 K-blocks, two padding blocks of rows at the end).
 * paired != 0: the source is in the [k/64][rows][2] order described at ASCB200_SCALE_A_PAIRED.
 * out_dev must be 16-byte aligned and hold ascb200_mx_scale_prepacked_bytes(rows, k) bytes; k a multiple of 64.  Pass out_dev as
 * scale_a_dev / scale_b_dev with the matching ASCB200_SCALE_*_PREPACKED flag. */
ASCB200_API size_t ascb200_mx_scale_prepacked_bytes(int32_t rows, int32_t k);
ASCB200_API int ascb200_mx_scale_prepack(const void* scale_dev, int32_t rows, int32_t k, int32_t paired, void* out_dev, size_t out_bytes,
                                         void* stream);
/* Transposes a packed fp4 matrix: src [rows][cols / 2 bytes] (two column-neighbours per byte, even column in the low nibble)
 * -> dst [cols][rows / 2 bytes] (two row-neighbours per byte, even row in the low nibble).  rows and cols even.  This turns the
 * reference's ND B of an MX Matmul ([K, N], two N-neighbours per byte:
 * 05_best_practices/01_matrix_compute/matmul_mxfp4_high_performance/scripts/gen_data.py:25-36,46) into the K-major [N, K] operand
 * the tensor core needs (and a transposed A, [K, M], into [M, K]).  ascb200_gemm does the same into its stream scratch on
 * every call when it is given trans_b == 0 (or trans_a == 1) with kind MXFP4; weights are better transposed once. */
ASCB200_API int ascb200_fp4_transpose(const void* src_dev, void* dst_dev, int32_t rows, int32_t cols, void* stream);

/* Grouped int8 matmul of the reference's QuantGroupMatmul example kernel
 * (examples/01_simd_cpp_api/05_best_practices/03_fusion_compute/quant_group_matmul_high_performance/
 *  quant_group_matmul_custom.asc:252-452): rows of A are split into `groups` consecutive groups by
 * group_counts_dev[g] (int64 row counts, not a cumulative sum; counts <= 0 are skipped); group g
 * uses B[g] ([n,k] when trans_b else [k,n]) and ch_scale_dev[g*n .. g*n+n).  `desc->m` is the row
 * capacity of A / C (>= sum of counts); kind must be S8 and epilogue DEQUANT_TOKEN_CHANNEL. */
ASCB200_API int ascb200_grouped_gemm(const ascb200_gemm_desc* desc, const int64_t* group_counts_dev, int32_t groups,
                                     void* stream);

/* MXFP4 Matmul for callers that must not allocate device memory.  (No counterpart in the reference:
 * its operators run on buffers the user kernel already owns.)
 *
 * Who needs it: a host that has handed all of the GPU's memory to its own pool or arena before this
 * library is touched (inference servers and training frameworks commonly do), or that runs inside a
 * latency-critical loop where cudaMalloc's implicit device synchronisation is not acceptable.  For
 * them ascb200_init (which allocates the status word) and ascb200_gemm (which grows a scratch block
 * for the re-tiled MX scale factors on first use) are both off limits.
 *
 * This entry point needs neither: its status word and its scale scratch live in one array that is
 * part of the library image (ASCB200_NOALLOC_MAX_SCALE_BYTES + 256 bytes on every GPU that loads the
 * library, held until the process exits).  It calls no cudaMalloc / cudaFree and needs no ascb200_init;
 * it works on the calling thread's current device.  Inputs and outputs are still the caller's.
 *
 *  - desc: exactly as for ascb200_gemm with kind == ASCB200_KIND_MXFP4 (other kinds: ASCB200_EUNSUPPORTED); it runs the same
 *    kernels as ascb200_gemm and gives the same bytes;
 *  - limit: the re-tiled scales take (ceil(m/128) + ceil(n/128) + 2) * 2*ceil(k/256) * 512 bytes (the 2 are padding blocks that
 *    tiles at the right edge read); if that exceeds ASCB200_NOALLOC_MAX_SCALE_BYTES the call returns ASCB200_ETOOBIG and launches
 *    nothing (m = n = k = 8192 needs 4,259,840 bytes and fits; a prepacked scale tensor does not count);
 *  - the first call on each device looks up the array's device address; make that first call outside
 *    any stream capture;
 *  - all calls on one device share the array, which keeps the previous call's contents (every scale byte a call reads is
 *    rewritten by that call first; the status word is a latch and needs no clearing): two calls whose GPU work
 *    may overlap - different streams, or different host threads - race on it; serialise them;
 *  - an expired device-side wait is latched in the array's first word, not in the word that ascb200_device_status reads:
 *    ascb200_noalloc_status (which allocates nothing either) copies it to *status_host after synchronising `stream`, returns
 *    ASCB200_ETIMEOUT when it is non-zero and clears it. */
#define ASCB200_NOALLOC_MAX_SCALE_BYTES ((4u << 20) + (512u << 10))
ASCB200_API int ascb200_gemm_mxfp4_noalloc(const ascb200_gemm_desc* desc, void* stream);
ASCB200_API int ascb200_noalloc_status(void* stream, uint32_t* status_host);

/* ---- several GPUs of one box ---------------------------------------------------------------------- */

/* The reference spreads a Matmul over AI cores with the multi-core tiling (MultiCoreMatmulTiling::SetDim / SetSingleShape,
 * include/adv_api/matmul/matmul_tiling.h:30-62; block offsets in examples/.../00_matmul/matmul/matmul.asc:114-141) and the grouped
 * matmul by handing group blocks to cores in turn (quant_group_matmul_custom.asc:254-286).  Across GPUs the same two splits
 * are used, both without communication; these are plain host functions (no device needed).
 *
 * N-slab: rank `rank` of `world` owns columns [*lo, *hi) of B / the per-channel parameters / C; slabs are equal multiples of
 * `align` columns, the last ranks get what is left (possibly nothing). */
ASCB200_API int ascb200_shard_nslab(int64_t n, int32_t rank, int32_t world, int32_t align, int64_t* lo, int64_t* hi);
/* Expert groups: greedy longest-processing-time assignment by row count (largest group first, each to the rank with the
 * fewest rows so far; ties go to the lower group / rank index).  counts_host[g] <= 0 counts as no rows.  owner_host[g] = rank. */
ASCB200_API int ascb200_shard_groups_lpt(const int64_t* counts_host, int32_t groups, int32_t world, int32_t* owner_host);

/* The optional collective of the path: every rank ends with the whole C.  Takes the role of the reference's kernel-side
 * Hccl<>::AllGather(sendBuf, recvBuf, sendCount, dataType, strideCount, repeat) (include/adv_api/hccl/hccl.h:103-105), whose
 * strideCount places each rank's piece at a stride in recvBuf.  Here: NCCL all-gather of the contiguous slabs into
 * gathered_dev ([ranks][m][n_loc]) followed by a local re-layout kernel into full_dev (row-major [m][ranks * n_loc], leading
 * dimension ld_full elements, 0 = packed); full_dev == NULL skips the re-layout.  All ranks call it with the same m, n_loc,
 * elem_bytes; both buffers are the caller's.  NCCL is loaded at run time (libnccl.so.2); without it these calls return
 * ASCB200_EUNSUPPORTED.  Communicators: ascb200_comm_unique_id on one rank (128 bytes, handed to the others by whatever means
 * the host has), then ascb200_comm_init on every rank with its device current; ascb200_comm_init_all creates the
 * communicators of `ndev` devices in one process (devices == NULL: 0 .. ndev-1), whose collective calls must then be
 * bracketed by ascb200_group_start / ascb200_group_end.  Inside such a group NCCL only records the all-gather and issues it
 * when the group is closed: pass full_dev == NULL there and call ascb200_interleave_slabs on every device afterwards. */
ASCB200_API int ascb200_comm_unique_id(void* id_out_128_bytes);
ASCB200_API int ascb200_comm_init(void** comm, int32_t world, int32_t rank, const void* unique_id_128_bytes);
ASCB200_API int ascb200_comm_init_all(void** comms, int32_t ndev, const int32_t* devices);
ASCB200_API int ascb200_comm_destroy(void* comm);
ASCB200_API int ascb200_group_start(void);
ASCB200_API int ascb200_group_end(void);
ASCB200_API int ascb200_allgather_slabs(void* comm, int32_t ranks, const void* slab_dev, int64_t m, int64_t n_loc, int32_t elem_bytes,
                                        void* gathered_dev, void* full_dev, int64_t ld_full, void* stream);
/* The re-layout by itself: [ranks][m][n_loc] -> [m][ld_full] with slab r in columns [r * n_loc, (r + 1) * n_loc).  HBM bound:
 * 2 * ranks * m * n_loc * elem_bytes bytes per launch. */
ASCB200_API int ascb200_interleave_slabs(const void* gathered_dev, void* full_dev, int32_t ranks, int64_t m, int64_t n_loc, int64_t ld_full,
                                         int32_t elem_bytes, void* stream);

/* ---- SoftMax ------------------------------------------------------------------------------------ */

/* Unpacks a fractal ("NZ") matrix [groups][n/C0][k/16][16][C0], C0 = 32 / elem_bytes columns per block (the format
 * CubeFormat::NZ of include/adv_api/matmul/matmul_config.h:26-37; the grouped matmul example stores its int8 weights so:
 * examples/.../quant_group_matmul_high_performance/scripts/gen_data.py:62), into row-major [groups][n][k] (to_nk = 1, the K-major
 * layout of trans_b = 1) or [groups][k][n] (to_nk = 0).  k must be a multiple of 16, n of C0; elem_bytes 1 or 2.  Replaces the
 * reference's on-the-fly NZ loads (impl/adv_api/detail/matmul/stage/copy_cube_in): weights are static, they are unpacked once. */
ASCB200_API int ascb200_nz_unpack(const void* src_nz_dev, void* dst_dev, int32_t groups, int32_t k, int32_t n, int32_t elem_bytes,
                                  int32_t to_nk, void* stream);

/* SoftMax<T>(dst, sum, max, src, tiling, shapeInfo) over the last axis of src[m,k]
 * (include/adv_api/activation/softmax.h:92-109,229-247).  dtype F16 or F32; k*sizeof(T) must be a
 * multiple of 32 bytes like in the reference (softmax_check_common.h:63-67).  sum/max are fp32:
 * stats_brc != 0 writes [m, 32/sizeof(float)] with the value repeated over one 32-byte block (the
 * reference default), stats_brc == 0 writes [m] (SoftmaxMode::SOFTMAX_OUTPUT_WITHOUT_BRC). */
ASCB200_API int ascb200_softmax(const void* src_dev, void* dst_dev, float* sum_dev, float* max_dev, int32_t m, int32_t k,
                                int32_t dtype, int32_t stats_brc, void* stream);

/* LogSoftMax<T>(dst, sum, max, src, sharedTmpBuffer, tiling, shapeInfo)
 * (include/adv_api/activation/logsoftmax.h:56-71; formula of LogSoftMax.md): per row max, e = exp(x - max), sum,
 * y = log10(e / sum), evaluated in fp32 as ln(.) * 0.4342944819 like the reference
 * (impl/adv_api/detail/activation/softmax/membase/common/logsoftmax_common_impl.h:277-376).  dtype F16 or F32;
 * sum/max have the SAME dtype as src (the reference's LocalTensor<T> statistics) and are written once per row
 * (stats_brc == 0) or broadcast over one 32-byte block (stats_brc != 0: 16 halves or 8 floats per row).
 * Same argument checks as ascb200_softmax. */
ASCB200_API int ascb200_log_softmax(const void* src_dev, void* dst_dev, void* sum_dev, void* max_dev, int32_t m, int32_t k,
                                    int32_t dtype, int32_t stats_brc, void* stream);

/* SimpleSoftMax<T>(dst, inSum, inMax, src, tiling, shapeInfo) (include/adv_api/activation/simplesoftmax.h:55-190):
 * y = exp(x - inMax) / inSum per row with statistics computed earlier, fp32 arithmetic, cast RINT
 * (impl/adv_api/detail/activation/softmax/membase/common/simple_softmax_common_impl.h:320-502).  dtype F16 or F32;
 * stats_dtype == dtype (the all-T overloads) or F32 beside F16 data (the half / float overloads); statistics hold one
 * value per row (stats_brc == 0) or one 32-byte block per row (stats_brc != 0).  k * sizeof(T) a multiple of 32. */
ASCB200_API int ascb200_simple_softmax(const void* src_dev, void* dst_dev, const void* in_sum_dev, const void* in_max_dev, int32_t m,
                                       int32_t k, int32_t dtype, int32_t stats_dtype, int32_t stats_brc, void* stream);

/* SoftmaxGrad<T>(dst, grad, src, tiling, isFront, shapeInfo) and SoftmaxGradFront<T>(dst, grad, src, tiling, shapeInfo)
 * (include/adv_api/activation/softmaxgrad.h:57-175): per row s = sum(grad * src) in fp32; is_front == 0 writes
 * dst[m, k] = (grad - s) * src, is_front != 0 writes dst[m, 32 / sizeof(T)] = s (one 32-byte block per row)
 * (impl/adv_api/detail/activation/softmax/membase/common/softmax_grad_nd_impl.h:27-60).  dtype F16 or F32;
 * k * sizeof(T) a multiple of 32. */
ASCB200_API int ascb200_softmax_grad(const void* grad_dev, const void* src_dev, void* dst_dev, int32_t m, int32_t k, int32_t dtype,
                                     int32_t is_front, void* stream);

/* ---- AscendQuant -------------------------------------------------------------------------------- */

/* AscendQuant per tensor: dst = int8(rint_sat(half(src) * half(scale) + half(offset))), arithmetic in fp16
 * (include/adv_api/quantization/ascend_quant.h; impl/.../quant/ascend_quant_3510_impl.h:34-120).
 * src dtype F16 / BF16 / F32; cal_count elements. */
ASCB200_API int ascb200_quant_per_tensor(const void* src_dev, int8_t* dst_dev, int64_t cal_count, int32_t dtype, float scale,
                                         float offset, void* stream);
/* AscendQuant per channel: src [rows, scale_count]; scale_dev (and offset_dev when not NULL) have
 * scale_count entries of the source dtype; with offset_dev == NULL the scalar `offset` (converted
 * to the source dtype) is used (impl/.../quant/ascend_quant_3510_impl.h:275-378,553-700). */
ASCB200_API int ascb200_quant_per_channel(const void* src_dev, int8_t* dst_dev, int32_t rows, int32_t scale_count, int32_t dtype,
                                          const void* scale_dev, const void* offset_dev, float offset, void* stream);

/* AscendQuant with a policy (include/adv_api/quantization/ascend_quant.h:682-790; AscendQuantPolicy of
 * include/adv_api/quantization/ascend_quant_utils.h:75-89; AscendQuantParam {m, n, calCount, groupSize}; implementation
 * impl/adv_api/detail/quantization/quant/ascend_quant_per_group_3510_impl.h): dst[i,j] = cast(src[i,j] * scale [+ offset]).
 *   ASCB200_QUANT_PER_TOKEN: scale / offset [m].
 *   ASCB200_QUANT_PER_GROUP: k_dim = 1 (config.kDim): scale [m, ceil(n / group_size)]; k_dim = 0: scale [ceil(m / group_size), n];
 *                            group_size a positive multiple of 32.
 * src: F16 / BF16 / F32; scale (and offset tensor): F32, or the source's 16-bit type (arithmetic then runs in that type);
 * dst: S8, FP8_E4M3, FP8_E5M2, or FP4_E2M1 (PER_GROUP only, two values per byte, n even, offset ignored like the reference).
 * has_offset = config.hasOffset; the offset is offset_tensor (scale's shape) or, when that is NULL, offset_scalar.
 * Rounding: CAST_RINT with saturation (the default config.roundMode). */
enum { ASCB200_QUANT_PER_TOKEN = 2, ASCB200_QUANT_PER_GROUP = 3 };  /* values of AscendQuantPolicy */
ASCB200_API int ascb200_quant_policy(const void* src_dev, void* dst_dev, int32_t m, int32_t n, int32_t src_dtype, int32_t scale_dtype,
                                     int32_t dst_dtype, int32_t policy, int32_t k_dim, int32_t group_size, const void* scale_dev,
                                     const void* offset_tensor_dev, float offset_scalar, int32_t has_offset, void* stream);
/* The same with config.roundMode (include/adv_api/quantization/ascend_quant_utils.h:55-64): round_mode takes the values of
 * RoundMode (impl/basic_api/utils/kernel_utils_mode.h:103-120): 0 CAST_NONE and 1 CAST_RINT nearest even, 2 CAST_FLOOR, 3 CAST_CEIL,
 * 4 CAST_ROUND halves away from zero, 5 CAST_TRUNC towards zero; all saturating.  Modes other than nearest even go with S8
 * destinations; CAST_ODD and the hybrid modes are not built (ASCB200_EUNSUPPORTED). */
ASCB200_API int ascb200_quant_policy_rm(const void* src_dev, void* dst_dev, int32_t m, int32_t n, int32_t src_dtype, int32_t scale_dtype,
                                        int32_t dst_dtype, int32_t policy, int32_t k_dim, int32_t group_size, const void* scale_dev,
                                        const void* offset_tensor_dev, float offset_scalar, int32_t has_offset, int32_t round_mode, void* stream);

/* AscendDequant with a policy (include/adv_api/quantization/ascend_dequant.h:293-318, AscendDeQuantPolicy / AscendDeQuantParam of
 * include/adv_api/quantization/ascend_dequant_utils.h:32-44): dst[i,j] = cast(float(src[i,j]) * float(scale)), scale per row
 * (PER_TOKEN: [m]) or per group (PER_GROUP: k_dim 1 -> [m, ceil(n / group_size)], k_dim 0 -> [ceil(m / group_size), n]).
 * src S32 / F32; scale F32 / F16 / BF16; dst F32 / F16 / BF16.  The interface's offset tensor is unused by the reference. */
enum { ASCB200_DEQUANT_PER_TOKEN = 0, ASCB200_DEQUANT_PER_GROUP = 1 };  /* values of AscendDeQuantPolicy */
ASCB200_API int ascb200_dequant_policy(const void* src_dev, void* dst_dev, int32_t m, int32_t n, int32_t src_dtype, int32_t scale_dtype,
                                       int32_t dst_dtype, int32_t policy, int32_t k_dim, int32_t group_size, const void* scale_dev,
                                       void* stream);

/* AscendAntiQuant<int8_t, OutputDataType, isTranspose>(dst, src, [offset,] scale, [sharedTmpBuffer,] k, shapeInfo)
 * (include/adv_api/quantization/ascend_antiquant.h:47-200): dst = scale * (src + offset), src int8 [rows, cols], dst F16 or BF16.
 *   mode 0  per tensor: scale_scalar / offset_scalar (rounded to the output type first, as the interface takes them in it);
 *   mode 1  per channel, isTranspose = false: src [K, N], scale_dev / offset_dev [N] of the output type, one pair per column;
 *   mode 2  per channel, isTranspose = true:  src [N, K], scale_dev / offset_dev [N], one pair per row.
 * offset_dev == NULL in modes 1 / 2 uses offset_scalar (0 for the overloads without offset).  Arithmetic follows the
 * reference's register code (impl/adv_api/detail/quantization/antiquant/ascend_antiquant_3510_impl.h): half outputs add and
 * multiply in half; bfloat16 outputs in bfloat16 for mode 1 and in fp32 with one rounding for modes 0 and 2.
 * cols must be a multiple of 32. */
ASCB200_API int ascb200_antiquant(const int8_t* src_dev, void* dst_dev, int32_t rows, int32_t cols, int32_t dst_dtype, int32_t mode,
                                  const void* scale_dev, const void* offset_dev, float scale_scalar, float offset_scalar, void* stream);

/* SoftmaxFlashV2<T, isUpdate>(dst, expSum, max, src, expMax, inExpSum, inMax, tiling, shapeInfo)
 * (include/adv_api/activation/softmaxflashv2.h:93-300): one step of the online softmax over rows [m, k].
 *   update == 0: max = rowmax(x); y = exp(x - max); expSum = rowsum(y).
 *   update == 1: max = max(inMax, rowmax(x)); y = exp(x - max); expMax = exp(inMax - max); expSum = expMax * inExpSum + rowsum(y).
 * dtype (x, y, expMax): F16 or F32; stats_dtype (max / sum tensors): the same, or F32 with F16 data (the half/float overload).
 * stats_brc = 1: every per-row value fills one 32-byte block ([m, 8] floats / [m, 16] halves, SOFTMAX_NORMAL);
 * 0: [m] (SOFTMAX_OUTPUT_WITHOUT_BRC).  k * sizeof(T) must be a multiple of 32 bytes; k up to 16384 halves / 8192 floats. */
ASCB200_API int ascb200_softmax_flash_v2(const void* src_dev, void* dst_dev, void* exp_sum_dev, void* max_dev, void* exp_max_dev,
                                         const void* in_exp_sum_dev, const void* in_max_dev, int32_t m, int32_t k, int32_t dtype,
                                         int32_t stats_dtype, int32_t update, int32_t stats_brc, void* stream);

/* SoftmaxFlash<T>(dst, sum, max, src, expMax, inSum, inMax, tiling, isUpdate, shapeInfo)
 * (include/adv_api/activation/softmaxflash.h:65-215, the first version, kept by the reference as deprecated; formulas of
 * SoftmaxFlash.md): the step above followed by the normalisation.
 *   update == 0: the same result as SoftMax (y = exp(x - max) / sum).
 *   update == 1: max = max(inMax, rowmax(x)); e = exp(x - max); sum = exp(inMax - max) * inSum + rowsum(e);
 *                expMax = exp(inMax - max) * inSum / sum; y = e / sum.
 * Arguments as ascb200_softmax_flash_v2. */
ASCB200_API int ascb200_softmax_flash(const void* src_dev, void* dst_dev, void* sum_dev, void* max_dev, void* exp_max_dev,
                                      const void* in_sum_dev, const void* in_max_dev, int32_t m, int32_t k, int32_t dtype,
                                      int32_t stats_dtype, int32_t update, int32_t stats_brc, void* stream);

/* SoftMax immediately followed by per-channel AscendQuant of its output, one pass over src:
 * writes the fp16 SoftMax result, sum, max and the int8 tensor.  Equivalent to calling
 * ascb200_softmax then ascb200_quant_per_channel (dtype F16). */
ASCB200_API int ascb200_softmax_quant(const void* src_dev, void* dst_dev, float* sum_dev, float* max_dev, int8_t* q_dev,
                                      const void* scale_dev, const void* offset_dev, float offset, int32_t m, int32_t k,
                                      int32_t stats_brc, void* stream);

/* ---- AscendDequant ------------------------------------------------------------------------------ */

/* AscendDequant<dstT, scaleT>(dst, src, deqScale, DequantParams{m, n, calCount}):
 * dst[i,j] = dstT(float(src[i,j]) * float(scale[j])), j < cal_count; src rows hold n int32, dst rows
 * hold n_dst elements (the reference pads dst rows to 32 bytes)
 * (include/adv_api/quantization/ascend_dequant.h; impl/.../dequant/ascend_dequant_common_impl.h:261-432).
 * scale_dtype F32 or BF16 for a [cal_count] tensor; scale_dev == NULL selects the scalar overload. */
ASCB200_API int ascb200_dequant(const int32_t* src_dev, void* dst_dev, int32_t m, int32_t n, int32_t cal_count, int32_t n_dst,
                                int32_t dst_dtype, const void* scale_dev, int32_t scale_dtype, float scale_scalar, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ASCB200_H */
