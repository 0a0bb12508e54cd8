// Shared host/device helpers of the ascb200 library (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ascb200.h"

namespace ascb200 {

// Per-device state created by ascb200_init.
struct DeviceState {
    bool ready = false;
    int device = -1;
    int sm_count = 0;
    long long l2_bytes = 0;
    uint32_t* status_dev = nullptr;  // bit 0: bounded wait expired inside a GEMM kernel
    // scratch for re-tiled MX scale factors, one block per stream that asked for one (grows on demand)
    struct StreamScratch {
        cudaStream_t stream = nullptr;
        void* dev = nullptr;
        size_t bytes = 0;
        unsigned long long last_use = 0;
    };
    static constexpr int kMaxStreamScratch = 64;
    StreamScratch scratch[kMaxStreamScratch];
    int scratch_count = 0;
    unsigned long long scratch_clock = 0;
};

DeviceState* current_state();           // nullptr (and ASCB200_ENODEV recorded) when init has not run
// Scratch of at least `bytes` that belongs to `stream` (see the note on MXFP4 scratch at ascb200_gemm).  Thread-safe.
int stream_scratch(DeviceState* st, size_t bytes, cudaStream_t stream, void** out);
int cuda_fail(cudaError_t e);           // records e, returns ASCB200_ECUDA
// packed fp4 [rows][cols / 2] -> [cols][rows / 2] (csrc/prepack.cu)
int fp4_transpose(const void* src, void* dst, int rows, int cols, cudaStream_t stream);
#define ASCB200_CUDA(call)                                   \
    do {                                                     \
        cudaError_t e__ = (call);                            \
        if (e__ != cudaSuccess) return ::ascb200::cuda_fail(e__); \
    } while (0)

// Launch with programmatic stream serialisation: the grid may be scheduled while the kernel before it in the stream is
// still draining, which hides the launch latency between back-to-back kernels.  The kernel must execute
// grid_dependency_wait() before it touches global memory; then nothing it reads or writes can race with its predecessor.
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// The same with the grid cut into clusters of `cluster_x` consecutive blocks (a run-time cluster shape: the kernel needs no
// __cluster_dims__; grid.x must be a multiple of cluster_x).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, unsigned cluster_x, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = cluster_x;
    attrs[1].val.clusterDim.y = 1;
    attrs[1].val.clusterDim.z = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Lets the next kernel of the stream start its launch, then waits until every kernel before this one has completed and its
// writes are visible.  A no-op pair when the kernel was launched without the attribute.
__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

static inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

#ifdef __CUDACC__
// ---- numeric conversions: one definition per rounding rule of the reference -----------------
// fp32 -> fp16, round to nearest even, overflow saturates to +-65504 (CAST_RINT with saturation).
__device__ __forceinline__ __half f32_to_f16_sat(float f)
{
    unsigned short b = __half_as_ushort(__float2half_rn(f));
    if ((b & 0x7FFFu) == 0x7C00u) b = (b & 0x8000u) | 0x7BFFu;  // +-inf -> +-65504, NaN untouched
    return __ushort_as_half(b);
}
__device__ __forceinline__ __nv_bfloat16 f32_to_bf16(float f) { return __float2bfloat16_rn(f); }
// fp32 -> int8, round to nearest even, saturating; NaN -> 0.
__device__ __forceinline__ int f32_to_s8(float f)
{
    int i = __float2int_rn(f);  // saturates to int32, NaN -> 0
    return max(-128, min(127, i));
}
// The (1,8,10) scale in bits [31:13] of a fixpipe quant parameter.
__device__ __forceinline__ float quant_alpha(uint64_t q) { return __uint_as_float(static_cast<uint32_t>(q) & 0xFFFFE000u); }
__device__ __forceinline__ float quant_offset(uint64_t q)
{
    int o = static_cast<int>((q >> 37) & 0x1FFu);
    return static_cast<float>((o & 0x100) ? o - 512 : o);
}
#endif

}  // namespace ascb200
