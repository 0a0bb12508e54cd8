// Self-test of the bounded device-side waits: a one-CTA kernel waits on an mbarrier that nothing will ever complete, with
// the same wait routine the GEMM kernels use but a limit of a fraction of a millisecond.  The wait gives up, the kernel
// records the fact in the device status word and in its own result word and returns normally; the context stays usable.
#include "tc_common.cuh"

namespace ascb200 {
namespace {

using namespace tc;

__global__ void __launch_bounds__(64) bounded_wait_selftest_kernel(uint32_t* status, uint32_t* result, long long limit_cycles)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_word;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);   // one arrival expected; no thread arrives
        abort_word = 0u;
        fence_barrier_init();
    }
    __syncthreads();
    // warp 0 waits with the polling form, warp 1 with the backing-off form; whichever gives up first sets the abort word,
    // the other then returns at its next check
    const long long t0 = clock64();
    bool ok;
    if (threadIdx.x < 32) ok = mbar_wait(smem_u32(&bar), 0u, &abort_word, status, limit_cycles);
    else ok = mbar_wait_relaxed(smem_u32(&bar), 0u, &abort_word, status);
    const long long waited = clock64() - t0;
    __syncthreads();
    if (threadIdx.x == 0) {
        result[0] = ok ? 0u : 1u;                     // 1: the wait was abandoned, as it must be
        result[1] = abort_word;                       // 1: the CTA-wide abort word was set
        result[2] = static_cast<uint32_t>(waited >> 10);   // cycles waited / 1024
    }
}

}  // namespace
}  // namespace ascb200

using namespace ascb200;

extern "C" int ascb200_selftest_bounded_wait(uint32_t* result_host3, void* stream)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    if (!result_host3) return ASCB200_EINVAL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint32_t* result_dev = st->status_dev + 16;   // inside the 256-byte status block, away from the status word
    ASCB200_CUDA(cudaMemsetAsync(result_dev, 0xFF, 3 * sizeof(uint32_t), s));
    bounded_wait_selftest_kernel<<<1, 64, 0, s>>>(st->status_dev, result_dev, 200000ll);   // about 0.1 ms
    ASCB200_CUDA(cudaGetLastError());
    ASCB200_CUDA(cudaMemcpyAsync(result_host3, result_dev, 3 * sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    ASCB200_CUDA(cudaStreamSynchronize(s));
    return ASCB200_OK;
}
