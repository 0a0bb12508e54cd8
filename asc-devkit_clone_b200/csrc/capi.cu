// Library state, error reporting and the memory / stream shims of the C ABI.
#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace ascb200 {

static DeviceState g_states[16];
static std::mutex g_mu;
static thread_local int t_last_cuda = 0;

int cuda_fail(cudaError_t e)
{
    t_last_cuda = static_cast<int>(e);
    (void)cudaGetLastError();
    return ASCB200_ECUDA;
}

DeviceState* current_state()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
    DeviceState* st = &g_states[dev];
    return st->ready ? st : nullptr;
}

int stream_scratch(DeviceState* st, size_t bytes, cudaStream_t stream, void** out)
{
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState::StreamScratch* e = nullptr;
    for (int i = 0; i < st->scratch_count; ++i)
        if (st->scratch[i].stream == stream) e = &st->scratch[i];
    if (!e) {
        if (st->scratch_count == DeviceState::kMaxStreamScratch) {
            // Table full: release the older half.  Their streams may still be running kernels that read the blocks.
            ASCB200_CUDA(cudaDeviceSynchronize());
            unsigned long long order[DeviceState::kMaxStreamScratch];
            for (int i = 0; i < st->scratch_count; ++i) order[i] = st->scratch[i].last_use;
            std::nth_element(order, order + st->scratch_count / 2, order + st->scratch_count);
            const unsigned long long cut = order[st->scratch_count / 2];
            int kept = 0;
            for (int i = 0; i < st->scratch_count; ++i) {
                if (st->scratch[i].last_use < cut) {
                    if (st->scratch[i].dev) (void)cudaFree(st->scratch[i].dev);
                } else {
                    st->scratch[kept++] = st->scratch[i];
                }
            }
            st->scratch_count = kept;
        }
        e = &st->scratch[st->scratch_count++];
        *e = DeviceState::StreamScratch();
        e->stream = stream;
    }
    e->last_use = ++st->scratch_clock;
    if (bytes > e->bytes) {
        // kernels queued on this stream may still read the old block
        if (e->dev) {
            ASCB200_CUDA(cudaStreamSynchronize(stream));
            ASCB200_CUDA(cudaFree(e->dev));
        }
        e->dev = nullptr;
        e->bytes = 0;
        const size_t want = bytes + (bytes >> 2);
        ASCB200_CUDA(cudaMalloc(&e->dev, want));
        e->bytes = want;
    }
    *out = e->dev;
    return ASCB200_OK;
}

}  // namespace ascb200

using namespace ascb200;

extern "C" {

int ascb200_init(int device)
{
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) {
        (void)cudaGetLastError();
        return ASCB200_ENODEV;
    }
    if (device < 0 || device >= count || device >= 16) return ASCB200_EINVAL;
    ASCB200_CUDA(cudaSetDevice(device));
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState* st = &g_states[device];
    if (st->ready) return ASCB200_OK;
    cudaDeviceProp prop;
    ASCB200_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return ASCB200_ENODEV;
    st->device = device;
    st->sm_count = prop.multiProcessorCount;
    st->l2_bytes = prop.l2CacheSize;
    ASCB200_CUDA(cudaMalloc(&st->status_dev, 256));
    ASCB200_CUDA(cudaMemset(st->status_dev, 0, 256));
    st->ready = true;
    return ASCB200_OK;
}

const char* ascb200_strerror(int code)
{
    switch (code) {
        case ASCB200_OK: return "ok";
        case ASCB200_EINVAL: return "invalid argument";
        case ASCB200_EALIGN: return "pointer or leading dimension not aligned as required";
        case ASCB200_EUNSUPPORTED: return "combination not supported";
        case ASCB200_ENODEV: return "no initialised sm_100 CUDA device (call ascb200_init)";
        case ASCB200_ECUDA: return "CUDA call failed";
        case ASCB200_ETIMEOUT: return "device-side wait expired";
        case ASCB200_ETOOBIG: return "extent beyond supported limit";
        default: return "unknown error";
    }
}

int ascb200_last_cuda_error(void) { return t_last_cuda; }

int ascb200_sm_count(void)
{
    DeviceState* st = current_state();
    return st ? st->sm_count : ASCB200_ENODEV;
}

int ascb200_device_status(void* stream, uint32_t* status_host)
{
    DeviceState* st = current_state();
    if (!st) return ASCB200_ENODEV;
    uint32_t v = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    ASCB200_CUDA(cudaMemcpyAsync(&v, st->status_dev, sizeof(v), cudaMemcpyDeviceToHost, s));
    ASCB200_CUDA(cudaStreamSynchronize(s));
    if (status_host) *status_host = v;
    if (v != 0) {
        ASCB200_CUDA(cudaMemsetAsync(st->status_dev, 0, sizeof(v), s));
        return ASCB200_ETIMEOUT;
    }
    return ASCB200_OK;
}

int ascb200_malloc(void** p, size_t bytes)
{
    if (!p) return ASCB200_EINVAL;
    ASCB200_CUDA(cudaMalloc(p, bytes ? bytes : 1));
    return ASCB200_OK;
}
int ascb200_free(void* p)
{
    ASCB200_CUDA(cudaFree(p));
    return ASCB200_OK;
}
int ascb200_malloc_host(void** p, size_t bytes)
{
    if (!p) return ASCB200_EINVAL;
    ASCB200_CUDA(cudaMallocHost(p, bytes ? bytes : 1));
    return ASCB200_OK;
}
int ascb200_free_host(void* p)
{
    ASCB200_CUDA(cudaFreeHost(p));
    return ASCB200_OK;
}
int ascb200_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream)
{
    ASCB200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
    return ASCB200_OK;
}
int ascb200_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream)
{
    ASCB200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    return ASCB200_OK;
}
int ascb200_memset(void* dst, int value, size_t bytes, void* stream)
{
    ASCB200_CUDA(cudaMemsetAsync(dst, value, bytes, static_cast<cudaStream_t>(stream)));
    return ASCB200_OK;
}
int ascb200_stream_create(void** stream)
{
    if (!stream) return ASCB200_EINVAL;
    cudaStream_t s;
    ASCB200_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return ASCB200_OK;
}
int ascb200_stream_destroy(void* stream)
{
    ASCB200_CUDA(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
    return ASCB200_OK;
}
int ascb200_stream_sync(void* stream)
{
    ASCB200_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return ASCB200_OK;
}
int ascb200_event_create(void** event)
{
    if (!event) return ASCB200_EINVAL;
    cudaEvent_t e;
    ASCB200_CUDA(cudaEventCreate(&e));
    *event = e;
    return ASCB200_OK;
}
int ascb200_event_destroy(void* event)
{
    ASCB200_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
    return ASCB200_OK;
}
int ascb200_event_record(void* event, void* stream)
{
    ASCB200_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
    return ASCB200_OK;
}
int ascb200_stream_wait_event(void* stream, void* event)
{
    ASCB200_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
    return ASCB200_OK;
}
int ascb200_event_elapsed_ms(void* start, void* stop, float* ms)
{
    if (!ms) return ASCB200_EINVAL;
    ASCB200_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(stop)));
    ASCB200_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
    return ASCB200_OK;
}

int ascb200_graph_begin(void* stream)
{
    ASCB200_CUDA(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal));
    return ASCB200_OK;
}
int ascb200_graph_end(void* stream, void** graph_exec)
{
    if (!graph_exec) return ASCB200_EINVAL;
    cudaGraph_t g = nullptr;
    ASCB200_CUDA(cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &g));
    cudaGraphExec_t e = nullptr;
    cudaError_t err = cudaGraphInstantiate(&e, g, 0);
    (void)cudaGraphDestroy(g);
    if (err != cudaSuccess) return cuda_fail(err);
    *graph_exec = e;
    return ASCB200_OK;
}
int ascb200_graph_launch(void* graph_exec, void* stream)
{
    ASCB200_CUDA(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph_exec), static_cast<cudaStream_t>(stream)));
    return ASCB200_OK;
}
int ascb200_graph_destroy(void* graph_exec)
{
    ASCB200_CUDA(cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph_exec)));
    return ASCB200_OK;
}

}  // extern "C"
