// Several GPUs of one box: the shard planners (N-slab for the large GEMMs, expert groups for the grouped matmul; both
// without communication) and the optional all-gather that gives every rank the whole C when it is asked for.
//
// The all-gather is NCCL's (over NVLink / NVSwitch) followed by one local re-layout kernel: column slabs of a row-major C
// are not contiguous, so the slabs arrive as [rank][M][N/ranks] and are interleaved into [M][N] on this GPU.  Every kernel
// here reads and writes this GPU's memory only.  NCCL is looked up at run time (dlopen of libnccl.so.2): hosts that never
// gather need no NCCL, and a process that already loaded one (a framework's bundled copy) shares it.
#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace ascb200 {
namespace {

// ---- NCCL entry points (types declared here: the library must build and load without NCCL's header) ----
typedef struct ncclComm* NcclComm;
struct NcclUniqueId { char internal[128]; };
typedef int (*GetUniqueIdFn)(NcclUniqueId*);
typedef int (*CommInitRankFn)(NcclComm*, int, NcclUniqueId, int);
typedef int (*CommInitAllFn)(NcclComm*, int, const int*);
typedef int (*CommDestroyFn)(NcclComm);
typedef int (*AllGatherFn)(const void*, void*, size_t, int /*ncclDataType_t*/, NcclComm, cudaStream_t);
typedef int (*GroupFn)(void);
constexpr int kNcclInt8 = 0;  // ncclInt8 / ncclChar

struct NcclApi {
    bool ok = false;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    CommInitAllFn comm_init_all = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    AllGatherFn all_gather = nullptr;
    GroupFn group_start = nullptr, group_end = nullptr;
};

const NcclApi& nccl()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        api.get_unique_id = reinterpret_cast<GetUniqueIdFn>(dlsym(h, "ncclGetUniqueId"));
        api.comm_init_rank = reinterpret_cast<CommInitRankFn>(dlsym(h, "ncclCommInitRank"));
        api.comm_init_all = reinterpret_cast<CommInitAllFn>(dlsym(h, "ncclCommInitAll"));
        api.comm_destroy = reinterpret_cast<CommDestroyFn>(dlsym(h, "ncclCommDestroy"));
        api.all_gather = reinterpret_cast<AllGatherFn>(dlsym(h, "ncclAllGather"));
        api.group_start = reinterpret_cast<GroupFn>(dlsym(h, "ncclGroupStart"));
        api.group_end = reinterpret_cast<GroupFn>(dlsym(h, "ncclGroupEnd"));
        api.ok = api.get_unique_id && api.comm_init_rank && api.comm_init_all && api.comm_destroy && api.all_gather && api.group_start && api.group_end;
    });
    return api;
}

// [ranks][m][row_bytes] -> [m][ld_bytes] with slab r at byte r * row_bytes of every row.  One thread moves one vector of V
// bytes; consecutive threads walk along a destination row, so both sides are read and written in whole lines.
template <typename V>
__global__ void __launch_bounds__(256) interleave_slabs_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int ranks, long long m,
                                                               long long row_bytes, long long ld_bytes)
{
    const long long vec_per_row = row_bytes / static_cast<long long>(sizeof(V)) * ranks;
    const long long vec_per_slab_row = row_bytes / static_cast<long long>(sizeof(V));
    const long long total = vec_per_row * m;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long row = i / vec_per_row, v = i % vec_per_row;
        const long long r = v / vec_per_slab_row, c = v % vec_per_slab_row;
        const V val = *reinterpret_cast<const V*>(src + (r * m + row) * row_bytes + c * sizeof(V));
        *reinterpret_cast<V*>(dst + row * ld_bytes + r * row_bytes + c * sizeof(V)) = val;
    }
}

int interleave(const void* gathered, void* full, int ranks, long long m, long long n_loc, long long ld_full, int elem_bytes, cudaStream_t stream)
{
    if (!gathered || !full || ranks <= 0 || m < 0 || n_loc < 0 || elem_bytes <= 0) return ASCB200_EINVAL;
    if (ld_full == 0) ld_full = n_loc * ranks;
    if (ld_full < n_loc * ranks) return ASCB200_EINVAL;
    if (m == 0 || n_loc == 0) return ASCB200_OK;
    const long long row_bytes = n_loc * elem_bytes, ld_bytes = ld_full * elem_bytes;
    const uint8_t* src = static_cast<const uint8_t*>(gathered);
    uint8_t* dst = static_cast<uint8_t*>(full);
    int sms = 148;
    if (DeviceState* st = current_state()) sms = st->sm_count;
    auto grid_for = [&](long long vecs) { return static_cast<int>(std::min<long long>((vecs + 255) / 256, static_cast<long long>(sms) * 16)); };
    if (row_bytes % 16 == 0 && ld_bytes % 16 == 0 && aligned_to(src, 16) && aligned_to(dst, 16)) {
        interleave_slabs_kernel<uint4><<<grid_for(row_bytes / 16 * ranks * m), 256, 0, stream>>>(src, dst, ranks, m, row_bytes, ld_bytes);
    } else if (row_bytes % 4 == 0 && ld_bytes % 4 == 0 && aligned_to(src, 4) && aligned_to(dst, 4)) {
        interleave_slabs_kernel<uint32_t><<<grid_for(row_bytes / 4 * ranks * m), 256, 0, stream>>>(src, dst, ranks, m, row_bytes, ld_bytes);
    } else {
        interleave_slabs_kernel<uint8_t><<<grid_for(row_bytes * ranks * m), 256, 0, stream>>>(src, dst, ranks, m, row_bytes, ld_bytes);
    }
    ASCB200_CUDA(cudaGetLastError());
    return ASCB200_OK;
}

}  // namespace
}  // namespace ascb200

using namespace ascb200;

extern "C" {

int ascb200_shard_nslab(int64_t n, int32_t rank, int32_t world, int32_t align, int64_t* lo, int64_t* hi)
{
    if (n < 0 || world <= 0 || rank < 0 || rank >= world || align <= 0 || !lo || !hi) return ASCB200_EINVAL;
    int64_t per = (n + world - 1) / world;
    per = (per + align - 1) / align * align;
    *lo = std::min<int64_t>(n, static_cast<int64_t>(rank) * per);
    *hi = std::min<int64_t>(n, *lo + per);
    return ASCB200_OK;
}

int ascb200_shard_groups_lpt(const int64_t* counts_host, int32_t groups, int32_t world, int32_t* owner_host)
{
    if (groups < 0 || world <= 0 || (groups > 0 && (!counts_host || !owner_host))) return ASCB200_EINVAL;
    std::vector<int32_t> order(groups);
    for (int32_t g = 0; g < groups; ++g) order[g] = g;
    auto rows = [&](int32_t g) { return std::max<int64_t>(counts_host[g], 0); };
    std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return rows(a) > rows(b); });
    std::vector<int64_t> load(world, 0);
    for (int32_t g : order) {
        const int32_t r = static_cast<int32_t>(std::min_element(load.begin(), load.end()) - load.begin());  // first of the least loaded
        owner_host[g] = r;
        load[r] += rows(g);
    }
    return ASCB200_OK;
}

int ascb200_comm_unique_id(void* id_out)
{
    if (!id_out) return ASCB200_EINVAL;
    const NcclApi& api = nccl();
    if (!api.ok) return ASCB200_EUNSUPPORTED;
    NcclUniqueId id;
    if (api.get_unique_id(&id) != 0) return ASCB200_ECUDA;
    memcpy(id_out, &id, sizeof(id));
    return ASCB200_OK;
}

int ascb200_comm_init(void** comm, int32_t world, int32_t rank, const void* unique_id)
{
    if (!comm || !unique_id || world <= 0 || rank < 0 || rank >= world) return ASCB200_EINVAL;
    const NcclApi& api = nccl();
    if (!api.ok) return ASCB200_EUNSUPPORTED;
    NcclUniqueId id;
    memcpy(&id, unique_id, sizeof(id));
    NcclComm c = nullptr;
    if (api.comm_init_rank(&c, world, id, rank) != 0) return ASCB200_ECUDA;
    *comm = c;
    return ASCB200_OK;
}

int ascb200_comm_init_all(void** comms, int32_t ndev, const int32_t* devices)
{
    if (!comms || ndev <= 0) return ASCB200_EINVAL;
    const NcclApi& api = nccl();
    if (!api.ok) return ASCB200_EUNSUPPORTED;
    std::vector<NcclComm> c(ndev, nullptr);
    std::vector<int> devs(ndev);
    for (int i = 0; i < ndev; ++i) devs[i] = devices ? devices[i] : i;
    if (api.comm_init_all(c.data(), ndev, devs.data()) != 0) return ASCB200_ECUDA;
    for (int i = 0; i < ndev; ++i) comms[i] = c[i];
    return ASCB200_OK;
}

int ascb200_comm_destroy(void* comm)
{
    if (!comm) return ASCB200_OK;
    const NcclApi& api = nccl();
    if (!api.ok) return ASCB200_EUNSUPPORTED;
    return api.comm_destroy(static_cast<NcclComm>(comm)) == 0 ? ASCB200_OK : ASCB200_ECUDA;
}

int ascb200_group_start(void)
{
    const NcclApi& api = nccl();
    if (!api.ok) return ASCB200_EUNSUPPORTED;
    return api.group_start() == 0 ? ASCB200_OK : ASCB200_ECUDA;
}

int ascb200_group_end(void)
{
    const NcclApi& api = nccl();
    if (!api.ok) return ASCB200_EUNSUPPORTED;
    return api.group_end() == 0 ? ASCB200_OK : ASCB200_ECUDA;
}

int ascb200_interleave_slabs(const void* gathered_dev, void* full_dev, int32_t ranks, int64_t m, int64_t n_loc, int64_t ld_full, int32_t elem_bytes,
                             void* stream)
{
    return interleave(gathered_dev, full_dev, ranks, m, n_loc, ld_full, elem_bytes, static_cast<cudaStream_t>(stream));
}

int ascb200_allgather_slabs(void* comm, int32_t ranks, const void* slab_dev, int64_t m, int64_t n_loc, int32_t elem_bytes, void* gathered_dev,
                            void* full_dev, int64_t ld_full, void* stream)
{
    if (!comm || !slab_dev || !gathered_dev || ranks <= 0 || m < 0 || n_loc < 0 || elem_bytes <= 0) return ASCB200_EINVAL;
    const NcclApi& api = nccl();
    if (!api.ok) return ASCB200_EUNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t bytes = static_cast<size_t>(m) * static_cast<size_t>(n_loc) * static_cast<size_t>(elem_bytes);
    if (api.all_gather(slab_dev, gathered_dev, bytes, kNcclInt8, static_cast<NcclComm>(comm), s) != 0) return ASCB200_ECUDA;
    if (!full_dev) return ASCB200_OK;  // the caller wants the slabs as they arrive: [ranks][m][n_loc]
    return interleave(gathered_dev, full_dev, ranks, m, n_loc, ld_full, elem_bytes, s);
}

}  // extern "C"
