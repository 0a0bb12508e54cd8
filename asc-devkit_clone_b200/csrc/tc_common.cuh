// sm_100a building blocks shared by the tensor-core GEMM kernels: mbarriers with bounded waits,
// TMA tile loads (never with cluster multicast), tcgen05 MMA / TMEM helpers, descriptors.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace ascb200 {
namespace tc {

// ---- bounded waits -------------------------------------------------------------------------
// Every spin in these kernels gives up after a time limit.  The first waiter that gives up sets
// the CTA-wide abort word in shared memory and bit 0 of the device status word; every later wait
// returns at once, all roles leave their loops and the CTA frees its TMEM and exits normally.
// The limit is counted in SM clock cycles (clock64 is a cheap per-SM register; the global
// nanosecond timer costs hundreds of cycles per read and must stay out of the polling path):
// 4e9 cycles is about 2 s at the maximum SM clock and about 3.5 s at the lowest clock seen under load.
constexpr long long kWaitLimitCycles = 4000000000ll;

__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// ---- bulk tensor stores (shared -> global) -----------------------------------------------------
// x * element size must be a multiple of 16 bytes; coordinates are never negative here.
// The lines written are marked evict-first in L2: outputs are written once and should not push the
// operands, which every tile re-reads, out of the cache.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y)
{
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;"
                 :: "l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "l"(policy) : "memory");
}
// Same copy as a reduction: global = global + shared, element-wise in the tensor map's data type.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, uint32_t src, int x, int y)
{
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y) : "memory");
}
// Element-wise maximum / minimum into global memory (enAtomic = 2 / 3); the element type comes from the tensor map.
__device__ __forceinline__ void tma_reduce_max_2d(const CUtensorMap* m, uint32_t src, int x, int y)
{
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.max.tile.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_reduce_min_2d(const CUtensorMap* m, uint32_t src, int x, int y)
{
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.min.tile.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once all but the newest N bulk groups of this thread have finished reading shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
// Makes this thread's shared-memory writes visible to the asynchronous (TMA) proxy.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void ld_shared_v4(uint32_t addr, float& a, float& b, float& c, float& d)
{
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(a), "=f"(b), "=f"(c), "=f"(d) : "r"(addr));
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" :: "r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// One lane of a converged warp (elect.sync).  Unlike a test of the lane index, the compiler knows
// that the guarded code runs on a single thread and keeps its operands in uniform registers, which
// the tcgen05 / TMA instructions take; this shortens the issue path of every such instruction.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred P1;\n"
        "elect.sync _|P1, 0xFFFFFFFF;\n"
        "selp.u32 %0, 1, 0, P1;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// Non-blocking probe of the barrier phase.  try_wait may put the warp to sleep for a hardware-chosen
// interval when the phase is not complete yet; the wake-up costs hundreds of cycles, which the
// two warps that drive the pipeline cannot afford on every K block, so they poll with test_wait.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Slow path shared by both wait flavours: called once every few hundred failed polls.
static __device__ __noinline__ bool mbar_wait_expired(long long t0, volatile uint32_t* abort_smem, uint32_t* status, long long limit = kWaitLimitCycles)
{
    if (*abort_smem) return true;
    if (clock64() - t0 > limit) {
        *abort_smem = 1u;
        atomicOr(status, 1u);
        return true;
    }
    return false;
}
// Returns false when the wait was abandoned (abort already set, or the time limit ran out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_smem, uint32_t* status,
                                          long long limit = kWaitLimitCycles)
{
    if (mbar_test_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t it = 0;
    while (true) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((++it & 1023u) == 0u && mbar_wait_expired(t0, abort_smem, status, limit)) return false;
    }
}

// Same contract, for waits that are expected to last long (an epilogue warp waiting for a whole
// main loop): backs off between polls so that it does not take issue slots from the warps that
// feed the tensor cores.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile uint32_t* abort_smem, uint32_t* status)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t it = 0;
    while (true) {
        __nanosleep(64);
        if (mbar_try_wait(bar, parity)) return true;
        if ((++it & 255u) == 0u && mbar_wait_expired(t0, abort_smem, status)) return false;
    }
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- TMA (tile mode, single CTA destination) ---------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, int x, int y, int z, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}
// Untiled bulk copy global -> shared (16-byte aligned addresses, size multiple of 16).
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

// ---- tcgen05 ---------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrives on `bar` once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- CTA pairs (cta_group::2) -------------------------------------------------------------------
// Two CTAs of a cluster drive one 256-row MMA: each holds its 128 rows of A and half of B's rows in
// its own shared memory, the even CTA (the leader) issues the instructions.  Shared-memory addresses
// of the odd CTA carry bit 24 inside the cluster window; clearing it names the same offset in the leader.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on a barrier that may live in the other CTA of the pair (address in the cluster window).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// The same for an arrival that hands back a TMEM accumulator stage: no data written through the generic proxy is published
// by it (the tcgen05 fence before it orders the TMEM reads), so the default form (release at CTA scope) is enough.  The
// cluster-scope release above first waits until all of the thread's earlier memory traffic is visible across the cluster,
// about 1400 cycles per tile in an epilogue warp.
__device__ __forceinline__ void mbar_arrive_cluster_tmem(uint32_t cluster_bar)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// Waits that observe data written by the other CTA of the pair (acquire at cluster scope).
__device__ __forceinline__ bool mbar_test_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded like mbar_wait; `relaxed` backs off between polls (for waits that are expected to last long).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, bool relaxed, volatile uint32_t* abort_smem, uint32_t* status)
{
    if (mbar_test_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t it = 0;
    while (true) {
        if (relaxed) __nanosleep(64);
        if (mbar_test_wait_cluster(bar, parity)) return true;
        if ((++it & 255u) == 0u && mbar_wait_expired(t0, abort_smem, status)) return false;
    }
}
// The address, in the cluster's shared-memory window, of `addr` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Tile load issued by either CTA of a pair: data lands in the issuing CTA, the bytes are counted on
// the leader's barrier.  No multicast: every CTA fetches exactly the rows it owns.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* m, int x, int y, int z, uint32_t leader_bar)
{
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(leader_bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t leader_bar)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(leader_bar)
                 : "memory");
}
// Pair forms of the block-scaled MMA and of the scale-factor copy: every CTA of the pair copies
// from its own shared memory into its own TMEM.
__device__ __forceinline__ void mma_mxf4_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                              uint32_t sfb_tmem, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t sdesc)
{
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask)
                 : "memory");
}

enum : int { KIND_F16 = 0, KIND_I8 = 1, KIND_MXF4 = 2, KIND_MXF8 = 3 };

template <int KIND>
__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    if constexpr (KIND == KIND_F16) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

template <int KIND>
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    if constexpr (KIND == KIND_F16) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
// Block-scaled fp4: one ue8m0 scale per 32 K elements, two per 64-deep instruction.
__device__ __forceinline__ void mma_mxf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                         uint32_t sfb_tmem, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}
// Shared memory -> TMEM copy of 32 rows x 16 bytes, replicated into the four 32-lane quadrants.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// TMEM -> registers: lane i of the warp reads 32 consecutive 32-bit columns of TMEM lane (base lane + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- lean issue path ---------------------------------------------------------------------------
// One thread feeds the tensor cores; every instruction it spends between two MMAs is time the
// tensor pipe may sit idle.  These forms take descriptors as (low word, high word) pairs so that the
// per-instruction work is one 32-bit add on the low word (start address in 16-byte units).
template <int KIND, bool PAIR>
__device__ __forceinline__ void mma_issue(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                          uint32_t accumulate)
{
#define ASCB200_MMA_ASM(GROUP, KINDSTR)                                                                       \
    asm volatile(                                                                                             \
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"  \
        "setp.ne.b32 p, %6, 0;\n\t"                                                                            \
        "tcgen05.mma.cta_group::" GROUP ".kind::" KINDSTR " [%0], da, db, %5, p;\n\t}"                         \
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)                \
        : "memory")
    if constexpr (KIND == KIND_F16) {
        if constexpr (PAIR) ASCB200_MMA_ASM("2", "f16");
        else ASCB200_MMA_ASM("1", "f16");
    } else {
        if constexpr (PAIR) ASCB200_MMA_ASM("2", "i8");
        else ASCB200_MMA_ASM("1", "i8");
    }
#undef ASCB200_MMA_ASM
}
#ifndef ASCB200_MXF4_KIND
#define ASCB200_MXF4_KIND "mxf4"
#endif
template <bool PAIR>
__device__ __forceinline__ void mma_issue_mxf4(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate)
{
#define ASCB200_MMA_ASM(GROUP)                                                                                \
    asm volatile(                                                                                             \
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"  \
        "setp.ne.b32 p, %8, 0;\n\t"                                                                            \
        "tcgen05.mma.cta_group::" GROUP ".kind::" ASCB200_MXF4_KIND ".block_scale.scale_vec::2X [%0], da, db, %5, [%6], [%7], p;\n\t}" \
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate) \
        : "memory")
    if constexpr (PAIR) ASCB200_MMA_ASM("2");
    else ASCB200_MMA_ASM("1");
#undef ASCB200_MMA_ASM
}
// Block-scaled fp8 (e4m3 / e5m2 operands, one ue8m0 scale per 32 K elements = one per 32-deep instruction).
__device__ __forceinline__ void mma_issue_mxf8(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %8, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, %5, [%6], [%7], p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void sf_copy_issue(uint32_t taddr, uint32_t s_lo, uint32_t s_hi)
{
    if constexpr (PAIR)
        asm volatile("{\n\t.reg .b64 d;\n\tmov.b64 d, {%1, %2};\n\ttcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d;\n\t}" ::"r"(taddr), "r"(s_lo), "r"(s_hi) : "memory");
    else
        asm volatile("{\n\t.reg .b64 d;\n\tmov.b64 d, {%1, %2};\n\ttcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n\t}" ::"r"(taddr), "r"(s_lo), "r"(s_hi) : "memory");
}
template <bool PAIR>
__device__ __forceinline__ void commit_issue(uint32_t bar)
{
    if constexpr (PAIR) tc_commit_pair(bar);
    else tc_commit(bar);
}

// ---- descriptors -----------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
// lbo / sbo in bytes.  K-major tiles: rows of 128 bytes, 8-row groups sbo = 1024 apart, lbo unused.
// MN-major tiles: 128 bytes along M/N per row, 8 k-rows per 1024-byte group (sbo), lbo = distance
// between consecutive 128-byte M/N chunks.
__host__ __device__ constexpr uint64_t smem_desc_sw128(uint32_t lbo, uint32_t sbo)
{
    return (static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16) | (static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32) |
           (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
}
// No-swizzle descriptor (layout type 0) used for the scale-factor copies.
__host__ __device__ constexpr uint64_t smem_desc_noswizzle(uint32_t lbo, uint32_t sbo)
{
    return (static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16) | (static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32) |
           (static_cast<uint64_t>(1) << 46);
}
__device__ __forceinline__ uint64_t desc_at(uint64_t desc_hi, uint32_t smem_addr)
{
    return desc_hi | static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
}

// Instruction descriptor, kind::f16 / kind::i8.  c_fmt: 1 fp32, 2 int32; ab_fmt: f16 0, bf16 1, s8 1.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t c_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn, uint32_t b_mn,
                                                   uint32_t m, uint32_t n)
{
    return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// Instruction descriptor, kind::mxf4 block scaled: e2m1 operands (format 1), ue8m0 scales (bit 23),
// K-major A and B; the scale-factor byte selectors (bits 4-5 for B, 29-30 for A) are added per instruction.
__host__ __device__ constexpr uint32_t make_idesc_mxf4(uint32_t m, uint32_t n)
{
    return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24);
}
// Instruction descriptor, kind::mxf8f6f4 block scaled: operand formats e4m3 = 0, e5m2 = 1; ue8m0 scales (bit 23); the
// scale-factor byte selectors (bits 4-5 for B, 29-30 for A: which of a TMEM column's four bytes) are added per instruction.
__host__ __device__ constexpr uint32_t make_idesc_mxf8(uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn, uint32_t b_mn, uint32_t m, uint32_t n)
{
    return (a_fmt << 7) | (b_fmt << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24);
}

}  // namespace tc
}  // namespace ascb200
