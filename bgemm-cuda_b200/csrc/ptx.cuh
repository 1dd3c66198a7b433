// Thin inline-PTX wrappers for sm_100a: mbarrier, bulk/TMA copies, tcgen05 (TMEM + UMMA).
// Every wait in this library is time-bounded: a wait that runs out sets a CTA-wide abort flag and a
// device status word, after which all later waits return at once and the kernel drains and exits.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace bgemm {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Default wait budget in SM clocks (~0.2 s at 2 GHz). Far above any legitimate wait of these kernels.
constexpr long long kWaitBudgetClocks = 400000000LL;
// The budget in force lives in shared memory, 12 bytes behind the CTA's abort flag (8-byte aligned there): the kernel
// prologue stores the default, or the shorter budget a test asked for (bgemm_debug_set_wait_test).
__device__ __forceinline__ long long wait_budget_of(volatile int* abort_flag) {
    return *reinterpret_cast<volatile long long*>(abort_flag + 3);
}
__device__ __forceinline__ void set_wait_budget(volatile int* abort_flag, long long requested) {
    *reinterpret_cast<volatile long long*>(abort_flag + 3) = requested > 0 ? requested : kWaitBudgetClocks;
}

// One blocking probe: the thread is suspended by the hardware (no issue slots burnt) until the phase
// completes or a short, implementation-defined time passes.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait. `abort_flag` lives in shared memory; once any thread sets it every wait falls through.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status_word,
                                          int where) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64(), budget = wait_budget_of(abort_flag);
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > budget) {
            *abort_flag = 1;
            if (status_word) atomicCAS(status_word, 0, where);
            return false;
        }
    }
    return true;
}

// The same for waiters that are not on the critical path (producers waiting for a free stage, epilogue warps waiting
// for the next accumulator): they back off between probes instead of polling, which leaves issue slots and power to
// the warps that feed the tensor pipe.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status_word,
                                                  int where) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64(), budget = wait_budget_of(abort_flag);
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(64);
        if (*abort_flag) return false;
        if (clock64() - t0 > budget) {
            *abort_flag = 1;
            if (status_word) atomicCAS(status_word, 0, where);
            return false;
        }
    }
    return true;
}

// ---- bulk (TMA) copies: every CTA fetches its own tiles -----------------------------------------------
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst_smem),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}
// Orders this thread's generic-proxy accesses to shared memory (ld/st.shared) with async-proxy accesses (TMA, bulk
// copies) that follow in synchronisation order: needed before a TMA store reads what threads wrote, and before a
// buffer that threads have READ is handed back to a producer whose next bulk copy overwrites it -- an mbarrier
// arrive alone does not order the two proxies.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tcgen05: tensor memory + UMMA ---------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t holder_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major shared-memory operand descriptor, 128-byte swizzle: rows 128 B apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;            // leading byte offset (unused for swizzled K-major), encoded 16 B
    d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;            // descriptor version for sm_100
    d |= (uint64_t)2 << 61;            // SWIZZLE_128B
    return d;
}
// kind::i8 instruction descriptor: D = s32, A = u8 (K-major, from TMEM), B = s8 (K-major), M = 128.
__host__ __device__ constexpr uint32_t umma_idesc_u8s8(int n) {
    return (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
// D[tmem_d] (+)= A[tmem_a] * B[smem desc]; A comes from tensor memory (".ts" form).
__device__ __forceinline__ void umma_i8_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(v[0]), "r"(v[1]),
                 "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// ---- register reallocation between the warp groups of a CTA --------------------------------------------------------
// Every warp of a group of four consecutive warps (0-3, 4-7, ...) must execute the same one of these. Registers that one
// group gives up become available to the groups that ask for more (they block until enough have been released).
template <int N>
__device__ __forceinline__ void regs_release() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void regs_request() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

// ---- L2 residency hints ------------------------------------------------------------------------------------------
// Policy for data that is written early in a kernel and read back at its end (partial sums handed between CTAs): keep
// it in L2 while the kernel streams its operands and results through.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void st_global_hint(int* addr, int v, uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.b32 [%0], %1, %2;" ::"l"(addr), "r"(v), "l"(policy) : "memory");
}
__device__ __forceinline__ int ld_global_hint(const int* addr, uint64_t policy) {
    int v;
    asm volatile("ld.global.L2::cache_hint.b32 %0, [%1], %2;" : "=r"(v) : "l"(addr), "l"(policy) : "memory");
    return v;
}

// ---- CTA pairs (cta_group::2): one UMMA over the two SMs of a 2-CTA cluster -----------------------------------------
// Both CTAs allocate (and free) the same tensor-memory columns together; each keeps its own 128 rows of A and D and
// half of the B tile in its own shared memory, and one thread of the even CTA issues the instruction for both.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t holder_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// kind::i8 instruction descriptor for an M-row tile (256 = 128 rows in each CTA of a pair).
__host__ __device__ constexpr uint32_t umma_idesc_u8s8_m(int n, int m) {
    return (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// kind::i8 instruction descriptor with the operand signedness spelled out (0 = u8, 1 = s8), both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_i8(int a_signed, int b_signed, int n, int m) {
    return (2u << 4) | ((uint32_t)a_signed << 7) | ((uint32_t)b_signed << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_i8_ts_pair(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
// Both operands from shared memory (the same descriptors are applied in both CTAs of the pair).
__device__ __forceinline__ void umma_i8_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0)
        : "memory");
}
// Arrival on `bar` (a shared::cluster address: this CTA's or the partner's barrier) once every UMMA this thread has
// issued so far has been executed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}
// The same arrival on the barrier at this offset in every CTA of `cta_mask` (only signals are multicast here; every
// CTA loads its own data).
__device__ __forceinline__ void umma_commit_pair_mask(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(cta_mask)
                 : "memory");
}
// Plain arrival on a barrier anywhere in the cluster (address from mapa_shared).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
// Tile load into this CTA's shared memory whose byte count is credited to a barrier of either CTA of the pair.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst_smem, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst_smem),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar_cluster)
        : "memory");
}

// ---- thread-block cluster: barrier and distributed shared memory ------------------------------------------------
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ int4 ld_dsmem_v4(uint32_t addr) {
    int4 v;
    asm volatile("ld.shared::cluster.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void st_dsmem_s32(uint32_t addr, int v) {
    asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// Programmatic dependent launch: no-ops unless the kernel was launched with the stream-serialization attribute.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ int ld_dsmem_s32(uint32_t addr) {
    int v;
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// Barrier over `nthreads` threads that also ORs a predicate: every participant gets the same answer, so a
// group can leave a loop together when any member has given up.
__device__ __forceinline__ bool named_bar_or(int id, int nthreads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n.reg .pred p, q;\nsetp.ne.b32 q, %3, 0;\nbar.red.or.pred p, %1, %2, q;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(r)
        : "r"(id), "r"(nthreads), "r"((uint32_t)pred)
        : "memory");
    return r != 0;
}

}  // namespace bgemm
