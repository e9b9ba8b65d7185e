// PTX wrappers shared by the tensor-core kernels (sm_100a): mbarriers with bounded waits, TMA bulk
// tensor copies (never with cluster multicast), tcgen05 MMA / commit / TMEM allocation and loads,
// shared-memory matrix descriptors.
#pragma once

#include "pg_internal.h"

#ifndef PG_SUSPEND_HINT_NS
#define PG_SUSPEND_HINT_NS 1000
#endif

namespace pgb {

constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;   // every wait gives up after 2 s

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bar is a shared::cluster address (possibly of the peer CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive on a barrier of another CTA of the cluster, publishing this thread's earlier writes to that CTA's
// shared memory (release at cluster scope); bar is a shared::cluster address.
__device__ __forceinline__ void mbar_arrive_release_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One try of a wait whose completion makes other CTAs' writes to this CTA's shared memory visible.
__device__ __forceinline__ uint32_t mbar_try_acquire_cluster(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Upper bound, in nanoseconds, that the hardware may keep a waiting thread suspended inside one
// try_wait before it returns "not yet" (a hint; the wait still ends as soon as the phase completes).
constexpr uint32_t g_suspend_hint_ns = PG_SUSPEND_HINT_NS;

// Spins on try_wait inside one asm block (so that the compiler sees straight-line, warp-uniform
// code around it) for at most `tries` attempts; returns 1 if the phase completed.
__device__ __forceinline__ uint32_t mbar_spin(uint32_t bar, uint32_t parity, uint32_t tries) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b32 n;\n\t"
        "mov.b32 n, %3;\n"
        "PG_WAIT_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %4;\n\t"
        "@p bra PG_WAIT_DONE;\n\t"
        "sub.u32 n, n, 1;\n\t"
        "setp.ne.u32 p, n, 0;\n\t"
        "@p bra PG_WAIT_LOOP;\n\t"
        "setp.ne.u32 p, n, 0;\n"          // n == 0 here: p = false
        "PG_WAIT_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(tries), "r"(g_suspend_hint_ns)
        : "memory");
    return done;
}
// The same with a caller-chosen suspend hint.
__device__ __forceinline__ uint32_t mbar_spin_hint(uint32_t bar, uint32_t parity, uint32_t tries, uint32_t hint_ns) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b32 n;\n\t"
        "mov.b32 n, %3;\n"
        "PG_WAITH_LOOP:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %4;\n\t"
        "@p bra PG_WAITH_DONE;\n\t"
        "sub.u32 n, n, 1;\n\t"
        "setp.ne.u32 p, n, 0;\n\t"
        "@p bra PG_WAITH_LOOP;\n\t"
        "setp.ne.u32 p, n, 0;\n"
        "PG_WAITH_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(tries), "r"(hint_ns)
        : "memory");
    return done;
}
// Bounded wait, executed by a whole (converged) warp; the result is the same in every lane.
// Returns false when the CTA is aborting (this or another wait ran out of time).
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                            uint32_t *status, uint32_t err_bit) {
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        const uint32_t done = mbar_spin(bar, parity, 1024);
        if (__all_sync(0xffffffffu, done)) return true;
        uint32_t give_up = *abort_flag;
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) give_up = 1;
        if (__any_sync(0xffffffffu, give_up)) {
            if ((threadIdx.x & 31) == 0) {
                *abort_flag = 1;
                atomicOr(status, err_bit);
            }
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t *status, uint32_t err_bit) {
    const uint32_t done = mbar_spin(bar, parity, 1u << 14);
    if (__all_sync(0xffffffffu, done)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, err_bit);
}
// For hand-overs whose latency is on the critical path (a consumer that starts as soon as its producer
// signals): the hardware may keep a waiting thread suspended for up to the hint before it looks again, so
// the hint is a few tens of nanoseconds here.
__device__ __forceinline__ bool mbar_wait_quick(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                                uint32_t *status, uint32_t err_bit, uint32_t hint_ns) {
    const uint32_t done = mbar_spin_hint(bar, parity, 1u << 16, hint_ns);
    if (__all_sync(0xffffffffu, done)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status, err_bit);
}
// For waits that normally last tens of microseconds (the epilogue waiting for a whole main loop):
// sleep between polls so that the waiting warps do not burn issue slots and power.
__device__ __forceinline__ bool mbar_wait_patient(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                                  uint32_t *status, uint32_t err_bit) {
    uint32_t done = mbar_spin(bar, parity, 4);
    if (__all_sync(0xffffffffu, done)) return true;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        __nanosleep(256);
        done = mbar_spin(bar, parity, 2);
        if (__all_sync(0xffffffffu, done)) return true;
        uint32_t give_up = *abort_flag;
        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) give_up = 1;
        if (__any_sync(0xffffffffu, give_up)) {
            if ((threadIdx.x & 31) == 0) {
                *abort_flag = 1;
                atomicOr(status, err_bit);
            }
            return false;
        }
    }
}
// One lane per warp, chosen by the hardware; unlike `lane == 0` the compiler knows the enclosing
// code stays warp-uniform, which lets descriptors and loop state live in uniform registers.
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
        "elect.sync rx|px, 0xFFFFFFFF;\n\t"
        "@px mov.s32 %0, 1;\n\t}"
        : "+r"(pred));
    return pred;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    if constexpr (CG == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (CG == 1)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    if constexpr (CG == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]
template <int CG>
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (CG == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Same, with each 64-bit descriptor passed as its two 32-bit halves (the high half is constant for
// an operand; only the address field in the low half moves), which keeps the issuing thread's
// arithmetic in 32 bits.
template <int CG>
__device__ __forceinline__ void umma_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                          uint32_t idesc, uint32_t accumulate) {
    if constexpr (CG == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\tsetp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\tsetp.ne.b32 p, %6, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on `bar` (same offset in every CTA of the pair) once all MMAs issued so far have completed.
template <int CG>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    if constexpr (CG == 1) {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    } else {
        const uint16_t mask = 3;  // both CTAs of the pair
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     ::"r"(bar), "h"(mask) : "memory");
    }
}

// L2 eviction-priority policies for the bulk copies
__device__ __forceinline__ uint64_t l2_policy(int kind) {   // 0 normal, 1 evict_first, 2 evict_last
    uint64_t pol;
    if (kind == 1) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    else if (kind == 2) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    else asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// TMA tile load global -> shared, completion counted on `bar` (for CG == 2 the barrier of the
// leader CTA, a shared::cluster address).
template <int CG>
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int32_t c0, int32_t c1, int32_t c2, uint64_t policy) {
    if constexpr (CG == 1)
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
            " [%0], [%1, {%3, %4, %5}], [%2], %6;"
            ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy) : "memory");
    else
        asm volatile(
            "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
            " [%0], [%1, {%3, %4, %5}], [%2], %6;"
            ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int32_t c0, int32_t c1, int32_t c2,
                                             uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3, %4}], [%1], %5;"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "l"(policy) : "memory");
}
// C tile += smem tile, performed by the TMA unit in L2
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap *map, uint32_t src, int32_t c0, int32_t c1, int32_t c2) {
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a 128-byte-swizzled tile (version 1 = Blackwell).
//   K-major : rows of 64 elements (128 B), 8-row groups 1024 B apart (SBO), LBO unused.
//   MN-major: [MN/64 chunks][BK k-rows][64 elements]; k-rows 128 B apart, 8-k groups 1024 B apart
//             (SBO), chunks BK*128 B apart (LBO).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;   // descriptor version
    d |= (uint64_t)2 << 61;   // SWIZZLE_128B
    return d;
}


}  // namespace pgb
