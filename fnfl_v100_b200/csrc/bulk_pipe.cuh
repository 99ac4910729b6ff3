// Bulk-copy (TMA) pipeline primitives for sm_100a: mbarrier phases in shared memory and the untiled
// cp.async.bulk global -> shared copy that signals them.  Every kernel here reads only its own GPU's memory and
// every copy is issued by one CTA for itself (no cluster-wide forms).
//
// Waits are bounded: a wait that does not complete within its poll limit records FNB_ERR_TIMEOUT in the caller's
// error word and returns false, and the kernel unwinds instead of spinning forever.  Two limits: the waits of the
// data path (mbar_wait) use kPrimarySpinLimit, the waits a producer makes while unwinding - for the copies it has
// already issued into its shared memory to land before the CTA exits - use kSpinLimit.  They are the same number
// in the product; a build that defines FNB_PRIMARY_SPIN_LIMIT as a few polls makes the data path give up at once
// while the unwinding stays patient, which is how the give-up path is exercised on a GPU without leaving a copy in
// flight.
#pragma once

#include "common.cuh"

namespace fnb {

// A failed poll suspends the thread for up to kPollNs, so the hint is also the granularity with which a waiter
// notices completion: 2 us made a latency-sensitive pipeline (consumers faster than memory) three times slower.
constexpr uint32_t kSpinLimit = 1u << 24;  // polls of at most kPollNs each: about a second in the worst case
#ifndef FNB_PRIMARY_SPIN_LIMIT
#define FNB_PRIMARY_SPIN_LIMIT (1u << 24)
#endif
constexpr uint32_t kPrimarySpinLimit = FNB_PRIMARY_SPIN_LIMIT;
#ifndef FNB_POLL_NS
#define FNB_POLL_NS 64
#endif
constexpr uint32_t kPollNs = FNB_POLL_NS;

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t * bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals) : "memory");
}
// makes freshly initialised barriers visible to the copy engine; follow with a block barrier
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t * bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t * bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t * bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kPollNs)
        : "memory");
    return done != 0;
}
// one look at the barrier without suspending the thread
__device__ __forceinline__ bool mbar_test_wait(uint64_t * bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// bounded wait for the phase with the given parity; false (and FNB_ERR_TIMEOUT in *err) when it gives up.  A build
// with a limit of a few polls looks without suspending (a suspended poll may last as long as the hardware likes,
// which is long enough for a copy to land), so that its waits really run out.
__device__ __forceinline__ bool mbar_wait(uint64_t * bar, uint32_t parity, uint32_t * err) {
    for (uint32_t i = 0; i < kPrimarySpinLimit; ++i) {
        if (kPrimarySpinLimit < 1024u ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
    }
    if (err != nullptr) atomicOr(err, FNB_ERR_TIMEOUT);
    return false;
}
// the unwinding wait: the producer's last look at a stage it has issued a copy into (always the full limit)
__device__ __forceinline__ bool mbar_wait_landed(uint64_t * bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// barrier among the first `threads` threads of the CTA (whole warps) on hardware barrier `id` (1 .. 15; 0 is
// __syncthreads'): lets the consumer warps wait for state only they need while the producer already streams
template <int ID>
__device__ __forceinline__ void named_barrier(int threads) {
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "r"(threads) : "memory");
}

// L2 policy for data that is read once: evict first
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// global -> this CTA's shared memory; src and dst 16-byte aligned, bytes a multiple of 16; completion is
// counted on `bar` in bytes
__device__ __forceinline__ void bulk_g2s(void * dst_smem, const void * src_gmem, uint32_t bytes, uint64_t * bar,
                                         uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

}  // namespace fnb
