// Bulk asynchronous copies (TMA, non-tensor form) and the mbarrier plumbing they need, for
// sm_100a.  Only CTA-local, non-multicast forms are used: global -> this CTA's shared memory
// with completion counted on an mbarrier, and shared -> global tracked by bulk groups.
//
// Rules kept by every user of this header:
//  * both addresses 16-byte aligned, size a multiple of 16 bytes;
//  * every wait is bounded: a wait that runs out records ISPORE_DEV_TIMEOUT in the device
//    status word and the caller unwinds (waits once more for what it has in flight, then
//    returns) instead of spinning forever;
//  * shared memory written by ordinary stores is fenced (fence.proxy.async) before a bulk
//    store reads it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ispore {
namespace tma {

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// Makes a freshly initialised mbarrier visible to the asynchronous proxy.
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One arrival plus the number of bytes the bulk copies bound to this barrier will deliver.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

// One try: true when the phase with the given parity has completed.  A thread that finds it
// incomplete is parked by the hardware until the phase completes or, at the latest, until the
// suspend-time hint (nanoseconds) has passed — without the hint the parking time is a short
// system default and a CTA of waiting threads keeps re-issuing the instruction, which takes issue
// slots from the warps of other CTAs on the SM that have work to do.
#ifndef ISPORE_MBAR_HINT_NS
#define ISPORE_MBAR_HINT_NS 1000000  // 1 ms per try; 0 = no hint
#endif
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
#if ISPORE_MBAR_HINT_NS > 0
    asm volatile(
        "{\n"
        "  .reg .pred p;\n"
        "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "  selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity), "r"(static_cast<uint32_t>(ISPORE_MBAR_HINT_NS))
        : "memory");
#else
    asm volatile(
        "{\n"
        "  .reg .pred p;\n"
        "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "  selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
#endif
    return done != 0;
}

// Bounded wait for the phase with the given parity: kMaxTries parked tries add up to about a
// second (with the 1 ms hint; the un-hinted default parks for far shorter, hence the larger
// count), far beyond any legitimate DRAM latency.
#if ISPORE_MBAR_HINT_NS > 0
constexpr uint32_t kMaxTries = 1024;
#else
constexpr uint32_t kMaxTries = 1u << 20;
#endif
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kMaxTries; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// global -> shared (this CTA), completion reported to `bar` as `bytes` of transaction count.
__device__ __forceinline__ void load(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// shared (this CTA) -> global, joined to the current bulk group of the issuing thread.
__device__ __forceinline__ void store(void* dst_gmem, const void* src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem),
                 "r"(smem_addr(src_smem)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Waits until at most N of this thread's bulk groups still have shared-memory reads pending.
template <int N>
__device__ __forceinline__ void wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Orders ordinary shared-memory writes before later asynchronous-proxy reads of them.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace tma
}  // namespace ispore
