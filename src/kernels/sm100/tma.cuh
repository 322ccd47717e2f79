// Bulk asynchronous copies (TMA, untiled form) and the mbarrier that tracks them.
// Only the plain forms are used: global → shared::cta (completion on an mbarrier of the same CTA)
// and shared::cta → global (bulk async-group), both on this GPU's own memory. No multicast
// qualifier appears anywhere in this library.
// Both addresses must be 16-byte aligned and the size a multiple of 16 bytes.
#pragma once

#include <cstdint>

namespace b200ccl::dev {

__device__ __forceinline__ unsigned smem_addr(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait: returns false when the phase did not complete within `max_polls` tries.
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, unsigned parity, unsigned max_polls) {
    for (unsigned i = 0; i < max_polls; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global → shared bulk copy; completes `bytes` transaction bytes on `bar`.
__device__ __forceinline__ void tma_load_bulk(void* smem_dst, const void* gmem_src, unsigned bytes,
                                              unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// shared -> global bulk copy, tracked by the thread's bulk async-group.
__device__ __forceinline__ void tma_store_bulk(void* gmem_dst, const void* smem_src, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_addr(smem_src)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void tma_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most kPending of the thread's bulk groups have not finished READING their source.
template <int kPending>
__device__ __forceinline__ void tma_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
// Waits until at most kPending of the thread's bulk groups have not COMPLETED (writes performed).
template <int kPending>
__device__ __forceinline__ void tma_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kPending) : "memory");
}
// Waits until every bulk group of the thread has completed (its writes are performed).
__device__ __forceinline__ void tma_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Orders this thread's earlier generic-proxy accesses before later async-proxy (TMA) accesses.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

}  // namespace b200ccl::dev
