// System-scope signalling between GPUs: release/acquire accesses, a per-CTA barrier across all
// ranks and the bounded wait every spin in this library goes through.
//
// Parity: nano-nccl's ld.acquire.sys / st.release.sys step accessors and its abort poll
// (src/transport/simple/step.h:14-37; wait loops src/kernels/ring_simple_kernel.cuh:586-748).
// Differences: waits are bounded by %globaltimer and end with a status record instead of
// spinning for ever, and flags are monotonic epochs that are never reset.
#pragma once

#include "kernels/sm100/dev_types.h"

namespace b200ccl::dev {

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_volatile_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Records the first failure of this rank and tells every rank to stop waiting.
__device__ __forceinline__ void report_failure(Status* status, ControlBlock* own, ControlBlock* const* ctrl,
                                               int nranks, unsigned int code, unsigned int peer,
                                               unsigned int where, unsigned long long epoch,
                                               unsigned long long waited_ns) {
    // The first failure of a rank is the one recorded; a plan mismatch also replaces an earlier
    // "aborted" record, which is only its echo from another CTA.
    if (status != nullptr && own != nullptr &&
        (atomicCAS(&own->fail_once, 0u, 1u) == 0u || (code == kStatusPlanMismatch && status->code != kStatusPlanMismatch))) {
        status->cta = blockIdx.x;
        status->peer = peer;
        status->where = where;
        status->epoch = epoch;
        status->waited_ns = waited_ns;
        __threadfence_system();
        status->code = code;  // written last: the host treats a non-zero code as "record complete"
        __threadfence_system();
    }
    if ((code == kStatusTimeout || code == kStatusPlanMismatch) && ctrl != nullptr) {
        for (int q = 0; q < nranks; ++q) st_relaxed_sys_u32(&ctrl[q]->abort_flag, 1u);
    }
}

// Spins until *flag >= want. Returns false after `timeout_ns`, or when the local abort flag (or
// `net_abort`, the host word a failed network proxy raises) is set; the caller must then leave
// the kernel. The clock and the abort words are read once every 64 polls.
__device__ __forceinline__ bool wait_at_least(const unsigned long long* flag, unsigned long long want,
                                              ControlBlock* own, unsigned long long timeout_ns,
                                              Status* status, ControlBlock* const* ctrl, int nranks,
                                              unsigned int peer, unsigned int where,
                                              const unsigned int* net_abort = nullptr) {
    const unsigned int* abort_flag = own != nullptr ? &own->abort_flag : nullptr;
    if (ld_acquire_sys(flag) >= want) return true;
    const unsigned long long t0 = global_timer_ns();
    unsigned int polls = 0;
    for (;;) {
        if (ld_acquire_sys(flag) >= want) return true;
        if ((++polls & 63u) == 0u) {
            if ((abort_flag != nullptr && ld_volatile_u32(abort_flag) != 0u) ||
                (net_abort != nullptr && ld_volatile_u32(net_abort) != 0u)) {
                report_failure(status, own, nullptr, 0, kStatusAborted, peer, where, want, global_timer_ns() - t0);
                return false;
            }
            const unsigned long long waited = global_timer_ns() - t0;
            if (waited > timeout_ns) {
                report_failure(status, own, ctrl, nranks, kStatusTimeout, peer, where, want, waited);
                return false;
            }
        }
    }
}

// Barrier among the CTAs with the same blockIdx.x on every rank. Thread p signals rank p and
// waits for rank p. Everything the CTA stored before the call is visible to every rank's CTA
// after it (release on the signal, acquire on the poll, bar.sync on both sides).
// Returns false (to every thread of the CTA) when the wait gave up.
// plan_hash != 0: CTA 0 also publishes the fingerprint of this launch's plan with the signal and
// compares it with every peer's after the wait; a difference ends the collective on every rank
// with kStatusPlanMismatch (the other CTAs leave through the abort word).
__device__ __forceinline__ bool cta_barrier_all_ranks(ControlBlock* const* ctrl, int rank, int nranks,
                                                      unsigned long long epoch, unsigned long long timeout_ns,
                                                      Status* status, unsigned int where,
                                                      unsigned long long plan_hash = 0ull) {
    __syncthreads();
    int ok = 1;
    if (threadIdx.x < (unsigned)nranks) {
        const int p = threadIdx.x;
        const bool check = plan_hash != 0ull && blockIdx.x == 0;
        if (check) st_relaxed_sys(&ctrl[p]->plan_hash[rank], plan_hash);
        st_release_sys(&ctrl[p]->barrier[blockIdx.x][rank], epoch);
        ok = wait_at_least(&ctrl[rank]->barrier[blockIdx.x][p], epoch, ctrl[rank], timeout_ns,
                           status, ctrl, nranks, (unsigned)p, where)
                 ? 1 : 0;
        if (ok && check && ld_relaxed_sys(&ctrl[rank]->plan_hash[p]) != plan_hash) {
            report_failure(status, ctrl[rank], ctrl, nranks, kStatusPlanMismatch, (unsigned)p, where, epoch, 0ull);
            ok = 0;
        }
    }
    return __syncthreads_and(ok) != 0;
}

}  // namespace b200ccl::dev
