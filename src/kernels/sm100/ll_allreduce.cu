// Low-latency AllReduce for small messages (up to 128 KiB): no barrier at all. Every rank stores
// each 4-byte word of its input, paired with the number of this call, straight into a slot of
// every rank's receive area (one 8-byte store, which arrives whole). A receiver spins on the slot
// until the call number matches, so the data is its own "ready" flag and the whole exchange costs
// one NVLink crossing instead of the two barrier round-trips of the one-shot kernel. Slots
// alternate between two parities: a rank can be at most one call ahead of a peer (it cannot finish
// a call without that peer's data for it), so a slot is never overwritten while it may still be read.
// Neither input nor output needs to be addressable by peers: only the receive areas are.
//
// The reference has no counterpart (its smallest latency is 2(N-1) ring hops); the idea is the
// flag-in-data "LL" protocol known from NCCL, written here for direct all-to-all exchange.
#include "kernels/sm100/ll_allreduce.h"

#include "kernels/sm100/sync.cuh"
#include "kernels/sm100/vec.cuh"

namespace b200ccl::kernels {

using namespace b200ccl::dev;

namespace {

using u64 = unsigned long long;

__device__ __forceinline__ void st_slot(u64* p, unsigned data, unsigned flag) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(data), "r"(flag) : "memory");
}
__device__ __forceinline__ uint2 ld_slot(const u64* p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

template <typename T>
struct Word;  // one 4-byte word ↔ fp32 lanes
template <>
struct Word<float> {
    static constexpr int kLanes = 1;
    static __device__ __forceinline__ void unpack(unsigned w, float (&f)[1]) { f[0] = __uint_as_float(w); }
    static __device__ __forceinline__ unsigned pack(const float (&f)[1]) { return __float_as_uint(f[0]); }
};
template <>
struct Word<__half> {
    static constexpr int kLanes = 2;
    static __device__ __forceinline__ void unpack(unsigned w, float (&f)[2]) { float2 v = h2_to_f2(w); f[0] = v.x; f[1] = v.y; }
    static __device__ __forceinline__ unsigned pack(const float (&f)[2]) { return f2_to_h2(f[0], f[1]); }
};
template <>
struct Word<__nv_bfloat16> {
    static constexpr int kLanes = 2;
    static __device__ __forceinline__ void unpack(unsigned w, float (&f)[2]) { float2 v = b2_to_f2(w); f[0] = v.x; f[1] = v.y; }
    static __device__ __forceinline__ unsigned pack(const float (&f)[2]) { return f2_to_b2(f[0], f[1]); }
};

template <typename T, typename Op, typename ParamT>
__global__ void __launch_bounds__(kBlockThreads) ll_kernel(const __grid_constant__ ParamT param) {
    const LlArgs* ap;
    if constexpr (sizeof(ParamT) == sizeof(LlArgs)) ap = reinterpret_cast<const LlArgs*>(&param);
    else ap = reinterpret_cast<const LlArgs*>(&param) + blockIdx.y;
    const LlArgs& a = *ap;
    const int n = a.nranks, rank = a.rank;
    // Every thread reads the CTA's call counter; thread 0 writes it back at the end.
    const u64 call = a.own_ctrl->ll_epoch[blockIdx.x] + 1;
    const unsigned flag = static_cast<unsigned>(call % 0xffffffffull) + 1u;  // never 0: a zeroed area matches no call
    const u64 parity = call & 1ull;
    const unsigned* in = static_cast<const unsigned*>(a.in);
    unsigned* out = static_cast<unsigned*>(a.out);
    const unsigned stride = kLlCtas * kBlockThreads;
    const unsigned first = blockIdx.x * kBlockThreads + threadIdx.x;

    // 1. Publish: word w of this rank goes to slot (parity, rank, w) of every rank.
    for (unsigned w = first; w < a.nwords; w += stride) {
        const unsigned v = in[w];
        const u64 slot = (parity * (u64)n + (u64)rank) * kLlMaxWords + w;
        for (int k = 0; k < n; ++k) {
            int q = rank + k;
            if (q >= n) q -= n;
            st_slot(a.area[q] + slot, v, flag);
        }
    }
    // 2. Collect: the slots of all sources are loaded together (n loads in flight), then only the
    //    sources whose call number has not arrived yet are polled again; combine in rank order.
    bool ok = true;
    const u64 t0 = global_timer_ns();
    const u64* own_area = a.area[rank] + parity * (u64)n * kLlMaxWords;
    for (unsigned w = first; ok && w < a.nwords; w += stride) {
        uint2 v[kMaxRanks];
        unsigned pending = (1u << n) - 1u;
        unsigned polls = 0;
        while (pending != 0u) {
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p)
                if (pending & (1u << p)) v[p] = ld_slot(own_area + (u64)p * kLlMaxWords + w);
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p)
                if ((pending & (1u << p)) && v[p].y == flag) pending &= ~(1u << p);
            if (pending != 0u && (++polls & 255u) == 0u) {
                const unsigned who = (unsigned)(__ffs((int)pending) - 1);
                if (ld_volatile_u32(&a.own_ctrl->abort_flag) != 0u) {
                    report_failure(a.status, a.own_ctrl, nullptr, 0, kStatusAborted, who, 20u, call, global_timer_ns() - t0);
                    ok = false;
                    break;
                }
                const u64 waited = global_timer_ns() - t0;
                if (waited > a.timeout_ns) {
                    report_failure(a.status, a.own_ctrl, a.ctrl, n, kStatusTimeout, who, 20u, call, waited);
                    ok = false;
                    break;
                }
            }
        }
        if (!ok) break;
        float acc[Word<T>::kLanes];
        Word<T>::unpack(v[0].x, acc);
#pragma unroll
        for (int p = 1; p < kMaxRanks; ++p) {
            if (p < n) {
                float f[Word<T>::kLanes];
                Word<T>::unpack(v[p].x, f);
#pragma unroll
                for (int e = 0; e < Word<T>::kLanes; ++e) acc[e] = Op::apply(acc[e], f[e]);
            }
        }
        if (a.scale != 1.0f) {
#pragma unroll
            for (int e = 0; e < Word<T>::kLanes; ++e) acc[e] *= a.scale;
        }
        out[w] = Word<T>::pack(acc);
    }
    // A CTA whose wait gave up leaves its counter alone: the communicator is poisoned anyway.
    if (__syncthreads_and(ok ? 1 : 0) && threadIdx.x == 0) a.own_ctrl->ll_epoch[blockIdx.x] = call;
}

template <typename T, typename Op>
cudaError_t launch_ll_t(const LlArgs* args, int loop_ranks, cudaStream_t stream) {
    dim3 grid(kLlCtas, loop_ranks > 0 ? loop_ranks : 1, 1), block(kBlockThreads, 1, 1);
    if (loop_ranks > 0) {
        if (loop_ranks > kMaxRanks) return cudaErrorInvalidValue;
        LoopPack<LlArgs> pack;
        for (int r = 0; r < loop_ranks; ++r) pack.r[r] = args[r];
        void* params[] = {&pack};
        return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(ll_kernel<T, Op, LoopPack<LlArgs>>), grid, block, params, 0, stream);
    }
    ll_kernel<T, Op, LlArgs><<<grid, block, 0, stream>>>(args[0]);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_ll_op(RedOp op, const LlArgs* args, int loop_ranks, cudaStream_t stream) {
    switch (op) {
        case RedOp::Sum:
        case RedOp::Avg: return launch_ll_t<T, OpAdd>(args, loop_ranks, stream);
        case RedOp::Max: return launch_ll_t<T, OpMax>(args, loop_ranks, stream);
        case RedOp::Min: return launch_ll_t<T, OpMin>(args, loop_ranks, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

std::size_t ll_area_bytes(int nranks) { return std::size_t(2) * nranks * kLlMaxWords * sizeof(unsigned long long); }

cudaError_t launch_ll_all_reduce(DType dtype, RedOp op, const LlArgs* args, int loop_ranks, cudaStream_t stream) {
    switch (dtype) {
        case DType::Float: return launch_ll_op<float>(op, args, loop_ranks, stream);
        case DType::Float16: return launch_ll_op<__half>(op, args, loop_ranks, stream);
        case DType::BFloat16: return launch_ll_op<__nv_bfloat16>(op, args, loop_ranks, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace b200ccl::kernels
