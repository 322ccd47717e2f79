// Direct collectives for sm_100a: AllReduce (one-shot, two-shot, NVLS), ReduceScatter and
// AllGather as single kernels that load and store peer GPUs' memory over NVLink / NVSwitch.
//
// What is fused into the one launch per rank: the cross-GPU barriers, the peer loads, the fp32
// widening and accumulation, the avg 1/N scale, the rounding, the stores to peers (or the
// multimem broadcast), and, for buffers that peers cannot address, the copy into and out of the
// staging arena. No separate elementwise kernel runs.
//
// Parity: replaces nano-nccl's only kernel, ring_simple_kernel (src/kernels/
// ring_simple_kernel.cuh:1118-1237), whose 2(N-1) neighbour hops become two hops (pull the own
// shard from every peer, push the result to every peer) or one (every rank pulls everything).
// The reference's pivot step "reduce + scale + write output + forward" (kernel:433-481) is the
// store_all branch below. Its 4-CTA launch (communicator.cu:1094-1095) becomes a grid sized by
// the tuner.
#include "kernels/sm100/direct_collectives.h"

#include "kernels/sm100/sync.cuh"
#include "kernels/sm100/vec.cuh"

namespace b200ccl::kernels {

using namespace b200ccl::dev;

namespace {

using u64 = unsigned long long;

// A kernel parameter is either one rank's arguments, or (loopback emulation) the arguments of
// every emulated rank, of which the CTA picks the one of rank blockIdx.y.
template <typename A>
__device__ __forceinline__ const A& select_args(const A& one) { return one; }
template <typename A>
__device__ __forceinline__ const A& select_args(const LoopPack<A>& all) { return all.r[blockIdx.y]; }

// Copies the packs first, first+stripe, ... below len, four loads in flight per thread. One side is
// the caller's own buffer (16-byte aligned at most), the other the staging arena.
template <typename P, bool kFromUser>
__device__ __forceinline__ void copy_stripes(void* dst, u64 dst0, const void* src, u64 src0, u64 first, u64 len, u64 stripe) {
    for (u64 j = first; j < len; j += stripe * 4) {
        typename P::Raw v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (j + (u64)u * stripe < len) {
                if constexpr (kFromUser) v[u] = P::load_user(src, src0 + j + (u64)u * stripe);
                else v[u] = P::load(src, src0 + j + (u64)u * stripe);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (j + (u64)u * stripe < len) {
                if constexpr (kFromUser) P::store(dst, dst0 + j + (u64)u * stripe, v[u]);
                else P::store_user(dst, dst0 + j + (u64)u * stripe, v[u]);
            }
        }
    }
}

// Packs in flight per thread and peer: fewer ranks, or narrower packs, leave room for more.
template <int N, int kPackBytes>
struct UnrollFor {
    static constexpr int k16 = N == 0 ? 1 : (N >= 8 ? 1 : (N >= 4 ? 2 : (N >= 2 ? 4 : 8)));
    static constexpr int value = kPackBytes == 32 ? (k16 > 1 ? k16 / 2 : 1) : k16;
};

#if defined(B200CCL_DEBUG_BOUNDS)
// Checking builds: an index beyond the extent that the host passed is recorded (first one wins) and
// the access is skipped; the kernel still runs to its end, so no wait is left hanging.
#define B2_IN_BOUNDS(index, extent, where_)                                                                    \
    ((extent) == 0ull || (index) < (extent) ||                                                                \
     (report_failure(a.status, own, nullptr, 0, kStatusBadArgs, (unsigned)rank, (where_), (index), 0ull), false))
#else
#define B2_IN_BOUNDS(index, extent, where_) true
#endif

// One template for one-shot / two-shot / ReduceScatter / NVLS; the differences are data:
// shard_mode picks the range this rank reduces, store_all picks who receives the result.
template <typename T, typename Op, int N, template <class> class PackT, bool kNvls, typename ParamT>
__global__ void __launch_bounds__(kBlockThreads)
reduce_kernel(const __grid_constant__ ParamT param) {
    using P = PackT<T>;
    using Raw = typename P::Raw;
    constexpr int kElems = P::kElems;
    constexpr int NN = N > 0 ? N : kMaxRanks;
    // For the multimem variant the N slot carries the unroll factor (the rank count is a run-time value there).
    constexpr int kU = kNvls ? (N > 0 ? N : 4) : UnrollFor<N, P::kBytes>::value;

    __shared__ u64 s_epoch;
    const CollArgs& a = select_args(param);

    const int n = (N > 0 && !kNvls) ? N : a.nranks;
    const int rank = a.rank;
    ControlBlock* own = a.ctrl[rank];
    if (threadIdx.x == 0) s_epoch = own->epoch[blockIdx.x];
    __syncthreads();
    u64 epoch = s_epoch;

    const u64 stripe = (u64)gridDim.x * blockDim.x;
    const u64 first = (u64)blockIdx.x * blockDim.x + threadIdx.x;
    const int mode = a.shard_mode;
    const int nshards = mode == kShardWhole ? 1 : n;
    const int mine = mode == kShardWhole ? 0 : rank;
    auto shard_lo = [&](int s) -> u64 { return mode == kShardSplit ? (a.len * (u64)s) / (u64)n : 0; };
    auto shard_len = [&](int s) -> u64 {
        return mode == kShardSplit ? (a.len * (u64)(s + 1)) / (u64)n - (a.len * (u64)s) / (u64)n : a.len;
    };

    // 1. Staged input: this CTA copies exactly the packs that the same-numbered CTA of each
    //    peer will read, so the per-CTA barrier below is all the ordering that is needed.
    if (a.user_in != nullptr) {
        void* stage = const_cast<void*>(a.in[rank]);
        for (int s = 0; s < nshards; ++s) {
            const u64 lo = shard_lo(s), len = shard_len(s);
            const u64 dst0 = lo + (u64)s * a.in_stride, src0 = lo + (u64)s * a.uin_stride;
            copy_stripes<P, true>(stage, dst0, a.user_in, src0, first, len, stripe);
        }
    }

    // 2. Every rank's input is ready (and every rank's previous use of `out` is over).
    ++epoch;
    if (!cta_barrier_all_ranks(a.ctrl, rank, n, epoch, a.timeout_ns, a.status, 1u, a.plan_hash)) return;

    // 3. Reduce the own shard.
    {
        const u64 lo = shard_lo(mine), len = shard_len(mine);
        const u64 in0 = lo + (u64)mine * a.in_stride;
        const u64 out0 = mode == kShardBlocks ? 0 : lo;
        const bool scaled = a.scale != 1.0f;
        if constexpr (kNvls) {
            const uint4* mc_in = static_cast<const uint4*>(a.mc_in) + in0;
            uint4* mc_out = static_cast<uint4*>(a.mc_out) + out0;
            for (u64 j = first; j < len; j += stripe * kU) {
                uint4 r[kU];
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const u64 jj = j + (u64)u * stripe;
                    if (jj < len) r[u] = multimem_ld_reduce_add<T>(mc_in + jj);
                }
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const u64 jj = j + (u64)u * stripe;
                    if (jj < len) {
                        uint4 v = r[u];
                        if (scaled) {
                            float f[kElems];
                            P::unpack(v, f);
#pragma unroll
                            for (int e = 0; e < kElems; ++e) f[e] *= a.scale;
                            v = P::pack(f);
                        }
                        if (a.store_all) multimem_st16(mc_out + jj, v);
                        else P::store(a.out[rank], out0 + jj, v);
                    }
                }
            }
        } else {
            for (u64 j = first; j < len; j += stripe * kU) {
                Raw r[kU][NN];
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const u64 jj = j + (u64)u * stripe;
                    if (jj < len && B2_IN_BOUNDS(in0 + jj, a.in_extent, 30u)) {
#pragma unroll
                        for (int p = 0; p < NN; ++p)
                            if (p < n) r[u][p] = P::load(a.in[p], in0 + jj);
                    }
                }
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const u64 jj = j + (u64)u * stripe;
                    if (jj < len && B2_IN_BOUNDS(in0 + jj, a.in_extent, 30u) && B2_IN_BOUNDS(out0 + jj, a.out_extent, 31u)) {
                        // Fixed order 0..n-1: every rank computes bit-identical results.
                        float acc[kElems];
                        P::unpack(r[u][0], acc);
#pragma unroll
                        for (int p = 1; p < NN; ++p) {
                            if (p < n) {
                                float f[kElems];
                                P::unpack(r[u][p], f);
#pragma unroll
                                for (int e = 0; e < kElems; ++e) acc[e] = Op::apply(acc[e], f[e]);
                            }
                        }
                        if (scaled) {
#pragma unroll
                            for (int e = 0; e < kElems; ++e) acc[e] *= a.scale;
                        }
                        const Raw v = P::pack(acc);
                        if (a.store_all) {
#pragma unroll
                            for (int k = 0; k < NN; ++k) {
                                if (k < n) {
                                    int q = rank + k;  // start with the own copy, then spread over peers
                                    if (q >= n) q -= n;
                                    P::store(a.out[q], out0 + jj, v);
                                }
                            }
                        } else {
                            P::store(a.out[rank], out0 + jj, v);
                        }
                    }
                }
            }
        }
    }

    // 4. Every rank has finished reading inputs and its stores to peers are visible.
    ++epoch;
    if (!cta_barrier_all_ranks(a.ctrl, rank, n, epoch, a.timeout_ns, a.status, 2u)) return;

    // 5. Staged output: copy what the same-numbered CTAs of all ranks stored into the arena.
    if (a.user_out != nullptr) {
        for (int s = 0; s < nshards; ++s) {
            const u64 lo = shard_lo(s), len = shard_len(s);
            copy_stripes<P, false>(a.user_out, lo, a.out[rank], lo, first, len, stripe);
        }
    }
    if (threadIdx.x == 0) own->epoch[blockIdx.x] = epoch;
}

// AllGather: bytes only. push: store the own block into every rank's output; pull: load every
// rank's block into the own output; nvls: one multimem.st per pack reaches every rank.
template <typename RawT, typename ParamT>
__global__ void __launch_bounds__(kBlockThreads)
gather_kernel(const __grid_constant__ ParamT param) {
    __shared__ u64 s_epoch;
    const GatherArgs& a = select_args(param);
    const int n = a.nranks, rank = a.rank;
    ControlBlock* own = a.ctrl[rank];
    if (threadIdx.x == 0) s_epoch = own->epoch[blockIdx.x];
    __syncthreads();
    u64 epoch = s_epoch;
    const u64 stripe = (u64)gridDim.x * blockDim.x;
    const u64 first = (u64)blockIdx.x * blockDim.x + threadIdx.x;
    constexpr bool kWide = sizeof(RawT) == 16;
    auto load = [](const void* base, u64 i) -> RawT {
        if constexpr (kWide) return ld16_stream(static_cast<const uint4*>(base) + i);
        else return *(static_cast<const volatile RawT*>(base) + i);
    };
    auto store = [](void* base, u64 i, RawT v) {
        if constexpr (kWide) st16(static_cast<uint4*>(base) + i, v);
        else static_cast<RawT*>(base)[i] = v;
    };

    if (a.mode == 1 && a.user_in != nullptr) {
        void* stage = const_cast<void*>(a.in[rank]);
        for (u64 j = first; j < a.len; j += stripe) store(stage, j, load(a.user_in, j));
    }
    ++epoch;
    if (!cta_barrier_all_ranks(a.ctrl, rank, n, epoch, a.timeout_ns, a.status, 1u, a.plan_hash)) return;

    if (a.mode == 0) {
        const u64 base = (u64)rank * a.out_stride;
        for (u64 j = first; j < a.len; j += stripe * 2) {
            const u64 j1 = j + stripe;
            RawT v0 = load(a.in[rank], j), v1;
            if (j1 < a.len) v1 = load(a.in[rank], j1);
            for (int k = 0; k < n; ++k) {
                int q = rank + k;
                if (q >= n) q -= n;
                store(a.out[q], base + j, v0);
                if (j1 < a.len) store(a.out[q], base + j1, v1);
            }
        }
    } else if (a.mode == 1) {
        for (int k = 0; k < n; ++k) {
            int p = rank + k;
            if (p >= n) p -= n;
            const u64 base = (u64)p * a.out_stride;
            for (u64 j = first; j < a.len; j += stripe * 4) {
                RawT v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (j + u * stripe < a.len) v[u] = load(a.in[p], j + u * stripe);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (j + u * stripe < a.len) store(a.out[rank], base + j + u * stripe, v[u]);
            }
        }
    } else {
        if constexpr (kWide) {
            uint4* mc = static_cast<uint4*>(a.mc_out) + (u64)rank * a.out_stride;
            for (u64 j = first; j < a.len; j += stripe) multimem_st16(mc + j, load(a.in[rank], j));
        }
    }

    ++epoch;
    if (!cta_barrier_all_ranks(a.ctrl, rank, n, epoch, a.timeout_ns, a.status, 2u)) return;
    if (threadIdx.x == 0) own->epoch[blockIdx.x] = epoch;
}

// ---- launch helpers ------------------------------------------------------------------------

template <typename ParamT>
cudaError_t launch(void (*kernel)(ParamT), const ParamT& param, const LaunchConfig& cfg) {
    dim3 grid(cfg.grid, cfg.loop_ranks > 0 ? cfg.loop_ranks : 1, 1);
    dim3 block(cfg.block, 1, 1);
    if (cfg.loop_ranks > 0) {
        // The emulated ranks wait for one another inside one launch: all CTAs must be resident,
        // which a cooperative launch checks.
        void* params[] = {const_cast<ParamT*>(&param)};
        return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, params, 0,
                                           cfg.stream);
    }
    kernel<<<grid, block, 0, cfg.stream>>>(param);
    return cudaGetLastError();
}

template <typename T, typename Op, template <class> class PackT, bool kNvls, typename ParamT>
cudaError_t launch_reduce_n(int nranks, const ParamT& param, const LaunchConfig& cfg) {
    if constexpr (kNvls) {
        if (cfg.nvls_unroll >= 8) return launch(reduce_kernel<T, Op, 8, PackT, true, ParamT>, param, cfg);
        if (cfg.nvls_unroll <= 1) return launch(reduce_kernel<T, Op, 1, PackT, true, ParamT>, param, cfg);
        if (cfg.nvls_unroll <= 2) return launch(reduce_kernel<T, Op, 2, PackT, true, ParamT>, param, cfg);
        return launch(reduce_kernel<T, Op, 4, PackT, true, ParamT>, param, cfg);
    } else if constexpr (PackT<T>::kBytes < 16) {
        return launch(reduce_kernel<T, Op, 0, PackT, false, ParamT>, param, cfg);
    } else {
        switch (nranks) {
            case 1: return launch(reduce_kernel<T, Op, 1, PackT, false, ParamT>, param, cfg);
            case 2: return launch(reduce_kernel<T, Op, 2, PackT, false, ParamT>, param, cfg);
            case 4: return launch(reduce_kernel<T, Op, 4, PackT, false, ParamT>, param, cfg);
            case 8: return launch(reduce_kernel<T, Op, 8, PackT, false, ParamT>, param, cfg);
            default: return launch(reduce_kernel<T, Op, 0, PackT, false, ParamT>, param, cfg);
        }
    }
}

template <typename T, template <class> class PackT, typename ParamT>
cudaError_t launch_reduce_op(RedOp op, int nranks, const ParamT& param, const LaunchConfig& cfg) {
    switch (op) {
        case RedOp::Sum:
        case RedOp::Avg: return launch_reduce_n<T, OpAdd, PackT, false>(nranks, param, cfg);
        case RedOp::Max: return launch_reduce_n<T, OpMax, PackT, false>(nranks, param, cfg);
        case RedOp::Min: return launch_reduce_n<T, OpMin, PackT, false>(nranks, param, cfg);
    }
    return cudaErrorInvalidValue;
}

template <typename T, typename ParamT>
cudaError_t launch_reduce_pack(RedOp op, int pack_bytes, int n, const ParamT& param, const LaunchConfig& cfg) {
    if (pack_bytes == 32) return launch_reduce_op<T, Wide32>(op, n, param, cfg);
    if (pack_bytes == 16) return launch_reduce_op<T, Wide>(op, n, param, cfg);
    return launch_reduce_op<T, Narrow>(op, n, param, cfg);
}

template <typename T>
cudaError_t launch_reduce_t(RedOp op, int pack_bytes, bool nvls, const CollArgs* args, const LaunchConfig& cfg) {
    const int n = args[0].nranks;
    if (cfg.loop_ranks > 0) {
        if (nvls || cfg.loop_ranks > kMaxRanks) return cudaErrorInvalidValue;
        LoopPack<CollArgs> pack;
        for (int r = 0; r < cfg.loop_ranks; ++r) pack.r[r] = args[r];
        return launch_reduce_pack<T>(op, pack_bytes, n, pack, cfg);
    }
    if (nvls) {
        if (pack_bytes != 16 || (op != RedOp::Sum && op != RedOp::Avg)) return cudaErrorInvalidValue;
        return launch_reduce_n<T, OpAdd, Wide, true>(n, args[0], cfg);
    }
    return launch_reduce_pack<T>(op, pack_bytes, n, args[0], cfg);
}

template <typename RawT>
cudaError_t launch_gather_t(const GatherArgs* args, const LaunchConfig& cfg) {
    if (cfg.loop_ranks > 0) {
        if (cfg.loop_ranks > kMaxRanks) return cudaErrorInvalidValue;
        LoopPack<GatherArgs> pack;
        for (int r = 0; r < cfg.loop_ranks; ++r) pack.r[r] = args[r];
        return launch(gather_kernel<RawT, LoopPack<GatherArgs>>, pack, cfg);
    }
    return launch(gather_kernel<RawT, GatherArgs>, args[0], cfg);
}

}  // namespace

cudaError_t launch_reduce(DType dtype, RedOp op, int pack_bytes, bool nvls, const CollArgs* args,
                          const LaunchConfig& cfg) {
    if (pack_bytes != 32 && pack_bytes != 16 && pack_bytes != static_cast<int>(dtype_size(dtype))) return cudaErrorInvalidValue;
    switch (dtype) {
        case DType::Float: return launch_reduce_t<float>(op, pack_bytes, nvls, args, cfg);
        case DType::Float16: return launch_reduce_t<__half>(op, pack_bytes, nvls, args, cfg);
        case DType::BFloat16: return launch_reduce_t<__nv_bfloat16>(op, pack_bytes, nvls, args, cfg);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_gather(const GatherArgs* args, const LaunchConfig& cfg) {
    if (args[0].mode == 2 && (args[0].pack_bytes != 16 || cfg.loop_ranks > 0)) return cudaErrorInvalidValue;
    switch (args[0].pack_bytes) {
        case 16: return launch_gather_t<uint4>(args, cfg);
        case 4: return launch_gather_t<unsigned int>(args, cfg);
        case 2: return launch_gather_t<unsigned short>(args, cfg);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace b200ccl::kernels

// ---------------------------------------------------------------------------------------------
// Allocation-free single-GPU all-reduce (declaration and contract: kernels/sm100/no_alloc.h).
// Same kernel as the communicator's single-GPU emulation; the control blocks live in the array
// below instead of in memory obtained from the driver.

#include "kernels/sm100/no_alloc.h"

#include <cstdint>
#include <cstring>
#include <mutex>
#include <string>

namespace b200ccl::kernels {
// Message of the calling thread's last failure, shared with the C interface (b2_last_error).
void set_last_error_message(const std::string& message);
}  // namespace b200ccl::kernels

namespace {

// The scratch: one control block per emulated rank. In host code this name is only a stand-in
// for the device object; its device address is obtained once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_no_alloc_scratch[B2_NO_ALLOC_MAX_RANKS * sizeof(b200ccl::dev::ControlBlock)];

constexpr int kNoAllocMaxDevices = 64;
std::mutex g_no_alloc_mutex;
void* g_no_alloc_address[kNoAllocMaxDevices] = {nullptr};  // device address of the array, per device ordinal

// Device address of the scratch array on the current device (resolved on first use).
cudaError_t no_alloc_scratch_address(void** out) {
    int device = 0;
    cudaError_t st = cudaGetDevice(&device);
    if (st != cudaSuccess) return st;
    if (device < 0 || device >= kNoAllocMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_no_alloc_mutex);
    if (g_no_alloc_address[device] == nullptr) {
        void* ptr = nullptr;
        st = cudaGetSymbolAddress(&ptr, g_no_alloc_scratch);
        if (st != cudaSuccess) return st;
        g_no_alloc_address[device] = ptr;
    }
    *out = g_no_alloc_address[device];
    return cudaSuccess;
}

}  // namespace

extern "C" int b2_local_all_reduce_no_alloc(const void* const* inputs, void* const* outputs, int nranks, size_t count,
                                            int dtype, int redop, void* stream, void* status_record) {
    using namespace b200ccl;
    using namespace b200ccl::dev;
    auto reject = [](const std::string& why) {
        kernels::set_last_error_message("b2_local_all_reduce_no_alloc: " + why);
        return 2;
    };
    if (nranks < 1 || nranks > B2_NO_ALLOC_MAX_RANKS)
        return reject("nranks = " + std::to_string(nranks) + " is outside 1.." + std::to_string(B2_NO_ALLOC_MAX_RANKS) +
                      " (the fixed scratch array holds " + std::to_string(B2_NO_ALLOC_MAX_RANKS) + " control blocks)");
    if (count == 0) return reject("count must be positive");
    if (dtype < 0 || dtype > 2) return reject("unsupported dtype");
    if (redop < 0 || redop > 3) return reject("unknown reduction operator");
    if (inputs == nullptr || outputs == nullptr) return reject("inputs and outputs must be non-null");
    const std::size_t elem_bytes = dtype_size(static_cast<DType>(dtype));
    if (count > SIZE_MAX / elem_bytes) return reject("count * element size does not fit in size_t");
    const std::size_t span = count * elem_bytes;
    // Byte ranges [ptr, ptr + span) of two buffers share at least one byte.
    auto overlap = [span](const void* a, const void* b) {
        const std::uintptr_t x = reinterpret_cast<std::uintptr_t>(a), y = reinterpret_cast<std::uintptr_t>(b);
        return x < y ? y - x < span : x - y < span;
    };
    for (int r = 0; r < nranks; ++r) {
        if (inputs[r] == nullptr || outputs[r] == nullptr) return reject("every buffer must be non-null");
        if (reinterpret_cast<std::uintptr_t>(inputs[r]) > UINTPTR_MAX - span ||
            reinterpret_cast<std::uintptr_t>(outputs[r]) > UINTPTR_MAX - span)
            return reject("a buffer's byte range wraps around the address space");
    }
    for (int r = 0; r < nranks; ++r) {
        for (int q = 0; q < nranks; ++q) {
            if (inputs[r] == outputs[q]) return reject("in-place operation is not supported");
            if (overlap(inputs[r], outputs[q]))
                return reject("input " + std::to_string(r) + " and output " + std::to_string(q) + " overlap");
            if (q > r && overlap(outputs[r], outputs[q]))
                return reject("outputs " + std::to_string(r) + " and " + std::to_string(q) + " overlap");
        }
    }
    void* scratch = nullptr;
    cudaError_t st = no_alloc_scratch_address(&scratch);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps the previous call's flags, epochs and abort word: start from zero.
    if (st == cudaSuccess) st = cudaMemsetAsync(scratch, 0, sizeof(ControlBlock) * B2_NO_ALLOC_MAX_RANKS, s);
    if (st != cudaSuccess) {
        kernels::set_last_error_message(std::string("b2_local_all_reduce_no_alloc: ") + cudaGetErrorString(st));
        (void)cudaGetLastError();
        return 1;
    }
    const DType dt = static_cast<DType>(dtype);
    const RedOp op = static_cast<RedOp>(redop);
    const std::size_t esz = dtype_size(dt);
    bool wide = (count * esz) % 16 == 0;
    for (int r = 0; r < nranks; ++r)
        wide = wide && ((reinterpret_cast<std::uintptr_t>(inputs[r]) | reinterpret_cast<std::uintptr_t>(outputs[r])) & 15u) == 0;
    const std::size_t pack = wide ? 16 : esz;
    const std::size_t bytes = count * esz;
    const bool oneshot = bytes <= (std::size_t(256) << 10);
    CollArgs args[B2_NO_ALLOC_MAX_RANKS];
    for (int r = 0; r < nranks; ++r) {
        CollArgs& a = args[r];
        std::memset(&a, 0, sizeof(a));
        for (int p = 0; p < nranks; ++p) {
            a.ctrl[p] = reinterpret_cast<ControlBlock*>(static_cast<unsigned char*>(scratch) + sizeof(ControlBlock) * p);
            a.in[p] = inputs[p];
            a.out[p] = oneshot ? nullptr : outputs[p];
        }
        a.out[r] = outputs[r];
        a.status = static_cast<Status*>(status_record);
        a.timeout_ns = static_cast<unsigned long long>(B2_NO_ALLOC_WAIT_MS) * 1000000ull;
        a.scale = op == RedOp::Avg ? 1.0f / static_cast<float>(nranks) : 1.0f;
        a.rank = r;
        a.nranks = nranks;
        a.len = bytes / pack;
        a.shard_mode = oneshot ? kShardWhole : kShardSplit;
        a.store_all = oneshot ? 0 : 1;
    }
    kernels::LaunchConfig cfg;
    const std::size_t per_cta = std::size_t(32) << 10;
    const std::size_t work = oneshot ? bytes : bytes / nranks;
    std::size_t grid = (work + per_cta - 1) / per_cta;
    const std::size_t cap = static_cast<std::size_t>(128 / nranks > 0 ? 128 / nranks : 1);
    cfg.grid = static_cast<int>(grid < 1 ? 1 : (grid > cap ? cap : grid));
    cfg.block = kBlockThreads;
    cfg.stream = s;
    cfg.loop_ranks = nranks;
    st = kernels::launch_reduce(dt, op, static_cast<int>(pack), false, args, cfg);
    if (st != cudaSuccess) {
        kernels::set_last_error_message(std::string("b2_local_all_reduce_no_alloc: launch failed: ") + cudaGetErrorString(st));
        (void)cudaGetLastError();
        return 1;
    }
    return 0;
}
