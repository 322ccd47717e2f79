// Ring collectives over Simple-protocol FIFOs for sm_100a.
//
// One CTA per channel. Data moves in slices through per-edge FIFOs that live in the receiver's
// memory (peer stores over NVLink) or in mapped host memory (SHM, socket and RDMA edges). Flow
// control is two monotonically growing step counters per edge, published with st.release.sys and
// polled with ld.acquire.sys; counters persist from launch to launch. The local operand of a
// reduce slice is prefetched into shared memory with bulk asynchronous copies (TMA) that are
// issued BEFORE the thread waits for the neighbour, so the local HBM read overlaps the wait.
//
// Parity: nano-nccl src/kernels/ring_simple_kernel.cuh:1118-1237 (schedule 1170-1230:
// direct_send, recv_reduce_send, recv_reduce_copy_send with the fused avg scale, recv_copy_send,
// direct_recv; credit rule 597-634; empty-slice elision 853-859; persistent steps 1152-1163,
// 1232-1236; abort poll 594-611). Differences: channel count is a run-time value; 16-bit types
// accumulate in fp32; every wait is bounded; ReduceScatter and AllGather schedules exist.
#include "kernels/sm100/ring_simple.h"

#include "kernels/sm100/sync.cuh"
#include "kernels/sm100/tma.cuh"
#include "kernels/sm100/vec.cuh"
#include "sched/ring_geometry.h"

namespace b200ccl::kernels {

using namespace b200ccl::dev;

namespace {

using u64 = unsigned long long;

constexpr int kRingThreads = 512;
constexpr unsigned kTileBytes = 32768;          // one TMA tile of the local operand
constexpr unsigned kTileVecs = kTileBytes / 16;
constexpr unsigned kMbarPolls = 1u << 24;       // bound on waiting for an own TMA copy

enum SliceFlags : unsigned {
    kRecv = 1u,        // take the slice from the incoming FIFO
    kLocal = 2u,       // take (or combine with) the local input
    kSend = 4u,        // forward into the outgoing FIFO
    kCopyOut = 8u,     // write into the local output
    kScale = 16u,      // multiply by args.scale before writing (avg, at the pivot only)
};

__device__ __forceinline__ uint4 ld16_volatile(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

struct ChannelState {
    RingChannel ch;
    u64 send_step;
    u64 recv_step;
};

struct Shared {
    alignas(128) unsigned char tile[2][kTileBytes];
    alignas(8) u64 mbar[2];
    u64 base_steps[2];
};

// Waits of the two flow-control threads; the outcome is shared through smem.
template <typename T>
__device__ __forceinline__ bool wait_flags(const RingArgs& a, ChannelState& st, unsigned flags, Shared& sm,
                                           u64& t_wait_recv, u64& t_wait_send) {
    int ok = 1;
    if ((flags & kRecv) && threadIdx.x == 0) {
        const u64 t0 = st.ch.stats ? global_timer_ns() : 0;
        ok = wait_at_least(st.ch.recv_tail, st.recv_step + ring::kSliceSteps, a.own_ctrl, a.timeout_ns, a.status, nullptr,
                           0, (unsigned)((a.rank + a.nranks - 1) % a.nranks), 10u, st.ch.abort_word) ? 1 : 0;
        if (ok && st.ch.abort_word && ld_volatile_u32(st.ch.abort_word) != 0u) ok = 0;
        if (st.ch.stats) t_wait_recv += global_timer_ns() - t0;
    }
    if ((flags & kSend) && threadIdx.x == 32) {
        const u64 t0 = st.ch.stats ? global_timer_ns() : 0;
        // credit: head + kFifoSteps >= step + kSliceSteps
        const u64 want = st.send_step + ring::kSliceSteps >= (u64)ring::kFifoSteps
                             ? st.send_step + ring::kSliceSteps - ring::kFifoSteps : 0;
        ok = wait_at_least(st.ch.send_head, want, a.own_ctrl, a.timeout_ns, a.status, nullptr, 0,
                           (unsigned)((a.rank + 1) % a.nranks), 11u, st.ch.abort_word) ? 1 : 0;
        if (ok && st.ch.abort_word && ld_volatile_u32(st.ch.abort_word) != 0u) ok = 0;
        if (st.ch.stats) t_wait_send += global_timer_ns() - t0;
    }
    return __syncthreads_and(ok) != 0;
}

// One slice: wait, move/combine `n` elements, publish. Returns false when a wait gave up.
template <typename T, typename Op, bool kWide>
__device__ bool run_slice(const RingArgs& a, ChannelState& st, Shared& sm, unsigned (&phase)[2], unsigned flags,
                          const T* local_in, T* local_out, u64 n) {
    if (n == 0) {  // empty slice: neither side waits, posts or advances
        if (st.ch.stats && threadIdx.x == 0) atomicAdd(&st.ch.stats->empty_slices, 1ull);
        return true;
    }
    const bool recv = flags & kRecv, send = flags & kSend, local = flags & kLocal, copy_out = flags & kCopyOut;
    const bool scaled = (flags & kScale) && a.scale != 1.0f;
    const T* fifo_in = recv ? static_cast<const T*>(st.ch.recv_fifo) + ring::slot_offset(st.recv_step, a.step_elems) : nullptr;
    T* fifo_out = send ? static_cast<T*>(st.ch.send_fifo) + ring::slot_offset(st.send_step, a.step_elems) : nullptr;
    u64 t_wait_recv = 0, t_wait_send = 0, t0 = 0;
    // Small received slices (one 16-byte vector per thread at most) return their FIFO slot to the
    // sender BEFORE they are combined and forwarded: the slot is read into registers, the credit is
    // posted, and only then does the slice go on. On host-memory and network edges, where a credit
    // takes microseconds to arrive, this takes the consumer's own work off the sender's critical path.
    // Parity: the reference's early-credit path for slices of at most 4096 bytes
    // (src/kernels/ring_simple_kernel.cuh:486-583, 912-927).
    bool early = false;

    bool ok = true;
    if constexpr (kWide) {
        constexpr int kElems = 16 / sizeof(T);
        const u64 nvec = n / kElems;  // wide path: n is a whole number of vectors
        const bool staged = local && recv;  // prefetch the local operand while waiting for the neighbour
        const unsigned ntiles = staged ? (unsigned)((nvec + kTileVecs - 1) / kTileVecs) : 0;
        auto issue = [&](unsigned t) {
            const u64 v0 = (u64)t * kTileVecs;
            const unsigned bytes = (unsigned)(((nvec - v0) < kTileVecs ? (nvec - v0) : kTileVecs) * 16);
            mbar_arrive_expect_tx(&sm.mbar[t & 1], bytes);
            tma_load_bulk(sm.tile[t & 1], reinterpret_cast<const uint4*>(local_in) + v0, bytes, &sm.mbar[t & 1]);
        };
        if (staged && threadIdx.x == 0) issue(0);
        ok = wait_flags<T>(a, st, flags, sm, t_wait_recv, t_wait_send);
        if (!ok) {
            // Leave only after the copy in flight has landed (bounded).
            if (staged) mbar_wait_bounded(&sm.mbar[0], phase[0], kMbarPolls);
            return false;
        }
        if (st.ch.stats && threadIdx.x == 0) t0 = global_timer_ns();
        early = recv && nvec <= (u64)kRingThreads;
        uint4 pre = make_uint4(0, 0, 0, 0);
        if (early) {
            int sink = 0;
            if (threadIdx.x < nvec) {
                pre = ld16_volatile(reinterpret_cast<const uint4*>(fifo_in) + threadIdx.x);
                sink = (pre.x ^ pre.y ^ pre.z ^ pre.w) == 0x5bd1e995u;  // a use of the value: the barrier below then follows the load's arrival
            }
            (void)__syncthreads_or(sink);  // every thread holds its part of the slot
            if (threadIdx.x == 0) st_release_sys(st.ch.recv_head, st.recv_step + ring::kSliceSteps);
        }
        auto combine_store = [&](u64 v, uint4 loc, bool have_loc) {
            uint4 out;
            if (recv) {
                const uint4 r = early ? pre : ld16_volatile(reinterpret_cast<const uint4*>(fifo_in) + v);
                if (have_loc || scaled) {
                    float acc[kElems], f[kElems];
                    Wide<T>::unpack(r, acc);
                    if (have_loc) {
                        Wide<T>::unpack(loc, f);
#pragma unroll
                        for (int e = 0; e < kElems; ++e) acc[e] = Op::apply(f[e], acc[e]);
                    }
                    if (scaled) {
#pragma unroll
                        for (int e = 0; e < kElems; ++e) acc[e] *= a.scale;
                    }
                    out = Wide<T>::pack(acc);
                } else {
                    out = r;
                }
            } else {
                out = loc;
            }
            if (copy_out) st16(reinterpret_cast<uint4*>(local_out) + v, out);
            if (send) st16(reinterpret_cast<uint4*>(fifo_out) + v, out);
        };
        if (staged) {
            for (unsigned t = 0; t < ntiles; ++t) {
                if (t + 1 < ntiles && threadIdx.x == 0) issue(t + 1);
                const unsigned b = t & 1;
                int got = mbar_wait_bounded(&sm.mbar[b], phase[b], kMbarPolls) ? 1 : 0;
                phase[b] ^= 1u;
                if (!__syncthreads_and(got)) {
                    if (threadIdx.x == 0)
                        report_failure(a.status, a.own_ctrl, nullptr, 0, kStatusTimeout, (unsigned)a.rank, 12u, st.recv_step, 0);
                    if (t + 1 < ntiles) mbar_wait_bounded(&sm.mbar[b ^ 1], phase[b ^ 1], kMbarPolls);
                    return false;
                }
                const u64 v0 = (u64)t * kTileVecs;
                const u64 vend = (nvec - v0) < kTileVecs ? (nvec - v0) : kTileVecs;
                const uint4* tile = reinterpret_cast<const uint4*>(sm.tile[b]);
                for (u64 i = threadIdx.x; i < vend; i += kRingThreads) combine_store(v0 + i, tile[i], true);
                __syncthreads();  // the tile may be refilled only after every thread has read it
            }
        } else {
            for (u64 v = threadIdx.x; v < nvec; v += kRingThreads) {
                uint4 loc = make_uint4(0, 0, 0, 0);
                if (local) loc = ld16_stream(reinterpret_cast<const uint4*>(local_in) + v);
                combine_store(v, loc, local);
            }
        }
    } else {
        ok = wait_flags<T>(a, st, flags, sm, t_wait_recv, t_wait_send);
        if (!ok) return false;
        if (st.ch.stats && threadIdx.x == 0) t0 = global_timer_ns();
        for (u64 i = threadIdx.x; i < n; i += kRingThreads) {
            float acc[1];
            if (recv) {
                const T r = Narrow<T>::load(fifo_in, i);
                Narrow<T>::unpack(r, acc);
                if (local) acc[0] = Op::apply(Elem<T>::to_f(local_in[i]), acc[0]);
            } else {
                acc[0] = Elem<T>::to_f(local_in[i]);
            }
            if (scaled) acc[0] *= a.scale;
            const T out = Elem<T>::from_f(acc[0]);
            if (copy_out) local_out[i] = out;
            if (send) fifo_out[i] = out;
        }
    }

    // Publish: all data stores of the CTA happen-before the counters (bar.sync, then release).
    __syncthreads();
    u64 t1 = 0;
    if (st.ch.stats && threadIdx.x == 0) t1 = global_timer_ns();
    if (recv) {
        if (!early && threadIdx.x == 0) st_release_sys(st.ch.recv_head, st.recv_step + ring::kSliceSteps);
        st.recv_step += ring::kSliceSteps;
    }
    if (send) {
        if (threadIdx.x == 32) {
            if (st.ch.send_sizes) {
                st.ch.send_sizes[st.send_step % ring::kFifoSteps] = (unsigned)(n * sizeof(T));
            }
            st_release_sys(st.ch.send_tail, st.send_step + ring::kSliceSteps);
        }
        st.send_step += ring::kSliceSteps;
    }
    if (st.ch.stats && threadIdx.x == 0) {
        RingTurnaroundStats* s = st.ch.stats;
        atomicAdd(&s->wait_recv_ns, t_wait_recv);
        atomicAdd(&s->compute_ns, t1 - t0);
        atomicAdd(&s->post_ns, global_timer_ns() - t1);
        atomicAdd(&s->slices, 1ull);
    }
    if (st.ch.stats && threadIdx.x == 32 && t_wait_send) atomicAdd(&st.ch.stats->wait_send_ns, t_wait_send);
    return true;
}

// A chunk travels as kSlicesPerChunk slices.
template <typename T, typename Op, bool kWide>
__device__ __forceinline__ bool run_chunk(const RingArgs& a, ChannelState& st, Shared& sm, unsigned (&phase)[2],
                                          unsigned flags, const T* local_in, T* local_out, u64 n) {
    const u64 sl = ring::slice_elems(n, sizeof(T), a.step_elems);
#pragma unroll 1
    for (int s = 0; s < ring::kSlicesPerChunk; ++s) {
        const u64 off = (u64)s * sl;
        const u64 sn = ring::clamp_elems(sl, n, off);
        if (!run_slice<T, Op, kWide>(a, st, sm, phase, flags, local_in ? local_in + off : nullptr,
                                     local_out ? local_out + off : nullptr, sn))
            return false;
    }
    return true;
}

template <typename T, typename Op, bool kWide, typename ParamT>
__global__ void __launch_bounds__(kRingThreads) ring_kernel(const __grid_constant__ ParamT param) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Shared& sm = *reinterpret_cast<Shared*>(smem_raw);
    const RingArgs* ap;
    if constexpr (sizeof(ParamT) == sizeof(RingArgs)) ap = reinterpret_cast<const RingArgs*>(&param);
    else ap = reinterpret_cast<const RingArgs*>(&param) + blockIdx.y;
    const RingArgs& a = *ap;
    const int c = blockIdx.x;
    const int n = a.nranks, r = a.rank;

    ChannelState st;
    st.ch = a.channels[c];
    if (threadIdx.x == 0) {
        sm.base_steps[0] = *st.ch.send_base;
        sm.base_steps[1] = *st.ch.recv_base;
        mbar_init(&sm.mbar[0], 1);
        mbar_init(&sm.mbar[1], 1);
        mbar_fence_init();
    }
    __syncthreads();
    st.send_step = sm.base_steps[0];
    st.recv_step = sm.base_steps[1];
    unsigned phase[2] = {0u, 0u};

    const T* in = static_cast<const T*>(a.input);
    T* out = static_cast<T*>(a.output);
    // On the 16-byte path parts are cut in whole vectors so that every offset stays aligned.
    constexpr u64 kVecElems = kWide ? 16 / sizeof(T) : 1;
    ring::Part part = ring::channel_part(a.count / kVecElems, c, a.nchannels);
    part.offset *= kVecElems;
    part.count *= kVecElems;
    bool ok = true;
    auto mod = [n](int v) { return ((v % n) + n) % n; };

    if (a.collective == (int)Collective::AllReduce) {
        const u64 cs = ring::all_reduce_chunk_elems(part.count, n, sizeof(T), a.step_elems);
        for (u64 w0 = 0; ok && cs > 0 && w0 < part.count; w0 += cs * (u64)n) {
            auto chunk = [&](int k, u64* off, u64* len) {
                *off = w0 + (u64)k * cs;
                *len = ring::clamp_elems(cs, part.count, *off);
                *off += part.offset;
            };
            u64 off, len;
            chunk(mod(r - 1), &off, &len);
            ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kLocal | kSend, in + off, nullptr, len);
            for (int j = 2; ok && j < n; ++j) {
                chunk(mod(r - j), &off, &len);
                ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kRecv | kLocal | kSend, in + off, nullptr, len);
            }
            if (ok) {  // pivot: final value → output and onwards
                chunk(r, &off, &len);
                ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kRecv | kLocal | kSend | kCopyOut | kScale, in + off, out + off, len);
            }
            for (int j = 1; ok && j < n - 1; ++j) {
                chunk(mod(r - j), &off, &len);
                ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kRecv | kSend | kCopyOut, nullptr, out + off, len);
            }
            if (ok) {
                chunk(mod(r + 1), &off, &len);
                ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kRecv | kCopyOut, nullptr, out + off, len);
            }
        }
    } else if (a.collective == (int)Collective::ReduceScatter) {
        const u64 cs = ring::block_chunk_elems(part.count, sizeof(T), a.step_elems);
        for (u64 w0 = 0; ok && cs > 0 && w0 < part.count; w0 += cs) {
            const u64 len = ring::clamp_elems(cs, part.count, w0);
            auto blk = [&](int k) { return (u64)k * a.count + part.offset + w0; };
            ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kLocal | kSend, in + blk(mod(r - 1)), nullptr, len);
            for (int j = 2; ok && j < n; ++j)
                ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kRecv | kLocal | kSend, in + blk(mod(r - j)), nullptr, len);
            if (ok)
                ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kRecv | kLocal | kCopyOut | kScale, in + blk(r),
                                             out + part.offset + w0, len);
        }
    } else {  // AllGather
        const u64 cs = ring::block_chunk_elems(part.count, sizeof(T), a.step_elems);
        for (u64 w0 = 0; ok && cs > 0 && w0 < part.count; w0 += cs) {
            const u64 len = ring::clamp_elems(cs, part.count, w0);
            auto blk = [&](int k) { return (u64)k * a.count + part.offset + w0; };
            ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kLocal | kSend | kCopyOut, in + part.offset + w0, out + blk(r), len);
            for (int j = 1; ok && j < n - 1; ++j)
                ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kRecv | kSend | kCopyOut, nullptr, out + blk(mod(r - j)), len);
            if (ok) ok = run_chunk<T, Op, kWide>(a, st, sm, phase, kRecv | kCopyOut, nullptr, out + blk(mod(r + 1)), len);
        }
    }

    // Progress persists only when the whole schedule ran (an aborted launch leaves the
    // communicator poisoned, as in the reference, kernel:1186-1188).
    if (ok && threadIdx.x == 0) {
        *st.ch.send_base = st.send_step;
        *st.ch.recv_base = st.recv_step;
    }
}

template <typename T, typename Op, bool kWide>
cudaError_t launch_ring_t(const RingArgs* args, const RingLaunch& cfg) {
    const size_t smem = sizeof(Shared);
    dim3 grid(args[0].nchannels, cfg.loop_ranks > 0 ? cfg.loop_ranks : 1, 1);
    dim3 block(kRingThreads, 1, 1);
    if (cfg.loop_ranks > 0) {
        if (cfg.loop_ranks > kMaxRanks) return cudaErrorInvalidValue;
        LoopPack<RingArgs> pack;
        for (int i = 0; i < cfg.loop_ranks; ++i) pack.r[i] = args[i];
        auto kernel = ring_kernel<T, Op, kWide, LoopPack<RingArgs>>;
        cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (st != cudaSuccess) return st;
        void* params[] = {&pack};
        return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, params, smem, cfg.stream);
    }
    auto kernel = ring_kernel<T, Op, kWide, RingArgs>;
    // The attribute belongs to the current device's copy of the function: set it on every launch
    // (a process may drive several GPUs).
    cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (st != cudaSuccess) return st;
    kernel<<<grid, block, smem, cfg.stream>>>(args[0]);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_ring_op(RedOp op, const RingArgs* args, const RingLaunch& cfg) {
    const bool wide = args[0].wide != 0;
    switch (op) {
        case RedOp::Sum:
        case RedOp::Avg:
            return wide ? launch_ring_t<T, OpAdd, true>(args, cfg) : launch_ring_t<T, OpAdd, false>(args, cfg);
        case RedOp::Max:
            return wide ? launch_ring_t<T, OpMax, true>(args, cfg) : launch_ring_t<T, OpMax, false>(args, cfg);
        case RedOp::Min:
            return wide ? launch_ring_t<T, OpMin, true>(args, cfg) : launch_ring_t<T, OpMin, false>(args, cfg);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

int ring_block_threads() { return kRingThreads; }

cudaError_t launch_ring(DType dtype, RedOp op, const RingArgs* args, const RingLaunch& cfg) {
    switch (dtype) {
        case DType::Float: return launch_ring_op<float>(op, args, cfg);
        case DType::Float16: return launch_ring_op<__half>(op, args, cfg);
        case DType::BFloat16: return launch_ring_op<__nv_bfloat16>(op, args, cfg);
    }
    return cudaErrorInvalidValue;
}

}  // namespace b200ccl::kernels
