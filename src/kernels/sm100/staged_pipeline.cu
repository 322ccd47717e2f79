// AllReduce of buffers that peers cannot address (ordinary allocations of another process), as a
// three-stage tile pipeline inside ONE kernel per rank:
//
//   copy-in   one elected thread moves tile k of the caller's input into this rank's staging arena
//             with TMA bulk copies (global -> shared -> global, own memory only),
//   reduce    fourteen warps reduce this rank's shard of tile k across all ranks' arenas and store
//             the result into every rank's arena: multimem.ld_reduce / multimem.st through the
//             NVSwitch, or plain peer loads and stores (two ranks, max/min, no multicast),
//   copy-out  one elected thread moves tile k of this rank's arena into the caller's output, again
//             with TMA bulk copies,
//
// all three running at once on different tiles. The stages of the same CTA index on every rank
// meet through three monotonic counters per (CTA, source rank) in peer memory (PipeFlags), written
// with st.release.sys and polled with ld.acquire.sys: "tile copied in", "shard reduced and stored
// everywhere", "tile copied out". A slot of the arena is reused once the counter that marks its last
// reader has passed. The arena is a ring, so a message of any size streams through it in one launch.
//
// What is fused into the one launch: both staging copies, the cross-GPU synchronisation, the loads
// from every rank, the fp32 widening and accumulation, the avg 1/N scale, the single rounding and
// the broadcast of the result.
//
// The reference has no counterpart: it is single-process, so every buffer is peer-addressable, and
// it moves data through per-edge FIFOs (src/kernels/ring_simple_kernel.cuh:1170-1230). The nearest
// relative is its pivot step, which reduces, scales, writes the output and forwards in one pass
// (kernel:433-481); here that pass is the reduce stage.
#include "kernels/sm100/staged_pipeline.h"

#include "kernels/sm100/sync.cuh"
#include "kernels/sm100/tma.cuh"
#include "kernels/sm100/vec.cuh"

namespace b200ccl::kernels {

using namespace b200ccl::dev;

namespace {

using u64 = unsigned long long;
using uchar = unsigned char;

constexpr int kThreads = 512;
constexpr int kCopyWarps = 2;                               // warp 0 copies in, warp 1 copies out
constexpr int kReduceThreads = kThreads - 32 * kCopyWarps;  // 448
constexpr int kStages = 3;                                  // shared-memory stages per copy direction
constexpr unsigned kChunk = 32768;                          // bytes per TMA bulk copy
constexpr unsigned kPolls = 1u << 20;                       // bound on waiting for an own bulk copy

struct CopyRing {
    alignas(128) uchar tile[kStages][kChunk];
    alignas(8) u64 full[kStages];
};

struct Shared {
    CopyRing in;
    CopyRing out;
    int reduce_ok;
    int failed;
};

template <typename A>
__device__ __forceinline__ const A& select_args(const A& one) { return one; }
template <typename A>
__device__ __forceinline__ const A& select_args(const LoopPack<A>& all) { return all.r[blockIdx.y]; }

// Stage timing uses the SM's own cycle counter: %globaltimer is one chip-wide register whose reads
// from many SMs at once queue up for microseconds each, which would distort what is measured.
__device__ __forceinline__ u64 stage_clock() { return (u64)clock64(); }

__device__ __forceinline__ void reducers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kReduceThreads) : "memory"); }

// kN: rank count the peer-load loop is unrolled for (0: any, decided at run time). kU: packs in
// flight per thread and peer. The two copy rings take most of an SM's shared memory, so one CTA
// runs per SM and its threads may use the whole register file.
template <typename T, typename Op, bool kNvls, int kN, int kU, typename ParamT>
__global__ void __launch_bounds__(kThreads, 1) pipeline_kernel(const __grid_constant__ ParamT param) {
    using P = Wide<T>;
    constexpr int kElems = P::kElems;
    constexpr int NN = kN > 0 ? kN : kMaxRanks;
    extern __shared__ __align__(128) uchar smem_raw[];
    Shared& sm = *reinterpret_cast<Shared*>(smem_raw);
    __shared__ u64 s_epoch, s_base;

    const PipeArgs& a = select_args(param);
    const int n = (kN > 0 && !kNvls) ? kN : a.nranks;
    const int rank = a.rank;
    const unsigned cta = blockIdx.x;
    ControlBlock* own = a.ctrl[rank];
    PipeFlags* mine = a.flags[rank];
    if (threadIdx.x == 0) {
        s_epoch = own->epoch[cta];
        s_base = mine->base[cta];
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.in.full[s], 1);
            mbar_init(&sm.out.full[s], 1);
        }
        mbar_fence_init();
        sm.failed = 0;
        sm.reduce_ok = 1;
    }
    __syncthreads();
    const u64 epoch = s_epoch + 1;
    const u64 base = s_base;
    const u64 t_kernel = a.stats != nullptr ? stage_clock() : 0;

    // Every rank is inside this call (so nobody still uses the arena for an earlier one) and
    // launched it with the same plan.
    if (!cta_barrier_all_ranks(a.ctrl, rank, n, epoch, a.timeout_ns, a.status, 50u, a.plan_hash)) return;

    const u64 total_tiles = (a.bytes + a.tile_bytes - 1) / a.tile_bytes;
    const u64 K = cta < total_tiles ? (total_tiles - cta + gridDim.x - 1) / gridDim.x : 0;  // tiles cta, cta + grid, ...
    const u64 S = (u64)a.slots;
    auto tile_off = [&](u64 k) { return ((u64)cta + k * gridDim.x) * a.tile_bytes; };
    auto tile_len = [&](u64 k) {
        const u64 off = tile_off(k);
        return a.bytes - off < a.tile_bytes ? a.bytes - off : a.tile_bytes;
    };
    auto slot_off = [&](u64 k) { return ((u64)cta * S + (k % S)) * a.tile_bytes; };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    bool ok = true;
    const bool timed = a.stats != nullptr;

    if (warp <= 1) {
        // ---- the two copy stages: one elected thread each, a continuous stream of chunks ------------
        // Chunks flow through the shared-memory ring without a pause at tile borders: loads run up to
        // kStages chunks ahead of stores, a stage is refilled once the store that drained it has read
        // it, and a tile is announced as soon as the stores (copy-in) or loads (copy-out) of its last
        // chunk are known to be complete.
        if (lane == 0) {
            const bool in = warp == 0;
            CopyRing& ring = in ? sm.in : sm.out;
            const uchar* src = in ? static_cast<const uchar*>(a.user_in) : static_cast<const uchar*>(a.arena_out[rank]);
            uchar* dst = in ? static_cast<uchar*>(a.arena_in[rank]) : static_cast<uchar*>(a.user_out);
            auto chunks_of = [&](u64 k) { return (tile_len(k) + kChunk - 1) / kChunk; };
            auto chunk_len = [&](u64 k, u64 j) {
                const u64 left = tile_len(k) - j * kChunk;
                return (unsigned)(left < kChunk ? left : kChunk);
            };
            u64 total = 0;
            for (u64 k = 0; k < K; ++k) total += chunks_of(k);
            // A tile is announced to every rank with one fence and n relaxed stores (a release).
            auto announce = [&](unsigned long long (PipeFlags::*row)[kMaxCtas][kMaxRanks], u64 tiles) {
                fence_acq_rel_sys();
                for (int p = 0; p < n; ++p) st_relaxed_sys(&(a.flags[p]->*row)[cta][rank], base + tiles);
            };
            auto wait_all = [&](unsigned long long (*row)[kMaxRanks], u64 want, unsigned where) {
                for (int p = 0; p < n; ++p)
                    if (!wait_at_least(&row[cta][p], want, own, a.timeout_ns, a.status, a.ctrl, n, (unsigned)p, where)) return false;
                return true;
            };
            u64 lk = 0, lj = 0, issued = 0;       // next chunk to load
            u64 sk = 0, sj = 0, stores = 0;        // next chunk to store
            u64 freed = 0;                         // chunks whose store has finished reading its stage
            u64 closed = 0;                        // tiles all of whose stores have been issued (copy-in) / loads have landed (copy-out)
            u64 announced = 0;                     // tiles announced to the other ranks
            u64 t_wait = 0, t_busy = 0, t_mark = timed ? stage_clock() : 0;
            while (ok && stores < total) {
                // 1. Loads, as far ahead as stages and the arena slots allow.
                while (ok && issued < total && issued < freed + kStages) {
                    if (lj == 0) {
                        const u64 t0 = timed ? stage_clock() : 0;
                        if (in) {
                            if (lk >= S) {
                                // The slot held tile lk - S: every rank must have reduced it, which needs this
                                // rank's own copy of that tile to be announced first.
                                const u64 need = lk - S + 1;
                                if (closed < need) break;  // its stores are not even issued: store first
                                if (announced < need) {
                                    tma_wait_group_all();
                                    freed = stores;
                                    announce(&PipeFlags::in_ready, closed);
                                    announced = closed;
                                }
                                ok = wait_all(mine->reduced, base + need, 51u);
                            }
                        } else {
                            // Tile lk must have been reduced by every rank, which (from tile S on) needs this
                            // rank to have announced that it drained tile lk - S.
                            if (lk >= S && announced < lk - S + 1) break;
                            ok = wait_all(mine->reduced, base + lk + 1, 53u);
                            // Peers wrote the slot through the generic proxy; the bulk copies below read it
                            // through the asynchronous one.
                            fence_proxy_async();
                        }
                        if (timed) t_wait += stage_clock() - t0;
                        if (!ok) break;
                    }
                    const int s = (int)(issued % kStages);
                    const unsigned len = chunk_len(lk, lj);
                    mbar_arrive_expect_tx(&ring.full[s], len);
                    tma_load_bulk(ring.tile[s], src + (in ? tile_off(lk) : slot_off(lk)) + lj * kChunk, len, &ring.full[s]);
                    ++issued;
                    if (++lj == chunks_of(lk)) { ++lk; lj = 0; }
                }
                if (!ok) break;
                // 2. The next chunk has landed: store it.
                const int s = (int)(stores % kStages);
                if (!mbar_wait_bounded(&ring.full[s], (unsigned)((stores / kStages) & 1), kPolls)) {
                    report_failure(a.status, own, a.ctrl, n, kStatusTimeout, (unsigned)rank, in ? 52u : 56u, base + sk, 0ull);
                    ok = false;
                    break;
                }
                const bool last_of_tile = sj + 1 == chunks_of(sk);
                if (!in && last_of_tile) {
                    // Every load of the tile has landed in shared memory: its arena slot may be reused.
                    ++closed;
                    announce(&PipeFlags::drained, closed);
                    announced = closed;
                }
                const u64 closed_before = closed;
                tma_store_bulk(dst + (in ? slot_off(sk) : tile_off(sk)) + sj * kChunk, ring.tile[s], chunk_len(sk, sj));
                tma_commit_group();
                ++stores;
                if (last_of_tile) {
                    if (in) ++closed;
                    ++sk;
                    sj = 0;
                } else {
                    ++sj;
                }
                if (in && closed_before > announced) {
                    // Tiles closed by an earlier store: complete once all groups but the newest are.
                    tma_wait_group<1>();
                    freed = stores - 1;
                    announce(&PipeFlags::in_ready, closed_before);
                    announced = closed_before;
                } else if (stores >= 2) {
                    tma_wait_group_read<1>();
                    freed = stores - 1;
                }
            }
            // Stores read shared memory (and must be complete before the kernel's results count).
            if (!ok)
                for (u64 g = stores + 1; g < issued; ++g) mbar_wait_bounded(&ring.full[g % kStages], (unsigned)((g / kStages) & 1), kPolls);
            tma_wait_group_all();
            if (ok && in && announced < closed) announce(&PipeFlags::in_ready, closed);
            if (timed) {
                t_busy = stage_clock() - t_mark - t_wait;
                if (in) {
                    atomicAdd(&a.stats->in_wait_slot_ns, t_wait);
                    atomicAdd(&a.stats->in_copy_ns, t_busy);
                    atomicAdd(&a.stats->tiles, K);
                    atomicAdd(&a.stats->calls, 1ull);
                } else {
                    atomicAdd(&a.stats->out_wait_ns, t_wait);
                    atomicAdd(&a.stats->out_copy_ns, t_busy);
                }
            }
        }
    } else {
        // ---- reduce: own shard of the tile, all ranks' arenas -> all ranks' arenas --------------------
        const u64 rt = threadIdx.x - 32 * kCopyWarps;
        const bool scaled = a.scale != 1.0f;
        u64 t_wait = 0, t_work = 0;
        const bool clock = timed && rt == 0;  // one reader: %globaltimer is a slow read that serialises
        for (u64 k = 0; k < K; ++k) {
            const u64 t0 = clock ? stage_clock() : 0;
            if (warp == kCopyWarps) {
                int good = 1;
                if (lane < n)  // every rank's copy of tile k is in its arena
                    good = wait_at_least(&mine->in_ready[cta][lane], base + k + 1, own, a.timeout_ns, a.status, a.ctrl, n,
                                         (unsigned)lane, 54u) ? 1 : 0;
                else if (lane >= 16 && lane < 16 + n && k >= S)  // every rank has copied tile k - S out of the slot
                    good = wait_at_least(&mine->drained[cta][lane - 16], base + k - S + 1, own, a.timeout_ns, a.status, a.ctrl,
                                         n, (unsigned)(lane - 16), 55u) ? 1 : 0;
                good = __all_sync(0xffffffffu, good);
                if (lane == 0) sm.reduce_ok = good;
            }
            reducers_sync();
            if (!sm.reduce_ok) { ok = false; break; }
            const u64 t1 = clock ? stage_clock() : 0;
            const u64 packs = tile_len(k) / 16;
            const u64 lo = packs * (u64)rank / (u64)n, hi = packs * (u64)(rank + 1) / (u64)n;
            const u64 s0 = slot_off(k) / 16;
            if constexpr (kNvls) {
                const uint4* mc_in = static_cast<const uint4*>(a.mc_in) + s0;
                uint4* mc_out = static_cast<uint4*>(a.mc_out) + s0;
                for (u64 j = lo + rt; j < hi; j += (u64)kReduceThreads * kU) {
                    uint4 r[kU];
#pragma unroll
                    for (int u = 0; u < kU; ++u) {
                        const u64 jj = j + (u64)u * kReduceThreads;
                        if (jj < hi) r[u] = multimem_ld_reduce_add<T>(mc_in + jj);
                    }
#pragma unroll
                    for (int u = 0; u < kU; ++u) {
                        const u64 jj = j + (u64)u * kReduceThreads;
                        if (jj < hi) {
                            uint4 v = r[u];
                            if (scaled) {
                                float f[kElems];
                                P::unpack(v, f);
#pragma unroll
                                for (int e = 0; e < kElems; ++e) f[e] *= a.scale;
                                v = P::pack(f);
                            }
                            multimem_st16(mc_out + jj, v);
                        }
                    }
                }
            } else {
                for (u64 j = lo + rt; j < hi; j += (u64)kReduceThreads * kU) {
                    uint4 r[kU][NN];
#pragma unroll
                    for (int u = 0; u < kU; ++u) {
                        const u64 jj = j + (u64)u * kReduceThreads;
                        if (jj < hi) {
#pragma unroll
                            for (int p = 0; p < NN; ++p)
                                if (p < n) r[u][p] = P::load(a.arena_in[p], s0 + jj);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kU; ++u) {
                        const u64 jj = j + (u64)u * kReduceThreads;
                        if (jj < hi) {
                            float acc[kElems];  // fixed order 0..n-1: bit-identical results on every rank
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
                            const uint4 v = P::pack(acc);
#pragma unroll
                            for (int q = 0; q < NN; ++q) {
                                if (q < n) {
                                    int dstr = rank + q;  // start with the own copy, then spread over peers
                                    if (dstr >= n) dstr -= n;
                                    P::store(a.arena_out[dstr], s0 + jj, v);
                                }
                            }
                        }
                    }
                }
            }
            reducers_sync();  // every reducer's stores happen-before the release below
            if (warp == kCopyWarps && lane < n) st_release_sys(&a.flags[lane]->reduced[cta][rank], base + k + 1);
            if (clock) { t_wait += t1 - t0; t_work += stage_clock() - t1; }
        }
        if (clock) {
            atomicAdd(&a.stats->red_wait_ns, t_wait);
            atomicAdd(&a.stats->red_work_ns, t_work);
        }
    }

    if (!ok) *(volatile int*)&sm.failed = 1;
    __syncthreads();
    // Progress persists only when every stage ran to its end (a failed call leaves the communicator unusable).
    if (threadIdx.x == 0 && *(volatile int*)&sm.failed == 0) {
        own->epoch[cta] = epoch;
        mine->base[cta] = base + K;
    }
    if (threadIdx.x == 0 && cta == 0 && a.stats != nullptr) atomicAdd(&a.stats->kernel_ns, stage_clock() - t_kernel);
}

template <typename KernelT, typename ParamT>
cudaError_t launch_kernel(KernelT kernel, const ParamT& param, const PipeLaunch& cfg) {
    const std::size_t smem = sizeof(Shared);
    // The attribute belongs to the current device's copy of the function: set it on every launch.
    cudaError_t st = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (st != cudaSuccess) return st;
    dim3 grid(cfg.grid, cfg.loop_ranks > 0 ? cfg.loop_ranks : 1, 1), block(kThreads, 1, 1);
    if (cfg.loop_ranks > 0) {
        void* params[] = {const_cast<ParamT*>(&param)};
        return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), grid, block, params, smem, cfg.stream);
    }
    kernel<<<grid, block, smem, cfg.stream>>>(param);
    return cudaGetLastError();
}

template <typename T, typename Op, int kN, int kU>
cudaError_t launch_peer_n(const PipeArgs* args, const PipeLaunch& cfg) {
    if (cfg.loop_ranks > 0) {
        if (cfg.loop_ranks > kMaxRanks) return cudaErrorInvalidValue;
        LoopPack<PipeArgs> pack;
        for (int r = 0; r < cfg.loop_ranks; ++r) pack.r[r] = args[r];
        return launch_kernel(pipeline_kernel<T, Op, false, kN, kU, LoopPack<PipeArgs>>, pack, cfg);
    }
    return launch_kernel(pipeline_kernel<T, Op, false, kN, kU, PipeArgs>, args[0], cfg);
}

// Fewer ranks leave registers for more packs in flight per peer.
template <typename T, typename Op>
cudaError_t launch_peer(const PipeArgs* args, const PipeLaunch& cfg) {
    switch (args[0].nranks) {
        case 2: return launch_peer_n<T, Op, 2, 8>(args, cfg);
        case 4: return launch_peer_n<T, Op, 4, 4>(args, cfg);
        case 8: return launch_peer_n<T, Op, 8, 2>(args, cfg);
        default: return launch_peer_n<T, Op, 0, 2>(args, cfg);
    }
}

template <typename T>
cudaError_t launch_t(RedOp op, const PipeArgs* args, const PipeLaunch& cfg) {
    if (cfg.nvls) {
        if (cfg.loop_ranks > 0 || (op != RedOp::Sum && op != RedOp::Avg) || args[0].mc_in == nullptr || args[0].mc_out == nullptr)
            return cudaErrorInvalidValue;
        if (cfg.nvls_unroll >= 8) return launch_kernel(pipeline_kernel<T, OpAdd, true, 0, 8, PipeArgs>, args[0], cfg);
        if (cfg.nvls_unroll <= 1) return launch_kernel(pipeline_kernel<T, OpAdd, true, 0, 1, PipeArgs>, args[0], cfg);
        if (cfg.nvls_unroll <= 2) return launch_kernel(pipeline_kernel<T, OpAdd, true, 0, 2, PipeArgs>, args[0], cfg);
        return launch_kernel(pipeline_kernel<T, OpAdd, true, 0, 4, PipeArgs>, args[0], cfg);
    }
    switch (op) {
        case RedOp::Sum:
        case RedOp::Avg: return launch_peer<T, OpAdd>(args, cfg);
        case RedOp::Max: return launch_peer<T, OpMax>(args, cfg);
        case RedOp::Min: return launch_peer<T, OpMin>(args, cfg);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

std::size_t pipeline_smem_bytes() { return sizeof(Shared); }

cudaError_t launch_staged_pipeline(DType dtype, RedOp op, const PipeArgs* args, const PipeLaunch& cfg) {
    const PipeArgs& a = args[0];
    if (a.bytes == 0 || a.bytes % 16 != 0 || a.tile_bytes == 0 || a.tile_bytes % 16 != 0 || a.slots < 1 || cfg.grid < 1 ||
        cfg.grid > kMaxCtas)
        return cudaErrorInvalidValue;
    switch (dtype) {
        case DType::Float: return launch_t<float>(op, args, cfg);
        case DType::Float16: return launch_t<__half>(op, args, cfg);
        case DType::BFloat16: return launch_t<__nv_bfloat16>(op, args, cfg);
    }
    return cudaErrorInvalidValue;
}

}  // namespace b200ccl::kernels
