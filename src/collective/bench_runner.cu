// Benchmark runner and its device helpers (seeded fill, recomputing verifier).
#include "b200ccl/bench.h"

#include "b200ccl/traits.h"
#include "collective/bench_profiling.h"
#include "core/buffers.h"
#include "core/check.h"
#include "core/datagen.h"
#include "core/env.h"
#include "core/stream.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>

namespace b200ccl {

namespace {

template <DType D>
__global__ void fill_kernel(typename DTypeTraits<D>::type* buf, std::size_t count, bool uniform, std::uint64_t seed,
                            int rank, std::uint64_t first) {
    for (std::size_t i = blockIdx.x * (std::size_t)blockDim.x + threadIdx.x; i < count;
         i += (std::size_t)gridDim.x * blockDim.x)
        buf[i] = DTypeTraits<D>::from_float(datagen::value(uniform, seed, rank, first + i));
}

template <DType D>
__device__ float rounded_input(bool uniform, std::uint64_t seed, int rank, std::uint64_t index) {
    return DTypeTraits<D>::to_float(DTypeTraits<D>::from_float(datagen::value(uniform, seed, rank, index)));
}

template <DType D>
__global__ void verify_kernel(const typename DTypeTraits<D>::type* out, std::size_t count, RedOp op, bool uniform,
                              std::uint64_t seed, int nranks, int src_rank, std::uint64_t first, float eps,
                              unsigned long long* wrong, unsigned int* max_abs_bits) {
    unsigned long long bad = 0;
    float worst = 0.0f;
    for (std::size_t i = blockIdx.x * (std::size_t)blockDim.x + threadIdx.x; i < count;
         i += (std::size_t)gridDim.x * blockDim.x) {
        double expect;
        if (src_rank >= 0) {
            expect = rounded_input<D>(uniform, seed, src_rank, first + i);
        } else {
            expect = rounded_input<D>(uniform, seed, 0, first + i);
            for (int r = 1; r < nranks; ++r) {
                const double v = rounded_input<D>(uniform, seed, r, first + i);
                if (op == RedOp::Max) expect = v > expect ? v : expect;
                else if (op == RedOp::Min) expect = v < expect ? v : expect;
                else expect += v;
            }
            if (op == RedOp::Avg) expect /= nranks;
        }
        const float got = DTypeTraits<D>::to_float(out[i]);
        const float err = fabsf(got - static_cast<float>(expect));
        if (!(err <= eps)) ++bad;
        if (err > worst || err != err) worst = err != err ? INFINITY : err;
    }
    if (bad) atomicAdd(wrong, bad);
    atomicMax(max_abs_bits, __float_as_uint(worst));  // non-negative floats order like their bit patterns
}

int grid_for(std::size_t count) {
    return static_cast<int>(std::min<std::size_t>((count + 255) / 256, 148 * 8));
}

// Debug aid (B200CCL_DEBUG_FIRST_WRONG=1, as NANO_NCCL_DEBUG_FIRST_WRONG in the reference's
// ring_simple.cu:80, 91-95): after a failed verification, find the first mismatching element on the
// host and print it. Runs only when something is already wrong.
template <DType D>
void report_first_wrong_t(const void* device_out, std::size_t count, RedOp op, bool uniform, std::uint64_t seed, int nranks,
                          int src_rank, std::uint64_t first, float eps, int rank) {
    using T = typename DTypeTraits<D>::type;
    std::vector<T> host(count);
    if (cudaMemcpy(host.data(), device_out, count * sizeof(T), cudaMemcpyDeviceToHost) != cudaSuccess) {
        (void)cudaGetLastError();
        return;
    }
    auto input = [&](int r, std::uint64_t i) {
        return static_cast<double>(DTypeTraits<D>::to_float(DTypeTraits<D>::from_float(datagen::value(uniform, seed, r, i))));
    };
    for (std::size_t i = 0; i < count; ++i) {
        double expect;
        if (src_rank >= 0) {
            expect = input(src_rank, first + i);
        } else {
            expect = input(0, first + i);
            for (int r = 1; r < nranks; ++r) {
                const double v = input(r, first + i);
                if (op == RedOp::Max) expect = v > expect ? v : expect;
                else if (op == RedOp::Min) expect = v < expect ? v : expect;
                else expect += v;
            }
            if (op == RedOp::Avg) expect /= nranks;
        }
        const float got = DTypeTraits<D>::to_float(host[i]);
        if (!(std::fabs(got - static_cast<float>(expect)) <= eps)) {
            std::fprintf(stderr, "first wrong element: rank %d index %zu got %.9g expected %.9g (eps %g)\n", rank, i,
                         static_cast<double>(got), expect, static_cast<double>(eps));
            return;
        }
    }
}

void report_first_wrong(const void* out, std::size_t count, DType dtype, RedOp op, bool uniform, std::uint64_t seed,
                        int nranks, int src_rank, std::uint64_t first, float eps, int rank) {
    switch (dtype) {
        case DType::Float: report_first_wrong_t<DType::Float>(out, count, op, uniform, seed, nranks, src_rank, first, eps, rank); break;
        case DType::Float16: report_first_wrong_t<DType::Float16>(out, count, op, uniform, seed, nranks, src_rank, first, eps, rank); break;
        case DType::BFloat16: report_first_wrong_t<DType::BFloat16>(out, count, op, uniform, seed, nranks, src_rank, first, eps, rank); break;
    }
}

}  // namespace

void bench_fill(void* buf, std::size_t count, DType dtype, bool uniform, std::uint64_t seed, int rank,
                std::uint64_t first_index, cudaStream_t stream) {
    const int g = std::max(grid_for(count), 1);
    switch (dtype) {
        case DType::Float:
            fill_kernel<DType::Float><<<g, 256, 0, stream>>>(static_cast<float*>(buf), count, uniform, seed, rank, first_index);
            break;
        case DType::Float16:
            fill_kernel<DType::Float16><<<g, 256, 0, stream>>>(static_cast<__half*>(buf), count, uniform, seed, rank, first_index);
            break;
        case DType::BFloat16:
            fill_kernel<DType::BFloat16><<<g, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(buf), count, uniform, seed, rank, first_index);
            break;
    }
    B2_CUDA(cudaGetLastError());
}

void bench_verify(const void* out, std::size_t count, DType dtype, RedOp redop, bool uniform, std::uint64_t seed,
                  int nranks, int src_rank, std::uint64_t first_index, float eps, unsigned long long* wrong,
                  unsigned int* max_abs_bits, cudaStream_t stream) {
    const int g = std::max(grid_for(count), 1);
    switch (dtype) {
        case DType::Float:
            verify_kernel<DType::Float><<<g, 256, 0, stream>>>(static_cast<const float*>(out), count, redop, uniform, seed,
                                                                nranks, src_rank, first_index, eps, wrong, max_abs_bits);
            break;
        case DType::Float16:
            verify_kernel<DType::Float16><<<g, 256, 0, stream>>>(static_cast<const __half*>(out), count, redop, uniform, seed,
                                                                  nranks, src_rank, first_index, eps, wrong, max_abs_bits);
            break;
        case DType::BFloat16:
            verify_kernel<DType::BFloat16><<<g, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(out), count, redop,
                                                                   uniform, seed, nranks, src_rank, first_index, eps, wrong,
                                                                   max_abs_bits);
            break;
    }
    B2_CUDA(cudaGetLastError());
}

namespace {

struct RankState {
    int device = 0;
    std::unique_ptr<Stream> own_stream;  // null for emulated ranks, which share rank 0's stream
    cudaStream_t stream = nullptr;
    std::unique_ptr<Event> start_ev, stop_ev;  // timing events on `stream`
    cudaEvent_t start = nullptr, stop = nullptr;
    std::vector<void*> send, recv;  // one per buffer set
    DeviceBuffer<unsigned long long> wrong_buf;
    DeviceBuffer<unsigned int> max_abs_buf;
    unsigned long long* wrong = nullptr;
    unsigned int* max_abs = nullptr;
};

constexpr std::uint64_t kSeed = 20240611;

}  // namespace

int run_collective_bench(const BenchConfig& config, std::vector<BenchResult>* results) {
    if (!results) return 2;
    int visible = 0;
    if (cudaGetDeviceCount(&visible) != cudaSuccess || visible == 0) {
        (void)cudaGetLastError();
        std::fprintf(stderr, "bench: no CUDA device\n");
        return 3;
    }
    const int nranks = config.nranks > 0 ? config.nranks : visible;
    CommunicatorConfig cc;
    cc.transport = config.transport;
    Algo algo = Algo::Auto;
    if (!parse_algo(config.algo.c_str(), &algo)) {
        std::fprintf(stderr, "bench: unknown algo '%s'\n", config.algo.c_str());
        return 2;
    }
    cc.algo = algo;
    if (config.loopback) {
        cc.loopback = true;
        cc.loopback_ranks = nranks;
        cc.devices = {0};
    } else {
        if (nranks > visible) {
            std::fprintf(stderr, "bench: %d ranks requested, %d GPUs visible\n", nranks, visible);
            return 3;
        }
        for (int d = 0; d < nranks; ++d) cc.devices.push_back(d);
    }
    auto comm = create_communicator(cc);
    const std::size_t esz = dtype_size(config.dtype);
    const float eps = config.epsilon > 0 ? config.epsilon : dtype_default_epsilon(config.dtype);
    const Collective coll = config.collective;
    const std::size_t in_mult = coll == Collective::ReduceScatter ? nranks : 1;
    const std::size_t out_mult = coll == Collective::AllGather ? nranks : 1;

    std::vector<RankState> ranks(nranks);
    for (int r = 0; r < nranks; ++r) {
        ranks[r].device = config.loopback ? 0 : r;
        RankState& st = ranks[r];
        if (!config.loopback || r == 0) {
            st.own_stream.reset(new Stream(st.device));
            st.stream = st.own_stream->get();
        } else {
            st.stream = ranks[0].stream;  // one launch plays all ranks: they share rank 0's stream
        }
        st.start_ev.reset(new Event(st.device, /*timing=*/true));
        st.stop_ev.reset(new Event(st.device, /*timing=*/true));
        st.start = st.start_ev->get();
        st.stop = st.stop_ev->get();
        st.wrong_buf.reset(st.device, 1);
        st.max_abs_buf.reset(st.device, 1);
        st.wrong = st.wrong_buf.get();
        st.max_abs = st.max_abs_buf.get();
    }
    auto sync_all = [&] {
        for (int r = 0; r < nranks; ++r) {
            DeviceGuard guard(ranks[r].device);
            B2_CUDA(cudaStreamSynchronize(ranks[r].stream));
        }
    };

    PinnedBuffer<unsigned long long> readback(2);
    int rc = 0;
    for (std::size_t bytes : make_sizes(config.min_bytes, config.max_bytes, config.factor)) {
        const std::size_t count = std::max<std::size_t>(bytes / esz, 1);
        const std::size_t in_bytes = count * esz * in_mult, out_bytes = count * esz * out_mult;
        // Rotate over several buffer sets so that successive iterations do not hit a warm L2
        // (126 MB): at least 512 MiB of working set where memory allows, at most 8 sets.
        std::size_t sets = std::min<std::size_t>(8, std::max<std::size_t>(1, (std::size_t(512) << 20) / (in_bytes + out_bytes)));
        std::vector<std::vector<void*>> sym_in, sym_out;
        try {
            for (std::size_t s = 0; s < sets; ++s) {
                if (config.symmetric) {
                    sym_in.push_back(comm->alloc_symmetric(in_bytes));
                    sym_out.push_back(comm->alloc_symmetric(out_bytes));
                    for (int r = 0; r < nranks; ++r) {
                        ranks[r].send.push_back(sym_in.back()[r]);
                        ranks[r].recv.push_back(sym_out.back()[r]);
                    }
                } else {
                    for (int r = 0; r < nranks; ++r) {
                        DeviceGuard guard(ranks[r].device);
                        void *a = nullptr, *b = nullptr;
                        B2_CUDA(cudaMalloc(&a, in_bytes));
                        B2_CUDA(cudaMalloc(&b, out_bytes));
                        ranks[r].send.push_back(a);
                        ranks[r].recv.push_back(b);
                    }
                }
            }
            for (int r = 0; r < nranks; ++r) {
                DeviceGuard guard(ranks[r].device);
                for (std::size_t s = 0; s < sets; ++s) {
                    bench_fill(ranks[r].send[s], count * in_mult, config.dtype, config.uniform_data, kSeed, r, 0, ranks[r].stream);
                    B2_CUDA(cudaMemsetAsync(ranks[r].recv[s], 0xff, out_bytes, ranks[r].stream));
                }
            }
            sync_all();

            auto issue = [&](std::size_t set) {
                CollectiveArgs a;
                a.count = count;
                a.dtype = config.dtype;
                a.redop = config.redop;
                for (int r = 0; r < nranks; ++r) {
                    a.send_buffers.push_back(ranks[r].send[set]);
                    a.recv_buffers.push_back(ranks[r].recv[set]);
                    a.streams.push_back(ranks[r].stream);
                }
                switch (coll) {
                    case Collective::AllReduce: comm->all_reduce(a); break;
                    case Collective::ReduceScatter: comm->reduce_scatter(a); break;
                    case Collective::AllGather: comm->all_gather(a); break;
                }
            };
            for (int i = 0; i < config.warmup_iters; ++i) issue(i % sets);
            sync_all();
            comm->check_async_error();
            const int record_ranks = config.loopback ? 1 : nranks;
            for (int r = 0; r < record_ranks; ++r) {
                DeviceGuard guard(ranks[r].device);
                B2_CUDA(cudaEventRecord(ranks[r].start, ranks[r].stream));
            }
            if (config.graph) {
                // The whole batch is captured once per rank stream and replayed: launch cost leaves the
                // measurement and what remains is the device time of the collectives.
                std::vector<GraphExec> graphs;
                for (int r = 0; r < record_ranks; ++r) {
                    DeviceGuard guard(ranks[r].device);
                    B2_CUDA(cudaStreamBeginCapture(ranks[r].stream, cudaStreamCaptureModeRelaxed));
                }
                for (int i = 0; i < config.iters; ++i) issue(i % sets);
                for (int r = 0; r < record_ranks; ++r) {
                    DeviceGuard guard(ranks[r].device);
                    cudaGraph_t g = nullptr;
                    B2_CUDA(cudaStreamEndCapture(ranks[r].stream, &g));
                    graphs.emplace_back(g);
                    B2_CUDA(cudaGraphDestroy(g));
                }
                for (int pass = 0; pass < 2; ++pass) {  // first replay warms up, second is timed
                    if (pass == 1)
                        for (int r = 0; r < record_ranks; ++r) {
                            DeviceGuard guard(ranks[r].device);
                            B2_CUDA(cudaEventRecord(ranks[r].start, ranks[r].stream));
                        }
                    for (int r = 0; r < record_ranks; ++r) {
                        DeviceGuard guard(ranks[r].device);
                        graphs[r].launch(ranks[r].stream);
                    }
                    if (pass == 0) sync_all();
                }
            } else {
                // Capture window and ranges cover the measured batch only (no-ops in normal builds).
                ProfilerSession session;
                NvtxRange size_range(bench_range_name(collective_name(coll), count * esz));
                for (int i = 0; i < config.iters; ++i) {
                    NvtxRange iter_range(bench_range_name(collective_name(coll), count * esz, i));
                    issue(i % sets);
                }
            }
            for (int r = 0; r < record_ranks; ++r) {
                DeviceGuard guard(ranks[r].device);
                B2_CUDA(cudaEventRecord(ranks[r].stop, ranks[r].stream));
            }
            sync_all();
            comm->check_async_error();
            float worst_ms = 0;
            for (int r = 0; r < record_ranks; ++r) {
                float ms = 0;
                B2_CUDA(cudaEventElapsedTime(&ms, ranks[r].start, ranks[r].stop));
                worst_ms = std::max(worst_ms, ms);
            }

            // Verify the last-written set of every rank.
            const std::size_t last_set = (config.iters > 0 ? (config.iters - 1) : 0) % sets;
            unsigned long long wrong_total = 0;
            float max_abs = 0;
            for (int r = 0; r < nranks; ++r) {
                DeviceGuard guard(ranks[r].device);
                B2_CUDA(cudaMemsetAsync(ranks[r].wrong, 0, sizeof(unsigned long long), ranks[r].stream));
                B2_CUDA(cudaMemsetAsync(ranks[r].max_abs, 0, sizeof(unsigned int), ranks[r].stream));
                readback.get()[0] = readback.get()[1] = 0;
                if (coll == Collective::AllGather) {
                    for (int src = 0; src < nranks; ++src)
                        bench_verify(static_cast<char*>(ranks[r].recv[last_set]) + src * count * esz, count, config.dtype,
                                     config.redop, config.uniform_data, kSeed, nranks, src, 0, eps, ranks[r].wrong,
                                     ranks[r].max_abs, ranks[r].stream);
                } else {
                    const std::uint64_t first = coll == Collective::ReduceScatter ? (std::uint64_t)r * count : 0;
                    bench_verify(ranks[r].recv[last_set], count, config.dtype, config.redop, config.uniform_data, kSeed, nranks,
                                 -1, first, eps, ranks[r].wrong, ranks[r].max_abs, ranks[r].stream);
                }
                // Read the two counters back through pinned memory (a truly asynchronous copy).
                unsigned long long* host = readback.get();
                B2_CUDA(cudaMemcpyAsync(&host[0], ranks[r].wrong, sizeof(unsigned long long), cudaMemcpyDeviceToHost, ranks[r].stream));
                B2_CUDA(cudaMemcpyAsync(&host[1], ranks[r].max_abs, sizeof(unsigned int), cudaMemcpyDeviceToHost, ranks[r].stream));
                B2_CUDA(cudaStreamSynchronize(ranks[r].stream));
                if (host[0] != 0 && wrong_total == 0 && env::get_bool("B200CCL_DEBUG_FIRST_WRONG", false, "NANO_NCCL_DEBUG_FIRST_WRONG")) {
                    if (coll == Collective::AllGather) {
                        for (int src = 0; src < nranks; ++src)
                            report_first_wrong(static_cast<char*>(ranks[r].recv[last_set]) + src * count * esz, count, config.dtype,
                                               config.redop, config.uniform_data, kSeed, nranks, src, 0, eps, r);
                    } else {
                        const std::uint64_t first = coll == Collective::ReduceScatter ? (std::uint64_t)r * count : 0;
                        report_first_wrong(ranks[r].recv[last_set], count, config.dtype, config.redop, config.uniform_data, kSeed,
                                           nranks, -1, first, eps, r);
                    }
                }
                wrong_total += host[0];
                const unsigned int m = static_cast<unsigned int>(host[1] & 0xffffffffull);
                float mf;
                std::memcpy(&mf, &m, sizeof(mf));
                max_abs = std::max(max_abs, mf);
            }

            BenchResult res;
            res.algo = algo_name(comm->last_call().algo);
            res.collective = coll;
            res.dtype = config.dtype;
            res.redop = config.redop;
            res.transport = comm->transport();
            res.nranks = nranks;
            res.bytes = count * esz;
            res.count = count;
            res.time_us = config.iters > 0 ? worst_ms * 1e3 / config.iters : 0;
            const std::size_t alg_bytes = coll == Collective::AllReduce ? res.bytes : res.bytes * nranks;
            res.algbw = algbw_gbs(alg_bytes, res.time_us);
            res.busbw = busbw_gbs(coll, res.algbw, nranks);
            res.wrong = static_cast<long long>(wrong_total);
            res.max_abs_error = max_abs;
            results->push_back(res);
        } catch (const std::exception& e) {
            std::fprintf(stderr, "bench: size %zu failed: %s\n", bytes, e.what());
            rc = 1;
        }
        // Release this size's buffers.
        sync_all();
        for (auto& v : sym_in) comm->free_symmetric(v);
        for (auto& v : sym_out) comm->free_symmetric(v);
        for (int r = 0; r < nranks; ++r) {
            if (!config.symmetric) {
                DeviceGuard guard(ranks[r].device);
                for (void* p : ranks[r].send) cudaFree(p);
                for (void* p : ranks[r].recv) cudaFree(p);
            }
            ranks[r].send.clear();
            ranks[r].recv.clear();
        }
        if (rc != 0) break;
    }
    comm.reset();  // waits for work in flight; streams, events and counters are released by their owners
    return rc;
}

int run_all_reduce_bench(const BenchConfig& config, std::vector<BenchResult>* results) {
    BenchConfig c = config;
    c.collective = Collective::AllReduce;
    return run_collective_bench(c, results);
}

}  // namespace b200ccl
