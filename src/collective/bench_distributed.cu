// Multi-process benchmark runner: one process per GPU (or per group of GPUs), joined by the TCP
// rendezvous, every process timing its own ranks and all of them agreeing on the numbers.
//
// Parity: the MPI variant of nano-nccl's benchmark (benchmarks/all_reduce_bench.cu:84-316):
// constant inputs of value global_rank + 1, a barrier before the timed batch, the maximum over
// ranks of the measured time (MPI_Allreduce(MAX) there, an all-gather over the rendezvous here),
// verification against the closed-form result, and one exit status for all processes. Differences:
// the batch is timed with CUDA events on the launching stream instead of the host clock,
// ReduceScatter and AllGather are covered, and #wrong counts elements.
#include "b200ccl/bench.h"
#include "b200ccl/bootstrap.h"
#include "core/buffers.h"
#include "core/check.h"
#include "core/stream.h"
#include "kernels/sm100/vec.cuh"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <type_traits>

namespace b200ccl {

namespace {

template <typename T>
__global__ void fill_constant_kernel(T* buf, std::size_t count, float value) {
    const T v = dev::Elem<T>::from_f(value);
    for (std::size_t i = blockIdx.x * (std::size_t)blockDim.x + threadIdx.x; i < count; i += (std::size_t)gridDim.x * blockDim.x)
        buf[i] = v;
}

// Counts elements of buf[0, count) further than eps from `expect` (blocks of `block` elements may
// each have their own expectation: expect + block_step * (i / block), for AllGather).
template <typename T>
__global__ void count_wrong_kernel(const T* buf, std::size_t count, float expect, float block_step, std::size_t block,
                                   float eps, unsigned long long* wrong, unsigned int* max_abs_bits) {
    unsigned long long mine = 0;
    float worst = 0.0f;
    for (std::size_t i = blockIdx.x * (std::size_t)blockDim.x + threadIdx.x; i < count; i += (std::size_t)gridDim.x * blockDim.x) {
        const float want = expect + block_step * static_cast<float>(i / block);
        const float err = fabsf(dev::Elem<T>::to_f(buf[i]) - want);
        if (!(err <= eps)) ++mine;  // a NaN counts as wrong
        worst = fmaxf(worst, err);
    }
    if (mine) atomicAdd(wrong, mine);
    atomicMax(max_abs_bits, __float_as_uint(worst));  // non-negative floats order like their bit patterns
}

template <typename Fn>
void by_dtype(DType dtype, Fn&& fn) {
    switch (dtype) {
        case DType::Float: fn(static_cast<float*>(nullptr)); break;
        case DType::Float16: fn(static_cast<__half*>(nullptr)); break;
        case DType::BFloat16: fn(static_cast<__nv_bfloat16*>(nullptr)); break;
    }
}

int launch_grid(std::size_t count) {
    return static_cast<int>(std::min<std::size_t>(1184, std::max<std::size_t>(1, (count + 255) / 256)));
}

}  // namespace

int run_distributed_bench(Bootstrap& bootstrap, int device, const BenchConfig& config, std::vector<BenchResult>* results) {
    if (!results) return 2;
    const int world = bootstrap.size();
    Algo algo = Algo::Auto;
    if (!parse_algo(config.algo.c_str(), &algo)) {
        std::fprintf(stderr, "bench: unknown algo '%s'\n", config.algo.c_str());
        return 2;
    }
    // Failures before the first collective are agreed on, so that no process waits for one that gave up.
    std::string local_error;
    std::unique_ptr<Communicator> comm;
    try {
        B2_CUDA(cudaSetDevice(device));
        CommunicatorConfig cc;
        cc.devices = {device};
        cc.transport = config.transport;
        cc.algo = algo;
        comm = create_communicator_from_bootstrap(bootstrap, cc);
    } catch (const std::exception& e) {
        local_error = e.what();
    }
    const std::string agreed = bootstrap.error_consensus(local_error);
    if (!agreed.empty()) {
        std::fprintf(stderr, "bench: communicator setup failed: %s\n", agreed.c_str());
        return 3;
    }
    const int nranks = comm->global_rank_count();
    const int rank = comm->first_global_rank();
    const std::size_t esz = dtype_size(config.dtype);
    const float eps = config.epsilon > 0 ? config.epsilon : dtype_default_epsilon(config.dtype);
    const Collective coll = config.collective;
    const std::size_t in_mult = coll == Collective::ReduceScatter ? nranks : 1;
    const std::size_t out_mult = coll == Collective::AllGather ? nranks : 1;
    // Closed-form result of reducing the values 1..n.
    float expect = 0.0f;
    switch (config.redop) {
        case RedOp::Sum: expect = 0.5f * nranks * (nranks + 1); break;
        case RedOp::Avg: expect = 0.5f * (nranks + 1); break;
        case RedOp::Max: expect = static_cast<float>(nranks); break;
        case RedOp::Min: expect = 1.0f; break;
    }

    Stream stream(device);
    Event start(device, /*timing=*/true), stop(device, /*timing=*/true);
    DeviceBuffer<unsigned long long> wrong_dev(device, 1);
    DeviceBuffer<unsigned int> max_abs_dev(device, 1);
    int rc = 0;
    for (std::size_t bytes : make_sizes(config.min_bytes, config.max_bytes, config.factor)) {
        const std::size_t count = std::max<std::size_t>(bytes / esz, 1);
        const std::size_t in_bytes = count * esz * in_mult, out_bytes = count * esz * out_mult;
        // Rotate over buffer sets so that successive iterations do not find their data in L2 (126 MB).
        const std::size_t sets = std::min<std::size_t>(8, std::max<std::size_t>(1, (std::size_t(512) << 20) / (in_bytes + out_bytes)));
        std::vector<void*> send, recv;
        std::vector<std::vector<void*>> symmetric;
        double seconds = 0.0;
        unsigned long long wrong = 0;
        unsigned int max_abs_bits = 0;
        CallInfo info;
        std::string failure;
        try {
            for (std::size_t s = 0; s < sets; ++s) {
                void *a = nullptr, *b = nullptr;
                if (config.symmetric) {
                    symmetric.push_back(comm->alloc_symmetric(in_bytes));
                    a = symmetric.back()[0];
                    symmetric.push_back(comm->alloc_symmetric(out_bytes));
                    b = symmetric.back()[0];
                } else {
                    B2_CUDA(cudaMalloc(&a, in_bytes));
                    send.push_back(a);
                    B2_CUDA(cudaMalloc(&b, out_bytes));
                    recv.push_back(b);
                }
                if (config.symmetric) {
                    send.push_back(a);
                    recv.push_back(b);
                }
                by_dtype(config.dtype, [&](auto* tag) {
                    using T = std::remove_pointer_t<decltype(tag)>;
                    fill_constant_kernel<T><<<launch_grid(count * in_mult), 256, 0, stream.get()>>>(
                        static_cast<T*>(a), count * in_mult, static_cast<float>(rank + 1));
                });
                B2_CUDA(cudaGetLastError());
                B2_CUDA(cudaMemsetAsync(b, 0xff, out_bytes, stream.get()));
            }
            CollectiveArgs args;
            args.count = count;
            args.dtype = config.dtype;
            args.redop = config.redop;
            args.streams = {stream.get()};
            auto run_once = [&](std::size_t s) {
                args.send_buffers = {send[s % sets]};
                args.recv_buffers = {recv[s % sets]};
                switch (coll) {
                    case Collective::AllReduce: comm->all_reduce(args); break;
                    case Collective::ReduceScatter: comm->reduce_scatter(args); break;
                    case Collective::AllGather: comm->all_gather(args); break;
                }
            };
            for (int i = 0; i < config.warmup_iters; ++i) run_once(static_cast<std::size_t>(i));
            B2_CUDA(cudaStreamSynchronize(stream.get()));
            comm->check_async_error();
            bootstrap.barrier();
            B2_CUDA(cudaEventRecord(start.get(), stream.get()));
            for (int i = 0; i < config.iters; ++i) run_once(static_cast<std::size_t>(i));
            B2_CUDA(cudaEventRecord(stop.get(), stream.get()));
            B2_CUDA(cudaStreamSynchronize(stream.get()));
            comm->check_async_error();
            float ms = 0.0f;
            B2_CUDA(cudaEventElapsedTime(&ms, start.get(), stop.get()));
            seconds = ms * 1e-3 / std::max(config.iters, 1);
            info = comm->last_call();
            // Verify the set written last.
            const std::size_t last = static_cast<std::size_t>(std::max(config.iters, 1) - 1) % sets;
            wrong_dev.zero();
            max_abs_dev.zero();
            by_dtype(config.dtype, [&](auto* tag) {
                using T = std::remove_pointer_t<decltype(tag)>;
                const bool gather = coll == Collective::AllGather;
                count_wrong_kernel<T><<<launch_grid(count * out_mult), 256, 0, stream.get()>>>(
                    static_cast<const T*>(recv[last]), count * out_mult, gather ? 1.0f : expect, gather ? 1.0f : 0.0f,
                    gather ? count : count * out_mult + 1, eps, wrong_dev.get(), max_abs_dev.get());
            });
            B2_CUDA(cudaGetLastError());
            B2_CUDA(cudaMemcpyAsync(&wrong, wrong_dev.get(), sizeof(wrong), cudaMemcpyDeviceToHost, stream.get()));
            B2_CUDA(cudaMemcpyAsync(&max_abs_bits, max_abs_dev.get(), sizeof(max_abs_bits), cudaMemcpyDeviceToHost, stream.get()));
            B2_CUDA(cudaStreamSynchronize(stream.get()));
        } catch (const std::exception& e) {
            failure = e.what();
        }
        // One row for all processes: slowest rank's time, every rank's wrong elements, or the first failure.
        struct Report {
            double seconds;
            unsigned long long wrong;
            unsigned int max_abs_bits;
            int failed;
        } mine{seconds, wrong, max_abs_bits, failure.empty() ? 0 : 1};
        std::vector<Report> all(static_cast<std::size_t>(world));
        bootstrap.allgather(&mine, all.data(), sizeof(Report));
        const std::string first_failure = bootstrap.error_consensus(failure);
        for (void* p : send)
            if (!config.symmetric) cudaFree(p);
        for (void* p : recv)
            if (!config.symmetric) cudaFree(p);
        if (!first_failure.empty()) {
            std::fprintf(stderr, "bench: size %zu failed: %s\n", bytes, first_failure.c_str());
            rc = 1;
            break;  // the communicator of a failed collective refuses further work
        }
        for (auto& ptrs : symmetric) comm->free_symmetric(ptrs);
        BenchResult r;
        r.algo = algo_name(info.algo);
        r.collective = coll;
        r.dtype = config.dtype;
        r.redop = config.redop;
        r.transport = comm->transport();
        r.nranks = nranks;
        r.bytes = count * esz;
        r.count = count;
        unsigned int worst_bits = 0;
        for (const Report& rep : all) {
            r.time_us = std::max(r.time_us, rep.seconds * 1e6);
            r.wrong += static_cast<long long>(rep.wrong);
            worst_bits = std::max(worst_bits, rep.max_abs_bits);
        }
        float worst = 0.0f;
        static_assert(sizeof(worst) == sizeof(worst_bits), "float bits");
        std::memcpy(&worst, &worst_bits, sizeof(worst));
        r.max_abs_error = worst;
        const std::size_t total = coll == Collective::AllReduce ? r.bytes : r.bytes * static_cast<std::size_t>(nranks);
        r.algbw = algbw_gbs(total, r.time_us);
        r.busbw = busbw_gbs(coll, r.algbw, nranks);
        results->push_back(r);
    }
    comm.reset();
    // The exit status is the same everywhere (all_reduce_bench.cu:414-428 of the reference).
    for (const auto& r : *results)
        if (r.wrong != 0) rc = std::max(rc, 1);
    std::vector<int> codes(static_cast<std::size_t>(world));
    bootstrap.allgather(&rc, codes.data(), sizeof(int));
    return *std::max_element(codes.begin(), codes.end());
}

}  // namespace b200ccl
