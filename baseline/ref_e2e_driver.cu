// Harness around the UNMODIFIED reference library (nano-nccl), used by `bench.py --impl reference`.
// It calls only the reference's public API (create_communicator, Communicator::all_reduce,
// check_async_error) and times two things with CUDA events on every rank's stream (maximum over
// ranks): K back-to-back all_reduce calls, and the same K steps end to end, where every step
// first copies its input from pinned host memory to the device and finally reads the first
// 4 KiB of the result back. The reference's stock benchmark has no host-to-device path, which is
// why this file exists; nothing of this project's library is linked into it.
//
// usage: ref_e2e_n<N> <bytes> <steps> <warmup> <auto|p2p|shm>
#include "nano_nccl/communicator.h"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#define CK(x)                                                                             \
    do {                                                                                  \
        cudaError_t e_ = (x);                                                             \
        if (e_ != cudaSuccess) {                                                          \
            std::fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));          \
            return 3;                                                                     \
        }                                                                                 \
    } while (0)

int main(int argc, char** argv) {
    if (argc < 5) {
        std::fprintf(stderr, "usage: %s bytes steps warmup transport\n", argv[0]);
        return 2;
    }
    const std::size_t bytes = std::strtoull(argv[1], nullptr, 10);
    const int steps = std::atoi(argv[2]), warmup = std::atoi(argv[3]);
    nano_nccl::TransportKind transport;
    if (!nano_nccl::parse_transport(argv[4], &transport)) return 2;
    const int n = nano_nccl::kRanks;
    const std::size_t count = bytes / sizeof(float);
    const std::size_t back = 4096;

    nano_nccl::CommunicatorConfig cfg;
    for (int d = 0; d < n; ++d) cfg.devices.push_back(d);
    cfg.transport = transport;
    std::unique_ptr<nano_nccl::Communicator> comm;
    try {
        comm = nano_nccl::create_communicator(cfg);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "create_communicator: %s\n", e.what());
        return 4;
    }

    std::vector<float*> send(n), recv(n), host_in(n), host_out(n);
    std::vector<cudaStream_t> streams(n);
    std::vector<cudaEvent_t> start(n), stop(n);
    for (int r = 0; r < n; ++r) {
        CK(cudaSetDevice(r));
        CK(cudaMalloc(&send[r], bytes));
        CK(cudaMalloc(&recv[r], bytes));
        CK(cudaMallocHost(&host_in[r], bytes));
        CK(cudaMallocHost(&host_out[r], back));
        CK(cudaStreamCreateWithFlags(&streams[r], cudaStreamNonBlocking));
        CK(cudaEventCreate(&start[r]));
        CK(cudaEventCreate(&stop[r]));
        for (std::size_t i = 0; i < count; ++i) host_in[r][i] = static_cast<float>((i * 131 + r * 17) % 1000) / 1000.0f - 0.5f;
        CK(cudaMemcpyAsync(send[r], host_in[r], bytes, cudaMemcpyHostToDevice, streams[r]));
        CK(cudaStreamSynchronize(streams[r]));
    }
    nano_nccl::CollectiveArgs args;
    for (int r = 0; r < n; ++r) {
        args.send_buffers.push_back(send[r]);
        args.recv_buffers.push_back(recv[r]);
        args.streams.push_back(streams[r]);
    }
    args.count = count;
    args.dtype = nano_nccl::DType::Float;
    args.redop = nano_nccl::RedOp::Sum;

    auto sync_all = [&]() -> int {
        for (int r = 0; r < n; ++r) {
            CK(cudaSetDevice(r));
            CK(cudaStreamSynchronize(streams[r]));
        }
        return 0;
    };
    auto run = [&](bool e2e, int k) -> int {
        for (int i = 0; i < k; ++i) {
            if (e2e)
                for (int r = 0; r < n; ++r) {
                    CK(cudaSetDevice(r));
                    CK(cudaMemcpyAsync(send[r], host_in[r], bytes, cudaMemcpyHostToDevice, streams[r]));
                }
            comm->all_reduce(args);
            if (e2e)
                for (int r = 0; r < n; ++r) {
                    CK(cudaSetDevice(r));
                    CK(cudaMemcpyAsync(host_out[r], recv[r], back, cudaMemcpyDeviceToHost, streams[r]));
                }
        }
        return 0;
    };
    double ms[2] = {0, 0};
    try {
        for (int mode = 0; mode < 2; ++mode) {
            if (run(mode == 1, warmup)) return 3;
            if (sync_all()) return 3;
            for (int r = 0; r < n; ++r) {
                CK(cudaSetDevice(r));
                CK(cudaEventRecord(start[r], streams[r]));
            }
            if (run(mode == 1, steps)) return 3;
            for (int r = 0; r < n; ++r) {
                CK(cudaSetDevice(r));
                CK(cudaEventRecord(stop[r], streams[r]));
            }
            if (sync_all()) return 3;
            comm->check_async_error();
            for (int r = 0; r < n; ++r) {
                float t = 0;
                CK(cudaEventElapsedTime(&t, start[r], stop[r]));
                if (t / steps > ms[mode]) ms[mode] = t / steps;
            }
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "all_reduce: %s\n", e.what());
        return 5;
    }
    // Spot check of the read-back slice of rank 0.
    long wrong = 0;
    for (std::size_t i = 0; i < back / sizeof(float) && i < count; ++i) {
        float expect = 0;
        for (int r = 0; r < n; ++r) expect += host_in[r][i];
        if (std::fabs(host_out[0][i] - expect) > 1e-4f) ++wrong;
    }
    std::printf("REF_E2E ranks %d bytes %zu steps %d warmup %d transport %s kernel_ms_per_step %.6f e2e_ms_per_step %.6f "
                "h2d_bytes %zu d2h_bytes %zu wrong %ld\n",
                n, bytes, steps, warmup, nano_nccl::transport_name(comm->transport()), ms[0], ms[1], bytes, back, wrong);
    comm.reset();
    return wrong ? 1 : 0;
}
