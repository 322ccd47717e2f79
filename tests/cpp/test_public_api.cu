// C++ public API on one GPU (four ranks emulated by one launch): configuration and argument
// errors, the three collectives, NaN propagation, back-to-back launches without a
// synchronisation, moving a communicator while work is in flight, destroying it with
// unsynchronised streams, symmetric allocation, and the nano_nccl:: alias headers.
// Modelled on the reference's tests/public_api.cu:668-916. Returns 77 without a GPU.
#include "check.h"
#include "nano_nccl/communicator.h"
#include "nano_nccl/types.h"

#include <cmath>
#include <vector>

namespace nn = nano_nccl;  // the alias namespace must be usable as the reference's was

#define CK(x) T_CHECK((x) == cudaSuccess)

namespace {

constexpr int kRanks = 4;

struct Buffers {
    std::vector<float*> in, out;
    std::vector<const void*> send;
    std::vector<void*> recv;
    std::vector<cudaStream_t> streams;
    std::size_t count;
    Buffers(std::size_t n, cudaStream_t s, std::size_t in_mult = 1, std::size_t out_mult = 1) : count(n) {
        for (int r = 0; r < kRanks; ++r) {
            float *a, *b;
            CK(cudaMalloc(&a, n * in_mult * sizeof(float)));
            CK(cudaMalloc(&b, n * out_mult * sizeof(float)));
            std::vector<float> h(n * in_mult);
            for (std::size_t i = 0; i < h.size(); ++i) h[i] = static_cast<float>((i % 97) + r * 1000);
            CK(cudaMemcpy(a, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice));
            in.push_back(a); out.push_back(b); send.push_back(a); recv.push_back(b); streams.push_back(s);
        }
    }
    ~Buffers() { for (auto p : in) cudaFree(p); for (auto p : out) cudaFree(p); }
    nn::CollectiveArgs args(nn::RedOp op = nn::RedOp::Sum) const {
        nn::CollectiveArgs a;
        a.send_buffers = send; a.recv_buffers = recv; a.streams = streams; a.count = count;
        a.dtype = nn::DType::Float; a.redop = op;
        return a;
    }
    std::vector<float> host(int r, std::size_t n) const {
        std::vector<float> h(n);
        T_CHECK(cudaMemcpy(h.data(), out[r], n * sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess);
        return h;
    }
};

nn::CommunicatorConfig loop_config() {
    nn::CommunicatorConfig cfg;
    cfg.devices = {0};
    cfg.loopback = true;
    cfg.loopback_ranks = kRanks;
    cfg.wait_timeout_ms = 3000;
    return cfg;
}

}  // namespace

int main() {
    int devices = 0;
    if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) {
        std::puts("no GPU: skipped");
        return 77;
    }
    // configuration errors
    {
        nn::CommunicatorConfig bad;
        t_expect_throw([&] { nn::create_communicator(bad); }, "at least one device", "empty config");
        bad.devices = {0, 99};
        t_expect_throw([&] { nn::create_communicator(bad); }, "visible sequence", "device out of range");
        bad = loop_config();
        bad.transport = nn::TransportKind::Mixed;
        t_expect_throw([&] { nn::create_communicator(bad); }, "mixed", "mixed requested");
    }
    cudaStream_t s;
    CK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    auto comm = nn::create_communicator(loop_config());
    T_CHECK(comm->global_rank_count() == kRanks && comm->local_rank_count() == kRanks);
    T_CHECK(comm->transport() == nn::TransportKind::P2p);
    T_CHECK(comm->describe().find("transport") != std::string::npos);

    // argument errors leave the communicator usable
    Buffers b(1 << 14, s);
    {
        auto a = b.args(); a.streams.pop_back();
        t_expect_throw([&] { comm->all_reduce(a); }, "one entry per rank", "sizes");
        a = b.args(); a.count = 0;
        t_expect_throw([&] { comm->all_reduce(a); }, "positive", "count");
        a = b.args(); a.recv_buffers[2] = nullptr;
        t_expect_throw([&] { comm->all_reduce(a); }, "non-null", "null");
        a = b.args(); a.recv_buffers[1] = const_cast<void*>(a.send_buffers[1]);
        t_expect_throw([&] { comm->all_reduce(a); }, "in-place", "in-place");
        a = b.args(); a.redop = static_cast<nn::RedOp>(11);
        t_expect_throw([&] { comm->all_reduce(a); }, "reduction", "redop");
        a = b.args(); a.dtype = static_cast<nn::DType>(5);
        t_expect_throw([&] { comm->all_reduce(a); }, "unsupported dtype", "dtype");
    }
    // two rounds of sum, then max / avg / min
    for (int round = 0; round < 2; ++round) {
        comm->all_reduce(b.args());
        CK(cudaStreamSynchronize(s));
        comm->check_async_error();
        for (int r = 0; r < kRanks; ++r) {
            auto h = b.host(r, b.count);
            for (std::size_t i = 0; i < b.count; i += 997) T_CHECK(std::fabs(h[i] - (4.0f * (i % 97) + 6000.0f)) < 1e-3f);
        }
    }
    comm->all_reduce(b.args(nn::RedOp::Max));
    CK(cudaStreamSynchronize(s));
    T_CHECK(b.host(1, 8)[5] == 5.0f + 3000.0f);
    comm->all_reduce(b.args(nn::RedOp::Avg));
    CK(cudaStreamSynchronize(s));
    T_CHECK(std::fabs(b.host(2, 8)[5] - (5.0f + 1500.0f)) < 1e-3f);
    comm->all_reduce(b.args(nn::RedOp::Min));
    CK(cudaStreamSynchronize(s));
    T_CHECK(b.host(3, 8)[5] == 5.0f);

    // reduce_scatter and all_gather are implemented (the reference throws for both)
    {
        Buffers rs(4096, s, kRanks, 1);
        comm->reduce_scatter(rs.args());
        CK(cudaStreamSynchronize(s));
        for (int r = 0; r < kRanks; ++r) {
            auto h = rs.host(r, 4096);
            const std::size_t gi = static_cast<std::size_t>(r) * 4096 + 7;
            T_CHECK(std::fabs(h[7] - (4.0f * (gi % 97) + 6000.0f)) < 1e-3f);
        }
        Buffers ag(4096, s, 1, kRanks);
        comm->all_gather(ag.args());
        CK(cudaStreamSynchronize(s));
        auto h = ag.host(0, 4096 * kRanks);
        for (int r = 0; r < kRanks; ++r) T_CHECK(h[r * 4096 + 11] == 11.0f + r * 1000.0f);
        comm->check_async_error();
    }
    // NaN injected on rank 1 propagates through max and min
    {
        Buffers n(32, s);
        const float nanv = std::nanf("");
        for (int i : {3, 11, 19, 27}) CK(cudaMemcpy(n.in[1] + i, &nanv, sizeof(float), cudaMemcpyHostToDevice));
        for (nn::RedOp op : {nn::RedOp::Max, nn::RedOp::Min}) {
            comm->all_reduce(n.args(op));
            CK(cudaStreamSynchronize(s));
            for (int r = 0; r < kRanks; ++r) {
                auto h = n.host(r, 32);
                for (int i = 0; i < 32; ++i) T_CHECK(std::isnan(h[i]) == (i == 3 || i == 11 || i == 19 || i == 27));
            }
        }
    }
    // back-to-back launches without synchronisation, then move while in flight
    {
        Buffers big(1 << 22, s);
        for (int i = 0; i < 8; ++i) comm->all_reduce(big.args());
        auto moved = std::move(comm);  // work is still running
        moved->all_reduce(big.args());
        CK(cudaStreamSynchronize(s));
        moved->check_async_error();
        auto h = big.host(0, 16);
        T_CHECK(std::fabs(h[9] - (4.0f * 9 + 6000.0f)) < 1e-3f);
        comm = std::move(moved);
    }
    // symmetric allocation: one pointer per local rank, usable as a collective buffer
    {
        auto in = comm->alloc_symmetric(1 << 16);
        auto out = comm->alloc_symmetric(1 << 16);
        T_CHECK(in.size() == static_cast<std::size_t>(kRanks));
        nn::CollectiveArgs a;
        for (int r = 0; r < kRanks; ++r) {
            CK(cudaMemset(in[r], 0, 1 << 16));
            a.send_buffers.push_back(in[r]); a.recv_buffers.push_back(out[r]); a.streams.push_back(s);
        }
        a.count = (1 << 16) / 4;
        comm->all_reduce(a);
        CK(cudaStreamSynchronize(s));
        comm->check_async_error();
        comm->free_symmetric(in);
        comm->free_symmetric(out);
        t_expect_throw([&] { comm->free_symmetric(out); }, "live window", "double free");
    }
    // destruction with unsynchronised streams waits for the work
    {
        Buffers big(1 << 22, s);
        auto other = nn::create_communicator(loop_config());
        for (int i = 0; i < 4; ++i) other->all_reduce(big.args());
        other.reset();  // no stream synchronisation before this
        auto h = big.host(2, 16);
        T_CHECK(std::fabs(h[4] - (4.0f * 4 + 6000.0f)) < 1e-3f);
    }
    comm.reset();
    cudaStreamDestroy(s);
    std::puts("public api ok");
    return 0;
}
