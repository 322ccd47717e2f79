// Ring edge sets without a GPU: every ring edge of a three-rank, two-channel ring is looped
// through the socket transport (real TCP on 127.0.0.1, HELLO matching, proxy threads) and then
// through the RDMA transport (in-process verbs backend, both data planes), while host threads play
// the kernels' part of the Simple protocol on the mapped FIFOs: credit wait, payload, size, tail on
// the sending side; tail wait, check, head on the receiving side. More slices than the FIFO holds
// are sent, so credit must flow back through the proxies.
#include "check.h"
#include "sched/ring_geometry.h"
#include "transport/net_edge.h"

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

using namespace b200ccl;
using namespace b200ccl::transport;

namespace {

constexpr int kRanks = 3, kChannels = 2, kSlices = 11;
constexpr std::size_t kFifoBytes = 64 << 10;  // 8 steps of 8 KiB

unsigned long long load(const unsigned long long* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
void store(unsigned long long* p, unsigned long long v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }

bool spin_until(const std::function<bool()>& pred) {
    const auto end = std::chrono::steady_clock::now() + std::chrono::seconds(20);
    while (!pred()) {
        if (std::chrono::steady_clock::now() > end) return false;
        std::this_thread::yield();
    }
    return true;
}

unsigned char pattern(int src, int channel, int slice, std::size_t i) {
    return static_cast<unsigned char>(src * 61 + channel * 17 + slice * 7 + i);
}

void run_ring(TransportKind kind) {
    NetEdgeConfig cfg;
    cfg.kind = kind;
    cfg.nranks = kRanks;
    cfg.channels = kChannels;
    cfg.fifo_bytes = kFifoBytes;
    cfg.all_edges = true;
    for (int r = 0; r < kRanks; ++r) cfg.local.push_back({r, 0});
    auto edges = create_net_edges(cfg, nullptr);
    edges->start();
    const std::size_t step_bytes = kFifoBytes / ring::kFifoSteps;
    std::atomic<int> failures{0};
    std::vector<std::thread> threads;
    for (int r = 0; r < kRanks; ++r) {
        for (int c = 0; c < kChannels; ++c) {
            const NetHalf* out = edges->send_half(r, c);
            const NetHalf* in = edges->recv_half(r, c);
            T_CHECK(out && in && out->fifo && in->fifo && out->sizes);
            threads.emplace_back([=, &failures] {  // sending side of rank r
                for (int s = 0; s < kSlices; ++s) {
                    const unsigned long long step = static_cast<unsigned long long>(s) * ring::kSliceSteps;
                    if (!spin_until([&] { return ring::send_credit_ok(load(out->head), step); })) { ++failures; return; }
                    const std::size_t n = 1000 + 37 * s + r;  // different payload sizes, within two steps
                    auto* slot = static_cast<unsigned char*>(out->fifo) + ring::slot_offset(step, step_bytes);
                    for (std::size_t i = 0; i < n; ++i) slot[i] = pattern(r, c, s, i);
                    out->sizes[step % ring::kFifoSteps] = static_cast<unsigned int>(n);
                    store(out->tail, step + ring::kSliceSteps);
                }
            });
            threads.emplace_back([=, &failures] {  // receiving side of rank r: data comes from rank r-1
                const int src = (r + kRanks - 1) % kRanks;
                for (int s = 0; s < kSlices; ++s) {
                    const unsigned long long step = static_cast<unsigned long long>(s) * ring::kSliceSteps;
                    if (!spin_until([&] { return ring::recv_ready_ok(load(in->tail), step); })) { ++failures; return; }
                    const std::size_t n = 1000 + 37 * s + src;
                    const auto* slot = static_cast<const unsigned char*>(in->fifo) + ring::slot_offset(step, step_bytes);
                    for (std::size_t i = 0; i < n; ++i)
                        if (slot[i] != pattern(src, c, s, i)) { ++failures; return; }
                    store(in->head, step + ring::kSliceSteps);
                }
            });
        }
    }
    for (auto& t : threads) t.join();
    T_CHECK(failures.load() == 0);
    T_CHECK(edges->first_error().empty());
    T_CHECK(__atomic_load_n(edges->abort_word(), __ATOMIC_ACQUIRE) == 0u);
    edges->stop();
    edges.reset();
}

}  // namespace

int main() {
    run_ring(TransportKind::Socket);
    setenv("B200CCL_RDMA_BACKEND", "fake", 1);
    run_ring(TransportKind::Rdma);
    setenv("B200CCL_RDMA_USE_WRITE", "1", 1);
    setenv("B200CCL_RDMA_SHARED_PROGRESS", "1", 1);
    run_ring(TransportKind::Rdma);
    // a transport that cannot carry ring edges is refused
    NetEdgeConfig bad;
    bad.kind = TransportKind::Shm;
    bad.all_edges = true;
    t_expect_throw([&] { create_net_edges(bad, nullptr); }, "socket or rdma", "kind");
    std::puts("net edges ok");
    return 0;
}
