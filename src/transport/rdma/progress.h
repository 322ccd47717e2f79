// Drives RDMA proxies: either one host thread per proxy (default) or a single shared thread that
// visits every proxy, receivers first, and pauses the CPU when a whole round did nothing
// (B200CCL_RDMA_SHARED_PROGRESS=1).
// Parity: nano-nccl src/transport/rdma/rdma_progress.cc:14-111.
#pragma once

#include "transport/rdma/proxy.h"

#include <atomic>
#include <thread>
#include <vector>

namespace b200ccl::transport::rdma {

class ProgressEngine {
public:
    explicit ProgressEngine(bool shared, int numa_node = -1) : shared_(shared), numa_node_(numa_node) {}
    ~ProgressEngine() { stop(); }
    ProgressEngine(const ProgressEngine&) = delete;
    ProgressEngine& operator=(const ProgressEngine&) = delete;
    void add(RdmaProxy* proxy);     // before start()
    void start_receivers();         // prepare() + threads of the receive side
    void start_senders();           // threads of the send side (shared mode: starts the one thread)
    void stop() noexcept;           // ask every loop to end and join
    bool shared() const { return shared_; }
    std::size_t thread_count() const { return threads_.size(); }
    std::uint64_t idle_rounds() const { return idle_rounds_.load(); }

private:
    void run_one(RdmaProxy* p);
    void run_all();
    bool shared_;
    int numa_node_;
    std::vector<RdmaProxy*> receivers_, senders_;
    std::vector<std::thread> threads_;
    std::atomic<bool> stop_{false};
    std::atomic<bool> senders_live_{false};
    std::atomic<std::uint64_t> idle_rounds_{0};
};

}  // namespace b200ccl::transport::rdma
