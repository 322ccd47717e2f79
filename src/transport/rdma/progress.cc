#include "transport/rdma/progress.h"

#include "core/numa.h"

#if defined(__x86_64__)
#include <immintrin.h>
#endif

namespace b200ccl::transport::rdma {

namespace {
inline void cpu_relax() {
#if defined(__x86_64__)
    _mm_pause();
#else
    std::this_thread::yield();
#endif
}
}  // namespace

void ProgressEngine::add(RdmaProxy* proxy) { (proxy->is_receiver() ? receivers_ : senders_).push_back(proxy); }

void ProgressEngine::run_one(RdmaProxy* p) {
    numa::pin_current_thread_to_node(numa_node_);
    while (!stop_.load(std::memory_order_acquire)) {
        if (p->failed()) break;
        if (!p->progress()) cpu_relax();
    }
}

void ProgressEngine::run_all() {
    numa::pin_current_thread_to_node(numa_node_);
    while (!stop_.load(std::memory_order_acquire)) {
        bool did = false;
        for (RdmaProxy* p : receivers_) did = p->progress() || did;
        if (senders_live_.load(std::memory_order_acquire))
            for (RdmaProxy* p : senders_) did = p->progress() || did;
        if (!did) {
            idle_rounds_.fetch_add(1, std::memory_order_relaxed);
            cpu_relax();
        }
    }
}

void ProgressEngine::start_receivers() {
    for (RdmaProxy* p : receivers_) p->prepare();
    if (shared_) {
        threads_.emplace_back([this] { run_all(); });
    } else {
        for (RdmaProxy* p : receivers_) threads_.emplace_back([this, p] { run_one(p); });
    }
}

void ProgressEngine::start_senders() {
    senders_live_.store(true, std::memory_order_release);
    if (!shared_)
        for (RdmaProxy* p : senders_) threads_.emplace_back([this, p] { run_one(p); });
}

void ProgressEngine::stop() noexcept {
    stop_.store(true, std::memory_order_release);
    for (auto& t : threads_)
        if (t.joinable()) t.join();
    threads_.clear();
}

}  // namespace b200ccl::transport::rdma
