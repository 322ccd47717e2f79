// Host-side timeline of the RDMA proxies: per event kind a count, total, maximum and a 12-bin
// histogram of durations (bin edges 250 ns … 30 µs), plus histograms of the in-flight depth at
// post time. Hooks in the proxies are compiled only with B200CCL_ENABLE_TIMELINE and recorded
// only when B200CCL_RDMA_PROXY_TIMELINE is exactly "1", so release binaries carry no
// instrumentation. Dumped as text when the edge set is destroyed.
//
// Parity: nano-nccl src/transport/rdma/rdma_proxy_timeline.h:11-101 / .cc:12-192.
#pragma once

#include <array>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <string>

namespace b200ccl::transport::rdma {

enum class TimelineEvent : int {
    ReadyToPost = 0,   // slice became sendable → work request posted
    InterPost,         // between two consecutive posts
    PostToCqe,         // post → its completion seen
    CqeToPublish,      // completion seen → counter published
    TailArmToPost,     // kernel published tail → post (send side)
    CtsWait,           // waiting for a clear-to-send grant
    CtsGrant,          // slot freed → grant written (receive side)
    kCount
};
const char* timeline_event_name(TimelineEvent e);

constexpr int kTimelineBins = 12;
// Upper edges in ns of bins 0..10; bin 11 is "longer".
extern const std::array<std::uint64_t, kTimelineBins - 1> kTimelineBinEdgesNs;
constexpr int kDepthBins = 9;  // in-flight depth 0..7, 8+

struct TimelineCounter {
    std::atomic<std::uint64_t> count{0}, total_ns{0}, max_ns{0};
    std::array<std::atomic<std::uint64_t>, kTimelineBins> bins{};
};

class ProxyTimeline {
public:
    ProxyTimeline(std::string label = "") : label_(std::move(label)) {}
    void record(TimelineEvent e, std::uint64_t ns);
    void record_depth(int in_flight);
    std::uint64_t count(TimelineEvent e) const { return counters_[static_cast<int>(e)].count.load(); }
    std::uint64_t total_ns(TimelineEvent e) const { return counters_[static_cast<int>(e)].total_ns.load(); }
    std::uint64_t max_ns(TimelineEvent e) const { return counters_[static_cast<int>(e)].max_ns.load(); }
    std::uint64_t bin(TimelineEvent e, int b) const { return counters_[static_cast<int>(e)].bins[b].load(); }
    std::uint64_t depth_bin(int b) const { return depth_[b].load(); }
    // "rdma proxy timeline v1 <label>" header, then one line per event kind and one depth line.
    std::string dump() const;
    static int bin_for(std::uint64_t ns);

private:
    std::string label_;
    std::array<TimelineCounter, static_cast<int>(TimelineEvent::kCount)> counters_{};
    std::array<std::atomic<std::uint64_t>, kDepthBins> depth_{};
};

// Measures a scope and records it on destruction (no-op with a null timeline).
class TimelineScope {
public:
    TimelineScope(ProxyTimeline* t, TimelineEvent e) : t_(t), e_(e), t0_(std::chrono::steady_clock::now()) {}
    ~TimelineScope() {
        if (t_) t_->record(e_, static_cast<std::uint64_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(
                                   std::chrono::steady_clock::now() - t0_).count()));
    }
private:
    ProxyTimeline* t_;
    TimelineEvent e_;
    std::chrono::steady_clock::time_point t0_;
};

bool timeline_enabled_from_env();  // B200CCL_RDMA_PROXY_TIMELINE (or NANO_NCCL_…) exactly "1"

}  // namespace b200ccl::transport::rdma
