#include "transport/rdma/timeline.h"

#include "core/env.h"

#include <cstring>
#include <sstream>

namespace b200ccl::transport::rdma {

const std::array<std::uint64_t, kTimelineBins - 1> kTimelineBinEdgesNs = {250,  500,  1000,  2000,  3000, 5000,
                                                                           7500, 10000, 15000, 20000, 30000};

const char* timeline_event_name(TimelineEvent e) {
    switch (e) {
        case TimelineEvent::ReadyToPost: return "ready_to_post";
        case TimelineEvent::InterPost: return "inter_post";
        case TimelineEvent::PostToCqe: return "post_to_cqe";
        case TimelineEvent::CqeToPublish: return "cqe_to_publish";
        case TimelineEvent::TailArmToPost: return "tail_arm_to_post";
        case TimelineEvent::CtsWait: return "cts_wait";
        case TimelineEvent::CtsGrant: return "cts_grant";
        default: return "unknown";
    }
}

int ProxyTimeline::bin_for(std::uint64_t ns) {
    for (int b = 0; b < kTimelineBins - 1; ++b)
        if (ns <= kTimelineBinEdgesNs[b]) return b;
    return kTimelineBins - 1;
}

void ProxyTimeline::record(TimelineEvent e, std::uint64_t ns) {
    TimelineCounter& c = counters_[static_cast<int>(e)];
    c.count.fetch_add(1, std::memory_order_relaxed);
    c.total_ns.fetch_add(ns, std::memory_order_relaxed);
    std::uint64_t prev = c.max_ns.load(std::memory_order_relaxed);
    while (ns > prev && !c.max_ns.compare_exchange_weak(prev, ns, std::memory_order_relaxed)) {
    }
    c.bins[bin_for(ns)].fetch_add(1, std::memory_order_relaxed);
}

void ProxyTimeline::record_depth(int in_flight) {
    const int b = in_flight < 0 ? 0 : (in_flight >= kDepthBins - 1 ? kDepthBins - 1 : in_flight);
    depth_[b].fetch_add(1, std::memory_order_relaxed);
}

std::string ProxyTimeline::dump() const {
    std::ostringstream os;
    os << "rdma proxy timeline v1 " << label_ << "\n";
    for (int e = 0; e < static_cast<int>(TimelineEvent::kCount); ++e) {
        const TimelineCounter& c = counters_[e];
        const std::uint64_t n = c.count.load();
        os << "  " << timeline_event_name(static_cast<TimelineEvent>(e)) << " count=" << n << " avg_ns=" << (n ? c.total_ns.load() / n : 0)
           << " max_ns=" << c.max_ns.load() << " hist=";
        for (int b = 0; b < kTimelineBins; ++b) os << (b ? "," : "") << c.bins[b].load();
        os << "\n";
    }
    os << "  depth hist=";
    for (int b = 0; b < kDepthBins; ++b) os << (b ? "," : "") << depth_[b].load();
    os << "\n";
    return os.str();
}

bool timeline_enabled_from_env() {
    const char* v = env::get("B200CCL_RDMA_PROXY_TIMELINE", "NANO_NCCL_RDMA_PROXY_TIMELINE");
    return v && std::strcmp(v, "1") == 0;
}

}  // namespace b200ccl::transport::rdma
