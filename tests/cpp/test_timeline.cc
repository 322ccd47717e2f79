// Observability units without a GPU: proxy timeline counters, histogram bins, scope timing and
// dump format. Modelled on the reference's tests/rdma_proxy_timeline_test.cc.
#include "check.h"
#include "transport/rdma/timeline.h"

#include <chrono>
#include <cstdlib>
#include <thread>

using namespace b200ccl::transport::rdma;

int main() {
    ProxyTimeline t("send source=0 destination=1 channel=2");
    t.record(TimelineEvent::PostToCqe, 100);
    t.record(TimelineEvent::PostToCqe, 900);
    t.record(TimelineEvent::PostToCqe, 50000);
    T_CHECK(t.count(TimelineEvent::PostToCqe) == 3 && t.total_ns(TimelineEvent::PostToCqe) == 51000 &&
            t.max_ns(TimelineEvent::PostToCqe) == 50000);
    T_CHECK(ProxyTimeline::bin_for(250) == 0 && ProxyTimeline::bin_for(251) == 1 && ProxyTimeline::bin_for(30000) == 10 &&
            ProxyTimeline::bin_for(30001) == 11);
    T_CHECK(t.bin(TimelineEvent::PostToCqe, 0) == 1 && t.bin(TimelineEvent::PostToCqe, 2) == 1 && t.bin(TimelineEvent::PostToCqe, 11) == 1);
    t.record_depth(0); t.record_depth(3); t.record_depth(3); t.record_depth(40);
    T_CHECK(t.depth_bin(0) == 1 && t.depth_bin(3) == 2 && t.depth_bin(kDepthBins - 1) == 1);
    {
        TimelineScope scope(&t, TimelineEvent::CtsWait);
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
    T_CHECK(t.count(TimelineEvent::CtsWait) == 1 && t.total_ns(TimelineEvent::CtsWait) >= 1000000);
    { TimelineScope none(nullptr, TimelineEvent::CtsWait); }
    const std::string d = t.dump();
    T_CHECK(d.find("rdma proxy timeline v1 send source=0 destination=1 channel=2") == 0);
    T_CHECK(d.find("post_to_cqe count=3 avg_ns=17000 max_ns=50000") != std::string::npos);
    T_CHECK(d.find("depth hist=1,0,0,2") != std::string::npos);
    for (int e = 0; e < static_cast<int>(TimelineEvent::kCount); ++e)
        T_CHECK(d.find(timeline_event_name(static_cast<TimelineEvent>(e))) != std::string::npos);
    unsetenv("B200CCL_RDMA_PROXY_TIMELINE"); unsetenv("NANO_NCCL_RDMA_PROXY_TIMELINE");
    T_CHECK(!timeline_enabled_from_env());
    setenv("B200CCL_RDMA_PROXY_TIMELINE", "true", 1);
    T_CHECK(!timeline_enabled_from_env());  // exactly "1"
    setenv("B200CCL_RDMA_PROXY_TIMELINE", "1", 1);
    T_CHECK(timeline_enabled_from_env());
    std::puts("timeline ok");
    return 0;
}
