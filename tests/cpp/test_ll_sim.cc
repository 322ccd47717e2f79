// The low-latency AllReduce protocol on host threads (sim/ll_sim.h): call lengths that change from
// call to call, every operator, a slow rank (so that the others get a call ahead and both slot
// parities are in use at once), and a rank that stops (the others' waits run out and name it).
#include "check.h"
#include "sim/ll_sim.h"

using namespace b200ccl;
using namespace b200ccl::sim;

int main() {
    const std::vector<std::size_t> lengths = {1, 1000, 7, 1024, 3, 512, 1024, 1, 64, 999, 2, 1024};
    for (int n : {2, 4, 8}) {
        for (RedOp op : {RedOp::Sum, RedOp::Avg, RedOp::Max, RedOp::Min}) {
            LlSimConfig c;
            c.nranks = n;
            c.ctas = n == 8 ? 2 : 3;
            c.redop = op;
            c.call_words = lengths;
            c.slow_rank = n - 1;
            const LlSimResult r = run_ll_sim(c);
            T_CHECK(r.wrong == 0 && !r.timed_out);
            T_CHECK(r.max_lead <= 1);  // nobody can finish a call without everyone's data for it
        }
    }
    {   // many short calls back to back: the parities alternate 200 times
        LlSimConfig c;
        c.nranks = 4;
        c.call_words.assign(200, 33);
        c.slow_rank = 1;
        const LlSimResult r = run_ll_sim(c);
        T_CHECK(r.wrong == 0 && !r.timed_out && r.max_lead <= 1);
    }
    {   // rank 2 leaves before call 3: someone's wait runs out in call 3 and names rank 2
        LlSimConfig c;
        c.nranks = 4;
        c.call_words.assign(6, 100);
        c.stall_rank = 2;
        c.stall_at_call = 3;
        c.wait_timeout_ms = 200.0;
        const LlSimResult r = run_ll_sim(c);
        T_CHECK(r.timed_out && r.timeout_peer == 2 && r.timeout_call == 3 && r.timeout_rank != 2);
        T_CHECK(r.wrong == 0);  // the three calls before it were right
        T_CHECK(r.message.find("waiting for rank 2") != std::string::npos);
    }
    {   // bad configurations are refused
        LlSimConfig c;
        c.call_words = {0};
        T_CHECK(run_ll_sim(c).wrong == -1);
        c.call_words = {2000};
        T_CHECK(run_ll_sim(c).wrong == -1);
    }
    std::printf("ll sim ok\n");
    return 0;
}
