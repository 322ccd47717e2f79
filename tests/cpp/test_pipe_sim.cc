// The staged tile pipeline's three-counter protocol on host threads (sim/pipe_sim.h): messages from
// one ragged tile to many tiles per CTA, several calls in a row without resetting a counter, two and
// four arena slots, every operator, a rank whose copy-in dawdles, and a rank whose copy-in stops (the
// others' bounded waits run out and name it). Run under ThreadSanitizer it also checks that every
// access to an arena slot is ordered by one of the counters.
#include "check.h"
#include "sim/pipe_sim.h"

using namespace b200ccl;
using namespace b200ccl::sim;

int main() {
    const std::vector<std::size_t> lengths = {1, 64, 65, 1000, 4096 + 3, 7, 640, 2048};
    for (int n : {2, 4, 8}) {
        for (RedOp op : {RedOp::Sum, RedOp::Avg, RedOp::Max, RedOp::Min}) {
            for (int slots : {2, 4}) {
                PipeSimConfig c;
                c.nranks = n;
                c.ctas = n == 8 ? 2 : 3;
                c.slots = slots;
                c.tile_elems = 64;
                c.redop = op;
                c.call_elems = lengths;
                c.slow_rank = n - 1;
                const PipeSimResult r = run_pipe_sim(c);
                T_CHECK(r.wrong == 0 && !r.timed_out);
                long long tiles = 0;
                for (std::size_t len : lengths) tiles += static_cast<long long>((len + 63) / 64);
                T_CHECK(r.tiles == tiles * n);
                // copy-in runs at most `slots` tiles ahead of reduce, reduce at most `slots` ahead of copy-out
                T_CHECK(r.max_tiles_in_flight >= 1 && r.max_tiles_in_flight <= 2 * slots);
            }
        }
    }
    {   // many calls back to back: the counters only grow
        PipeSimConfig c;
        c.nranks = 4;
        c.ctas = 2;
        c.call_elems.assign(100, 700);
        const PipeSimResult r = run_pipe_sim(c);
        T_CHECK(r.wrong == 0 && !r.timed_out);
    }
    {   // rank 1's copy-in stops at call 2: someone's wait runs out and names rank 1; the calls before were right
        PipeSimConfig c;
        c.nranks = 4;
        c.ctas = 2;
        c.call_elems.assign(5, 1000);
        c.stall_rank = 1;
        c.stall_at_call = 2;
        c.wait_timeout_ms = 200.0;
        const PipeSimResult r = run_pipe_sim(c);
        T_CHECK(r.timed_out && r.timeout_peer == 1 && r.wrong == 0);
        T_CHECK(r.message.find("waiting for rank 1") != std::string::npos);
    }
    {   // bad configurations are refused
        PipeSimConfig c;
        c.call_elems = {0};
        T_CHECK(run_pipe_sim(c).wrong == -1);
        c.call_elems = {10};
        c.slots = 0;
        T_CHECK(run_pipe_sim(c).wrong == -1);
    }
    std::printf("pipe sim ok\n");
    return 0;
}
