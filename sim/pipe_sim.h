// CPU-only simulator of the staged tile pipeline of src/kernels/sm100/staged_pipeline.cu: every
// (rank, CTA) pair runs three host threads (copy-in, reduce, copy-out) that meet the same stages
// of the same CTA index on every other rank through three monotonic counters per (CTA, source
// rank), exactly the device's PipeFlags: "tile copied in", "shard reduced and stored everywhere",
// "tile copied out". std::atomic with release stores and acquire loads stands for st.release.sys /
// ld.acquire.sys; the arenas are plain memory, so a missing happens-before edge is a data race
// that ThreadSanitizer reports. Slot reuse follows the device's rules (a slot of the input half is
// refilled once every rank has reduced the tile it held, a slot of the output half is rewritten
// once every rank has copied its tile out), calls follow one another without resetting anything,
// and a rank whose copy-in stage stops makes the others' bounded waits run out with its identity.
//
// The reference has no such protocol and no simulator.
#pragma once

#include "b200ccl/types.h"

#include <cstddef>
#include <string>
#include <vector>

namespace b200ccl::sim {

struct PipeSimConfig {
    int nranks = 4;
    int ctas = 2;                          // CTAs per rank
    int slots = 2;                         // arena slots per CTA and half
    std::size_t tile_elems = 64;           // fp32 elements per tile
    RedOp redop = RedOp::Sum;
    std::vector<std::size_t> call_elems;   // one entry per call: message length in elements (> 0)
    double wait_timeout_ms = 2000.0;
    int slow_rank = -1;                    // this rank's copy-in stage dawdles (skew between ranks)
    int stall_rank = -1;                   // failure injection: this rank's copy-in stage stops ...
    int stall_at_call = 0;                 // ... at this call (0-based)
};

struct PipeSimResult {
    long long wrong = 0;          // wrong elements over all ranks and calls (-1: bad configuration)
    bool timed_out = false;
    int timeout_rank = -1;        // first rank whose wait ran out
    int timeout_peer = -1;        // the rank it was waiting for
    int timeout_stage = -1;       // 0 copy-in, 1 reduce, 2 copy-out
    long long tiles = 0;          // tiles taken through the pipeline (all ranks, CTAs and calls)
    int max_tiles_in_flight = 0;  // most tiles one CTA had between copy-in and copy-out at once
    std::string message;
};

PipeSimResult run_pipe_sim(const PipeSimConfig& config);

}  // namespace b200ccl::sim
