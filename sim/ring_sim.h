// CPU-only simulator of the ring + Simple protocol: every (rank, channel) pair is a host thread
// that runs the same schedule as the device kernel (same geometry header), with FIFOs in host
// memory and step counters as std::atomic with release/acquire ordering. It needs no GPU.
//
// Uses: (1) an oracle and timing baseline for the plumbing (4 ranks, 4 channels, 1 Mi floats per
// rank, values uniform[-1,1) from seed = rank); (2) a place to run the flag protocol under a
// thread sanitizer; (3) failure tests: a rank that stops makes its neighbours' bounded waits run
// out, and the result names who waited for whom.
//
// The reference has no simulator; its protocol checks need a GPU (tests/simple_protocol.cu).
#pragma once

#include "b200ccl/types.h"

#include <cstddef>
#include <cstdint>
#include <string>

namespace b200ccl::sim {

struct RingSimConfig {
    int nranks = 4;
    int channels = 4;
    std::size_t count = 1u << 20;          // floats per rank
    std::size_t fifo_bytes = 4u << 20;     // per channel and edge
    RedOp redop = RedOp::Sum;
    Collective collective = Collective::AllReduce;
    double wait_timeout_ms = 5000.0;
    int stall_rank = -1;                   // failure injection: this rank stops ...
    long long stall_after_slices = 0;      // ... after this many slices (on every channel)
};

struct RingSimResult {
    double seconds = 0.0;
    long long wrong = 0;          // elements off by more than 1e-5 against the host reduction
    float max_abs_error = 0.0f;
    bool timed_out = false;
    int timeout_rank = -1;        // first rank whose wait ran out
    int timeout_peer = -1;        // rank it was waiting for
    int timeout_channel = -1;
    unsigned long long timeout_step = 0;
    unsigned long long slices = 0;        // non-empty slices processed, all threads
    unsigned long long empty_slices = 0;  // elided
    std::string message;
};

RingSimResult run_ring_sim(const RingSimConfig& config);

}  // namespace b200ccl::sim
