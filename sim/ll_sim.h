// CPU-only simulator of the low-latency (flag-in-data) AllReduce protocol of
// src/kernels/sm100/ll_allreduce.cu: every (rank, CTA) pair is a host thread; receive slots are
// std::atomic<uint64_t> {data, call number} written and polled with relaxed ordering (the device
// uses one 8-byte relaxed system-scope store / load per slot); a rank's CTAs meet between calls as
// the kernels of one stream do, but RANKS run free, so a fast rank gets one call ahead of a slow one
// and the two slot parities are really exercised. It checks every call's result against a host
// reduction, and a rank that stops makes the others' bounded waits run out with its identity.
//
// The reference has no such protocol and no simulator.
#pragma once

#include "b200ccl/types.h"

#include <cstddef>
#include <string>
#include <vector>

namespace b200ccl::sim {

struct LlSimConfig {
    int nranks = 4;
    int ctas = 2;                         // CTAs per rank (the device kernel uses 8)
    int lanes = 4;                        // "threads" per CTA: word w belongs to CTA (w / lanes) % ctas
    RedOp redop = RedOp::Sum;
    std::vector<std::size_t> call_words;  // one entry per call: message length in 4-byte words (> 0)
    std::size_t max_words = 1024;         // slot capacity per source (device: 32768)
    double wait_timeout_ms = 2000.0;
    int slow_rank = -1;                   // this rank sleeps a little before every call (skew)
    int stall_rank = -1;                  // failure injection: this rank never starts ...
    int stall_at_call = 0;                // ... this call (0-based) nor any later one
};

struct LlSimResult {
    long long wrong = 0;           // wrong words over all ranks and calls
    bool timed_out = false;
    int timeout_rank = -1;         // first rank whose wait ran out
    int timeout_peer = -1;         // the source it was waiting for
    long long timeout_call = -1;   // 0-based
    int max_lead = 0;              // largest number of calls one rank was observed ahead of another
    std::string message;
};

LlSimResult run_ll_sim(const LlSimConfig& config);

}  // namespace b200ccl::sim
