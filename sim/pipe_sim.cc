#include "sim/pipe_sim.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <memory>
#include <mutex>
#include <thread>

namespace b200ccl::sim {

namespace {

using Clock = std::chrono::steady_clock;
using u64 = std::uint64_t;

float apply(RedOp op, float a, float b) {
    switch (op) {
        case RedOp::Max: return (a != a) ? a : ((b != b) ? b : (a > b ? a : b));
        case RedOp::Min: return (a != a) ? a : ((b != b) ? b : (a < b ? a : b));
        default: return a + b;
    }
}

// Small integers: every reduction is exact in fp32 whatever the order.
float input_value(int rank, std::size_t call, std::size_t i) {
    return static_cast<float>(static_cast<int>((i * 5 + call * 7 + static_cast<std::size_t>(rank) * 3) % 19) - 9);
}

struct Flags {  // one per rank: row [cta * nranks + src] is written by `src`, read by the owner
    std::unique_ptr<std::atomic<u64>[]> start, in_ready, reduced, drained;
};

struct Shared {
    const PipeSimConfig* cfg = nullptr;
    std::vector<Flags> flags;
    std::vector<std::vector<float>> arena_in, arena_out;   // [rank][(cta * slots + slot) * tile + j]
    std::vector<std::vector<float>> user_in, user_out;     // [rank][i], refilled per call
    // Threads of one rank meet here between calls (a kernel ends when all of its CTAs have).
    std::vector<std::unique_ptr<std::atomic<u64>>> rank_arrivals;
    std::vector<std::unique_ptr<std::atomic<u64>[]>> cta_arrivals;  // [rank][cta]: the three stages of one CTA
    std::vector<std::unique_ptr<std::atomic<long long>[]>> in_flight;  // [rank][cta]
    std::atomic<bool> abort{false};
    std::atomic<long long> wrong{0};
    std::atomic<long long> tiles{0};
    std::atomic<int> max_in_flight{0};
    std::mutex mu;
    PipeSimResult* result = nullptr;
};

void record_timeout(Shared& sh, int rank, int peer, int stage) {
    std::lock_guard<std::mutex> lock(sh.mu);
    if (!sh.result->timed_out) {
        sh.result->timed_out = true;
        sh.result->timeout_rank = rank;
        sh.result->timeout_peer = peer;
        sh.result->timeout_stage = stage;
        static const char* names[] = {"copy-in", "reduce", "copy-out"};
        sh.result->message = "rank " + std::to_string(rank) + " (" + names[stage] + ") gave up waiting for rank " + std::to_string(peer);
    }
    sh.abort.store(true, std::memory_order_release);
}

// The device's bounded wait: acquire loads until the counter reaches `want`, the abort word is
// raised, or time runs out (then this thread raises abort for everyone).
bool wait_at_least(Shared& sh, const std::atomic<u64>& flag, u64 want, int rank, int peer, int stage) {
    const auto deadline = Clock::now() + std::chrono::microseconds(static_cast<long long>(sh.cfg->wait_timeout_ms * 1000.0));
    unsigned polls = 0;
    while (flag.load(std::memory_order_acquire) < want) {
        if ((++polls & 63u) == 0u) {
            if (sh.abort.load(std::memory_order_acquire)) return false;
            if (Clock::now() > deadline) {
                record_timeout(sh, rank, peer, stage);
                return false;
            }
            std::this_thread::yield();
        }
    }
    return true;
}

// Meeting point of `parties` threads that is passed `generation` times; abortable.
bool meet(Shared& sh, std::atomic<u64>& arrivals, u64 parties, u64 generation) {
    arrivals.fetch_add(1, std::memory_order_acq_rel);
    unsigned polls = 0;
    while (arrivals.load(std::memory_order_acquire) < parties * generation) {
        if ((++polls & 63u) == 0u) {
            if (sh.abort.load(std::memory_order_acquire)) return false;
            std::this_thread::yield();
        }
    }
    return true;
}

void stage_thread(Shared& sh, int rank, int cta, int stage) {
    const PipeSimConfig& cfg = *sh.cfg;
    const int n = cfg.nranks, G = cfg.ctas;
    const u64 S = static_cast<u64>(cfg.slots);
    const std::size_t T = cfg.tile_elems;
    auto row = [&](std::unique_ptr<std::atomic<u64>[]>& a, int src) -> std::atomic<u64>& { return a[cta * n + src]; };
    Flags& mine = sh.flags[rank];
    u64 base = 0, epoch = 0, rank_gen = 0, cta_gen = 0;
    const u64 rank_parties = static_cast<u64>(G) * 3;

    for (std::size_t call = 0; call < cfg.call_elems.size(); ++call) {
        const std::size_t count = cfg.call_elems[call];
        const u64 total_tiles = (count + T - 1) / T;
        const u64 K = static_cast<u64>(cta) < total_tiles ? (total_tiles - cta + G - 1) / G : 0;
        auto tile_off = [&](u64 k) { return (static_cast<u64>(cta) + k * G) * T; };
        auto tile_len = [&](u64 k) { return std::min<u64>(T, count - tile_off(k)); };
        auto slot_off = [&](u64 k) { return (static_cast<u64>(cta) * S + (k % S)) * T; };

        // Inputs of this call (one thread per rank fills them), then the rank's threads start together.
        if (cta == 0 && stage == 0) {
            sh.user_in[rank].resize(count);
            sh.user_out[rank].assign(count, -12345.0f);
            for (std::size_t i = 0; i < count; ++i) sh.user_in[rank][i] = input_value(rank, call, i);
        }
        if (!meet(sh, *sh.rank_arrivals[rank], rank_parties, ++rank_gen)) return;
        if (stage == 0 && rank == cfg.stall_rank && static_cast<int>(call) >= cfg.stall_at_call) return;  // this stage stops

        // Start barrier of the call among the CTAs of this index on every rank (the copy-in thread
        // speaks for its CTA), then the CTA's three stages go on together.
        ++epoch;
        if (stage == 0) {
            for (int p = 0; p < n; ++p) sh.flags[p].start[cta * n + rank].store(epoch, std::memory_order_release);
            for (int p = 0; p < n; ++p)
                if (!wait_at_least(sh, row(mine.start, p), epoch, rank, p, 0)) return;
        }
        if (!meet(sh, sh.cta_arrivals[rank][cta], 3, ++cta_gen)) return;

        for (u64 k = 0; k < K; ++k) {
            const u64 so = slot_off(k), len = tile_len(k);
            if (stage == 0) {
                if (rank == cfg.slow_rank) std::this_thread::sleep_for(std::chrono::microseconds(200));
                if (k >= S)
                    for (int p = 0; p < n; ++p)
                        if (!wait_at_least(sh, row(mine.reduced, p), base + k - S + 1, rank, p, 0)) return;
                for (u64 j = 0; j < len; ++j) sh.arena_in[rank][so + j] = sh.user_in[rank][tile_off(k) + j];
                const long long now = sh.in_flight[rank][cta].fetch_add(1, std::memory_order_relaxed) + 1;
                int seen = sh.max_in_flight.load(std::memory_order_relaxed);
                while (now > seen && !sh.max_in_flight.compare_exchange_weak(seen, static_cast<int>(now), std::memory_order_relaxed)) {}
                for (int p = 0; p < n; ++p) sh.flags[p].in_ready[cta * n + rank].store(base + k + 1, std::memory_order_release);
            } else if (stage == 1) {
                for (int p = 0; p < n; ++p)
                    if (!wait_at_least(sh, row(mine.in_ready, p), base + k + 1, rank, p, 1)) return;
                if (k >= S)
                    for (int p = 0; p < n; ++p)
                        if (!wait_at_least(sh, row(mine.drained, p), base + k - S + 1, rank, p, 1)) return;
                const u64 lo = len * static_cast<u64>(rank) / n, hi = len * static_cast<u64>(rank + 1) / n;
                for (u64 j = lo; j < hi; ++j) {
                    float acc = sh.arena_in[0][so + j];
                    for (int p = 1; p < n; ++p) acc = apply(cfg.redop, acc, sh.arena_in[p][so + j]);
                    if (cfg.redop == RedOp::Avg) acc *= 1.0f / static_cast<float>(n);
                    for (int q = 0; q < n; ++q) sh.arena_out[q][so + j] = acc;
                }
                for (int p = 0; p < n; ++p) sh.flags[p].reduced[cta * n + rank].store(base + k + 1, std::memory_order_release);
            } else {
                for (int p = 0; p < n; ++p)
                    if (!wait_at_least(sh, row(mine.reduced, p), base + k + 1, rank, p, 2)) return;
                for (u64 j = 0; j < len; ++j) sh.user_out[rank][tile_off(k) + j] = sh.arena_out[rank][so + j];
                sh.in_flight[rank][cta].fetch_sub(1, std::memory_order_relaxed);
                sh.tiles.fetch_add(1, std::memory_order_relaxed);
                for (int p = 0; p < n; ++p) sh.flags[p].drained[cta * n + rank].store(base + k + 1, std::memory_order_release);
            }
        }
        base += K;

        // The rank's "kernel" ends when all its stages have; then one thread checks the result.
        if (!meet(sh, *sh.rank_arrivals[rank], rank_parties, ++rank_gen)) return;
        if (cta == 0 && stage == 2) {
            long long bad = 0;
            for (std::size_t i = 0; i < count; ++i) {
                float want = input_value(0, call, i);
                for (int p = 1; p < n; ++p) want = apply(cfg.redop, want, input_value(p, call, i));
                if (cfg.redop == RedOp::Avg) want *= 1.0f / static_cast<float>(n);
                if (sh.user_out[rank][i] != want) ++bad;
            }
            if (bad) sh.wrong.fetch_add(bad, std::memory_order_relaxed);
        }
        if (!meet(sh, *sh.rank_arrivals[rank], rank_parties, ++rank_gen)) return;
    }
}

}  // namespace

PipeSimResult run_pipe_sim(const PipeSimConfig& config) {
    PipeSimResult result;
    const int n = config.nranks, G = config.ctas;
    bool bad = n < 1 || n > kMaxRanks || G < 1 || G > 16 || config.slots < 1 || config.tile_elems == 0 || config.call_elems.empty();
    for (std::size_t c : config.call_elems) bad = bad || c == 0;
    if (bad) {
        result.wrong = -1;
        result.message = "bad configuration";
        return result;
    }
    Shared sh;
    sh.cfg = &config;
    sh.result = &result;
    sh.flags.resize(n);
    const std::size_t arena = static_cast<std::size_t>(G) * config.slots * config.tile_elems;
    for (int r = 0; r < n; ++r) {
        for (auto* f : {&sh.flags[r].start, &sh.flags[r].in_ready, &sh.flags[r].reduced, &sh.flags[r].drained}) {
            f->reset(new std::atomic<u64>[static_cast<std::size_t>(G) * n]);
            for (int i = 0; i < G * n; ++i) (*f)[i].store(0, std::memory_order_relaxed);
        }
        sh.arena_in.emplace_back(arena, 0.0f);
        sh.arena_out.emplace_back(arena, 0.0f);
        sh.user_in.emplace_back();
        sh.user_out.emplace_back();
        sh.rank_arrivals.emplace_back(new std::atomic<u64>(0));
        sh.cta_arrivals.emplace_back(new std::atomic<u64>[G]);
        sh.in_flight.emplace_back(new std::atomic<long long>[G]);
        for (int c = 0; c < G; ++c) {
            sh.cta_arrivals.back()[c].store(0, std::memory_order_relaxed);
            sh.in_flight.back()[c].store(0, std::memory_order_relaxed);
        }
    }
    std::vector<std::thread> threads;
    for (int r = 0; r < n; ++r)
        for (int c = 0; c < G; ++c)
            for (int s = 0; s < 3; ++s) threads.emplace_back(stage_thread, std::ref(sh), r, c, s);
    for (auto& t : threads) t.join();
    result.wrong = sh.wrong.load();
    result.tiles = sh.tiles.load();
    result.max_tiles_in_flight = sh.max_in_flight.load();
    return result;
}

}  // namespace b200ccl::sim
