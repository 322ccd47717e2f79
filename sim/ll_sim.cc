#include "sim/ll_sim.h"

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
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
float input_value(int rank, std::size_t call, std::size_t w) {
    return static_cast<float>(static_cast<int>((w * 7 + call * 3 + static_cast<std::size_t>(rank) * 5) % 23) - 11);
}

struct Shared {
    const LlSimConfig* cfg = nullptr;
    // area[rank][(parity * nranks + source) * max_words + w]
    std::vector<std::unique_ptr<std::atomic<u64>[]>> area;
    std::vector<std::unique_ptr<std::atomic<u64>[]>> epoch;       // [rank][cta]: calls seen (device: ll_epoch)
    std::vector<std::unique_ptr<std::atomic<u64>>> arrived;       // per rank: CTAs that finished, all calls
    std::vector<std::unique_ptr<std::atomic<long long>>> progress;  // per rank: calls completed
    std::atomic<bool> abort{false};
    std::atomic<long long> wrong{0};
    std::atomic<int> max_lead{0};
    std::mutex mu;
    LlSimResult* result = nullptr;
};

void record_timeout(Shared& sh, int rank, int peer, long long call) {
    std::lock_guard<std::mutex> lock(sh.mu);
    if (!sh.result->timed_out) {
        sh.result->timed_out = true;
        sh.result->timeout_rank = rank;
        sh.result->timeout_peer = peer;
        sh.result->timeout_call = call;
        sh.result->message = "rank " + std::to_string(rank) + " gave up waiting for rank " + std::to_string(peer) +
                             " in call " + std::to_string(call);
    }
    sh.abort.store(true, std::memory_order_release);
}

void cta_thread(Shared& sh, int rank, int cta) {
    const LlSimConfig& cfg = *sh.cfg;
    const int n = cfg.nranks;
    const std::size_t stride = static_cast<std::size_t>(cfg.ctas) * cfg.lanes;
    const auto timeout = std::chrono::duration<double, std::milli>(cfg.wait_timeout_ms);
    std::vector<float> out;
    for (std::size_t k = 0; k < cfg.call_words.size(); ++k) {
        if (rank == cfg.stall_rank && static_cast<int>(k) >= cfg.stall_at_call) return;  // the rank is gone
        if (rank == cfg.slow_rank) std::this_thread::sleep_for(std::chrono::microseconds(300));
        const std::size_t nwords = cfg.call_words[k];
        const u64 call = sh.epoch[rank][cta].load(std::memory_order_relaxed) + 1;
        const std::uint32_t flag = static_cast<std::uint32_t>(call % 0xffffffffull) + 1u;
        const u64 parity = call & 1u;

        // How far ahead of the slowest rank is this one? (diagnostic only)
        long long slowest = static_cast<long long>(k);
        for (int p = 0; p < n; ++p) slowest = std::min(slowest, sh.progress[p]->load(std::memory_order_relaxed));
        int lead = static_cast<int>(static_cast<long long>(k) - slowest);
        int seen = sh.max_lead.load(std::memory_order_relaxed);
        while (lead > seen && !sh.max_lead.compare_exchange_weak(seen, lead, std::memory_order_relaxed)) {}

        // 1. publish (lane by lane, as the threads of a CTA would)
        for (int lane = 0; lane < cfg.lanes; ++lane) {
            for (std::size_t w = static_cast<std::size_t>(cta) * cfg.lanes + lane; w < nwords; w += stride) {
                const float v = input_value(rank, k, w);
                std::uint32_t bits;
                std::memcpy(&bits, &v, 4);
                const u64 word = (static_cast<u64>(flag) << 32) | bits;
                const std::size_t slot = (parity * n + rank) * cfg.max_words + w;
                for (int q = 0; q < n; ++q) sh.area[(rank + q) % n][slot].store(word, std::memory_order_relaxed);
            }
        }
        // 2. collect
        const auto t0 = Clock::now();
        bool ok = true;
        for (int lane = 0; ok && lane < cfg.lanes; ++lane) {
            for (std::size_t w = static_cast<std::size_t>(cta) * cfg.lanes + lane; ok && w < nwords; w += stride) {
                float acc = 0.0f;
                for (int p = 0; ok && p < n; ++p) {
                    const std::atomic<u64>& slot = sh.area[rank][(parity * n + p) * cfg.max_words + w];
                    u64 word = slot.load(std::memory_order_relaxed);
                    unsigned polls = 0;
                    while (static_cast<std::uint32_t>(word >> 32) != flag) {
                        if ((++polls & 63u) == 0u) {
                            if (sh.abort.load(std::memory_order_acquire)) ok = false;
                            else if (Clock::now() - t0 > timeout) {
                                record_timeout(sh, rank, p, static_cast<long long>(k));
                                ok = false;
                            }
                            if (!ok) break;
                            std::this_thread::yield();
                        }
                        word = slot.load(std::memory_order_relaxed);
                    }
                    if (!ok) break;
                    const std::uint32_t bits = static_cast<std::uint32_t>(word);
                    float f;
                    std::memcpy(&f, &bits, 4);
                    acc = p == 0 ? f : apply(cfg.redop, acc, f);
                }
                if (!ok) break;
                if (cfg.redop == RedOp::Avg) acc *= 1.0f / static_cast<float>(n);
                float expect = input_value(0, k, w);
                for (int p = 1; p < n; ++p) expect = apply(cfg.redop, expect, input_value(p, k, w));
                if (cfg.redop == RedOp::Avg) expect *= 1.0f / static_cast<float>(n);
                if (acc != expect) sh.wrong.fetch_add(1, std::memory_order_relaxed);
            }
        }
        if (!ok) return;
        sh.epoch[rank][cta].store(call, std::memory_order_relaxed);
        // Kernel boundary: the next call of this rank starts when all its CTAs are done with this one.
        const u64 target = static_cast<u64>(k + 1) * cfg.ctas;
        if (sh.arrived[rank]->fetch_add(1, std::memory_order_acq_rel) + 1 == target)
            sh.progress[rank]->store(static_cast<long long>(k + 1), std::memory_order_relaxed);
        while (sh.arrived[rank]->load(std::memory_order_acquire) < target) {
            if (sh.abort.load(std::memory_order_acquire)) return;
            std::this_thread::yield();
        }
    }
}

}  // namespace

LlSimResult run_ll_sim(const LlSimConfig& config) {
    LlSimResult res;
    if (config.nranks < 2 || config.nranks > kMaxRanks || config.ctas < 1 || config.lanes < 1 || config.max_words == 0) {
        res.wrong = -1;
        res.message = "ll simulator: bad configuration";
        return res;
    }
    for (std::size_t w : config.call_words) {
        if (w == 0 || w > config.max_words) {
            res.wrong = -1;
            res.message = "ll simulator: every call needs between 1 and max_words words";
            return res;
        }
    }
    Shared sh;
    sh.cfg = &config;
    sh.result = &res;
    const std::size_t slots = std::size_t(2) * config.nranks * config.max_words;
    for (int r = 0; r < config.nranks; ++r) {
        sh.area.emplace_back(new std::atomic<u64>[slots]);
        for (std::size_t i = 0; i < slots; ++i) sh.area.back()[i].store(0, std::memory_order_relaxed);
        sh.epoch.emplace_back(new std::atomic<u64>[config.ctas]);
        for (int c = 0; c < config.ctas; ++c) sh.epoch.back()[c].store(0, std::memory_order_relaxed);
        sh.arrived.emplace_back(new std::atomic<u64>(0));
        sh.progress.emplace_back(new std::atomic<long long>(0));
    }
    std::vector<std::thread> threads;
    for (int r = 0; r < config.nranks; ++r)
        for (int c = 0; c < config.ctas; ++c) threads.emplace_back(cta_thread, std::ref(sh), r, c);
    for (auto& t : threads) t.join();
    res.wrong = sh.wrong.load();
    res.max_lead = sh.max_lead.load();
    return res;
}

}  // namespace b200ccl::sim
