#include "sim/ring_sim.h"

#include "core/datagen.h"
#include "sched/ring_geometry.h"

#include <atomic>
#include <chrono>
#include <cmath>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace b200ccl::sim {

namespace {

using Clock = std::chrono::steady_clock;
using u64 = unsigned long long;

struct Edge {  // one channel of one directed edge e → e+1
    std::vector<float> fifo;
    alignas(64) std::atomic<u64> tail{0};  // written by the sender
    alignas(64) std::atomic<u64> head{0};  // written by the receiver
};

struct Shared {
    const RingSimConfig* cfg = nullptr;
    std::vector<std::unique_ptr<Edge>> edges;  // [e*channels + c]
    std::vector<std::vector<float>> input, output;
    std::atomic<bool> abort{false};
    std::mutex mu;
    RingSimResult* result = nullptr;
    std::atomic<u64> slices{0}, empty{0};
    std::size_t step_elems = 0;
};

float apply(RedOp op, float a, float b) {
    switch (op) {
        case RedOp::Max: return (a != a) ? a : ((b != b) ? b : (a > b ? a : b));
        case RedOp::Min: return (a != a) ? a : ((b != b) ? b : (a < b ? a : b));
        default: return a + b;
    }
}

enum : unsigned { kRecv = 1, kLocal = 2, kSend = 4, kCopyOut = 8, kScale = 16 };

class Worker {
public:
    Worker(Shared& sh, int rank, int channel) : sh_(sh), r_(rank), c_(channel) {
        const int n = sh.cfg->nranks, C = sh.cfg->channels;
        out_edge_ = sh.edges[r_ * C + c_].get();
        in_edge_ = sh.edges[((r_ + n - 1) % n) * C + c_].get();
    }

    void run() {
        const RingSimConfig& cfg = *sh_.cfg;
        const int n = cfg.nranks;
        const float* in = sh_.input[r_].data();
        float* out = sh_.output[r_].data();
        const ring::Part part = ring::channel_part(cfg.count, c_, cfg.channels);
        auto mod = [n](int v) { return ((v % n) + n) % n; };
        bool ok = true;
        if (cfg.collective == Collective::AllReduce) {
            const std::size_t cs = ring::all_reduce_chunk_elems(part.count, n, sizeof(float), sh_.step_elems);
            for (std::size_t w0 = 0; ok && cs > 0 && w0 < part.count; w0 += cs * n) {
                auto chunk = [&](int k, std::size_t* off, std::size_t* len) {
                    *off = w0 + static_cast<std::size_t>(k) * cs;
                    *len = ring::clamp_elems(cs, part.count, *off);
                    *off += part.offset;
                };
                std::size_t off, len;
                chunk(mod(r_ - 1), &off, &len);
                ok = run_chunk(kLocal | kSend, in + off, nullptr, len);
                for (int j = 2; ok && j < n; ++j) {
                    chunk(mod(r_ - j), &off, &len);
                    ok = run_chunk(kRecv | kLocal | kSend, in + off, nullptr, len);
                }
                if (ok) {
                    chunk(r_, &off, &len);
                    ok = run_chunk(kRecv | kLocal | kSend | kCopyOut | kScale, in + off, out + off, len);
                }
                for (int j = 1; ok && j < n - 1; ++j) {
                    chunk(mod(r_ - j), &off, &len);
                    ok = run_chunk(kRecv | kSend | kCopyOut, nullptr, out + off, len);
                }
                if (ok) {
                    chunk(mod(r_ + 1), &off, &len);
                    ok = run_chunk(kRecv | kCopyOut, nullptr, out + off, len);
                }
            }
        } else if (cfg.collective == Collective::ReduceScatter) {
            const std::size_t cs = ring::block_chunk_elems(part.count, sizeof(float), sh_.step_elems);
            for (std::size_t w0 = 0; ok && cs > 0 && w0 < part.count; w0 += cs) {
                const std::size_t len = ring::clamp_elems(cs, part.count, w0);
                auto blk = [&](int k) { return static_cast<std::size_t>(k) * cfg.count + part.offset + w0; };
                ok = run_chunk(kLocal | kSend, in + blk(mod(r_ - 1)), nullptr, len);
                for (int j = 2; ok && j < n; ++j) ok = run_chunk(kRecv | kLocal | kSend, in + blk(mod(r_ - j)), nullptr, len);
                if (ok) ok = run_chunk(kRecv | kLocal | kCopyOut | kScale, in + blk(r_), out + part.offset + w0, len);
            }
        } else {
            const std::size_t cs = ring::block_chunk_elems(part.count, sizeof(float), sh_.step_elems);
            for (std::size_t w0 = 0; ok && cs > 0 && w0 < part.count; w0 += cs) {
                const std::size_t len = ring::clamp_elems(cs, part.count, w0);
                auto blk = [&](int k) { return static_cast<std::size_t>(k) * cfg.count + part.offset + w0; };
                ok = run_chunk(kLocal | kSend | kCopyOut, in + part.offset + w0, out + blk(r_), len);
                for (int j = 1; ok && j < n - 1; ++j) ok = run_chunk(kRecv | kSend | kCopyOut, nullptr, out + blk(mod(r_ - j)), len);
                if (ok) ok = run_chunk(kRecv | kCopyOut, nullptr, out + blk(mod(r_ + 1)), len);
            }
        }
    }

private:
    bool wait(const std::atomic<u64>& flag, u64 want, int peer, u64 step) {
        const auto t0 = Clock::now();
        unsigned polls = 0;
        while (flag.load(std::memory_order_acquire) < want) {
            if ((++polls & 255u) == 0) {
                if (sh_.abort.load(std::memory_order_relaxed)) return false;
                const double ms = std::chrono::duration<double, std::milli>(Clock::now() - t0).count();
                if (ms > sh_.cfg->wait_timeout_ms) {
                    std::lock_guard<std::mutex> lock(sh_.mu);
                    if (!sh_.result->timed_out) {
                        sh_.result->timed_out = true;
                        sh_.result->timeout_rank = r_;
                        sh_.result->timeout_peer = peer;
                        sh_.result->timeout_channel = c_;
                        sh_.result->timeout_step = step;
                        sh_.result->message = "rank " + std::to_string(r_) + " channel " + std::to_string(c_) +
                                              " waited for rank " + std::to_string(peer) + " at step " + std::to_string(step);
                    }
                    sh_.abort.store(true, std::memory_order_relaxed);
                    return false;
                }
                std::this_thread::yield();
            }
        }
        return true;
    }

    bool run_chunk(unsigned flags, const float* local_in, float* local_out, std::size_t n) {
        const std::size_t sl = ring::slice_elems(n, sizeof(float), sh_.step_elems);
        for (int s = 0; s < ring::kSlicesPerChunk; ++s) {
            const std::size_t off = static_cast<std::size_t>(s) * sl;
            const std::size_t sn = ring::clamp_elems(sl, n, off);
            if (!run_slice(flags, local_in ? local_in + off : nullptr, local_out ? local_out + off : nullptr, sn)) return false;
        }
        return true;
    }

    bool run_slice(unsigned flags, const float* local_in, float* local_out, std::size_t n) {
        if (n == 0) {
            sh_.empty.fetch_add(1, std::memory_order_relaxed);
            return true;
        }
        const RingSimConfig& cfg = *sh_.cfg;
        if (cfg.stall_rank == r_ && static_cast<long long>(done_) >= cfg.stall_after_slices) return false;  // this rank "dies"
        const int nr = cfg.nranks;
        const bool recv = flags & kRecv, send = flags & kSend, local = flags & kLocal, copy_out = flags & kCopyOut;
        const float scale = (flags & kScale) && cfg.redop == RedOp::Avg ? 1.0f / nr : 1.0f;
        if (recv && !wait(in_edge_->tail, recv_step_ + ring::kSliceSteps, (r_ + nr - 1) % nr, recv_step_)) return false;
        if (send) {
            const u64 want = send_step_ + ring::kSliceSteps >= static_cast<u64>(ring::kFifoSteps)
                                 ? send_step_ + ring::kSliceSteps - ring::kFifoSteps : 0;
            if (!wait(out_edge_->head, want, (r_ + 1) % nr, send_step_)) return false;
        }
        const float* fin = recv ? in_edge_->fifo.data() + ring::slot_offset(recv_step_, sh_.step_elems) : nullptr;
        float* fout = send ? out_edge_->fifo.data() + ring::slot_offset(send_step_, sh_.step_elems) : nullptr;
        for (std::size_t i = 0; i < n; ++i) {
            float v;
            if (recv) v = local ? apply(cfg.redop, local_in[i], fin[i]) : fin[i];
            else v = local_in[i];
            if (scale != 1.0f) v *= scale;
            if (copy_out) local_out[i] = v;
            if (send) fout[i] = v;
        }
        if (recv) {
            in_edge_->head.store(recv_step_ + ring::kSliceSteps, std::memory_order_release);
            recv_step_ += ring::kSliceSteps;
        }
        if (send) {
            out_edge_->tail.store(send_step_ + ring::kSliceSteps, std::memory_order_release);
            send_step_ += ring::kSliceSteps;
        }
        ++done_;
        sh_.slices.fetch_add(1, std::memory_order_relaxed);
        return true;
    }

    Shared& sh_;
    int r_, c_;
    Edge* out_edge_ = nullptr;
    Edge* in_edge_ = nullptr;
    u64 send_step_ = 0, recv_step_ = 0, done_ = 0;
};

}  // namespace

RingSimResult run_ring_sim(const RingSimConfig& cfg) {
    RingSimResult result;
    if (cfg.nranks < 2 || cfg.nranks > kMaxRanks || cfg.channels < 1 || cfg.channels > kMaxChannels || cfg.count == 0) {
        result.message = "bad simulator configuration";
        result.wrong = -1;
        return result;
    }
    const int n = cfg.nranks, C = cfg.channels;
    Shared sh;
    sh.cfg = &cfg;
    sh.result = &result;
    sh.step_elems = ring::step_elems(cfg.fifo_bytes, sizeof(float));
    for (int i = 0; i < n * C; ++i) {
        sh.edges.emplace_back(new Edge());
        sh.edges.back()->fifo.assign(sh.step_elems * ring::kFifoSteps, 0.0f);
    }
    const std::size_t in_count = cfg.count * (cfg.collective == Collective::ReduceScatter ? n : 1);
    const std::size_t out_count = cfg.count * (cfg.collective == Collective::AllGather ? n : 1);
    sh.input.resize(n);
    sh.output.resize(n);
    for (int r = 0; r < n; ++r) {
        sh.input[r].resize(in_count);
        sh.output[r].assign(out_count, std::nanf(""));
        for (std::size_t i = 0; i < in_count; ++i) sh.input[r][i] = datagen::uniform_pm1(static_cast<std::uint64_t>(r), r, i);
    }
    std::vector<Worker> workers;
    workers.reserve(static_cast<std::size_t>(n) * C);
    for (int r = 0; r < n; ++r)
        for (int c = 0; c < C; ++c) workers.emplace_back(sh, r, c);
    const auto t0 = Clock::now();
    std::vector<std::thread> threads;
    for (auto& w : workers) threads.emplace_back([&w] { w.run(); });
    for (auto& t : threads) t.join();
    result.seconds = std::chrono::duration<double>(Clock::now() - t0).count();
    result.slices = sh.slices.load();
    result.empty_slices = sh.empty.load();
    if (result.timed_out || cfg.stall_rank >= 0) return result;

    // Host reference in double.
    for (int r = 0; r < n; ++r) {
        for (std::size_t i = 0; i < out_count; ++i) {
            double expect;
            if (cfg.collective == Collective::AllGather) {
                expect = sh.input[i / cfg.count][i % cfg.count];
            } else {
                const std::size_t idx = cfg.collective == Collective::ReduceScatter ? static_cast<std::size_t>(r) * cfg.count + i : i;
                expect = sh.input[0][idx];
                for (int q = 1; q < n; ++q) {
                    const double v = sh.input[q][idx];
                    if (cfg.redop == RedOp::Max) expect = v > expect ? v : expect;
                    else if (cfg.redop == RedOp::Min) expect = v < expect ? v : expect;
                    else expect += v;
                }
                if (cfg.redop == RedOp::Avg) expect /= n;
            }
            const float err = std::fabs(sh.output[r][i] - static_cast<float>(expect));
            if (!(err <= 1e-5f)) ++result.wrong;
            if (err > result.max_abs_error || err != err) result.max_abs_error = err != err ? INFINITY : err;
        }
    }
    return result;
}

}  // namespace b200ccl::sim
