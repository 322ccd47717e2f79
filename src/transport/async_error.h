// First-error latch shared by every proxy of a communicator. The first failure wins: its text
// (with the edge identity and the step) is kept, and a word in mapped host memory is set so that
// kernels spinning on this edge give up.
//
// Parity: nano-nccl SocketAsyncErrorState / RdmaAsyncErrorState
// (src/transport/socket/socket_proxy.cc:172-192, src/transport/rdma/rdma_proxy.cc:160-180);
// message shape "socket proxy source=7 destination=8 channel=2 step=0: <reason>" as asserted by
// the reference's tests/socket_protocol_test.cc:217-289.
#pragma once

#include <atomic>
#include <cstdint>
#include <mutex>
#include <string>

namespace b200ccl::transport {

struct ProxyIdentity {
    int source_rank = -1;
    int destination_rank = -1;
    int channel = -1;
};

class AsyncErrorState {
public:
    // `kind` prefixes messages ("socket", "rdma"); `abort_word` may be null.
    explicit AsyncErrorState(const char* kind, unsigned int* abort_word = nullptr) : kind_(kind), abort_word_(abort_word) {}
    AsyncErrorState(const AsyncErrorState&) = delete;
    AsyncErrorState& operator=(const AsyncErrorState&) = delete;

    void record_failure(const ProxyIdentity& id, std::uint64_t step, const std::string& reason) noexcept {
        bool expected = false;
        if (!claimed_.compare_exchange_strong(expected, true, std::memory_order_acq_rel)) return;
        try {
            std::lock_guard<std::mutex> lock(mutex_);
            message_ = std::string(kind_) + " proxy source=" + std::to_string(id.source_rank) + " destination=" +
                       std::to_string(id.destination_rank) + " channel=" + std::to_string(id.channel) + " step=" +
                       std::to_string(step) + ": " + reason;
        } catch (...) {
        }
        if (abort_word_) __atomic_store_n(abort_word_, 1u, __ATOMIC_RELEASE);
        has_error_.store(true, std::memory_order_release);
    }
    bool has_error() const noexcept { return has_error_.load(std::memory_order_acquire); }
    std::string message() const {
        if (!has_error()) return "";
        std::lock_guard<std::mutex> lock(mutex_);
        return message_;
    }
    static std::string format(const char* kind, const ProxyIdentity& id, std::uint64_t step, const std::string& reason) {
        AsyncErrorState tmp(kind);
        tmp.record_failure(id, step, reason);
        return tmp.message();
    }

private:
    const char* kind_;
    unsigned int* abort_word_;
    std::atomic<bool> claimed_{false};
    std::atomic<bool> has_error_{false};
    mutable std::mutex mutex_;
    std::string message_;
};

}  // namespace b200ccl::transport
