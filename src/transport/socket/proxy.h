// Host proxy threads of the socket transport: one thread per (edge, channel, direction) moves
// slices between a mapped host FIFO and a TCP connection.
//
// Send proxy: waits until the kernel's published tail passes the next slice, writes a 4-byte
// big-endian length and the payload straight from the FIFO slot, then publishes the head (credit
// back to the kernel). Receive proxy: waits for credit (head + slots >= step + increment),
// reads header and payload into the slot, stores the size, publishes the tail.
//
// Parity: nano-nccl src/transport/socket/socket_proxy.h:15-121 / .cc:243-283 (send loop),
// 334-361 (receive loop), 116-170 (framing, oversize check), 172-192 (error latch),
// 101-112 + 267-274 (test-only fault: close the socket after n good slices).
#pragma once

#include "transport/async_error.h"
#include "transport/socket/endpoint.h"

#include <atomic>
#include <cstdint>
#include <memory>
#include <thread>

namespace b200ccl::transport::socket {

struct ProxyFifo {
    std::uint8_t* data = nullptr;       // mapped host memory
    std::size_t slot_bytes = 0;         // bytes of one FIFO step
    std::size_t slot_count = 0;         // steps in the FIFO
    unsigned int* slot_sizes = nullptr; // payload bytes, indexed by step % slot_count
    std::size_t step_increment = 1;     // steps per slice
};

struct SendControl {
    unsigned long long* send_head = nullptr;  // proxy publishes
    unsigned long long* send_tail = nullptr;  // kernel publishes
};
struct RecvControl {
    unsigned long long* recv_head = nullptr;  // kernel publishes
    unsigned long long* recv_tail = nullptr;  // proxy publishes
};

class ProxyBase {
public:
    virtual ~ProxyBase();
    ProxyBase(const ProxyBase&) = delete;
    ProxyBase& operator=(const ProxyBase&) = delete;
    void start();
    void stop() noexcept;      // ask the loop to end
    void shutdown() noexcept;  // wake a blocked read/write
    void join() noexcept;
    std::uint64_t step() const noexcept { return step_.load(std::memory_order_acquire); }
    std::uint64_t slices() const noexcept { return slices_.load(std::memory_order_acquire); }

protected:
    ProxyBase(Fd connection, ProxyFifo fifo, ProxyIdentity identity, int numa_node, std::shared_ptr<AsyncErrorState> errors);
    virtual void loop() = 0;
    void run() noexcept;
    Fd connection_;
    ProxyFifo fifo_;
    ProxyIdentity identity_;
    int numa_node_;
    std::shared_ptr<AsyncErrorState> errors_;
    std::atomic<bool> stop_requested_{false};
    std::thread thread_;
    std::atomic<std::uint64_t> step_{0};
    std::atomic<std::uint64_t> slices_{0};
};

class SendProxy final : public ProxyBase {
public:
    SendProxy(Fd connection, ProxyFifo fifo, SendControl control, ProxyIdentity identity, int numa_node,
              std::shared_ptr<AsyncErrorState> errors);
    // Blocks until every slice the kernel has published so far is on the wire (or an error/stop).
    void drain() const;
    // Test hook: after `n` good slices the proxy closes its socket and fails. 0 disables.
    void fail_after_slices_for_testing(std::uint64_t n) { fail_after_ = n; }

private:
    void loop() override;
    SendControl control_;
    std::uint64_t fail_after_ = 0;
};

class RecvProxy final : public ProxyBase {
public:
    RecvProxy(Fd connection, ProxyFifo fifo, RecvControl control, ProxyIdentity identity, int numa_node,
              std::shared_ptr<AsyncErrorState> errors);

private:
    void loop() override;
    RecvControl control_;
};

// Value of B200CCL_SOCKET_FAIL_AFTER_SLICES (or NANO_NCCL_SOCKET_FAIL_AFTER_SLICES); honoured only
// in builds configured with B200CCL_SOCKET_TEST_FAULT_INJECTION, 0 otherwise.
std::uint64_t fault_injection_slices_from_env();

}  // namespace b200ccl::transport::socket
