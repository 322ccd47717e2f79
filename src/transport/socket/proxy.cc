#include "transport/socket/proxy.h"

#include "core/env.h"
#include "core/numa.h"

#include <sched.h>
#include <stdexcept>

namespace b200ccl::transport::socket {

namespace {
inline unsigned long long load_acquire(const unsigned long long* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline void store_release(unsigned long long* p, unsigned long long v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
}  // namespace

std::uint64_t fault_injection_slices_from_env() {
#if defined(B200CCL_SOCKET_TEST_FAULT_INJECTION)
    return static_cast<std::uint64_t>(env::get_int("B200CCL_SOCKET_FAIL_AFTER_SLICES", 0, "NANO_NCCL_SOCKET_FAIL_AFTER_SLICES"));
#else
    return 0;
#endif
}

ProxyBase::ProxyBase(Fd connection, ProxyFifo fifo, ProxyIdentity identity, int numa_node,
                     std::shared_ptr<AsyncErrorState> errors)
    : connection_(std::move(connection)), fifo_(fifo), identity_(identity), numa_node_(numa_node), errors_(std::move(errors)) {
    if (!fifo_.data || !fifo_.slot_bytes || !fifo_.slot_count || !fifo_.slot_sizes || !fifo_.step_increment)
        throw std::invalid_argument("socket proxy: incomplete FIFO description");
    set_tcp_nodelay(connection_.get());
}

ProxyBase::~ProxyBase() {
    stop();
    shutdown();
    join();
}

void ProxyBase::start() {
    if (!thread_.joinable()) thread_ = std::thread([this] { run(); });
}
void ProxyBase::stop() noexcept { stop_requested_.store(true, std::memory_order_release); }
void ProxyBase::shutdown() noexcept { connection_.shutdown_both(); }
void ProxyBase::join() noexcept {
    if (thread_.joinable()) thread_.join();
}

void ProxyBase::run() noexcept {
    numa::pin_current_thread_to_node(numa_node_);
    try {
        loop();
    } catch (const std::exception& e) {
        if (!stop_requested_) {
            errors_->record_failure(identity_, step_.load(), e.what());
            connection_.shutdown_both();  // the peer's proxy sees the connection end and fails too
        }
    } catch (...) {
        errors_->record_failure(identity_, step_.load(), "unknown failure");
        connection_.shutdown_both();
    }
}

SendProxy::SendProxy(Fd connection, ProxyFifo fifo, SendControl control, ProxyIdentity identity, int numa_node,
                     std::shared_ptr<AsyncErrorState> errors)
    : ProxyBase(std::move(connection), fifo, identity, numa_node, std::move(errors)), control_(control) {
    if (!control_.send_head || !control_.send_tail) throw std::invalid_argument("socket send proxy: missing counters");
    if (fail_after_ == 0) fail_after_ = fault_injection_slices_from_env();
}

void SendProxy::loop() {
    std::uint64_t step = 0;
    const std::size_t inc = fifo_.step_increment;
    while (!stop_requested_) {
        if (errors_->has_error()) return;
        if (load_acquire(control_.send_tail) >= step + inc) {
            const std::size_t slot = step % fifo_.slot_count;
            const unsigned int bytes = fifo_.slot_sizes[slot];
            if (bytes > inc * fifo_.slot_bytes) throw std::runtime_error("slice larger than its FIFO slots");
            if (fail_after_ != 0 && slices_.load() >= fail_after_) {
                connection_.reset();
                throw std::runtime_error("injected socket failure after " + std::to_string(fail_after_) + " slices");
            }
            send_slice(connection_.get(), fifo_.data + slot * fifo_.slot_bytes, bytes);
            step += inc;
            step_.store(step, std::memory_order_release);
            slices_.fetch_add(1, std::memory_order_acq_rel);
            store_release(control_.send_head, step);
        } else {
            sched_yield();
        }
    }
}

void SendProxy::drain() const {
    while (!stop_requested_ && !errors_->has_error() && step_.load(std::memory_order_acquire) < load_acquire(control_.send_tail))
        sched_yield();
}

RecvProxy::RecvProxy(Fd connection, ProxyFifo fifo, RecvControl control, ProxyIdentity identity, int numa_node,
                     std::shared_ptr<AsyncErrorState> errors)
    : ProxyBase(std::move(connection), fifo, identity, numa_node, std::move(errors)), control_(control) {
    if (!control_.recv_head || !control_.recv_tail) throw std::invalid_argument("socket recv proxy: missing counters");
}

void RecvProxy::loop() {
    std::uint64_t step = 0;
    const std::size_t inc = fifo_.step_increment;
    while (!stop_requested_) {
        if (errors_->has_error()) return;
        if (load_acquire(control_.recv_head) + fifo_.slot_count >= step + inc) {
            if (!wait_readable(connection_.get(), &stop_requested_)) return;
            const std::size_t slot = step % fifo_.slot_count;
            const std::uint32_t bytes = recv_slice(connection_.get(), fifo_.data + slot * fifo_.slot_bytes, inc * fifo_.slot_bytes);
            fifo_.slot_sizes[slot] = bytes;
            step += inc;
            step_.store(step, std::memory_order_release);
            slices_.fetch_add(1, std::memory_order_acq_rel);
            store_release(control_.recv_tail, step);
        } else {
            sched_yield();
        }
    }
}

}  // namespace b200ccl::transport::socket
