#include "transport/rdma/proxy.h"

#include <chrono>
#include <stdexcept>
#include <string>

namespace b200ccl::transport::rdma {

namespace {
inline unsigned long long load_acquire(const unsigned long long* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline void store_release(unsigned long long* p, unsigned long long v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
inline unsigned int load_u32(const unsigned int* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
constexpr int kPollBatch = 16;
constexpr unsigned kSignalEvery = 4;
}  // namespace

RdmaProxy::RdmaProxy(QueuePair* qp, CompletionQueue* cq, RdmaFifo fifo, ProxyIdentity id, DataPlane plane,
                     std::shared_ptr<AsyncErrorState> errors)
    : qp_(qp), cq_(cq), fifo_(fifo), id_(id), plane_(plane), errors_(std::move(errors)) {
    if (!qp_ || !cq_ || !fifo_.data || !fifo_.slot_bytes || !fifo_.slot_count || !fifo_.slot_sizes || !fifo_.step_increment ||
        fifo_.slot_count % fifo_.step_increment != 0)
        throw std::invalid_argument("rdma proxy: incomplete FIFO description");
}

bool RdmaProxy::guarded(bool (RdmaProxy::*body)()) {
    if (errors_->has_error()) return false;
    try {
        return (this->*body)();
    } catch (const std::exception& e) {
        errors_->record_failure(id_, step_.load(), e.what());
    } catch (...) {
        errors_->record_failure(id_, step_.load(), "unknown failure");
    }
    return false;
}

// ---- send ------------------------------------------------------------------------------------

RdmaSendProxy::RdmaSendProxy(QueuePair* qp, CompletionQueue* cq, RdmaFifo fifo, unsigned long long* send_head,
                             unsigned long long* send_tail, ProxyIdentity id, DataPlane plane, CtsLocalRing cts,
                             std::shared_ptr<AsyncErrorState> errors)
    : RdmaProxy(qp, cq, fifo, id, plane, std::move(errors)), send_head_(send_head), send_tail_(send_tail), cts_(cts) {
    if (!send_head_ || !send_tail_) throw std::invalid_argument("rdma send proxy: missing counters");
    if (plane_ == DataPlane::WriteCts && (!cts_.slots || cts_.count == 0))
        throw std::invalid_argument("rdma send proxy: WRITE plane needs a clear-to-send ring");
}

bool RdmaSendProxy::progress() { return guarded(static_cast<bool (RdmaProxy::*)()>(&RdmaSendProxy::body)); }

// Called from another thread than the one that drives progress(): reads only the atomic step.
bool RdmaSendProxy::drained() const { return failed() || step() >= load_acquire(send_tail_); }

bool RdmaSendProxy::body() {
    bool did = false;
    const std::uint64_t inc = fifo_.step_increment;

    // 1. Completions: in order on a reliable connection, so a signalled one retires all before it.
    Completion wc[kPollBatch];
    const int n = cq_->poll(kPollBatch, wc);
    if (n < 0) throw std::runtime_error("completion queue poll failed");
    for (int i = 0; i < n; ++i) {
        if (wc[i].status != 0) throw std::runtime_error("send completion with status " + std::to_string(wc[i].status));
        if (wc[i].opcode != WcOpcode::Send && wc[i].opcode != WcOpcode::RdmaWrite) continue;
        const std::uint64_t s = step_of_wr_id(wc[i].wr_id);
        if (s < next_complete_ || s >= next_post_ || (s - next_complete_) % inc != 0)
            throw std::runtime_error("unexpected completion step " + std::to_string(s));
        next_complete_ = s + inc;
        step_.store(next_complete_, std::memory_order_release);
        store_release(send_head_, next_complete_);
        did = true;
    }

    // 2. Post what the kernel has published, up to the flight limit.
    for (;;) {
        const std::uint64_t in_flight = (next_post_ - next_complete_) / inc;
        if (in_flight >= max_flight()) break;
        const std::uint64_t tail = load_acquire(send_tail_);
        if (tail < next_post_ + inc) break;
        const std::size_t slot = next_post_ % fifo_.slot_count;
        const std::uint32_t bytes = load_u32(fifo_.slot_sizes + slot);
        if (bytes > inc * fifo_.slot_bytes) throw std::runtime_error("send payload exceeds the FIFO slots of a slice");
        if (bytes == 0) {
            // Nothing to put on the wire. Retire it only at the completion head so that the
            // published head never overtakes sends still in flight.
            if (next_post_ != next_complete_) break;
            zero_payload_posts_.fetch_add(1, std::memory_order_relaxed);
            next_post_ += inc;
            next_complete_ += inc;
            step_.store(next_complete_, std::memory_order_release);
            store_release(send_head_, next_complete_);
            did = true;
            continue;
        }
        SendWr wr;
        wr.wr_id = wr_id_for_step(next_post_);
        wr.local_addr = fifo_.data + slot * fifo_.slot_bytes;
        wr.length = bytes;
        wr.lkey = fifo_.mr.lkey;
        if (plane_ == DataPlane::WriteCts) {
            RdmaCtsSlot& grant = cts_.slots[(next_post_ / inc) % cts_.count];
            if (__atomic_load_n(&grant.ready, __ATOMIC_ACQUIRE) != 1u || grant.step_tag != next_post_) break;
            if (bytes > grant.nbytes) throw std::runtime_error("clear-to-send grant smaller than the payload");
            wr.opcode = WrOpcode::RdmaWriteWithImm;
            wr.remote_addr = grant.raddr;
            wr.rkey = grant.rkey;
            wr.imm = bytes;
            __atomic_store_n(&grant.ready, 0u, __ATOMIC_RELEASE);  // cleared at post time: the slot may be granted again
        }
        // Selective signalling: every fourth post, when this post fills the flight window, or when
        // nothing further is ready behind it (end of a burst).
        ++since_signal_;
        const bool window_full = in_flight + 1 >= max_flight();
        const bool burst_tail = tail < next_post_ + 2 * inc;
        wr.signaled = since_signal_ >= kSignalEvery || window_full || burst_tail;
        if (wr.signaled) since_signal_ = 0;
#if defined(B200CCL_ENABLE_TIMELINE)
        if (timeline_) timeline_->record_depth(static_cast<int>(in_flight));
#endif
        qp_->post_send(wr);
        posts_.fetch_add(1, std::memory_order_relaxed);
        next_post_ += inc;
        did = true;
    }
    return did;
}

// ---- receive ---------------------------------------------------------------------------------

RdmaRecvProxy::RdmaRecvProxy(QueuePair* qp, CompletionQueue* cq, RdmaFifo fifo, unsigned long long* recv_head,
                             unsigned long long* recv_tail, ProxyIdentity id, DataPlane plane, CtsRemoteRing cts,
                             std::shared_ptr<AsyncErrorState> errors, bool elide_zero_payload)
    : RdmaProxy(qp, cq, fifo, id, plane, std::move(errors)), recv_head_(recv_head), recv_tail_(recv_tail), cts_(cts),
      elide_zero_(elide_zero_payload) {
    if (!recv_head_ || !recv_tail_) throw std::invalid_argument("rdma recv proxy: missing counters");
    if (plane_ == DataPlane::WriteCts && (cts_.addr == 0 || cts_.count == 0))
        throw std::invalid_argument("rdma recv proxy: WRITE plane needs the sender's clear-to-send ring");
}

void RdmaRecvProxy::prepare() {
    try {
        post_more();
    } catch (const std::exception& e) {
        errors_->record_failure(id_, step_.load(), e.what());
    }
}

bool RdmaRecvProxy::progress() { return guarded(static_cast<bool (RdmaProxy::*)()>(&RdmaRecvProxy::body)); }

void RdmaRecvProxy::post_cts(std::uint64_t step) {
    const std::uint64_t inc = fifo_.step_increment;
    const std::size_t slot = step % fifo_.slot_count;
    cts_staging_.raddr = reinterpret_cast<std::uint64_t>(fifo_.data + slot * fifo_.slot_bytes);
    cts_staging_.rkey = fifo_.mr.rkey;
    cts_staging_.nbytes = static_cast<std::uint32_t>(inc * fifo_.slot_bytes);
    cts_staging_.step_tag = step;
    cts_staging_.ready = 1;
    cts_staging_.reserved = 0;
    SendWr wr;
    wr.wr_id = wr_id_for_step(step);
    wr.opcode = WrOpcode::RdmaWrite;
    wr.local_addr = &cts_staging_;
    wr.length = sizeof(RdmaCtsSlot);
    wr.inline_data = true;  // the record is copied at post time, so the staging struct can be reused at once
    wr.remote_addr = cts_.addr + ((step / inc) % cts_.count) * sizeof(RdmaCtsSlot);
    wr.rkey = cts_.rkey;
    wr.signaled = ++cts_since_signal_ >= kSignalEvery;
    if (wr.signaled) cts_since_signal_ = 0;
    qp_->post_send(wr);
}

// Keeps one receive (and, on the WRITE plane, one grant) outstanding for every slice whose slots
// the kernel has given back.
bool RdmaRecvProxy::post_more() {
    bool did = false;
    const std::uint64_t inc = fifo_.step_increment;
    for (;;) {
        if ((next_post_ - next_complete_) / inc >= max_flight()) break;
        if (next_post_ + inc > load_acquire(recv_head_) + fifo_.slot_count) break;  // no credit
        const std::size_t slot = next_post_ % fifo_.slot_count;
        if (elide_zero_ && load_u32(fifo_.slot_sizes + slot) == 0) {
            if (next_post_ != next_complete_) break;  // keep the published tail in order
            zero_payload_posts_.fetch_add(1, std::memory_order_relaxed);
            next_post_ += inc;
            next_complete_ += inc;
            step_.store(next_complete_, std::memory_order_release);
            store_release(recv_tail_, next_complete_);
            did = true;
            continue;
        }
        RecvWr r;
        r.wr_id = wr_id_for_step(next_post_);
        r.lkey = fifo_.mr.lkey;
        if (plane_ == DataPlane::SendRecv) {
            r.addr = fifo_.data + slot * fifo_.slot_bytes;
            r.length = static_cast<std::uint32_t>(inc * fifo_.slot_bytes);
        } else {
            r.addr = fifo_.data;  // never written: a WRITE_WITH_IMM only consumes the work request
            r.length = 1;
        }
        qp_->post_recv(r);
        if (plane_ == DataPlane::WriteCts) post_cts(next_post_);
        posts_.fetch_add(1, std::memory_order_relaxed);
        next_post_ += inc;
        did = true;
    }
    return did;
}

bool RdmaRecvProxy::body() {
    bool did = post_more();
    const std::uint64_t inc = fifo_.step_increment;
    Completion wc[kPollBatch];
    const int n = cq_->poll(kPollBatch, wc);
    if (n < 0) throw std::runtime_error("completion queue poll failed");
    for (int i = 0; i < n; ++i) {
        if (wc[i].status != 0) throw std::runtime_error("receive completion with status " + std::to_string(wc[i].status));
        if (wc[i].opcode == WcOpcode::Send || wc[i].opcode == WcOpcode::RdmaWrite) continue;  // a signalled grant retired
        const std::uint64_t s = step_of_wr_id(wc[i].wr_id);
        if (s != next_complete_) throw std::runtime_error("unexpected completion step " + std::to_string(s));
        const std::uint32_t bytes = plane_ == DataPlane::WriteCts ? wc[i].imm : wc[i].byte_len;
        if (bytes > inc * fifo_.slot_bytes) throw std::runtime_error("received payload exceeds the FIFO slots of a slice");
        fifo_.slot_sizes[s % fifo_.slot_count] = bytes;
        next_complete_ = s + inc;
        step_.store(next_complete_, std::memory_order_release);
        store_release(recv_tail_, next_complete_);
        did = true;
    }
    if (did) did = post_more() || did;
    return did;
}

}  // namespace b200ccl::transport::rdma
