// Host proxies of the RDMA transport: state machines that move slices between a registered FIFO
// and a reliable-connection queue pair. Each proxy exposes progress(), which never blocks, so it
// can be driven by a thread of its own or by one shared progress thread.
//
// Two data planes (B200CCL_RDMA_USE_WRITE):
//  * SendRecv: the sender posts up to slot_count/step_increment SENDs in flight straight from the
//    FIFO slots, signalling selectively (every fourth post, when the flight limit is reached, at
//    the end of a burst); the receiver keeps full-slot RECVs posted as credit allows and takes the
//    payload size from the completion. Completions are in order, so one signalled completion
//    retires every earlier post; wr_id is the absolute step.
//  * WriteCts: for every free slot the receiver RDMA-writes (inline) a clear-to-send record into
//    the sender's CTS ring; the sender waits for ready==1 and the matching step tag, posts
//    RDMA_WRITE_WITH_IMM (immediate = payload bytes) to the granted address and clears `ready`
//    when it posts; the receiver harvests the immediates from 1-byte scratch RECVs.
// Zero-byte slices cause no network operation on either side.
//
// Parity: nano-nccl src/transport/rdma/rdma_proxy.h:24-281 / rdma_proxy.cc:330-784 (send),
// 879-1318 (receive), counters posts() / zero_payload_posts() (rdma_proxy.h:138-143).
#pragma once

#include "transport/async_error.h"
#include "transport/rdma/timeline.h"
#include "transport/rdma/verbs_backend.h"

#include <atomic>
#include <memory>

namespace b200ccl::transport::rdma {

struct RdmaFifo {
    std::uint8_t* data = nullptr;
    std::size_t slot_bytes = 0;      // bytes of one FIFO step
    std::size_t slot_count = 0;      // steps in the FIFO
    unsigned int* slot_sizes = nullptr;
    std::size_t step_increment = 1;  // steps per slice
    MemoryRegion mr;                 // registration covering `data`
};

struct CtsLocalRing {   // sender side: where grants arrive
    RdmaCtsSlot* slots = nullptr;
    std::size_t count = 0;
};
struct CtsRemoteRing {  // receiver side: where grants are written
    std::uint64_t addr = 0;
    std::uint32_t rkey = 0;
    std::size_t count = 0;
};

class RdmaProxy {
public:
    virtual ~RdmaProxy() = default;
    virtual void prepare() {}        // receive side: pre-post before the peer may send
    virtual bool progress() = 0;     // true when something was done; failures are latched, not thrown
    virtual bool is_receiver() const = 0;
    bool failed() const { return errors_->has_error(); }
    std::uint64_t step() const { return step_.load(std::memory_order_acquire); }
    std::uint64_t posts() const { return posts_.load(std::memory_order_relaxed); }
    std::uint64_t zero_payload_posts() const { return zero_payload_posts_.load(std::memory_order_relaxed); }
    void set_timeline(ProxyTimeline* t) { timeline_ = t; }

protected:
    RdmaProxy(QueuePair* qp, CompletionQueue* cq, RdmaFifo fifo, ProxyIdentity id, DataPlane plane,
              std::shared_ptr<AsyncErrorState> errors);
    bool guarded(bool (RdmaProxy::*body)());
    QueuePair* qp_;
    CompletionQueue* cq_;
    RdmaFifo fifo_;
    ProxyIdentity id_;
    DataPlane plane_;
    std::shared_ptr<AsyncErrorState> errors_;
    std::atomic<std::uint64_t> step_{0}, posts_{0}, zero_payload_posts_{0};
    ProxyTimeline* timeline_ = nullptr;
    std::size_t max_flight() const { return fifo_.slot_count / fifo_.step_increment; }
};

class RdmaSendProxy final : public RdmaProxy {
public:
    RdmaSendProxy(QueuePair* qp, CompletionQueue* cq, RdmaFifo fifo, unsigned long long* send_head,
                  unsigned long long* send_tail, ProxyIdentity id, DataPlane plane, CtsLocalRing cts,
                  std::shared_ptr<AsyncErrorState> errors);
    bool progress() override;
    bool is_receiver() const override { return false; }
    bool drained() const;  // everything the kernel published has completed

private:
    bool body();
    unsigned long long* send_head_;
    unsigned long long* send_tail_;
    CtsLocalRing cts_;
    std::uint64_t next_post_ = 0, next_complete_ = 0;
    unsigned since_signal_ = 0;
};

class RdmaRecvProxy final : public RdmaProxy {
public:
    // elide_zero_payload: a slot whose size entry is 0 when its turn comes is stepped locally,
    // without a posted receive (the sender skips the network for it too).
    RdmaRecvProxy(QueuePair* qp, CompletionQueue* cq, RdmaFifo fifo, unsigned long long* recv_head,
                  unsigned long long* recv_tail, ProxyIdentity id, DataPlane plane, CtsRemoteRing cts,
                  std::shared_ptr<AsyncErrorState> errors, bool elide_zero_payload = false);
    void prepare() override;
    bool progress() override;
    bool is_receiver() const override { return true; }

private:
    bool body();
    bool post_more();
    void post_cts(std::uint64_t step);
    unsigned long long* recv_head_;
    unsigned long long* recv_tail_;
    CtsRemoteRing cts_;
    bool elide_zero_;
    std::uint64_t next_post_ = 0, next_complete_ = 0;
    unsigned cts_since_signal_ = 0;
    RdmaCtsSlot cts_staging_{};
};

}  // namespace b200ccl::transport::rdma
