// In-process loopback implementation of VerbsBackend. Queue pairs created by one FakeVerbs
// object can connect to each other; sends are delivered by memcpy in posting order, with the
// reliable-connection rules the proxies depend on: a SEND or WRITE_WITH_IMM consumes one posted
// receive (and waits, in order, while none is posted), completions appear in order, unsignaled
// sends produce no completion, RDMA writes are checked against the registered region and rkey.
// Faults are injected on the host: the n-th send can complete with an error status.
#pragma once

#include "transport/rdma/verbs_backend.h"

#include <cstdint>
#include <memory>

namespace b200ccl::transport::rdma {

class FakeVerbs : public VerbsBackend {
public:
    FakeVerbs();
    ~FakeVerbs() override;
    std::string name() const override { return "fake"; }
    MemoryRegion register_memory(void* addr, std::size_t length) override;
    MemoryRegion register_device_memory(void* addr, std::size_t length) override;
    void deregister(const MemoryRegion& mr) override;
    std::unique_ptr<CompletionQueue> create_cq(int depth) override;
    std::unique_ptr<QueuePair> create_qp(CompletionQueue* cq, int max_send_wr, int max_recv_wr) override;

    // Test controls and counters.
    void fail_send_number(std::uint64_t n, int status);  // the n-th posted send (1-based) completes with `status`
    std::uint64_t sends_posted() const;
    std::uint64_t signaled_sends() const;
    std::uint64_t inline_sends() const;
    std::uint64_t recvs_posted() const;
    std::uint64_t registrations() const;
    bool allow_device_registration = true;  // false → register_device_memory throws "unavailable"

    struct Impl;

private:
    std::shared_ptr<Impl> impl_;
};

}  // namespace b200ccl::transport::rdma
