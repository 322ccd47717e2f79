// The subset of RDMA verbs the transport needs, as an interface. The proxies and the edge set are
// written against it; `FakeVerbs` (in-process loopback, always built) drives the unit tests and
// the self-connected ring, and an ibverbs implementation is compiled where libibverbs exists.
//
// Parity: the calls nano-nccl makes on libibverbs in src/transport/rdma/rdma_endpoint.cc:164-248
// (device/port/GID selection, PD, CQ), rdma_qp.cc:30-195 (RC QP, INIT→RTR→RTS), rdma_proxy.cc
// (ibv_post_send / ibv_post_recv / ibv_poll_cq) and rdma_gdr.cc:112-136 (memory registration).
#pragma once

#include "transport/rdma/protocol.h"

#include <cstdint>
#include <memory>
#include <string>

namespace b200ccl::transport::rdma {

struct MemoryRegion {
    void* addr = nullptr;
    std::size_t length = 0;
    std::uint32_t lkey = 0;
    std::uint32_t rkey = 0;
    std::uint64_t handle = 0;  // backend cookie
};

enum class WrOpcode { Send, RdmaWrite, RdmaWriteWithImm };

struct SendWr {
    std::uint64_t wr_id = 0;
    WrOpcode opcode = WrOpcode::Send;
    const void* local_addr = nullptr;
    std::uint32_t length = 0;
    std::uint32_t lkey = 0;
    bool signaled = false;
    bool inline_data = false;  // payload captured at post time (≤ max_inline_data bytes)
    std::uint64_t remote_addr = 0;
    std::uint32_t rkey = 0;
    std::uint32_t imm = 0;
};

struct RecvWr {
    std::uint64_t wr_id = 0;
    void* addr = nullptr;
    std::uint32_t length = 0;
    std::uint32_t lkey = 0;
};

enum class WcOpcode { Send, RdmaWrite, Recv, RecvRdmaWithImm };

struct Completion {
    std::uint64_t wr_id = 0;
    int status = 0;  // 0 = success; other values are the backend's error codes
    WcOpcode opcode = WcOpcode::Send;
    std::uint32_t byte_len = 0;
    std::uint32_t imm = 0;
};

constexpr std::uint32_t kMaxInlineData = 64;

class CompletionQueue {
public:
    virtual ~CompletionQueue() = default;
    virtual int poll(int max_entries, Completion* out) = 0;  // number of completions written, <0 on failure
};

class QueuePair {
public:
    virtual ~QueuePair() = default;
    virtual void fill_local_info(RdmaPeerInfo* info) const = 0;  // qpn, psn, lid, gid, mtu
    virtual void connect(const RdmaPeerInfo& remote) = 0;        // INIT → RTR → RTS
    virtual void post_send(const SendWr& wr) = 0;                // throws when the queue refuses
    virtual void post_recv(const RecvWr& wr) = 0;
};

class VerbsBackend {
public:
    virtual ~VerbsBackend() = default;
    virtual std::string name() const = 0;
    virtual MemoryRegion register_memory(void* addr, std::size_t length) = 0;
    // Device memory (GDR): dma-buf where the driver offers it, else peer-memory registration;
    // throws rather than falling back to host memory.
    virtual MemoryRegion register_device_memory(void* addr, std::size_t length) = 0;
    virtual void deregister(const MemoryRegion& mr) = 0;
    virtual std::unique_ptr<CompletionQueue> create_cq(int depth) = 0;
    // RC queue pair whose send and receive completions both go to `cq` (one shared CQ),
    // sq_sig_all = 0, max_inline_data = kMaxInlineData.
    virtual std::unique_ptr<QueuePair> create_qp(CompletionQueue* cq, int max_send_wr, int max_recv_wr) = 0;
};

// "fake" → FakeVerbs; "ibverbs" → the real backend (throws where it was not compiled in, or where
// no active HCA port is found). Default from B200CCL_RDMA_BACKEND, else ibverbs if compiled, else fake.
std::shared_ptr<VerbsBackend> create_backend(const std::string& name = "");

}  // namespace b200ccl::transport::rdma
