// Network edges of a ring: the ring edges that leave this process and therefore cannot be a
// peer store. Each such edge has, per channel, a host FIFO and counters in mapped host memory;
// a proxy thread moves slices between that FIFO and the wire (TCP socket or RDMA).
//
// Parity: the socket/RDMA wiring in nano-nccl's Communicator::Impl
// (src/collective/all_reduce/communicator.cu:295-396 setup_socket_transport, 490-785
// setup_rdma_transport, 1004-1051 pointer selection per edge kind).
#pragma once

#include "b200ccl/bootstrap.h"
#include "b200ccl/types.h"
#include "mem/symmetric.h"

#include <memory>
#include <string>
#include <vector>

namespace b200ccl::transport {

// What the ring kernel needs from one direction of one network edge and channel.
struct NetHalf {
    void* fifo = nullptr;                 // mapped host FIFO (kernel writes it when sending, reads it when receiving)
    unsigned long long* tail = nullptr;   // sending: kernel publishes; receiving: proxy publishes
    unsigned long long* head = nullptr;   // sending: proxy publishes (credit); receiving: kernel publishes
    unsigned int* sizes = nullptr;        // payload bytes per FIFO step slot
};

struct NetEdgeConfig {
    TransportKind kind = TransportKind::Socket;
    int nranks = 0;
    int channels = 0;
    std::size_t fifo_bytes = 0;
    std::vector<mem::LocalRankDesc> local;
    // Every ring edge goes over the network transport, also those between two ranks of this
    // process (loopback connections). Used when a single-process communicator asks for socket or
    // rdma: it exercises the whole kernel → proxy → wire → proxy → kernel path on one host.
    bool all_edges = false;
};

class NetEdgeSet {
public:
    virtual ~NetEdgeSet() = default;
    // Non-null when the edge `rank → rank+1` (send) / `rank-1 → rank` (recv) leaves this process.
    virtual const NetHalf* send_half(int global_rank, int channel) const = 0;
    virtual const NetHalf* recv_half(int global_rank, int channel) const = 0;
    virtual const unsigned int* abort_word() const = 0;  // mapped; non-zero after the first proxy failure
    virtual void start() = 0;                             // receive side first, then send side
    virtual void stop() = 0;                              // drain, shut down, join
    virtual std::string first_error() const = 0;
};

// Connects every cross-process ring edge (lower bootstrap rank connects, higher accepts) and
// builds the proxies. Throws on every process if any process failed (error consensus).
// `bootstrap` may be null for a single-process communicator (then all_edges must be set).
std::unique_ptr<NetEdgeSet> create_net_edges(const NetEdgeConfig& config, Bootstrap* bootstrap);

}  // namespace b200ccl::transport
