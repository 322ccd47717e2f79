// Ring + Simple-protocol engine: owns the per-edge FIFOs and runs the ring kernels. It is the
// path for transports without all-pairs peer access (SHM: FIFOs in mapped host memory) and an
// explicit choice (algo ring) on peer-to-peer transports (FIFOs in the receiver's memory).
//
// Parity: the FIFO sizing/wiring and launch part of nano-nccl's Communicator::Impl
// (src/collective/all_reduce/communicator.cu:894-941 ensure_fifo_buffers, 965-1099
// launch_ring_simple) and the P2P FIFO / SHM FIFO helpers (src/transport/p2p/p2p_fifo.cu:103-137,
// src/transport/shm/shm_fifo.h:9-32).
#pragma once

#include "b200ccl/communicator.h"
#include "kernels/sm100/dev_types.h"
#include "mem/symmetric.h"

#include <memory>
#include <string>
#include <vector>

namespace b200ccl {

struct RingEngineConfig {
    int nranks = 0;
    int channels = kDefaultChannels;
    unsigned long long timeout_ns = 0;
    bool use_host_fifo = false;  // SHM transport: FIFOs and counters in mapped pinned host memory
    bool loopback = false;
    // Socket or Rdma: ring edges that leave this process run over that network transport
    // (host FIFO + proxy threads); Auto: every edge is local or peer-mapped.
    TransportKind net_kind = TransportKind::Auto;
    std::vector<mem::LocalRankDesc> local;
    std::vector<dev::Status*> status;  // one per local rank
};

class RingEngine {
public:
    // `alloc` and `ctrl` may be null when use_host_fifo is set (no peer-mapped memory exists then).
    RingEngine(const RingEngineConfig& config, mem::SymmetricAllocator* alloc, const mem::SymmetricRegion* ctrl,
               Bootstrap* bootstrap);
    ~RingEngine();
    void launch(Collective collective, const CollectiveArgs& args);
    int channels() const;
    int block_threads() const;
    std::string async_error() const;  // first proxy/transport failure, "" when none

private:
    struct State;
    std::unique_ptr<State> state_;
};

}  // namespace b200ccl
