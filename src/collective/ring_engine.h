// Ring + Simple-protocol engine: owns the per-edge FIFOs and runs the ring kernels. Every edge is
// wired on its own: FIFO in the receiver's memory (peer stores over NVLink), in mapped host memory
// (SHM), or behind a network proxy; a ring may mix them. It is the path for transports without
// all-pairs peer access and an explicit choice (algo ring) otherwise.
//
// Parity: the FIFO sizing/wiring and launch part of nano-nccl's Communicator::Impl
// (src/collective/all_reduce/communicator.cu:894-941 ensure_fifo_buffers, 965-1099
// launch_ring_simple, per-edge pointer choice 1024-1031 and 1053-1060) and the P2P FIFO / SHM FIFO
// helpers (src/transport/p2p/p2p_fifo.cu:103-137, src/transport/shm/shm_fifo.h:9-32).
#pragma once

#include "b200ccl/communicator.h"
#include "kernels/sm100/dev_types.h"
#include "kernels/sm100/ring_simple.h"
#include "mem/symmetric.h"

#include <memory>
#include <string>
#include <vector>

namespace b200ccl {

struct RingEngineConfig {
    int nranks = 0;
    int channels = kDefaultChannels;
    unsigned long long timeout_ns = 0;
    // Kind of every directed ring edge e -> (e + 1) % nranks: P2p (FIFO in the receiver's device
    // memory, counters in device memory of the rank that polls them), Shm (FIFO and counters in
    // mapped pinned host memory on the receiver's NUMA node), or the network kind of edges that
    // leave this process. Empty: every edge P2p.
    std::vector<TransportKind> edge_kinds;
    bool loopback = false;
    // Socket or Rdma: ring edges that leave this process run over that network transport
    // (host FIFO + proxy threads); Auto: every edge is local or peer-mapped.
    TransportKind net_kind = TransportKind::Auto;
    std::vector<mem::LocalRankDesc> local;
    std::vector<dev::Status*> status;  // one per local rank
};

class RingEngine {
public:
    // `alloc` and `ctrl` may be null (no all-pairs peer-mapped memory, single process only): P2p edges
    // then get a plain device allocation on the receiver, reached through peer access enabled for
    // that pair alone, and every rank a private control block.
    RingEngine(const RingEngineConfig& config, mem::SymmetricAllocator* alloc, const mem::SymmetricRegion* ctrl,
               Bootstrap* bootstrap);
    ~RingEngine();
    void launch(Collective collective, const CollectiveArgs& args);
    int channels() const;
    int block_threads() const;
    std::string async_error() const;  // first proxy/transport failure, "" when none
    // The wiring of one local rank's channel, as the kernel receives it (tests check with
    // cudaPointerGetAttributes which GPU, or the host, owns each word).
    dev::RingChannelView channel_view(int local_index, int channel) const;

private:
    struct State;
    std::unique_ptr<State> state_;
};

}  // namespace b200ccl
