// Which transport each directed ring edge (e → e+1) uses, and the single kind a communicator
// reports for the whole ring ("mixed" when the edges differ). Pure host logic.
//
// Parity: nano-nccl RingTransportPlan / resolved_kind (src/transport/p2p/p2p_topology.h:13-36,
// p2p_topology.cu:134-177) and ProcessTopology with its validation (src/collective/all_reduce/
// topology.h:9-23, topology.cc:16-68: contiguous ranks per process, cross-process edges carry the
// network kind, one resolved kind per edge).
#pragma once

#include "b200ccl/types.h"

#include <string>
#include <vector>

namespace b200ccl::sched {

struct ProcessLayout {
    int nranks = 0;
    std::vector<int> first_rank;  // per process, ascending
    std::vector<int> rank_count;  // per process
    // Throws std::invalid_argument unless the processes' ranks tile 0..nranks-1 contiguously.
    void validate() const;
    int owner_of(int rank) const;  // process index, -1 when out of range
    bool distributed() const { return first_rank.size() > 1; }
};

struct RingTransportPlan {
    std::vector<TransportKind> edge_kinds;  // edge e goes from rank e to rank (e+1) % nranks
    // The one kind every edge has, else Mixed. An empty plan (one rank) reports `fallback`.
    TransportKind resolved_kind(TransportKind fallback = TransportKind::P2p) const;
    std::string describe() const;  // "edge 0->1: p2p\n..."
};

// local_kind: P2p or Shm, for edges inside one process. cross_kind: P2p (peer-mapped exported
// memory), Socket or Rdma, for edges between processes. loop_all_through_network: a single-process
// communicator that asked for socket/rdma routes every edge through that transport.
RingTransportPlan make_ring_transport_plan(const ProcessLayout& layout, TransportKind local_kind,
                                           TransportKind cross_kind, bool loop_all_through_network);

}  // namespace b200ccl::sched
