#include "sched/transport_plan.h"

#include <sstream>
#include <stdexcept>

namespace b200ccl::sched {

void ProcessLayout::validate() const {
    if (nranks < 1) throw std::invalid_argument("process layout: no ranks");
    if (first_rank.size() != rank_count.size() || first_rank.empty())
        throw std::invalid_argument("process layout: need one (first rank, count) pair per process");
    int expect = 0;
    for (std::size_t p = 0; p < first_rank.size(); ++p) {
        if (rank_count[p] < 1) throw std::invalid_argument("process layout: process " + std::to_string(p) + " owns no rank");
        if (first_rank[p] != expect)
            throw std::invalid_argument("process layout: ranks of process " + std::to_string(p) + " do not follow those of the previous process");
        expect += rank_count[p];
    }
    if (expect != nranks)
        throw std::invalid_argument("process layout: processes own " + std::to_string(expect) + " ranks, communicator has " +
                                    std::to_string(nranks));
}

int ProcessLayout::owner_of(int rank) const {
    for (std::size_t p = 0; p < first_rank.size(); ++p)
        if (rank >= first_rank[p] && rank < first_rank[p] + rank_count[p]) return static_cast<int>(p);
    return -1;
}

TransportKind RingTransportPlan::resolved_kind(TransportKind fallback) const {
    if (edge_kinds.empty()) return fallback;
    for (TransportKind k : edge_kinds)
        if (k != edge_kinds.front()) return TransportKind::Mixed;
    return edge_kinds.front();
}

std::string RingTransportPlan::describe() const {
    std::ostringstream os;
    const int n = static_cast<int>(edge_kinds.size());
    for (int e = 0; e < n; ++e) os << "edge " << e << "->" << (e + 1) % n << ": " << transport_name(edge_kinds[e]) << "\n";
    return os.str();
}

RingTransportPlan make_ring_transport_plan(const ProcessLayout& layout, TransportKind local_kind, TransportKind cross_kind,
                                           bool loop_all_through_network) {
    layout.validate();
    if (local_kind != TransportKind::P2p && local_kind != TransportKind::Shm)
        throw std::invalid_argument("transport plan: edges inside a process are p2p or shm");
    if (cross_kind != TransportKind::P2p && cross_kind != TransportKind::Socket && cross_kind != TransportKind::Rdma)
        throw std::invalid_argument("transport plan: edges between processes are p2p, socket or rdma");
    RingTransportPlan plan;
    if (layout.nranks < 2) return plan;
    for (int e = 0; e < layout.nranks; ++e) {
        const bool crosses = layout.owner_of(e) != layout.owner_of((e + 1) % layout.nranks);
        if (loop_all_through_network) plan.edge_kinds.push_back(cross_kind);
        else plan.edge_kinds.push_back(crosses ? cross_kind : local_kind);
    }
    return plan;
}

}  // namespace b200ccl::sched
