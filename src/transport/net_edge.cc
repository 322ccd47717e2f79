#include "transport/net_edge.h"

#include <stdexcept>

namespace b200ccl::transport {

std::unique_ptr<NetEdgeSet> create_socket_edges(const NetEdgeConfig& config, Bootstrap* bootstrap);
std::unique_ptr<NetEdgeSet> create_rdma_edges(const NetEdgeConfig& config, Bootstrap* bootstrap);

std::unique_ptr<NetEdgeSet> create_net_edges(const NetEdgeConfig& config, Bootstrap* bootstrap) {
    if (!bootstrap && !config.all_edges)
        throw std::invalid_argument("network edges need a multi-process communicator or all_edges");
    switch (config.kind) {
        case TransportKind::Socket: return create_socket_edges(config, bootstrap);
        case TransportKind::Rdma: return create_rdma_edges(config, bootstrap);
        default: throw std::invalid_argument("network edges: transport must be socket or rdma");
    }
}


}  // namespace b200ccl::transport
