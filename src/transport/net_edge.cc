#include "transport/net_edge.h"

#include <stdexcept>

namespace b200ccl::transport {

std::unique_ptr<NetEdgeSet> create_socket_edges(const NetEdgeConfig& config, Bootstrap* bootstrap);
std::unique_ptr<NetEdgeSet> create_rdma_edges(const NetEdgeConfig& config, Bootstrap* bootstrap);

std::unique_ptr<NetEdgeSet> create_net_edges(const NetEdgeConfig& config, Bootstrap* bootstrap) {
    if (!bootstrap) throw std::invalid_argument("network edges need a multi-process communicator");
    switch (config.kind) {
        case TransportKind::Socket: return create_socket_edges(config, bootstrap);
        case TransportKind::Rdma: return create_rdma_edges(config, bootstrap);
        default: throw std::invalid_argument("network edges: transport must be socket or rdma");
    }
}

// Placeholders until the socket and RDMA edge sets are linked in.
__attribute__((weak)) std::unique_ptr<NetEdgeSet> create_socket_edges(const NetEdgeConfig&, Bootstrap*) {
    throw std::runtime_error("socket transport is not part of this build");
}
__attribute__((weak)) std::unique_ptr<NetEdgeSet> create_rdma_edges(const NetEdgeConfig&, Bootstrap*) {
    throw std::runtime_error("rdma transport is not part of this build");
}

}  // namespace b200ccl::transport
