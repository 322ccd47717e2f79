#include "collective/validate.h"

#include <set>
#include <stdexcept>
#include <string>

namespace b200ccl {

void validate_collective_args(Collective collective, const CollectiveArgs& args, int local_ranks,
                              bool allow_in_place) {
    const std::string name = collective_name(collective);
    const std::size_t n = static_cast<std::size_t>(local_ranks);
    if (args.send_buffers.size() != n || args.recv_buffers.size() != n || args.streams.size() != n)
        throw std::invalid_argument(name + ": send_buffers, recv_buffers and streams need one entry per rank (" +
                                    std::to_string(local_ranks) + " local ranks)");
    if (args.count == 0) throw std::invalid_argument(name + ": count must be positive");
    switch (args.dtype) {
        case DType::Float:
        case DType::Float16:
        case DType::BFloat16: break;
        default: throw std::invalid_argument(name + ": unsupported dtype");
    }
    switch (args.redop) {
        case RedOp::Sum:
        case RedOp::Avg:
        case RedOp::Max:
        case RedOp::Min: break;
        default: throw std::invalid_argument(name + ": unknown reduction operator");
    }
    for (std::size_t r = 0; r < n; ++r) {
        if (args.send_buffers[r] == nullptr || args.recv_buffers[r] == nullptr)
            throw std::invalid_argument(name + ": buffers must be non-null (local rank " + std::to_string(r) + ")");
        if (args.send_buffers[r] == args.recv_buffers[r] && !(allow_in_place && collective == Collective::AllReduce))
            throw std::invalid_argument(name + ": in-place operation is not supported (send == recv on local rank " +
                                        std::to_string(r) + ")");
    }
}

void validate_config(const CommunicatorConfig& config, int visible_devices) {
    if (config.loopback) {
        if (config.devices.size() != 1)
            throw std::invalid_argument("loopback communicator takes exactly one device");
        if (config.loopback_ranks < 1 || config.loopback_ranks > kMaxRanks)
            throw std::invalid_argument("loopback_ranks must be between 1 and " + std::to_string(kMaxRanks));
    } else {
        if (config.devices.empty()) throw std::invalid_argument("communicator needs at least one device");
        if (static_cast<int>(config.devices.size()) > kMaxRanks)
            throw std::invalid_argument("communicator supports at most " + std::to_string(kMaxRanks) +
                                        " ranks per process");
    }
    if (config.max_ctas < 0) throw std::invalid_argument("max_ctas must not be negative");
    std::set<int> seen;
    for (int d : config.devices) {
        if (d < 0 || d >= visible_devices)
            throw std::invalid_argument("device " + std::to_string(d) + " is not in the visible sequence 0.." +
                                        std::to_string(visible_devices - 1));
        if (!seen.insert(d).second)
            throw std::invalid_argument("device " + std::to_string(d) + " is listed twice");
    }
    switch (config.transport) {
        case TransportKind::Auto:
        case TransportKind::Shm:
        case TransportKind::P2p:
        case TransportKind::Socket:
        case TransportKind::Rdma: break;
        default: throw std::invalid_argument("transport 'mixed' can be reported but not requested");
    }
}

}  // namespace b200ccl
