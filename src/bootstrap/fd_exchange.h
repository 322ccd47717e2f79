// Same-host descriptor passing on top of any control plane (see fd_exchange.cc).
#pragma once

#include "b200ccl/bootstrap.h"

#include <cstdint>
#include <vector>

namespace b200ccl {

class FdExchange {
public:
    // `control` must outlive this object; only its rank(), size(), allgather() and barrier() are used.
    FdExchange(Bootstrap& control, int timeout_ms);
    ~FdExchange();
    FdExchange(const FdExchange&) = delete;
    FdExchange& operator=(const FdExchange&) = delete;

    // The contract of Bootstrap::exchange_fds. At most 32 descriptors per call.
    std::vector<std::vector<int>> exchange(const std::vector<int>& fds);

private:
    void ensure_unix_listener();
    void send_fds_to(int peer, const std::vector<int>& fds);
    void recv_fds(std::vector<std::vector<int>>* result, int nf);

    Bootstrap& control_;
    int rank_;
    int size_;
    int timeout_ms_;
    int unix_fd_ = -1;
    std::uint64_t token_ = 0;
    std::uint32_t seq_ = 0;
};

}  // namespace b200ccl
