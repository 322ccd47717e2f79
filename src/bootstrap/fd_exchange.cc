// Descriptor passing between the processes of one host: one abstract AF_UNIX listener per
// process, descriptors sent as SCM_RIGHTS ancillary data. It needs nothing from the control plane
// but an all-gather and a barrier, so the TCP rendezvous and the MPI adapter share it.
#include "bootstrap/fd_exchange.h"

#include <cerrno>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <poll.h>
#include <random>
#include <stdexcept>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace b200ccl {

namespace {

[[noreturn]] void fail(const std::string& what) {
    throw std::runtime_error("bootstrap: " + what + ": " + std::strerror(errno));
}

struct FdHeader {
    int32_t src_rank;
    int32_t nfds;
    uint32_t seq;
    uint32_t valid_mask_lo;  // bit i set → entry i carries a descriptor (nfds ≤ 32 per call)
};

constexpr int kMaxFdsPerCall = 32;

sockaddr_un unix_addr(uint64_t token, int rank, socklen_t* len) {
    sockaddr_un sa{};
    sa.sun_family = AF_UNIX;
    char name[96];
    const int n = std::snprintf(name, sizeof(name), "b200ccl-%016llx-%d",
                                static_cast<unsigned long long>(token), rank);
    sa.sun_path[0] = '\0';  // abstract namespace: no file to clean up
    std::memcpy(sa.sun_path + 1, name, static_cast<std::size_t>(n));
    *len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + n);
    return sa;
}

}  // namespace

FdExchange::FdExchange(Bootstrap& control, int timeout_ms)
    : control_(control), rank_(control.rank()), size_(control.size()), timeout_ms_(timeout_ms) {}

FdExchange::~FdExchange() {
    if (unix_fd_ >= 0) ::close(unix_fd_);
}

std::vector<std::vector<int>> FdExchange::exchange(const std::vector<int>& fds) {
    const int nf = static_cast<int>(fds.size());
    if (nf > kMaxFdsPerCall) throw std::invalid_argument("bootstrap: too many descriptors in one exchange");
    std::vector<std::vector<int>> result(size_, std::vector<int>(nf, -1));
    for (int i = 0; i < nf; ++i) result[rank_][i] = fds[i] >= 0 ? ::dup(fds[i]) : -1;
    if (size_ == 1) return result;
    ensure_unix_listener();
    ++seq_;
    for (int p = 0; p < size_; ++p) {
        if (p != rank_) send_fds_to(p, fds);
    }
    for (int k = 0; k < size_ - 1; ++k) recv_fds(&result, nf);
    control_.barrier();  // nobody starts the next exchange while a peer still accepts this one
    return result;
}

void FdExchange::ensure_unix_listener() {
    if (unix_fd_ >= 0) return;
    uint64_t token = 0;
    if (rank_ == 0) {
        std::random_device rd;
        token = (static_cast<uint64_t>(rd()) << 32) ^ rd() ^ (static_cast<uint64_t>(::getpid()) << 20);
    }
    std::vector<uint64_t> all(size_);
    control_.allgather(&token, all.data(), sizeof(token));
    token_ = all[0];
    unix_fd_ = ::socket(AF_UNIX, SOCK_STREAM, 0);
    if (unix_fd_ < 0) fail("socket(AF_UNIX)");
    socklen_t len = 0;
    sockaddr_un sa = unix_addr(token_, rank_, &len);
    if (::bind(unix_fd_, reinterpret_cast<sockaddr*>(&sa), len) != 0) fail("bind(AF_UNIX)");
    if (::listen(unix_fd_, size_ + 8) != 0) fail("listen(AF_UNIX)");
    control_.barrier();  // every listener exists before anyone connects
}

void FdExchange::send_fds_to(int peer, const std::vector<int>& fds) {
    const int fd = ::socket(AF_UNIX, SOCK_STREAM, 0);
    if (fd < 0) fail("socket(AF_UNIX)");
    socklen_t len = 0;
    sockaddr_un sa = unix_addr(token_, peer, &len);
    if (::connect(fd, reinterpret_cast<sockaddr*>(&sa), len) != 0) {
        ::close(fd);
        fail("connect(AF_UNIX) to rank " + std::to_string(peer));
    }
    FdHeader h{};
    h.src_rank = rank_;
    h.nfds = static_cast<int32_t>(fds.size());
    h.seq = seq_;
    std::vector<int> valid;
    for (std::size_t i = 0; i < fds.size(); ++i) {
        if (fds[i] >= 0) {
            h.valid_mask_lo |= (1u << i);
            valid.push_back(fds[i]);
        }
    }
    msghdr msg{};
    iovec iov{&h, sizeof(h)};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * kMaxFdsPerCall)];
    if (!valid.empty()) {
        std::memset(ctrl, 0, sizeof(ctrl));
        msg.msg_control = ctrl;
        msg.msg_controllen = CMSG_SPACE(sizeof(int) * valid.size());
        cmsghdr* c = CMSG_FIRSTHDR(&msg);
        c->cmsg_level = SOL_SOCKET;
        c->cmsg_type = SCM_RIGHTS;
        c->cmsg_len = CMSG_LEN(sizeof(int) * valid.size());
        std::memcpy(CMSG_DATA(c), valid.data(), sizeof(int) * valid.size());
    }
    if (::sendmsg(fd, &msg, MSG_NOSIGNAL) != static_cast<ssize_t>(sizeof(h))) {
        ::close(fd);
        fail("sendmsg(SCM_RIGHTS)");
    }
    ::close(fd);
}

void FdExchange::recv_fds(std::vector<std::vector<int>>* result, int nf) {
    pollfd pfd{unix_fd_, POLLIN, 0};
    const int pr = ::poll(&pfd, 1, timeout_ms_);
    if (pr <= 0) throw std::runtime_error("bootstrap: timed out waiting for descriptors");
    const int fd = ::accept(unix_fd_, nullptr, nullptr);
    if (fd < 0) fail("accept(AF_UNIX)");
    FdHeader h{};
    msghdr msg{};
    iovec iov{&h, sizeof(h)};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * kMaxFdsPerCall)];
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    pollfd dfd{fd, POLLIN, 0};
    if (::poll(&dfd, 1, timeout_ms_) <= 0) {
        ::close(fd);
        throw std::runtime_error("bootstrap: timed out reading descriptors");
    }
    const ssize_t got = ::recvmsg(fd, &msg, MSG_WAITALL);
    ::close(fd);
    if (got != static_cast<ssize_t>(sizeof(h))) fail("recvmsg(SCM_RIGHTS)");
    std::vector<int> valid;
    for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
        if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
            const std::size_t k = (c->cmsg_len - CMSG_LEN(0)) / sizeof(int);
            valid.resize(k);
            std::memcpy(valid.data(), CMSG_DATA(c), k * sizeof(int));
        }
    }
    auto close_all = [&] { for (int v : valid) ::close(v); };
    if (h.src_rank < 0 || h.src_rank >= size_ || h.src_rank == rank_ || h.nfds != nf || h.seq != seq_) {
        close_all();
        throw std::runtime_error("bootstrap: descriptor exchange out of step with rank " +
                                 std::to_string(h.src_rank));
    }
    std::size_t vi = 0;
    for (int i = 0; i < nf; ++i) {
        if (h.valid_mask_lo & (1u << i)) {
            if (vi >= valid.size()) {
                close_all();
                throw std::runtime_error("bootstrap: fewer descriptors arrived than announced");
            }
            (*result)[h.src_rank][i] = valid[vi++];
        }
    }
}

}  // namespace b200ccl
