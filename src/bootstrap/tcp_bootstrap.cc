// TCP rendezvous: rank 0 is a star hub for all-gather/barrier; descriptor passing is done by
// FdExchange (one abstract AF_UNIX listener per process). This is the default control plane; it plays the role
// that the MPI C API plays for nano-nccl (src/collective/all_reduce/mpi_communicator.cc:
// 134-155 rank layout, 38-75 error consensus, 203-208 address all-gather).
#include "b200ccl/bootstrap.h"

#include "bootstrap/fd_exchange.h"
#include "core/check.h"

#include <arpa/inet.h>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <random>
#include <stdexcept>
#include <sys/socket.h>
#include <sys/un.h>
#include <thread>
#include <unistd.h>

namespace b200ccl {

namespace {

[[noreturn]] void fail(const std::string& what) {
    throw std::runtime_error("bootstrap: " + what + ": " + std::strerror(errno));
}

void write_all(int fd, const void* buf, std::size_t n) {
    const char* p = static_cast<const char*>(buf);
    while (n > 0) {
        const ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
        if (w < 0) {
            if (errno == EINTR) continue;
            fail("send");
        }
        p += w;
        n -= static_cast<std::size_t>(w);
    }
}

void read_all(int fd, void* buf, std::size_t n, int timeout_ms) {
    char* p = static_cast<char*>(buf);
    while (n > 0) {
        pollfd pfd{fd, POLLIN, 0};
        const int pr = ::poll(&pfd, 1, timeout_ms);
        if (pr == 0) throw std::runtime_error("bootstrap: timed out waiting for a peer process");
        if (pr < 0) {
            if (errno == EINTR) continue;
            fail("poll");
        }
        const ssize_t r = ::recv(fd, p, n, 0);
        if (r == 0) throw std::runtime_error("bootstrap: peer process closed the connection");
        if (r < 0) {
            if (errno == EINTR) continue;
            fail("recv");
        }
        p += r;
        n -= static_cast<std::size_t>(r);
    }
}


class TcpBootstrap final : public Bootstrap {
public:
    TcpBootstrap(const std::string& addr, int port, int rank, int size, int timeout_ms)
        : rank_(rank), size_(size), timeout_ms_(timeout_ms) {
        if (size < 1 || rank < 0 || rank >= size) throw std::invalid_argument("bootstrap: bad rank/size");
        if (size == 1) return;
        if (rank == 0) serve(addr, port);
        else connect_to_root(addr, port);
    }

    ~TcpBootstrap() override {
        for (int fd : clients_) if (fd >= 0) ::close(fd);
        if (root_fd_ >= 0) ::close(root_fd_);
        if (listen_fd_ >= 0) ::close(listen_fd_);
    }

    int rank() const override { return rank_; }
    int size() const override { return size_; }

    void allgather(const void* in, void* out, std::size_t bytes) override {
        char* o = static_cast<char*>(out);
        if (size_ == 1) {
            std::memcpy(o, in, bytes);
            return;
        }
        if (rank_ == 0) {
            std::memcpy(o, in, bytes);
            for (int r = 1; r < size_; ++r) read_all(clients_[r], o + r * bytes, bytes, timeout_ms_);
            for (int r = 1; r < size_; ++r) write_all(clients_[r], o, bytes * size_);
        } else {
            write_all(root_fd_, in, bytes);
            read_all(root_fd_, o, bytes * size_, timeout_ms_);
        }
    }

    void barrier() override {
        char c = 0;
        std::vector<char> all(size_);
        allgather(&c, all.data(), 1);
    }

    std::vector<std::vector<int>> exchange_fds(const std::vector<int>& fds) override {
        if (!fdx_) fdx_.reset(new FdExchange(*this, timeout_ms_));
        return fdx_->exchange(fds);
    }

private:
    void serve(const std::string& addr, int port) {
        listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
        if (listen_fd_ < 0) fail("socket");
        int one = 1;
        ::setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        sockaddr_in sa{};
        sa.sin_family = AF_INET;
        sa.sin_port = htons(static_cast<uint16_t>(port));
        if (addr.empty() || ::inet_pton(AF_INET, addr.c_str(), &sa.sin_addr) != 1)
            sa.sin_addr.s_addr = htonl(INADDR_ANY);
        if (::bind(listen_fd_, reinterpret_cast<sockaddr*>(&sa), sizeof(sa)) != 0) fail("bind");
        if (::listen(listen_fd_, size_ + 8) != 0) fail("listen");
        clients_.assign(size_, -1);
        for (int k = 1; k < size_; ++k) {
            pollfd pfd{listen_fd_, POLLIN, 0};
            const int pr = ::poll(&pfd, 1, timeout_ms_);
            if (pr <= 0) throw std::runtime_error("bootstrap: timed out waiting for ranks to connect");
            const int fd = ::accept(listen_fd_, nullptr, nullptr);
            if (fd < 0) fail("accept");
            ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
            int32_t r = -1;
            read_all(fd, &r, sizeof(r), timeout_ms_);
            if (r <= 0 || r >= size_ || clients_[r] >= 0) {
                ::close(fd);
                throw std::runtime_error("bootstrap: unexpected or duplicate rank " + std::to_string(r));
            }
            clients_[r] = fd;
        }
    }

    void connect_to_root(const std::string& addr, int port) {
        sockaddr_in sa{};
        sa.sin_family = AF_INET;
        sa.sin_port = htons(static_cast<uint16_t>(port));
        if (::inet_pton(AF_INET, addr.c_str(), &sa.sin_addr) != 1) {
            addrinfo hints{};
            hints.ai_family = AF_INET;
            hints.ai_socktype = SOCK_STREAM;
            addrinfo* res = nullptr;
            if (::getaddrinfo(addr.c_str(), nullptr, &hints, &res) != 0 || !res)
                throw std::runtime_error("bootstrap: cannot resolve '" + addr + "'");
            sa.sin_addr = reinterpret_cast<sockaddr_in*>(res->ai_addr)->sin_addr;
            ::freeaddrinfo(res);
        }
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms_);
        for (;;) {
            root_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
            if (root_fd_ < 0) fail("socket");
            if (::connect(root_fd_, reinterpret_cast<sockaddr*>(&sa), sizeof(sa)) == 0) break;
            ::close(root_fd_);
            root_fd_ = -1;
            if (std::chrono::steady_clock::now() > deadline)
                throw std::runtime_error("bootstrap: could not reach rank 0 at " + addr + ":" + std::to_string(port));
            std::this_thread::sleep_for(std::chrono::milliseconds(50));
        }
        int one = 1;
        ::setsockopt(root_fd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        const int32_t r = rank_;
        write_all(root_fd_, &r, sizeof(r));
    }

    int rank_;
    int size_;
    int timeout_ms_;
    int listen_fd_ = -1;
    int root_fd_ = -1;
    std::vector<int> clients_;
    std::unique_ptr<FdExchange> fdx_;
};

}  // namespace

std::string Bootstrap::error_consensus(const std::string& local_error) {
    constexpr std::size_t kLen = 256;
    char mine[kLen] = {0};
    std::strncpy(mine, local_error.c_str(), kLen - 1);
    std::vector<char> all(kLen * size());
    allgather(mine, all.data(), kLen);
    for (int r = 0; r < size(); ++r) {
        const char* s = all.data() + r * kLen;
        if (s[0] != '\0') return "process " + std::to_string(r) + ": " + std::string(s);
    }
    return "";
}

std::unique_ptr<Bootstrap> create_tcp_bootstrap(const std::string& addr, int port, int rank, int size,
                                                int timeout_ms) {
    return std::unique_ptr<Bootstrap>(new TcpBootstrap(addr, port, rank, size, timeout_ms));
}

}  // namespace b200ccl
