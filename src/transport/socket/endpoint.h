// Listening endpoint and connections of the socket transport.
//
// Parity: nano-nccl src/transport/socket/socket_endpoint.h:7-67 / .cc:63-92, 130-162, 187-237:
// RAII descriptors, an IPv4 listener on an ephemeral port bound to the single IPv4 address of the
// interface named by the environment (B200CCL_SOCKET_IFNAME, or NANO_NCCL_SOCKET_IFNAME), connect
// followed by HELLO, accept followed by HELLO validation. Without the variable the loopback
// address is used, which is enough for ranks on one host.
#pragma once

#include "transport/socket/wire.h"

#include <string>
#include <utility>

namespace b200ccl::transport::socket {

class Fd {
public:
    Fd() = default;
    explicit Fd(int fd) : fd_(fd) {}
    ~Fd() { reset(); }
    Fd(Fd&& o) noexcept : fd_(o.fd_) { o.fd_ = -1; }
    Fd& operator=(Fd&& o) noexcept { if (this != &o) { reset(); fd_ = o.fd_; o.fd_ = -1; } return *this; }
    Fd(const Fd&) = delete;
    Fd& operator=(const Fd&) = delete;
    int get() const { return fd_; }
    bool valid() const { return fd_ >= 0; }
    int release() { const int f = fd_; fd_ = -1; return f; }
    void reset();
    void shutdown_both() noexcept;
private:
    int fd_ = -1;
};

struct SocketAddress {  // what processes exchange through the bootstrap
    std::uint32_t ipv4_be = 0;
    std::uint16_t port_be = 0;
    std::uint16_t pad = 0;
};
static_assert(sizeof(SocketAddress) == 8, "address blob");

// IPv4 address of the interface: exactly one usable address is required; throws with the
// interface name otherwise. An empty name means loopback.
std::uint32_t interface_ipv4_be(const std::string& ifname);
std::string socket_ifname_from_env();

class Listener {
public:
    Listener() = default;
    static Listener create(const std::string& ifname);  // ephemeral port, backlog for every edge×channel
    const SocketAddress& address() const { return addr_; }
    // Accepts one connection and reads its HELLO (validated). `timeout_ms` bounds the wait.
    std::pair<Fd, WireHello> accept_hello(int timeout_ms) const;
    bool valid() const { return fd_.valid(); }
private:
    Fd fd_;
    SocketAddress addr_;
};

// Connects (retrying while the peer's listener comes up) and sends HELLO.
Fd connect_with_hello(const SocketAddress& peer, int channel, int source_rank, int destination_rank, int timeout_ms);

}  // namespace b200ccl::transport::socket
