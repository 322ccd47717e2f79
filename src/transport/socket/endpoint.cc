#include "transport/socket/endpoint.h"

#include "core/env.h"

#include <arpa/inet.h>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/in.h>
#include <poll.h>
#include <stdexcept>
#include <sys/socket.h>
#include <thread>
#include <unistd.h>

namespace b200ccl::transport::socket {

void Fd::reset() {
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
}
void Fd::shutdown_both() noexcept {
    if (fd_ >= 0) ::shutdown(fd_, SHUT_RDWR);
}

std::string socket_ifname_from_env() {
    return env::get_string("B200CCL_SOCKET_IFNAME", "", "NANO_NCCL_SOCKET_IFNAME");
}

std::uint32_t interface_ipv4_be(const std::string& ifname) {
    if (ifname.empty()) return htonl(INADDR_LOOPBACK);
    ifaddrs* list = nullptr;
    if (::getifaddrs(&list) != 0) throw std::runtime_error(std::string("getifaddrs: ") + std::strerror(errno));
    std::uint32_t found = 0;
    int count = 0;
    for (ifaddrs* it = list; it; it = it->ifa_next) {
        if (!it->ifa_addr || it->ifa_addr->sa_family != AF_INET || ifname != it->ifa_name) continue;
        if (!(it->ifa_flags & IFF_UP)) continue;
        found = reinterpret_cast<sockaddr_in*>(it->ifa_addr)->sin_addr.s_addr;
        ++count;
    }
    ::freeifaddrs(list);
    if (count != 1)
        throw std::runtime_error("socket interface '" + ifname + "' must have exactly one usable IPv4 address, found " +
                                 std::to_string(count));
    return found;
}

Listener Listener::create(const std::string& ifname) {
    Listener l;
    const std::uint32_t ip = interface_ipv4_be(ifname);
    l.fd_ = Fd(::socket(AF_INET, SOCK_STREAM, 0));
    if (!l.fd_.valid()) throw std::runtime_error(std::string("socket: ") + std::strerror(errno));
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = ip;
    sa.sin_port = 0;
    if (::bind(l.fd_.get(), reinterpret_cast<sockaddr*>(&sa), sizeof(sa)) != 0)
        throw std::runtime_error(std::string("bind: ") + std::strerror(errno));
    if (::listen(l.fd_.get(), 512) != 0) throw std::runtime_error(std::string("listen: ") + std::strerror(errno));
    socklen_t len = sizeof(sa);
    if (::getsockname(l.fd_.get(), reinterpret_cast<sockaddr*>(&sa), &len) != 0)
        throw std::runtime_error(std::string("getsockname: ") + std::strerror(errno));
    l.addr_.ipv4_be = sa.sin_addr.s_addr;
    l.addr_.port_be = sa.sin_port;
    return l;
}

std::pair<Fd, WireHello> Listener::accept_hello(int timeout_ms) const {
    pollfd pfd{fd_.get(), POLLIN, 0};
    const int pr = ::poll(&pfd, 1, timeout_ms);
    if (pr == 0) throw std::runtime_error("socket accept: timed out waiting for a peer");
    if (pr < 0) throw std::runtime_error(std::string("poll: ") + std::strerror(errno));
    Fd conn(::accept(fd_.get(), nullptr, nullptr));
    if (!conn.valid()) throw std::runtime_error(std::string("accept: ") + std::strerror(errno));
    set_tcp_nodelay(conn.get());
    WireHello h = recv_hello(conn.get());
    return {std::move(conn), h};
}

Fd connect_with_hello(const SocketAddress& peer, int channel, int source_rank, int destination_rank, int timeout_ms) {
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_addr.s_addr = peer.ipv4_be;
    sa.sin_port = peer.port_be;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    for (;;) {
        Fd fd(::socket(AF_INET, SOCK_STREAM, 0));
        if (!fd.valid()) throw std::runtime_error(std::string("socket: ") + std::strerror(errno));
        if (::connect(fd.get(), reinterpret_cast<sockaddr*>(&sa), sizeof(sa)) == 0) {
            set_tcp_nodelay(fd.get());
            send_hello(fd.get(), channel, source_rank, destination_rank);
            return fd;
        }
        if (std::chrono::steady_clock::now() > deadline)
            throw std::runtime_error(std::string("connect: ") + std::strerror(errno));
        std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
}

}  // namespace b200ccl::transport::socket
