#include "transport/socket/wire.h"

#include <arpa/inet.h>
#include <cerrno>
#include <cstring>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdexcept>
#include <string>
#include <sys/socket.h>
#include <sys/uio.h>

namespace b200ccl::transport::socket {

std::uint32_t to_big_endian(std::uint32_t v) { return htonl(v); }
std::uint32_t from_big_endian(std::uint32_t v) { return ntohl(v); }

void set_tcp_nodelay(int fd) {
    int one = 1;
    (void)::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
}

void send_all(int fd, const void* data, std::size_t bytes) {
    const char* p = static_cast<const char*>(data);
    while (bytes > 0) {
        const ssize_t w = ::send(fd, p, bytes, MSG_NOSIGNAL);
        if (w < 0) {
            if (errno == EINTR) continue;
            throw std::runtime_error(std::string("send: ") + std::strerror(errno));
        }
        p += w;
        bytes -= static_cast<std::size_t>(w);
    }
}

void recv_all(int fd, void* data, std::size_t bytes) {
    char* p = static_cast<char*>(data);
    while (bytes > 0) {
        const ssize_t r = ::recv(fd, p, bytes, 0);
        if (r == 0) throw std::runtime_error("recv: peer closed the connection");
        if (r < 0) {
            if (errno == EINTR) continue;
            throw std::runtime_error(std::string("recv: ") + std::strerror(errno));
        }
        p += r;
        bytes -= static_cast<std::size_t>(r);
    }
}

bool wait_readable(int fd, const std::atomic<bool>* stop) {
    for (;;) {
        if (stop && stop->load(std::memory_order_acquire)) return false;
        pollfd pfd{fd, POLLIN, 0};
        const int pr = ::poll(&pfd, 1, 20);
        if (pr > 0) return true;
        if (pr < 0 && errno != EINTR) throw std::runtime_error(std::string("poll: ") + std::strerror(errno));
    }
}

void send_slice(int fd, const void* payload, std::uint32_t payload_bytes) {
    SliceHeader h{to_big_endian(payload_bytes)};
    // Header and payload leave in one call straight from the FIFO slot: no bounce copy.
    iovec iov[2] = {{&h, sizeof(h)}, {const_cast<void*>(payload), payload_bytes}};
    msghdr msg{};
    msg.msg_iov = iov;
    msg.msg_iovlen = payload_bytes ? 2 : 1;
    std::size_t total = sizeof(h) + payload_bytes, sent = 0;
    while (sent < total) {
        const ssize_t w = ::sendmsg(fd, &msg, MSG_NOSIGNAL);
        if (w < 0) {
            if (errno == EINTR) continue;
            throw std::runtime_error(std::string("sendmsg: ") + std::strerror(errno));
        }
        sent += static_cast<std::size_t>(w);
        std::size_t skip = static_cast<std::size_t>(w);
        while (skip > 0 && msg.msg_iovlen > 0) {
            if (skip >= msg.msg_iov[0].iov_len) {
                skip -= msg.msg_iov[0].iov_len;
                ++msg.msg_iov;
                --msg.msg_iovlen;
            } else {
                msg.msg_iov[0].iov_base = static_cast<char*>(msg.msg_iov[0].iov_base) + skip;
                msg.msg_iov[0].iov_len -= skip;
                skip = 0;
            }
        }
    }
}

std::uint32_t recv_slice(int fd, void* payload, std::size_t capacity) {
    SliceHeader h{};
    recv_all(fd, &h, sizeof(h));
    const std::uint32_t n = from_big_endian(h.payload_bytes_be);
    if (n > capacity)
        throw std::runtime_error("oversized slice: header announces " + std::to_string(n) + " bytes, slot holds " +
                                 std::to_string(capacity));
    if (n) recv_all(fd, payload, n);
    return n;
}

void send_hello(int fd, int channel, int source_rank, int destination_rank) {
    WireHello h{};
    h.magic = to_big_endian(kHelloMagic);
    h.version = htons(kHelloVersion);
    h.channel = htons(static_cast<std::uint16_t>(channel));
    h.source_rank = to_big_endian(static_cast<std::uint32_t>(source_rank));
    h.destination_rank = to_big_endian(static_cast<std::uint32_t>(destination_rank));
    send_all(fd, &h, sizeof(h));
}

WireHello recv_hello(int fd) {
    WireHello h{};
    recv_all(fd, &h, sizeof(h));
    h.magic = from_big_endian(h.magic);
    h.version = ntohs(h.version);
    h.channel = ntohs(h.channel);
    h.source_rank = from_big_endian(h.source_rank);
    h.destination_rank = from_big_endian(h.destination_rank);
    if (h.magic != kHelloMagic) throw std::runtime_error("socket hello: bad magic");
    if (h.version != kHelloVersion) throw std::runtime_error("socket hello: unsupported version " + std::to_string(h.version));
    return h;
}

}  // namespace b200ccl::transport::socket
