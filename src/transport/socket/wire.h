// TCP wire format of the socket transport and blocking send/receive helpers.
//
// Parity (behavioural contract): 16-byte HELLO {magic 0x4e4e434c, version 1, channel, source,
// destination} (nano-nccl src/transport/socket/socket_endpoint.cc:21-29); slices framed by a
// 4-byte big-endian payload length (socket_protocol.h:8-18); a length above the receiver's
// capacity is rejected before any payload byte is copied (socket_proxy.cc:150-170); TCP_NODELAY.
#pragma once

#include <atomic>
#include <cstddef>
#include <cstdint>

namespace b200ccl::transport::socket {

constexpr std::uint32_t kHelloMagic = 0x4e4e434cu;
constexpr std::uint16_t kHelloVersion = 1;

struct WireHello {
    std::uint32_t magic;
    std::uint16_t version;
    std::uint16_t channel;
    std::uint32_t source_rank;
    std::uint32_t destination_rank;
};
static_assert(sizeof(WireHello) == 16, "HELLO is 16 bytes on the wire");

struct SliceHeader {
    std::uint32_t payload_bytes_be;
};
static_assert(sizeof(SliceHeader) == 4, "slice header is one big-endian 32-bit length");

std::uint32_t to_big_endian(std::uint32_t v);
std::uint32_t from_big_endian(std::uint32_t v);

void set_tcp_nodelay(int fd);  // ignored on non-TCP sockets (tests use AF_UNIX pairs)
// Blocking, complete transfers; throw std::runtime_error ("... peer closed ..." on EOF).
void send_all(int fd, const void* data, std::size_t bytes);
void recv_all(int fd, void* data, std::size_t bytes);
// Waits until `fd` is readable or `*stop` becomes true; returns false when stopped.
bool wait_readable(int fd, const std::atomic<bool>* stop);

void send_slice(int fd, const void* payload, std::uint32_t payload_bytes);
// Reads the header, rejects payload_bytes > capacity (throws, nothing copied), then the payload.
std::uint32_t recv_slice(int fd, void* payload, std::size_t capacity);

void send_hello(int fd, int channel, int source_rank, int destination_rank);
WireHello recv_hello(int fd);  // throws on bad magic or version

}  // namespace b200ccl::transport::socket
