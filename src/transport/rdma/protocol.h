// Wire structures and small pure helpers of the RDMA transport.
//
// Parity (behavioural contract): nano-nccl src/transport/rdma/rdma_protocol.h:12-53 — a 64-byte
// RdmaPeerInfo exchanged over the bootstrap connections, a 32-byte RdmaCtsSlot that the receiver
// RDMA-writes into the sender's clear-to-send ring, path MTU = min(local, remote), work-request
// ids that are the absolute step of the slice they carry.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace b200ccl::transport::rdma {

struct RdmaPeerInfo {
    std::uint32_t qpn;
    std::uint32_t psn;
    std::uint16_t lid;
    std::uint8_t gid_index;
    std::uint8_t active_mtu;     // ibv_mtu enumerator: 1=256 ... 5=4096
    std::uint32_t reserved0;
    std::uint8_t gid[16];
    std::uint64_t recv_fifo_addr;
    std::uint32_t recv_fifo_rkey;
    std::uint32_t recv_fifo_bytes;
    std::uint64_t cts_fifo_addr;
    std::uint32_t cts_fifo_rkey;
    std::uint32_t cts_fifo_slots;
};
static_assert(sizeof(RdmaPeerInfo) == 64, "peer info is 64 bytes on the wire");
static_assert(offsetof(RdmaPeerInfo, gid) == 16 && offsetof(RdmaPeerInfo, recv_fifo_addr) == 32 &&
              offsetof(RdmaPeerInfo, cts_fifo_addr) == 48, "peer info layout");

struct RdmaCtsSlot {
    std::uint64_t raddr;      // where the payload of this step must be written
    std::uint32_t rkey;
    std::uint32_t nbytes;     // capacity at raddr
    std::uint64_t step_tag;   // absolute step this grant is for
    std::uint32_t ready;      // 1 = grant valid; the sender clears it when it posts the write
    std::uint32_t reserved;
};
static_assert(sizeof(RdmaCtsSlot) == 32, "clear-to-send slot is 32 bytes");
static_assert(offsetof(RdmaCtsSlot, step_tag) == 16 && offsetof(RdmaCtsSlot, ready) == 24, "cts layout");

inline std::uint64_t wr_id_for_step(std::uint64_t step) { return step; }
inline std::uint64_t step_of_wr_id(std::uint64_t wr_id) { return wr_id; }

// MTU enumerators 1..5 (256..4096 bytes). Throws on values outside that range.
inline std::uint8_t negotiate_path_mtu(std::uint8_t local, std::uint8_t remote) {
    if (local < 1 || local > 5 || remote < 1 || remote > 5)
        throw std::invalid_argument("rdma: path MTU enumerator out of range (local " + std::to_string(local) +
                                    ", remote " + std::to_string(remote) + ")");
    return local < remote ? local : remote;
}

enum class DataPlane { SendRecv, WriteCts };
enum class FifoPlacement { HostPinned, Gdr };

// Environment (B200CCL_ names, NANO_NCCL_ spellings accepted): *_RDMA_USE_WRITE, *_RDMA_GDR,
// *_RDMA_SHARED_PROGRESS take 0/1/true/false/on/off and throw on anything else
// (rdma_proxy.cc:131-158, rdma_gdr.cc:50-61 of the reference).
DataPlane data_plane_from_env();
FifoPlacement fifo_placement_from_env();
bool shared_progress_from_env();

}  // namespace b200ccl::transport::rdma
