// Symmetric memory: one allocation of the same size on every rank of a communicator, mapped
// so that every local GPU can load and store every rank's copy, and, where the NVSwitch
// multicast engine is available, also reachable through one multicast address.
//
// Stands where nano-nccl allocates per-edge resources with cudaMalloc + peer access
// (src/transport/p2p/p2p_fifo.cu:103-137, p2p_step_counters.cu:53-74): those map ring
// neighbours only; here every rank maps every rank, because through NVSwitch all pairs are
// one hop apart at full bandwidth.
#pragma once

#include "b200ccl/bootstrap.h"

#include <cuda.h>

#include <cstddef>
#include <memory>
#include <string>
#include <vector>

namespace b200ccl::mem {

struct LocalRankDesc {
    int global_rank = 0;
    int device = 0;  // CUDA ordinal in this process
};

struct GroupDesc {
    int nranks = 0;
    std::vector<LocalRankDesc> local;  // ranks driven by this process, ascending global rank
    Bootstrap* bootstrap = nullptr;    // null → this process owns every rank
    bool want_multicast = true;
    bool loopback = false;  // all ranks live on local[0].device (single-GPU emulation)
};

class SymmetricRegion {
public:
    ~SymmetricRegion();
    SymmetricRegion(const SymmetricRegion&) = delete;
    SymmetricRegion& operator=(const SymmetricRegion&) = delete;

    std::size_t bytes() const { return bytes_; }
    // Address of rank g's copy, valid on every local device.
    void* rank_ptr(int g) const { return rank_va_[g]; }
    // Multicast address (stores reach every rank, ld_reduce combines every rank) or nullptr.
    void* multicast_ptr() const { return mc_va_; }
    bool contains(int g, const void* p, std::size_t len) const {
        const char* b = static_cast<const char*>(rank_va_[g]);
        const char* q = static_cast<const char*>(p);
        return q >= b && q + len <= b + bytes_;
    }

private:
    friend class SymmetricAllocator;
    SymmetricRegion() = default;
    std::size_t bytes_ = 0;
    std::vector<void*> rank_va_;
    void* mc_va_ = nullptr;
    // Backing state.
    bool vmm_ = false;
    std::vector<CUmemGenericAllocationHandle> handles_;  // per global rank (imported or own)
    std::vector<bool> handle_valid_;
    CUmemGenericAllocationHandle mc_handle_ = 0;
    bool mc_valid_ = false;
    std::vector<int> mc_bound_devices_;
    std::vector<int> owner_device_;  // per global rank: device to free on (cudaMalloc mode) or -1
};

class SymmetricAllocator {
public:
    explicit SymmetricAllocator(GroupDesc group);
    // Collective over every process of the group. Contents are zeroed.
    std::unique_ptr<SymmetricRegion> allocate(std::size_t bytes, const char* label);
    bool uses_vmm() const { return use_vmm_; }
    bool multicast_supported() const { return multicast_; }
    const GroupDesc& group() const { return group_; }
    const std::string& multicast_reason() const { return mc_reason_; }

private:
    std::unique_ptr<SymmetricRegion> allocate_vmm(std::size_t bytes, const char* label);
    std::unique_ptr<SymmetricRegion> allocate_plain(std::size_t bytes);
    void try_bind_multicast(SymmetricRegion& r, const char* label);
    GroupDesc group_;
    bool use_vmm_ = false;
    bool multicast_ = false;
    std::string mc_reason_;
    std::vector<int> local_devices_;  // unique device ordinals of this process
};

// cudaDeviceEnablePeerAccess for every ordered pair in `devices`; returns false (with a
// message) if some pair cannot reach each other. Already-enabled pairs are fine.
bool enable_all_peer_access(const std::vector<int>& devices, std::string* why);

}  // namespace b200ccl::mem
