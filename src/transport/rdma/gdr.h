// Placement and registration of an RDMA FIFO: pinned host memory (default) or device memory that
// the HCA reads and writes directly (B200CCL_RDMA_GDR=1). A GDR request that cannot be met fails;
// it never falls back to host memory silently.
// Parity: nano-nccl src/transport/rdma/rdma_gdr.cc:27-61, 112-136; communicator.cu:437-469.
#pragma once

#include "core/buffers.h"
#include "transport/rdma/verbs_backend.h"

#include <memory>

namespace b200ccl::transport::rdma {

class RegisteredFifo {
public:
    // device: CUDA ordinal whose memory (Gdr) or NUMA node (HostPinned) the FIFO uses.
    RegisteredFifo(std::shared_ptr<VerbsBackend> backend, FifoPlacement placement, std::size_t bytes, int device);
    ~RegisteredFifo();
    RegisteredFifo(const RegisteredFifo&) = delete;
    RegisteredFifo& operator=(const RegisteredFifo&) = delete;
    void* data() const { return data_; }
    std::size_t bytes() const { return bytes_; }
    const MemoryRegion& region() const { return mr_; }
    FifoPlacement placement() const { return placement_; }

private:
    std::shared_ptr<VerbsBackend> backend_;
    FifoPlacement placement_;
    std::size_t bytes_;
    void* data_ = nullptr;
    MappedBuffer<unsigned char> host_;
    DeviceBuffer<unsigned char> device_;
    MemoryRegion mr_;
};

}  // namespace b200ccl::transport::rdma
