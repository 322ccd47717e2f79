#include "transport/rdma/gdr.h"

#include "core/numa.h"

namespace b200ccl::transport::rdma {

RegisteredFifo::RegisteredFifo(std::shared_ptr<VerbsBackend> backend, FifoPlacement placement, std::size_t bytes, int device)
    : backend_(std::move(backend)), placement_(placement), bytes_(bytes) {
    if (placement_ == FifoPlacement::Gdr) {
        device_.reset(device, bytes);
        device_.zero();
        data_ = device_.get();
        mr_ = backend_->register_device_memory(data_, bytes);  // throws when the HCA cannot reach device memory
    } else {
        host_.reset(bytes, device >= 0 ? numa::gpu_node(device) : -1);
        data_ = host_.get();
        mr_ = backend_->register_memory(data_, bytes);
    }
}

RegisteredFifo::~RegisteredFifo() {
    if (mr_.addr) backend_->deregister(mr_);
}

}  // namespace b200ccl::transport::rdma
