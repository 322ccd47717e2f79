// Registration of ordinary device buffers of a multi-process communicator: every process exports
// the allocation that holds its buffer (CUDA IPC memory handle + offset of the buffer inside it),
// the processes exchange these records, and each maps its peers' allocations. Afterwards peers
// load and store the buffer directly, so collectives on it need no staging copy. (No multicast
// alias: only memory created through the virtual memory API can be bound to NVSwitch multicast.)
//
// The reference maps neighbours' cudaMalloc FIFOs inside one process only
// (src/transport/p2p/p2p_fifo.cu:103-137); sharing user buffers between processes is new here.
#pragma once

#include "b200ccl/bootstrap.h"
#include "mem/symmetric.h"

#include <cstddef>
#include <memory>
#include <vector>

namespace b200ccl::mem {

class IpcWindow {
public:
    ~IpcWindow();
    IpcWindow(const IpcWindow&) = delete;
    IpcWindow& operator=(const IpcWindow&) = delete;
    // Collective over all processes. `local_ptrs[i]` / `bytes` describe local rank i's buffer.
    // Throws on every process when any process cannot export or map (error consensus).
    static std::unique_ptr<IpcWindow> create(const GroupDesc& group, const std::vector<void*>& local_ptrs, std::size_t bytes);
    std::size_t bytes() const { return bytes_; }
    void* rank_ptr(int g) const { return rank_ptr_[g]; }

private:
    IpcWindow() = default;
    std::size_t bytes_ = 0;
    std::vector<void*> rank_ptr_;
    struct Opened { int device; void* base; };
    std::vector<Opened> opened_;  // mappings to close
};

}  // namespace b200ccl::mem
