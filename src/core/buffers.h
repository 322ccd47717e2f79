// RAII owners of the memory kinds the library uses: device, pinned host, mapped host (zero-copy,
// visible to every GPU, optionally placed on a NUMA node) and mapped 64/32-bit counter arrays.
//
// Parity: nano-nccl src/core/buffer.h:33-214 (DeviceBuffer, PinnedBuffer, MappedBuffer,
// MappedU64Array / MappedU32Array). The /dev/shm-backed RegisteredMappedBuffer of the reference
// (buffer.h:132-166) is unused by its product paths and has no counterpart here.
#pragma once

#include "core/check.h"
#include "core/numa.h"

#include <cstdlib>
#include <cstring>
#include <new>
#include <utility>

namespace b200ccl {

template <typename T>
class DeviceBuffer {
public:
    DeviceBuffer() = default;
    DeviceBuffer(int device, std::size_t count) { reset(device, count); }
    ~DeviceBuffer() { release(); }
    DeviceBuffer(DeviceBuffer&& o) noexcept { swap(o); }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept { if (this != &o) { release(); swap(o); } return *this; }
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    void reset(int device, std::size_t count) {
        release();
        if (count == 0) return;
        DeviceGuard guard(device);
        B2_CUDA(cudaMalloc(reinterpret_cast<void**>(&ptr_), count * sizeof(T)));
        device_ = device;
        count_ = count;
    }
    void zero() {
        if (!ptr_) return;
        DeviceGuard guard(device_);
        B2_CUDA(cudaMemset(ptr_, 0, count_ * sizeof(T)));
    }
    T* get() const { return ptr_; }
    std::size_t count() const { return count_; }
    int device() const { return device_; }
private:
    void release() {
        if (ptr_) {
            int prev = 0;
            cudaGetDevice(&prev);
            cudaSetDevice(device_);
            cudaFree(ptr_);
            cudaSetDevice(prev);
        }
        ptr_ = nullptr; count_ = 0;
    }
    void swap(DeviceBuffer& o) { std::swap(ptr_, o.ptr_); std::swap(count_, o.count_); std::swap(device_, o.device_); }
    T* ptr_ = nullptr;
    std::size_t count_ = 0;
    int device_ = 0;
};

// Host memory that every GPU can address (cudaHostAllocMapped | Portable). With a NUMA node the
// pages are placed there (the receiver's node for a FIFO, as communicator.cu:915-934 does).
template <typename T>
class MappedBuffer {
public:
    MappedBuffer() = default;
    explicit MappedBuffer(std::size_t count, int numa_node = -1) { reset(count, numa_node); }
    ~MappedBuffer() { release(); }
    MappedBuffer(MappedBuffer&& o) noexcept { swap(o); }
    MappedBuffer& operator=(MappedBuffer&& o) noexcept { if (this != &o) { release(); swap(o); } return *this; }
    MappedBuffer(const MappedBuffer&) = delete;
    MappedBuffer& operator=(const MappedBuffer&) = delete;
    void reset(std::size_t count, int numa_node = -1) {
        release();
        if (count == 0) return;
        numa::PreferNode prefer(numa_node);
        const cudaError_t st = cudaHostAlloc(reinterpret_cast<void**>(&ptr_), count * sizeof(T),
                                             cudaHostAllocMapped | cudaHostAllocPortable);
        if (st == cudaErrorNoDevice || st == cudaErrorInsufficientDriver) {
            // No GPU in this process (host-only tests of proxies and edge wiring): ordinary memory.
            (void)cudaGetLastError();
            if (posix_memalign(reinterpret_cast<void**>(&ptr_), 4096, count * sizeof(T)) != 0) throw std::bad_alloc();
            host_only_ = true;
        } else {
            B2_CUDA(st);
        }
        std::memset(ptr_, 0, count * sizeof(T));  // also touches the pages under the preferred policy
        count_ = count;
    }
    T* get() const { return ptr_; }            // valid on host and, under unified addressing, on every GPU
    T& operator[](std::size_t i) const { return ptr_[i]; }
    std::size_t count() const { return count_; }
    bool host_only() const { return host_only_; }
private:
    void release() {
        if (ptr_) {
            if (host_only_) std::free(ptr_);
            else cudaFreeHost(ptr_);
        }
        ptr_ = nullptr; count_ = 0; host_only_ = false;
    }
    void swap(MappedBuffer& o) { std::swap(ptr_, o.ptr_); std::swap(count_, o.count_); std::swap(host_only_, o.host_only_); }
    T* ptr_ = nullptr;
    std::size_t count_ = 0;
    bool host_only_ = false;
};

using MappedU64Array = MappedBuffer<unsigned long long>;
using MappedU32Array = MappedBuffer<unsigned int>;

template <typename T>
class PinnedBuffer {
public:
    PinnedBuffer() = default;
    explicit PinnedBuffer(std::size_t count) {
        if (count) B2_CUDA(cudaMallocHost(reinterpret_cast<void**>(&ptr_), count * sizeof(T)));
        count_ = count;
    }
    ~PinnedBuffer() { if (ptr_) cudaFreeHost(ptr_); }
    PinnedBuffer(PinnedBuffer&& o) noexcept { std::swap(ptr_, o.ptr_); std::swap(count_, o.count_); }
    PinnedBuffer& operator=(PinnedBuffer&& o) noexcept { std::swap(ptr_, o.ptr_); std::swap(count_, o.count_); return *this; }
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
    T* get() const { return ptr_; }
    std::size_t count() const { return count_; }
private:
    T* ptr_ = nullptr;
    std::size_t count_ = 0;
};

}  // namespace b200ccl
