#include "mem/symmetric.h"

#include "core/check.h"
#include "core/env.h"
#include "mem/cu_driver.h"

#include <algorithm>
#include <cstring>
#include <stdexcept>
#include <unistd.h>

namespace b200ccl::mem {

namespace {

std::size_t align_up(std::size_t v, std::size_t a) { return (v + a - 1) / a * a; }

CUmemAllocationProp device_prop(int device) {
    CUmemAllocationProp prop;
    std::memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

CUmulticastObjectProp multicast_prop(int ndevices, std::size_t size) {
    CUmulticastObjectProp prop;
    std::memset(&prop, 0, sizeof(prop));
    prop.numDevices = static_cast<unsigned>(ndevices);
    prop.size = size;
    prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

void set_access(CUdeviceptr va, std::size_t size, const std::vector<int>& devices) {
    std::vector<CUmemAccessDesc> descs(devices.size());
    for (std::size_t i = 0; i < devices.size(); ++i) {
        std::memset(&descs[i], 0, sizeof(CUmemAccessDesc));
        descs[i].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        descs[i].location.id = devices[i];
        descs[i].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    }
    cu::check(cu::api().MemSetAccess(va, size, descs.data(), descs.size()), "cuMemSetAccess");
}

void touch_context(int device) {
    B2_CUDA(cudaSetDevice(device));
    B2_CUDA(cudaFree(nullptr));
}

}  // namespace

bool enable_all_peer_access(const std::vector<int>& devices, std::string* why) {
    for (int a : devices) {
        for (int b : devices) {
            if (a == b) continue;
            int can = 0;
            B2_CUDA(cudaDeviceCanAccessPeer(&can, a, b));
            if (!can) {
                if (why)
                    *why = "device " + std::to_string(a) + " cannot access device " + std::to_string(b);
                return false;
            }
        }
    }
    for (int a : devices) {
        DeviceGuard guard(a);
        for (int b : devices) {
            if (a == b) continue;
            const cudaError_t st = cudaDeviceEnablePeerAccess(b, 0);
            if (st == cudaErrorPeerAccessAlreadyEnabled) {
                (void)cudaGetLastError();
            } else if (st != cudaSuccess) {
                if (why) *why = std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(st);
                (void)cudaGetLastError();
                return false;
            }
        }
    }
    return true;
}

SymmetricAllocator::SymmetricAllocator(GroupDesc group) : group_(std::move(group)) {
    B2_REQUIRE(group_.nranks >= 1, "symmetric group: need at least one rank");
    B2_REQUIRE(!group_.local.empty(), "symmetric group: this process owns no rank");
    for (const auto& l : group_.local) {
        if (std::find(local_devices_.begin(), local_devices_.end(), l.device) == local_devices_.end())
            local_devices_.push_back(l.device);
    }
    const bool multiprocess = group_.bootstrap != nullptr;
    const cu::Api& a = cu::api();
    use_vmm_ = a.vmm_ok && env::get_bool("B200CCL_VMM", true);
    if (use_vmm_) {
        for (int d : local_devices_) {
            if (!cu::device_attribute(d, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, 0) ||
                !cu::device_attribute(d, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, 0))
                use_vmm_ = false;
        }
    }
    if (multiprocess) {
        // Every process must take the same path.
        const std::string err = group_.bootstrap->error_consensus(
            use_vmm_ ? "" : "virtual memory management unavailable: " + a.why);
        if (!err.empty())
            throw std::runtime_error("multi-process communicator needs shareable allocations; " + err);
    }
    // Multicast: asked for, exposed by the driver, supported by every local device, one device
    // per rank (a device cannot be added to a multicast object twice, so loopback has none).
    multicast_ = false;
    if (!group_.want_multicast) mc_reason_ = "disabled by configuration";
    else if (!env::get_bool("B200CCL_NVLS", true, "B200CCL_NVLS_ENABLE")) mc_reason_ = "disabled by B200CCL_NVLS=0";
    else if (!use_vmm_) mc_reason_ = "needs virtual memory management";
    else if (!a.multicast_ok) mc_reason_ = "driver does not export cuMulticast*";
    else if (group_.loopback) mc_reason_ = "loopback emulation shares one device";
    else if (group_.nranks < 2) mc_reason_ = "single rank";
    else {
        multicast_ = true;
        for (int d : local_devices_) {
            if (!cu::device_attribute(d, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, 0)) {
                multicast_ = false;
                mc_reason_ = "device " + std::to_string(d) + " reports no multicast support";
            }
        }
    }
    if (multiprocess) {
        const std::string err = group_.bootstrap->error_consensus(multicast_ ? "" : mc_reason_);
        if (!err.empty()) {
            multicast_ = false;
            if (mc_reason_.empty()) mc_reason_ = "a peer process cannot use multicast (" + err + ")";
        }
    }
}

std::unique_ptr<SymmetricRegion> SymmetricAllocator::allocate(std::size_t bytes, const char* label) {
    B2_REQUIRE(bytes > 0, "symmetric allocation of zero bytes");
    auto region = use_vmm_ ? allocate_vmm(bytes, label) : allocate_plain(bytes);
    // Zero the local copies, then make sure every process has done so before anyone uses it.
    for (const auto& l : group_.local) {
        DeviceGuard guard(l.device);
        B2_CUDA(cudaMemset(region->rank_va_[l.global_rank], 0, region->bytes_));
        B2_CUDA(cudaDeviceSynchronize());
    }
    if (group_.bootstrap) group_.bootstrap->barrier();
    log_info("symmetric region '%s': %zu bytes per rank, %s, multicast %s", label, region->bytes_,
             region->vmm_ ? "vmm" : "cudaMalloc", region->mc_va_ ? "bound" : "none");
    return region;
}

std::unique_ptr<SymmetricRegion> SymmetricAllocator::allocate_plain(std::size_t bytes) {
    // Single process, no VMM: plain allocations reached through peer access.
    std::unique_ptr<SymmetricRegion> r(new SymmetricRegion());
    r->bytes_ = align_up(bytes, 256);
    r->rank_va_.assign(group_.nranks, nullptr);
    r->owner_device_.assign(group_.nranks, -1);
    for (const auto& l : group_.local) {
        DeviceGuard guard(l.device);
        void* p = nullptr;
        B2_CUDA(cudaMalloc(&p, r->bytes_));
        r->rank_va_[l.global_rank] = p;
        r->owner_device_[l.global_rank] = l.device;
    }
    return r;
}

std::unique_ptr<SymmetricRegion> SymmetricAllocator::allocate_vmm(std::size_t bytes, const char* label) {
    const cu::Api& a = cu::api();
    const int n = group_.nranks;
    Bootstrap* bs = group_.bootstrap;
    std::unique_ptr<SymmetricRegion> r(new SymmetricRegion());
    r->vmm_ = true;
    r->rank_va_.assign(n, nullptr);
    r->handles_.assign(n, 0);
    r->handle_valid_.assign(n, false);
    r->owner_device_.assign(n, -1);

    // Size: a multiple of both the allocation and the multicast granularity.
    std::size_t gran = 0;
    {
        CUmemAllocationProp prop = device_prop(group_.local[0].device);
        cu::check(a.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
                  "cuMemGetAllocationGranularity");
    }
    if (multicast_) {
        CUmulticastObjectProp mp = multicast_prop(n, align_up(bytes, gran));
        std::size_t mg = 0;
        if (a.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS && mg)
            gran = std::max(gran, mg);
    }
    const std::size_t size = align_up(bytes, gran);
    r->bytes_ = size;

    // Physical memory for the local ranks.
    for (const auto& l : group_.local) {
        touch_context(l.device);
        CUmemAllocationProp prop = device_prop(l.device);
        cu::check(a.MemCreate(&r->handles_[l.global_rank], size, &prop, 0), "cuMemCreate");
        r->handle_valid_[l.global_rank] = true;
    }

    // Handles of the other processes' ranks.
    if (bs) {
        std::vector<int> my_fds;
        for (const auto& l : group_.local) {
            int fd = -1;
            cu::check(a.MemExportToShareableHandle(&fd, r->handles_[l.global_rank],
                                                   CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
                      "cuMemExportToShareableHandle");
            my_fds.push_back(fd);
        }
        // Global ranks are contiguous per process, ordered by bootstrap rank.
        std::vector<int> counts(bs->size());
        const int mine = static_cast<int>(group_.local.size());
        bs->allgather(&mine, counts.data(), sizeof(int));
        auto all = bs->exchange_fds(my_fds);
        int g = 0;
        for (int p = 0; p < bs->size(); ++p) {
            for (int k = 0; k < counts[p]; ++k, ++g) {
                const int fd = all[p][k];
                if (p != bs->rank()) {
                    cu::check(a.MemImportFromShareableHandle(
                                  &r->handles_[g], reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
                              "cuMemImportFromShareableHandle");
                    r->handle_valid_[g] = true;
                }
                if (fd >= 0) ::close(fd);
            }
        }
        for (int fd : my_fds) ::close(fd);
    }

    // Map every rank's memory for every local device.
    for (int g = 0; g < n; ++g) {
        CUdeviceptr va = 0;
        cu::check(a.MemAddressReserve(&va, size, gran, 0, 0), "cuMemAddressReserve");
        cu::check(a.MemMap(va, size, 0, r->handles_[g], 0), "cuMemMap");
        set_access(va, size, local_devices_);
        r->rank_va_[g] = reinterpret_cast<void*>(va);
    }

    if (multicast_) try_bind_multicast(*r, label);
    return r;
}

void SymmetricAllocator::try_bind_multicast(SymmetricRegion& r, const char* label) {
    const cu::Api& a = cu::api();
    Bootstrap* bs = group_.bootstrap;
    const int n = group_.nranks;
    const std::size_t size = r.bytes_;
    std::string err;
    auto agree = [&](const std::string& e) -> bool {  // true when every process is fine
        const std::string all = bs ? bs->error_consensus(e) : e;
        if (!all.empty()) {
            log_warn("multicast for region '%s' unavailable: %s", label, all.c_str());
            mc_reason_ = all;
        }
        return all.empty();
    };
    auto drop = [&]() {
        for (int d : r.mc_bound_devices_) {
            CUdevice dev;
            if (a.DeviceGet(&dev, d) == CUDA_SUCCESS) a.MulticastUnbind(r.mc_handle_, dev, 0, size);
        }
        r.mc_bound_devices_.clear();
        if (r.mc_valid_) a.MemRelease(r.mc_handle_);
        r.mc_valid_ = false;
        multicast_ = false;  // later regions do not try again
    };

    // 1. The first process creates the object and shares it.
    const bool root = !bs || bs->rank() == 0;
    int export_fd = -1;
    if (root) {
        CUmulticastObjectProp mp = multicast_prop(n, size);
        const CUresult st = a.MulticastCreate(&r.mc_handle_, &mp);
        if (st != CUDA_SUCCESS) err = "cuMulticastCreate: " + cu::error_string(st);
        else r.mc_valid_ = true;
        if (r.mc_valid_ && bs) {
            const CUresult se = a.MemExportToShareableHandle(&export_fd, r.mc_handle_,
                                                             CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
            if (se != CUDA_SUCCESS) err = "export multicast handle: " + cu::error_string(se);
        }
    }
    if (!agree(err)) { if (export_fd >= 0) ::close(export_fd); drop(); return; }
    if (bs) {
        auto all = bs->exchange_fds({export_fd});
        if (!root) {
            const int fd = all[0][0];
            const CUresult si = a.MemImportFromShareableHandle(
                &r.mc_handle_, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            if (si != CUDA_SUCCESS) err = "import multicast handle: " + cu::error_string(si);
            else r.mc_valid_ = true;
        }
        for (auto& v : all) for (int fd : v) if (fd >= 0) ::close(fd);
        if (export_fd >= 0) ::close(export_fd);
        if (!agree(err)) { drop(); return; }
    }

    // 2. Every device joins; only when all have joined may memory be bound.
    for (const auto& l : group_.local) {
        CUdevice dev;
        CUresult st = a.DeviceGet(&dev, l.device);
        if (st == CUDA_SUCCESS) st = a.MulticastAddDevice(r.mc_handle_, dev);
        if (st != CUDA_SUCCESS) { err = "cuMulticastAddDevice: " + cu::error_string(st); break; }
    }
    if (!agree(err)) { drop(); return; }

    // 3. Bind the local ranks' memory at offset 0.
    for (const auto& l : group_.local) {
        touch_context(l.device);
        const CUresult st = a.MulticastBindMem(r.mc_handle_, 0, r.handles_[l.global_rank], 0, size, 0);
        if (st != CUDA_SUCCESS) { err = "cuMulticastBindMem: " + cu::error_string(st); break; }
        r.mc_bound_devices_.push_back(l.device);
    }
    if (!agree(err)) { drop(); return; }

    // 4. Map the multicast object.
    CUdeviceptr va = 0;
    std::size_t gran = 2u << 20;
    {
        CUmulticastObjectProp mp = multicast_prop(n, size);
        std::size_t mg = 0;
        if (a.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS && mg)
            gran = mg;
    }
    CUresult st = a.MemAddressReserve(&va, size, gran, 0, 0);
    if (st == CUDA_SUCCESS) {
        st = a.MemMap(va, size, 0, r.mc_handle_, 0);
        if (st == CUDA_SUCCESS) {
            try {
                set_access(va, size, local_devices_);
                r.mc_va_ = reinterpret_cast<void*>(va);
            } catch (const std::exception& e) {
                err = e.what();
                a.MemUnmap(va, size);
                a.MemAddressFree(va, size);
            }
        } else {
            err = "cuMemMap(multicast): " + cu::error_string(st);
            a.MemAddressFree(va, size);
        }
    } else {
        err = "cuMemAddressReserve(multicast): " + cu::error_string(st);
    }
    if (!agree(err)) {
        if (r.mc_va_) {
            a.MemUnmap(reinterpret_cast<CUdeviceptr>(r.mc_va_), size);
            a.MemAddressFree(reinterpret_cast<CUdeviceptr>(r.mc_va_), size);
            r.mc_va_ = nullptr;
        }
        drop();
    }
}

SymmetricRegion::~SymmetricRegion() {
    const cu::Api& a = cu::api();
    if (vmm_) {
        if (mc_va_) {
            a.MemUnmap(reinterpret_cast<CUdeviceptr>(mc_va_), bytes_);
            a.MemAddressFree(reinterpret_cast<CUdeviceptr>(mc_va_), bytes_);
        }
        for (int d : mc_bound_devices_) {
            CUdevice dev;
            if (a.DeviceGet(&dev, d) == CUDA_SUCCESS) a.MulticastUnbind(mc_handle_, dev, 0, bytes_);
        }
        if (mc_valid_) a.MemRelease(mc_handle_);
        for (std::size_t g = 0; g < rank_va_.size(); ++g) {
            if (rank_va_[g]) {
                a.MemUnmap(reinterpret_cast<CUdeviceptr>(rank_va_[g]), bytes_);
                a.MemAddressFree(reinterpret_cast<CUdeviceptr>(rank_va_[g]), bytes_);
            }
            if (handle_valid_[g]) a.MemRelease(handles_[g]);
        }
    } else {
        for (std::size_t g = 0; g < rank_va_.size(); ++g) {
            if (rank_va_[g] && owner_device_[g] >= 0) {
                int prev = 0;
                cudaGetDevice(&prev);
                cudaSetDevice(owner_device_[g]);
                cudaFree(rank_va_[g]);
                cudaSetDevice(prev);
            }
        }
    }
}

}  // namespace b200ccl::mem
