#include "mem/ipc_window.h"

#include "core/check.h"
#include "mem/cu_driver.h"

#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

namespace b200ccl::mem {

namespace {

struct Record {
    cudaIpcMemHandle_t handle;
    unsigned long long offset;  // of the buffer inside the exported allocation
    unsigned long long bytes;
    int valid;
    int pad;
};

// Base address of the allocation that contains `p` (IPC handles name whole allocations).
void* allocation_base(void* p) {
    using Fn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
        (void)cudaGetLastError();
        throw std::runtime_error("cuMemGetAddressRange is unavailable");
    }
    CUdeviceptr base = 0;
    size_t size = 0;
    cu::check(reinterpret_cast<Fn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(p)), "cuMemGetAddressRange");
    return reinterpret_cast<void*>(base);
}

// An allocation may hold several registered buffers (framework allocators carve tensors out of
// large segments). Each exported allocation is mapped once per process and reference-counted.
struct Mapping {
    void* base = nullptr;
    int refs = 0;
};
std::mutex g_map_mutex;
std::map<std::string, Mapping> g_mappings;  // key: raw bytes of the IPC handle

void* open_shared(const cudaIpcMemHandle_t& h) {
    const std::string key(reinterpret_cast<const char*>(&h), sizeof(h));
    std::lock_guard<std::mutex> lock(g_map_mutex);
    Mapping& m = g_mappings[key];
    if (m.refs == 0) {
        const cudaError_t st = cudaIpcOpenMemHandle(&m.base, h, cudaIpcMemLazyEnablePeerAccess);
        if (st != cudaSuccess) {
            g_mappings.erase(key);
            throw_cuda(st, "cudaIpcOpenMemHandle", __FILE__, __LINE__);
        }
    }
    ++m.refs;
    return m.base;
}

void close_shared(void* base) {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    for (auto it = g_mappings.begin(); it != g_mappings.end(); ++it) {
        if (it->second.base == base) {
            if (--it->second.refs == 0) {
                cudaIpcCloseMemHandle(base);
                g_mappings.erase(it);
            }
            return;
        }
    }
}

}  // namespace

std::unique_ptr<IpcWindow> IpcWindow::create(const GroupDesc& group, const std::vector<void*>& local_ptrs, std::size_t bytes) {
    Bootstrap* bs = group.bootstrap;
    if (!bs) throw std::invalid_argument("buffer registration is for multi-process communicators");
    if (local_ptrs.size() != group.local.size()) throw std::invalid_argument("register: one pointer per local rank");
    const int n = group.nranks;
    std::vector<Record> mine(n), all(static_cast<std::size_t>(n) * bs->size());
    std::memset(mine.data(), 0, sizeof(Record) * n);
    std::string err;
    try {
        for (std::size_t i = 0; i < group.local.size(); ++i) {
            DeviceGuard guard(group.local[i].device);
            void* base = allocation_base(local_ptrs[i]);
            Record& r = mine[group.local[i].global_rank];
            B2_CUDA(cudaIpcGetMemHandle(&r.handle, base));
            r.offset = static_cast<unsigned long long>(static_cast<char*>(local_ptrs[i]) - static_cast<char*>(base));
            r.bytes = bytes;
            r.valid = 1;
        }
    } catch (const std::exception& e) {
        (void)cudaGetLastError();
        err = std::string("cannot export the buffer (memory from the virtual-memory allocator cannot be shared this way): ") + e.what();
    }
    std::string all_err = bs->error_consensus(err);
    if (!all_err.empty()) throw std::runtime_error("register: " + all_err);
    bs->allgather(mine.data(), all.data(), sizeof(Record) * n);

    std::unique_ptr<IpcWindow> w(new IpcWindow());
    w->bytes_ = bytes;
    w->rank_ptr_.assign(n, nullptr);
    for (std::size_t i = 0; i < group.local.size(); ++i) w->rank_ptr_[group.local[i].global_rank] = local_ptrs[i];
    try {
        DeviceGuard guard(group.local[0].device);
        for (int p = 0; p < bs->size(); ++p) {
            if (p == bs->rank()) continue;
            for (int g = 0; g < n; ++g) {
                const Record& r = all[static_cast<std::size_t>(p) * n + g];
                if (!r.valid) continue;
                if (r.bytes != bytes) throw std::runtime_error("ranks registered buffers of different sizes");
                void* base = open_shared(r.handle);
                w->opened_.push_back({group.local[0].device, base});
                w->rank_ptr_[g] = static_cast<char*>(base) + r.offset;
            }
        }
    } catch (const std::exception& e) {
        (void)cudaGetLastError();
        err = std::string("cannot map a peer's buffer: ") + e.what();
    }
    all_err = bs->error_consensus(err);
    if (!all_err.empty()) throw std::runtime_error("register: " + all_err);
    for (int g = 0; g < n; ++g)
        if (!w->rank_ptr_[g]) throw std::runtime_error("register: a rank published no buffer");
    return w;
}

IpcWindow::~IpcWindow() {
    for (const Opened& o : opened_) {
        int prev = 0;
        cudaGetDevice(&prev);
        cudaSetDevice(o.device);
        close_shared(o.base);
        cudaSetDevice(prev);
    }
    (void)cudaGetLastError();
}

}  // namespace b200ccl::mem
