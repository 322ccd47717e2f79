#include "mem/cu_driver.h"

#include <cuda_runtime.h>

#include <stdexcept>

namespace b200ccl::cu {

namespace {

template <typename Fn>
bool resolve(const char* name, Fn* out) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    const cudaError_t st = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
    if (st != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
        (void)cudaGetLastError();
        *out = nullptr;
        return false;
    }
    *out = reinterpret_cast<Fn>(p);
    return true;
}

Api load() {
    Api a;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        (void)cudaGetLastError();
        a.why = "no CUDA device or driver";
        return a;
    }
    bool ok = true;
    ok &= resolve("cuGetErrorString", &a.GetErrorString);
    ok &= resolve("cuDeviceGet", &a.DeviceGet);
    ok &= resolve("cuDeviceGetAttribute", &a.DeviceGetAttribute);
    ok &= resolve("cuMemCreate", &a.MemCreate);
    ok &= resolve("cuMemRelease", &a.MemRelease);
    ok &= resolve("cuMemAddressReserve", &a.MemAddressReserve);
    ok &= resolve("cuMemAddressFree", &a.MemAddressFree);
    ok &= resolve("cuMemMap", &a.MemMap);
    ok &= resolve("cuMemUnmap", &a.MemUnmap);
    ok &= resolve("cuMemSetAccess", &a.MemSetAccess);
    ok &= resolve("cuMemGetAllocationGranularity", &a.MemGetAllocationGranularity);
    ok &= resolve("cuMemExportToShareableHandle", &a.MemExportToShareableHandle);
    ok &= resolve("cuMemImportFromShareableHandle", &a.MemImportFromShareableHandle);
    a.vmm_ok = ok;
    if (!ok) a.why = "driver does not export the cuMem* virtual memory API";
    bool mc = ok;
    mc &= resolve("cuMulticastCreate", &a.MulticastCreate);
    mc &= resolve("cuMulticastAddDevice", &a.MulticastAddDevice);
    mc &= resolve("cuMulticastBindMem", &a.MulticastBindMem);
    mc &= resolve("cuMulticastUnbind", &a.MulticastUnbind);
    mc &= resolve("cuMulticastGetGranularity", &a.MulticastGetGranularity);
    a.multicast_ok = mc;
    return a;
}

}  // namespace

const Api& api() {
    static const Api a = load();
    return a;
}

std::string error_string(CUresult r) {
    const char* s = nullptr;
    if (api().GetErrorString && api().GetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
    return "CUresult " + std::to_string(static_cast<int>(r));
}

void check(CUresult r, const char* what) {
    if (r != CUDA_SUCCESS) throw std::runtime_error(std::string(what) + ": " + error_string(r));
}

int device_attribute(int device, CUdevice_attribute attr, int dflt) {
    const Api& a = api();
    if (!a.DeviceGet || !a.DeviceGetAttribute) return dflt;
    CUdevice dev;
    if (a.DeviceGet(&dev, device) != CUDA_SUCCESS) return dflt;
    int v = dflt;
    if (a.DeviceGetAttribute(&v, attr, dev) != CUDA_SUCCESS) return dflt;
    return v;
}

}  // namespace b200ccl::cu
