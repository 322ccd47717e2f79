#include "topo/topology.h"

#include "core/check.h"
#include "mem/cu_driver.h"

#include <algorithm>
#include <cctype>
#include <dlfcn.h>
#include <fstream>
#include <sstream>

namespace b200ccl::topo {

namespace {

// The few NVML entry points used, resolved from libnvidia-ml.so.1 at run time so that the
// library neither links against NVML nor needs it to be present.
struct Nvml {
    using Device = void*;
    struct PciInfo {  // nvmlPciInfo_t
        char busIdLegacy[16];
        unsigned int domain, bus, device, pciDeviceId, pciSubSystemId;
        char busId[32];
    };
    void* lib = nullptr;
    int (*Init)() = nullptr;
    int (*Shutdown)() = nullptr;
    int (*DeviceGetHandleByPciBusId)(const char*, Device*) = nullptr;
    int (*DeviceGetNvLinkState)(Device, unsigned, unsigned*) = nullptr;
    int (*DeviceGetNvLinkVersion)(Device, unsigned, unsigned*) = nullptr;
    int (*DeviceGetNvLinkRemoteDeviceType)(Device, unsigned, unsigned*) = nullptr;
    bool ok = false;

    Nvml() {
        lib = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
        if (!lib) return;
        auto sym = [&](const char* n) { return dlsym(lib, n); };
        Init = reinterpret_cast<int (*)()>(sym("nvmlInit_v2"));
        Shutdown = reinterpret_cast<int (*)()>(sym("nvmlShutdown"));
        DeviceGetHandleByPciBusId =
            reinterpret_cast<int (*)(const char*, Device*)>(sym("nvmlDeviceGetHandleByPciBusId_v2"));
        DeviceGetNvLinkState = reinterpret_cast<int (*)(Device, unsigned, unsigned*)>(sym("nvmlDeviceGetNvLinkState"));
        DeviceGetNvLinkVersion =
            reinterpret_cast<int (*)(Device, unsigned, unsigned*)>(sym("nvmlDeviceGetNvLinkVersion"));
        DeviceGetNvLinkRemoteDeviceType =
            reinterpret_cast<int (*)(Device, unsigned, unsigned*)>(sym("nvmlDeviceGetNvLinkRemoteDeviceType"));
        if (Init && Shutdown && DeviceGetHandleByPciBusId && DeviceGetNvLinkState && Init() == 0) ok = true;
    }
    ~Nvml() {
        if (ok) Shutdown();
        if (lib) dlclose(lib);
    }
};

constexpr unsigned kNvmlMaxLinks = 18;
constexpr unsigned kRemoteTypeSwitch = 2;  // NVML_NVLINK_DEVICE_TYPE_SWITCH

}  // namespace

int gpu_numa_node_from_sysfs(const std::string& pci_bus_id, const std::string& sysfs_root) {
    std::string id = pci_bus_id;
    std::transform(id.begin(), id.end(), id.begin(), [](unsigned char c) { return std::tolower(c); });
    // CUDA prints 8-digit domains on some systems; sysfs uses 4.
    if (id.size() > 12 && id.find(':') == 8) id = id.substr(4);
    std::ifstream f(sysfs_root + "/bus/pci/devices/" + id + "/numa_node");
    int node = -1;
    if (!(f >> node) || node < 0) return 0;
    return node;
}

TopologyReport discover(const std::vector<int>& devices) {
    TopologyReport rep;
    Nvml nvml;
    rep.nvml_loaded = nvml.ok;
    std::ostringstream os;
    for (int d : devices) {
        GpuInfo g;
        g.device = d;
        cudaDeviceProp prop{};
        if (cudaGetDeviceProperties(&prop, d) == cudaSuccess) {
            g.name = prop.name;
            g.sm_count = prop.multiProcessorCount;
            g.cc_major = prop.major;
            g.cc_minor = prop.minor;
        } else {
            (void)cudaGetLastError();
        }
        char bus[32] = {0};
        if (cudaDeviceGetPCIBusId(bus, sizeof(bus), d) == cudaSuccess) g.pci_bus_id = bus;
        else (void)cudaGetLastError();
        g.numa_node = g.pci_bus_id.empty() ? 0 : gpu_numa_node_from_sysfs(g.pci_bus_id);
        g.multicast = cu::device_attribute(d, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, 0) != 0;
        if (nvml.ok && !g.pci_bus_id.empty()) {
            Nvml::Device h = nullptr;
            if (nvml.DeviceGetHandleByPciBusId(g.pci_bus_id.c_str(), &h) == 0) {
                for (unsigned link = 0; link < kNvmlMaxLinks; ++link) {
                    unsigned active = 0;
                    if (nvml.DeviceGetNvLinkState(h, link, &active) != 0 || !active) continue;
                    ++g.nvlink_active;
                    unsigned ver = 0;
                    if (nvml.DeviceGetNvLinkVersion && nvml.DeviceGetNvLinkVersion(h, link, &ver) == 0)
                        g.nvlink_version = static_cast<int>(ver);
                    unsigned type = 0;
                    if (nvml.DeviceGetNvLinkRemoteDeviceType &&
                        nvml.DeviceGetNvLinkRemoteDeviceType(h, link, &type) == 0 && type == kRemoteTypeSwitch)
                        ++g.nvlink_to_switch;
                }
            }
        }
        os << "gpu " << d << ": " << (g.name.empty() ? "?" : g.name) << " pci " << g.pci_bus_id << " numa " << g.numa_node
           << " sms " << g.sm_count << " nvlinks " << g.nvlink_active << " (to switch " << g.nvlink_to_switch
           << ", version id " << g.nvlink_version << ") multicast " << (g.multicast ? "yes" : "no") << "\n";
        rep.gpus.push_back(g);
    }
    const std::size_t n = devices.size();
    rep.peer_access.assign(n, std::vector<int>(n, 1));
    rep.native_atomics.assign(n, std::vector<int>(n, 1));
    rep.all_pairs_peer = true;
    for (std::size_t a = 0; a < n; ++a) {
        for (std::size_t b = 0; b < n; ++b) {
            if (a == b) continue;
            int can = 0, atom = 0;
            if (cudaDeviceCanAccessPeer(&can, devices[a], devices[b]) != cudaSuccess) (void)cudaGetLastError();
            if (cudaDeviceGetP2PAttribute(&atom, cudaDevP2PAttrNativeAtomicSupported, devices[a], devices[b]) != cudaSuccess)
                (void)cudaGetLastError();
            rep.peer_access[a][b] = can;
            rep.native_atomics[a][b] = atom;
            rep.all_pairs_peer &= can != 0;
        }
    }
    rep.nvswitch = !rep.gpus.empty();
    for (const auto& g : rep.gpus) rep.nvswitch &= g.nvlink_active > 0 && g.nvlink_to_switch == g.nvlink_active;
    os << "peer access: " << (rep.all_pairs_peer ? "all pairs" : "partial") << "; nvswitch " << (rep.nvswitch ? "yes" : "no")
       << "; nvml " << (rep.nvml_loaded ? "loaded" : "unavailable") << "\n";
    rep.text = os.str();
    return rep;
}

}  // namespace b200ccl::topo
