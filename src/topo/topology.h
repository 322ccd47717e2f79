// Run-time discovery of what connects the GPUs of this process: NUMA node per GPU (sysfs),
// NVLink links per GPU with the kind of device at the far end (NVML, loaded with dlopen), the
// CUDA peer-access matrix with native-atomics support, and NVSwitch multicast support.
//
// Parity: nano-nccl src/core/numa.cu:18-40 (GPU → NUMA node from sysfs, fallback 0) and
// src/transport/p2p/p2p_topology.cu:16-103 (NvmlSession, has_active_direct_nvlink). The
// reference accepts an NVLink only when its remote PCI device IS the peer GPU; through NVSwitch
// the remote device is the switch, so here a link to a switch counts for every peer.
#pragma once

#include <string>
#include <vector>

namespace b200ccl::topo {

struct GpuInfo {
    int device = 0;
    std::string name;
    std::string pci_bus_id;
    int numa_node = 0;           // 0 when sysfs has no answer (or says -1)
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    int nvlink_active = 0;       // active links (0 when NVML is unavailable)
    int nvlink_to_switch = 0;    // of those, links whose far end is an NVSwitch
    int nvlink_version = 0;
    bool multicast = false;      // CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED
};

struct TopologyReport {
    std::vector<GpuInfo> gpus;
    std::vector<std::vector<int>> peer_access;     // [a][b] 1 if a can map b's memory
    std::vector<std::vector<int>> native_atomics;  // [a][b] 1 if atomics over the link are native
    bool nvml_loaded = false;
    bool all_pairs_peer = false;
    bool nvswitch = false;       // every GPU has links and all of them end at a switch
    std::string text;            // human-readable, one line per fact
};

// Never throws for missing NVML/sysfs; missing facts are left at their defaults.
TopologyReport discover(const std::vector<int>& devices);

// GPU → NUMA node; `sysfs_root` is replaceable for tests. Returns 0 when unknown.
int gpu_numa_node_from_sysfs(const std::string& pci_bus_id, const std::string& sysfs_root = "/sys");

}  // namespace b200ccl::topo
