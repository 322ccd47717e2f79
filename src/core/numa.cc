#include "core/numa.h"

#include "topo/topology.h"

#include <cuda_runtime.h>

#include <fstream>
#include <sched.h>
#include <sstream>
#include <sys/syscall.h>
#include <unistd.h>

namespace b200ccl::numa {

namespace {
constexpr int kMpolDefault = 0;
constexpr int kMpolPreferred = 1;
}  // namespace

int gpu_node(int device) {
    char bus[32] = {0};
    if (cudaDeviceGetPCIBusId(bus, sizeof(bus), device) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return topo::gpu_numa_node_from_sysfs(bus);
}

bool set_preferred_node(int node) {
    if (node < 0 || node >= 1024) return false;
    unsigned long mask[16] = {0};
    mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
    return syscall(SYS_set_mempolicy, kMpolPreferred, mask, sizeof(mask) * 8) == 0;
}

void clear_preferred_node() { (void)syscall(SYS_set_mempolicy, kMpolDefault, nullptr, 0); }

std::vector<int> parse_cpulist(const std::string& text) {
    std::vector<int> cpus;
    std::stringstream ss(text);
    std::string item;
    while (std::getline(ss, item, ',')) {
        if (item.empty()) continue;
        const auto dash = item.find('-');
        try {
            if (dash == std::string::npos) {
                cpus.push_back(std::stoi(item));
            } else {
                const int lo = std::stoi(item.substr(0, dash)), hi = std::stoi(item.substr(dash + 1));
                for (int c = lo; c <= hi; ++c) cpus.push_back(c);
            }
        } catch (...) {
            return {};
        }
    }
    return cpus;
}

std::vector<int> node_cpus(int node, const std::string& sysfs_root) {
    std::ifstream f(sysfs_root + "/devices/system/node/node" + std::to_string(node) + "/cpulist");
    std::string line;
    if (!std::getline(f, line)) return {};
    return parse_cpulist(line);
}

bool pin_current_thread_to_node(int node) {
    if (node < 0) return false;
    const std::vector<int> cpus = node_cpus(node);
    if (cpus.empty()) return false;
    cpu_set_t set;
    CPU_ZERO(&set);
    for (int c : cpus)
        if (c >= 0 && c < CPU_SETSIZE) CPU_SET(c, &set);
    return sched_setaffinity(0, sizeof(set), &set) == 0;
}

}  // namespace b200ccl::numa
