// NUMA placement without libnuma: node of a GPU from sysfs, preferred-node memory policy through
// the set_mempolicy system call, thread pinning through sched_setaffinity and the node's cpulist.
//
// Parity: nano-nccl src/core/numa.h:6-14 / numa.cu:18-68 (gpu_numa_node, numa_set_prefer,
// pin_current_thread_to_numa_node), which link libnuma; the behaviour when NUMA information is
// missing is the same (node 0, calls become no-ops).
#pragma once

#include <string>
#include <vector>

namespace b200ccl::numa {

int gpu_node(int device);  // 0 when unknown
// Memory allocated by this thread afterwards prefers `node`. Returns false if the kernel refused.
bool set_preferred_node(int node);
void clear_preferred_node();
// CPUs of a node, parsed from <sysfs_root>/devices/system/node/node<N>/cpulist ("0-23,48-71").
std::vector<int> node_cpus(int node, const std::string& sysfs_root = "/sys");
std::vector<int> parse_cpulist(const std::string& text);
// Restricts the calling thread to the node's CPUs. No-op (returns false) when the list is empty.
bool pin_current_thread_to_node(int node);

// RAII: prefer `node` for allocations made in this scope.
class PreferNode {
public:
    explicit PreferNode(int node) : active_(node >= 0 && set_preferred_node(node)) {}
    ~PreferNode() { if (active_) clear_preferred_node(); }
    PreferNode(const PreferNode&) = delete;
    PreferNode& operator=(const PreferNode&) = delete;
private:
    bool active_;
};

}  // namespace b200ccl::numa
