// NUMA helpers against a fake sysfs tree, cpulist parsing, thread pinning; topology discovery
// must not throw on a machine without GPUs or NVML. Modelled on the NUMA-affinity case of the
// reference's tests/socket_protocol_test.cc:74-95.
#include "check.h"
#include "core/numa.h"
#include "topo/topology.h"

#include <cstdlib>
#include <fstream>
#include <sched.h>
#include <string>
#include <sys/stat.h>
#include <unistd.h>

using namespace b200ccl;

static void mkdirs(const std::string& path) {
    std::string cur;
    for (char ch : path) {
        cur += ch;
        if (ch == '/') mkdir(cur.c_str(), 0755);
    }
    mkdir(path.c_str(), 0755);
}

int main() {
    char tmpl[] = "/tmp/b2_sysfs_XXXXXX";
    const std::string root = mkdtemp(tmpl);
    mkdirs(root + "/bus/pci/devices/0000:1b:00.0");
    { std::ofstream(root + "/bus/pci/devices/0000:1b:00.0/numa_node") << "1\n"; }
    mkdirs(root + "/bus/pci/devices/0000:2c:00.0");
    { std::ofstream(root + "/bus/pci/devices/0000:2c:00.0/numa_node") << "-1\n"; }
    T_CHECK(topo::gpu_numa_node_from_sysfs("0000:1B:00.0", root) == 1);       // case-insensitive
    T_CHECK(topo::gpu_numa_node_from_sysfs("00000000:1b:00.0", root) == 1);   // 8-digit domain
    T_CHECK(topo::gpu_numa_node_from_sysfs("0000:2c:00.0", root) == 0);       // -1 → node 0
    T_CHECK(topo::gpu_numa_node_from_sysfs("0000:ff:00.0", root) == 0);       // absent → node 0

    const auto cpus = numa::parse_cpulist("0-3,8,10-11");
    T_CHECK(cpus.size() == 7 && cpus[4] == 8 && cpus.back() == 11);
    T_CHECK(numa::parse_cpulist("junk").empty());
    mkdirs(root + "/devices/system/node/node0");
    { std::ofstream(root + "/devices/system/node/node0/cpulist") << "0-1\n"; }
    T_CHECK(numa::node_cpus(0, root).size() == 2 && numa::node_cpus(7, root).empty());

    // Pinning to the real node 0 (when sysfs has it) leaves a non-empty affinity mask.
    if (!numa::node_cpus(0).empty()) {
        T_CHECK(numa::pin_current_thread_to_node(0));
        cpu_set_t set;
        T_CHECK(sched_getaffinity(0, sizeof(set), &set) == 0 && CPU_COUNT(&set) > 0);
    }
    T_CHECK(!numa::pin_current_thread_to_node(-1));
    { numa::PreferNode prefer(0); }  // must not throw whether or not the kernel accepts it

    const topo::TopologyReport rep = topo::discover({});
    T_CHECK(rep.gpus.empty() && !rep.text.empty());
    std::puts("numa/topology ok");
    return 0;
}
