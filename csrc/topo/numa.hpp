// NUMA and CPU placement helpers, read from sysfs and applied with plain system calls.
//
// Covers what the reference takes from hwloc (src/hwloc/hwloc_wrapper.hpp:42-78: NUMA node of
// a core, binding a thread's memory to a node, node-local allocation of staging buffers, PCI
// proximity of a device) and the automatic worker placement of src/common/env/env.cpp:1120-1347
// without a dependency on libhwloc: /sys/devices/system/node gives the node -> CPU lists,
// /sys/bus/pci/devices/<bdf>/numa_node the home node of a GPU or NIC, set_mempolicy / mbind
// do the binding.
#pragma once
#include <cstddef>
#include <string>
#include <vector>

namespace cclx {

class numa_info {
public:
    static numa_info& get();
    // for tests: read a tree laid out like sysfs from another root
    explicit numa_info(const std::string& sys_root);

    int node_count() const { return (int)nodes_.size(); }
    const std::vector<int>& cpus_of_node(int node) const;
    int node_of_cpu(int cpu) const;                   // -1 when unknown
    int node_of_pci(const std::string& bdf) const;    // "0000:1b:00.0"; -1 when unknown
    std::vector<int> allowed_cpus() const;            // affinity mask of the calling thread

    // worker placement for CCL_WORKER_AFFINITY=auto: the ranks of a host take disjoint cores
    // from the end of `cpus` (application threads usually sit on the first ones); an empty
    // result means that there are too few cores to pin anything
    static std::vector<int> auto_worker_cpus(const std::vector<int>& cpus, int local_rank, int local_size,
                                             int workers);

    // memory policy of the calling thread: prefer `node` (-1 restores the default)
    bool bind_thread_memory(int node) const;
    // page-aligned host buffer whose pages are placed on `node` (falls back to the default policy)
    void* alloc_on_node(size_t bytes, int node) const;
    void free_on_node(void* p, size_t bytes) const;

    static std::vector<int> parse_cpulist(const std::string& s);
    std::string describe() const;

private:
    std::string root_;
    std::vector<std::vector<int>> nodes_;
};

} // namespace cclx
