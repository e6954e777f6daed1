// Topology discovery of one node: GPUs, peer access, NVLink links, NVSwitch
// multicast capability.
//
// Counterpart of the reference topo_manager (src/topology/topo_manager.cpp:330-480,
// :947-1195), which derives "intra-card" and "inter-card" colours from Level Zero
// sub-devices and fabric ports to build pair / plane sub-communicators.  On an
// NVSwitch node every GPU reaches every peer at full bandwidth, so the hierarchy
// collapses: one plane, one colour per node; what remains is to verify that
// assumption (P2P matrix, active NVLink count per GPU via NVML when the library
// is present, multicast attribute) and to fall back to host staging when it
// does not hold.  CCL_TOPO_COLOR keeps the reference's modes: "fixed" (trust the
// assumption), "cuda" (query), "env" (reserved for explicit colour lists).
#pragma once
#include <string>
#include <vector>

namespace cclx {

struct gpu_info {
    int index = -1;
    std::string name;
    std::string pci_bus_id;
    int numa_node = -1; // home NUMA node of the device (sysfs), -1 when unknown
    int sm_count = 0;
    size_t mem_bytes = 0;
    int cc_major = 0, cc_minor = 0;
    int nvlink_active = -1; // active NVLink links (-1: NVML not available)
    bool multicast = false;
    int l2_bytes = 0;
};

class topo_info {
public:
    static const topo_info& local(); // discovered once per process
    int gpu_count() const { return (int)gpus.size(); }
    bool p2p(int a, int b) const;
    bool all_p2p() const;
    bool nvswitch_like() const; // every pair has native-atomic capable P2P
    std::string describe() const;

    std::vector<gpu_info> gpus;
    std::vector<char> p2p_matrix; // n x n
    std::vector<char> atomic_matrix;
    bool nvml_loaded = false;
};

} // namespace cclx
