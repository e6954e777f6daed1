#include "topo/topo.hpp"
#include "topo/numa.hpp"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nvml.h>

#include <mutex>
#include <sstream>

#include "core/env.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"

namespace cclx {

namespace {

// NVML is optional: loaded at run time like the reference loads its device libraries
struct nvml_api {
    void* lib = nullptr;
    nvmlReturn_t (*Init)() = nullptr;
    nvmlReturn_t (*Shutdown)() = nullptr;
    nvmlReturn_t (*DeviceGetHandleByPciBusId)(const char*, nvmlDevice_t*) = nullptr;
    nvmlReturn_t (*DeviceGetNvLinkState)(nvmlDevice_t, unsigned int, nvmlEnableState_t*) = nullptr;
    bool ok = false;
};

nvml_api load_nvml() {
    nvml_api a;
    a.lib = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
    if (!a.lib)
        return a;
    a.Init = (decltype(a.Init))dlsym(a.lib, "nvmlInit_v2");
    a.Shutdown = (decltype(a.Shutdown))dlsym(a.lib, "nvmlShutdown");
    a.DeviceGetHandleByPciBusId = (decltype(a.DeviceGetHandleByPciBusId))dlsym(a.lib, "nvmlDeviceGetHandleByPciBusId_v2");
    a.DeviceGetNvLinkState = (decltype(a.DeviceGetNvLinkState))dlsym(a.lib, "nvmlDeviceGetNvLinkState");
    a.ok = a.Init && a.Shutdown && a.DeviceGetHandleByPciBusId && a.DeviceGetNvLinkState && a.Init() == NVML_SUCCESS;
    return a;
}

topo_info discover() {
    topo_info t;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        n = 0;
    }
    const env_data& env = env_data::get();
    nvml_api nv;
    if (n > 0 && env.topo_color != "fixed")
        nv = load_nvml();
    t.nvml_loaded = nv.ok;
    const gpu::driver_api& d = gpu::driver();
    for (int i = 0; i < n; i++) {
        gpu_info g;
        g.index = i;
        cudaDeviceProp p;
        if (cudaGetDeviceProperties(&p, i) == cudaSuccess) {
            g.name = p.name;
            g.sm_count = p.multiProcessorCount;
            g.mem_bytes = p.totalGlobalMem;
            g.cc_major = p.major;
            g.cc_minor = p.minor;
            g.l2_bytes = p.l2CacheSize;
        }
        char bus[32] = { 0 };
        if (cudaDeviceGetPCIBusId(bus, sizeof(bus), i) == cudaSuccess)
            g.pci_bus_id = bus;
            g.numa_node = numa_info::get().node_of_pci(bus);
        if (d.loaded) {
            CUdevice cd;
            int mc = 0;
            if (d.DeviceGet(&cd, i) == CUDA_SUCCESS &&
                d.DeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd) == CUDA_SUCCESS)
                g.multicast = mc != 0;
        }
        if (nv.ok && !g.pci_bus_id.empty()) {
            nvmlDevice_t h;
            if (nv.DeviceGetHandleByPciBusId(g.pci_bus_id.c_str(), &h) == NVML_SUCCESS) {
                int active = 0;
                for (unsigned l = 0; l < NVML_NVLINK_MAX_LINKS; l++) {
                    nvmlEnableState_t st;
                    if (nv.DeviceGetNvLinkState(h, l, &st) == NVML_SUCCESS && st == NVML_FEATURE_ENABLED)
                        active++;
                }
                g.nvlink_active = active;
            }
        }
        t.gpus.push_back(g);
    }
    t.p2p_matrix.assign((size_t)n * n, 0);
    t.atomic_matrix.assign((size_t)n * n, 0);
    for (int a = 0; a < n; a++)
        for (int b = 0; b < n; b++) {
            if (a == b) {
                t.p2p_matrix[a * n + b] = t.atomic_matrix[a * n + b] = 1;
                continue;
            }
            if (env.topo_p2p_access == "1") {
                t.p2p_matrix[a * n + b] = 1;
                continue;
            }
            if (env.topo_p2p_access == "0")
                continue;
            int can = 0, atom = 0;
            if (cudaDeviceCanAccessPeer(&can, a, b) == cudaSuccess)
                t.p2p_matrix[a * n + b] = can != 0;
            if (cudaDeviceGetP2PAttribute(&atom, cudaDevP2PAttrNativeAtomicSupported, a, b) == cudaSuccess)
                t.atomic_matrix[a * n + b] = atom != 0;
        }
    (void)cudaGetLastError();
    if (nv.ok)
        nv.Shutdown();
    return t;
}

} // namespace

const topo_info& topo_info::local() {
    static topo_info inst = discover();
    return inst;
}

bool topo_info::p2p(int a, int b) const {
    const int n = gpu_count();
    return a >= 0 && b >= 0 && a < n && b < n && p2p_matrix[a * n + b];
}

bool topo_info::all_p2p() const {
    for (char c : p2p_matrix)
        if (!c)
            return false;
    return true;
}

bool topo_info::nvswitch_like() const {
    if (gpu_count() < 2)
        return false;
    for (char c : atomic_matrix)
        if (!c)
            return false;
    return all_p2p();
}

std::string topo_info::describe() const {
    std::ostringstream ss;
    const int n = gpu_count();
    ss << n << " GPU(s)";
    for (auto& g : gpus)
        ss << "\n  [" << g.index << "] " << g.name << " " << g.pci_bus_id << " numa " << g.numa_node << " sm_" << g.cc_major << g.cc_minor << " "
           << g.sm_count << " SMs " << (g.mem_bytes >> 30) << " GiB L2 " << (g.l2_bytes >> 20)
           << " MiB nvlink_active=" << g.nvlink_active << " multicast=" << g.multicast;
    if (n > 1) {
        ss << "\n  p2p:";
        for (int a = 0; a < n; a++) {
            ss << "\n   ";
            for (int b = 0; b < n; b++)
                ss << " " << (int)p2p_matrix[a * n + b];
        }
        ss << "\n  all-to-all peer access: " << all_p2p() << ", switch-like (native atomics everywhere): "
           << nvswitch_like();
    }
    return ss.str();
}

} // namespace cclx
