#include "topo/numa.hpp"

#include <dirent.h>
#include <sched.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cstdlib>
#include <fstream>
#include <sstream>

#include "core/log.hpp"

namespace cclx {

namespace {
// values of <linux/mempolicy.h>, which is not always installed
constexpr int MPOL_DEFAULT_ = 0, MPOL_PREFERRED_ = 1, MPOL_BIND_ = 2;

std::string read_line(const std::string& path) {
    std::ifstream f(path);
    std::string s;
    if (f)
        std::getline(f, s);
    return s;
}
} // namespace

std::vector<int> numa_info::parse_cpulist(const std::string& s) {
    std::vector<int> out;
    std::stringstream ss(s);
    std::string tok;
    while (std::getline(ss, tok, ',')) {
        if (tok.empty())
            continue;
        const size_t dash = tok.find('-');
        char* end = nullptr;
        const long a = std::strtol(tok.c_str(), &end, 10);
        long b = a;
        if (dash != std::string::npos)
            b = std::strtol(tok.c_str() + dash + 1, &end, 10);
        for (long c = a; c <= b && c >= 0 && out.size() < 65536; c++)
            out.push_back((int)c);
    }
    return out;
}

numa_info::numa_info(const std::string& sys_root) : root_(sys_root) {
    const std::string dir = root_ + "/devices/system/node";
    if (DIR* d = opendir(dir.c_str())) {
        while (dirent* e = readdir(d)) {
            int id = -1;
            if (std::sscanf(e->d_name, "node%d", &id) != 1 || id < 0 || id > 4095)
                continue;
            if ((size_t)id >= nodes_.size())
                nodes_.resize(id + 1);
            nodes_[id] = parse_cpulist(read_line(dir + "/" + e->d_name + "/cpulist"));
        }
        closedir(d);
    }
    if (nodes_.empty()) { // no NUMA information: one node with every online core
        nodes_.resize(1);
        nodes_[0] = parse_cpulist(read_line(root_ + "/devices/system/cpu/online"));
    }
}

numa_info& numa_info::get() {
    static numa_info inst("/sys");
    return inst;
}

const std::vector<int>& numa_info::cpus_of_node(int node) const {
    static const std::vector<int> none;
    return node >= 0 && node < (int)nodes_.size() ? nodes_[node] : none;
}

int numa_info::node_of_cpu(int cpu) const {
    for (size_t n = 0; n < nodes_.size(); n++)
        if (std::find(nodes_[n].begin(), nodes_[n].end(), cpu) != nodes_[n].end())
            return (int)n;
    return -1;
}

int numa_info::node_of_pci(const std::string& bdf) const {
    std::string id = bdf;
    std::transform(id.begin(), id.end(), id.begin(), [](unsigned char c) { return (char)std::tolower(c); });
    if (id.size() > 12 && id.compare(0, 4, "0000") == 0 && id[8] == ':') // NVML prints an 8-digit domain
        id = id.substr(4);
    const std::string s = read_line(root_ + "/bus/pci/devices/" + id + "/numa_node");
    if (s.empty())
        return -1;
    const int n = std::atoi(s.c_str());
    return n >= 0 && n < (int)nodes_.size() ? n : -1;
}

std::vector<int> numa_info::allowed_cpus() const {
    std::vector<int> out;
    cpu_set_t set;
    CPU_ZERO(&set);
    if (sched_getaffinity(0, sizeof(set), &set) == 0)
        for (int c = 0; c < CPU_SETSIZE; c++)
            if (CPU_ISSET(c, &set))
                out.push_back(c);
    return out;
}

std::vector<int> numa_info::auto_worker_cpus(const std::vector<int>& cpus, int local_rank, int local_size,
                                             int workers) {
    std::vector<int> out;
    const int need = local_size * workers;
    // pin only when every rank still keeps at least one core per worker for the application
    if (workers <= 0 || local_size <= 0 || local_rank < 0 || (int)cpus.size() < 2 * need)
        return out;
    for (int w = 0; w < workers; w++)
        out.push_back(cpus[cpus.size() - 1 - (size_t)(local_rank * workers + w)]);
    return out;
}

bool numa_info::bind_thread_memory(int node) const {
    if (node < 0)
        return syscall(SYS_set_mempolicy, MPOL_DEFAULT_, nullptr, 0) == 0;
    if (node >= 1024)
        return false;
    unsigned long mask[16] = { 0 };
    mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
    return syscall(SYS_set_mempolicy, MPOL_PREFERRED_, mask, 1024 + 1) == 0;
}

void* numa_info::alloc_on_node(size_t bytes, int node) const {
    void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    if (p == MAP_FAILED)
        return nullptr;
    if (node >= 0 && node < 1024 && node_count() > 1) {
        unsigned long mask[16] = { 0 };
        mask[node / (8 * sizeof(unsigned long))] |= 1ul << (node % (8 * sizeof(unsigned long)));
        if (syscall(SYS_mbind, p, bytes, MPOL_BIND_, mask, 1024 + 1, 0) != 0)
            LOG_DEBUG("mbind to node ", node, " failed; default placement");
    }
    return p;
}

void numa_info::free_on_node(void* p, size_t bytes) const {
    if (p)
        munmap(p, bytes);
}

std::string numa_info::describe() const {
    std::stringstream ss;
    ss << node_count() << " NUMA node(s)";
    for (size_t n = 0; n < nodes_.size(); n++)
        ss << "; node" << n << ": " << nodes_[n].size() << " cpus";
    return ss.str();
}

} // namespace cclx
