#include "comm/host_comm.hpp"

#include <unistd.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>

#include "core/env.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"
#include "gpu/device_comm.hpp"
#include "topo/topo.hpp"

namespace cclx {

// one transport per KVS rendezvous, shared by every communicator created on it
namespace {
std::mutex tr_mu;
std::map<std::string, std::weak_ptr<atl_transport>> transports;
} // namespace

std::shared_ptr<host_comm> host_comm::create(int size, int rank, std::shared_ptr<kvs::ikvs> store) {
    const env_data& env = env_data::get();
    auto pm = std::make_shared<pmi>(store, rank, size);
    logger::get().set_rank(rank);
    std::shared_ptr<atl_transport> tr;
    {
        std::lock_guard<std::mutex> lk(tr_mu);
        const std::string key = store->get_address().str() + "#" + std::to_string(size) + "#" + std::to_string(rank);
        auto it = transports.find(key);
        if (it != transports.end())
            tr = it->second.lock();
        if (!tr) {
            if (env.atl_transport == atl_transport_t::ofi) {
                std::string why;
                tr = create_ofi_transport(*pm, env.worker_count, why);
                if (!tr)
                    LOG_WARN("CCL_ATL_TRANSPORT=ofi: ", why, "; the socket transport carries the traffic");
            }
            else if (env.atl_transport == atl_transport_t::mpi) {
                std::string why;
                tr = create_mpi_transport(*pm, env.worker_count, why);
                if (!tr)
                    LOG_WARN("CCL_ATL_TRANSPORT=mpi: ", why, "; the socket transport carries the traffic");
            }
            if (!tr)
                tr = create_tcp_transport(*pm, env.worker_count);
            transports[key] = tr;
        }
    }
    // communicator id: agreed maximum of every rank's next free id
    uint64_t mine = atl_comm::next_comm_id();
    std::vector<uint64_t> all(size);
    pm->allgather(&mine, all.data(), sizeof(uint64_t));
    uint64_t id = *std::max_element(all.begin(), all.end());
    atl_comm::bump_comm_id(id + 1);
    std::vector<int> ranks(size);
    for (int i = 0; i < size; i++)
        ranks[i] = i;
    auto atl = std::make_shared<atl_comm>(tr, ranks, rank, id);
    executor::get().ensure_started(tr);
    auto c = std::make_shared<host_comm>(atl, pm);
    env.print(rank);
    return c;
}

host_comm::host_comm(std::shared_ptr<atl_comm> atl, std::shared_ptr<pmi> pm) : atl_(std::move(atl)), pm_(std::move(pm)) {
    send_seq_.assign(atl_->size(), 0);
    recv_seq_.assign(atl_->size(), 0);
}

host_comm::~host_comm() {
    release_device();
}

uint64_t host_comm::next_sched_id(bool internal) {
    std::lock_guard<std::mutex> lk(mu_);
    // external ids use the lower half of the tag field, internal ones the upper half
    const uint64_t half = atl_tag::MAX_SCHED / 2;
    if (internal)
        return half + (int_sched_++ % (half - 8));
    return ext_sched_++ % (half - atl_tag::UNORDERED_SPAN);
}

uint64_t host_comm::unordered_sched_id(uint64_t k) const {
    CCL_THROW_IF_NOT(k < atl_tag::UNORDERED_SPAN, "too many distinct match_ids on one communicator");
    return atl_tag::MAX_SCHED / 2 - atl_tag::UNORDERED_SPAN + k;
}

std::shared_ptr<host_comm> host_comm::split(int color, int key) {
    auto sub = atl_->split(color, key);
    return std::make_shared<host_comm>(sub, pm_);
}

void host_comm::build_hosts() {
    if (!host_idx_.empty())
        return;
    char host[64] = { 0 };
    gethostname(host, sizeof(host) - 1);
    // CCL_TOPO_FAKE_HOST lets a test place ranks of one machine on different "nodes"
    if (const char* fake = std::getenv("CCL_TOPO_FAKE_HOST"))
        std::snprintf(host, sizeof(host), "%s", fake);
    std::vector<char> all((size_t)size() * 64);
    atl_->allgather(host, all.data(), 64);
    std::vector<std::string> names;
    host_idx_.assign(size(), 0);
    for (int r = 0; r < size(); r++) {
        std::string h(&all[(size_t)r * 64], strnlen(&all[(size_t)r * 64], 64));
        auto it = std::find(names.begin(), names.end(), h);
        if (it == names.end()) {
            names.push_back(h);
            host_idx_[r] = (int)names.size() - 1;
        }
        else
            host_idx_[r] = (int)(it - names.begin());
    }
}

const std::vector<int>& host_comm::host_index() {
    build_hosts();
    return host_idx_;
}

std::shared_ptr<host_comm> host_comm::node_comm() {
    if (!node_) {
        build_hosts();
        node_ = split(host_idx_[rank()], rank());
    }
    return node_;
}

std::shared_ptr<host_comm> host_comm::r2r_comm() {
    if (!r2r_) {
        auto node = node_comm();
        r2r_ = split(node->rank(), rank());
    }
    return r2r_;
}

int host_comm::local_rank() {
    const env_data& env = env_data::get();
    if (env.local_rank >= 0)
        return env.local_rank;
    if (env.process_launcher == launcher_t::torchrun)
        if (const char* s = std::getenv("LOCAL_RANK"))
            return std::atoi(s);
    if (env.process_launcher == launcher_t::hydra)
        if (const char* s = std::getenv("MPI_LOCALRANKID"))
            return std::atoi(s);
    return node_comm()->rank();
}

int host_comm::local_size() {
    const env_data& env = env_data::get();
    if (env.local_size > 0)
        return env.local_size;
    if (env.process_launcher == launcher_t::torchrun)
        if (const char* s = std::getenv("LOCAL_WORLD_SIZE"))
            return std::atoi(s);
    if (env.process_launcher == launcher_t::hydra)
        if (const char* s = std::getenv("MPI_LOCALNRANKS"))
            return std::atoi(s);
    return node_comm()->size();
}

namespace {
// bootstrap exchange for the device communicator carried by the host transport
class atl_bootstrap : public gpu::bootstrap_if {
public:
    atl_bootstrap(atl_comm& a, std::shared_ptr<pmi> pm) : a_(a), pm_(std::move(pm)) {}
    int rank() const override { return a_.rank(); }
    int size() const override { return a_.size(); }
    void allgather(const void* s, void* r, size_t n) override { a_.allgather(s, r, n); }
    void barrier() override { a_.barrier(); }
    std::string job_id() override {
        char id[24] = { 0 };
        if (a_.rank() == 0)
            std::snprintf(id, sizeof(id), "%08x%08x", (unsigned)getpid(), (unsigned)(a_.id() * 2654435761u + counter_++));
        std::vector<char> all((size_t)a_.size() * 24);
        a_.allgather(id, all.data(), 24);
        return std::string(all.data());
    }

private:
    atl_comm& a_;
    std::shared_ptr<pmi> pm_;
    static unsigned counter_;
};
unsigned atl_bootstrap::counter_ = 0;
} // namespace

void host_comm::init_device() {
    if (dev_)
        return;
    build_hosts();
    for (int r = 0; r < size(); r++)
        CCL_THROW_IF_NOT(host_idx_[r] == host_idx_[rank()],
                         "the device communicator needs every rank on one node (NVLink domain); use the node "
                         "sub-communicator for multi-node jobs");
    if (env_data::get().topo_fabric_check && size() > 1) {
        // CCL_TOPO_FABRIC_VERTEX_CONNECTION_CHECK=1: name the pair of ranks without peer access before
        // any memory is mapped (off by default: mapping the heap reports an unreachable peer as well).
        // Devices are compared by PCI bus id, ordinals differ between processes.
        const topo_info& t = topo_info::local();
        int cur = 0;
        cudaGetDevice(&cur);
        char mine[32] = { 0 };
        if (cur >= 0 && cur < t.gpu_count())
            std::snprintf(mine, sizeof(mine), "%s", t.gpus[cur].pci_bus_id.c_str());
        std::vector<char> all((size_t)size() * 32);
        atl_->allgather(mine, all.data(), 32);
        auto ordinal = [&](int r) {
            for (int g = 0; g < t.gpu_count(); g++)
                if (t.gpus[g].pci_bus_id == &all[(size_t)r * 32])
                    return g;
            return -1; // not visible to this process: nothing to compare
        };
        for (int r = 0; r < size(); r++) {
            const int g = ordinal(r);
            CCL_THROW_IF_NOT(r == rank() || g < 0 || g == cur || t.p2p(cur, g), "rank ", rank(), " (GPU ", mine,
                             ") has no peer access to rank ", r, " (GPU ", &all[(size_t)r * 32], ")");
        }
    }
    dev_bs_.reset(new atl_bootstrap(*atl_, pm_));
    dev_.reset(new gpu::device_comm());
    dev_->init(*dev_bs_);
}

gpu::device_comm* host_comm::device() {
    if (!dev_)
        init_device();
    return dev_.get();
}

void host_comm::release_device() {
    if (dev_) {
        // every rank unbinds together: a peer must not touch my memory after I unmap it
        try {
            cudaDeviceSynchronize();
            if (!aborted_)
                atl_->barrier();
        }
        catch (...) {
        }
        for (auto& sc : dev_scratch_)
            sc.reset();
        dev_.reset();
    }
}

void host_comm::abort() {
    aborted_ = true;
    if (dev_)
        dev_->abort();
}

} // namespace cclx
