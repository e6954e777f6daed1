// Communicator: rank / size, transport view, schedule-id allocator, sub-communicators,
// schedule cache and (optionally) the device communicator of the node.
//
// Reference counterpart: ccl_comm (src/comm/comm.hpp:366-665, comm.cpp:115-309,
// :400-430): rank/size, comm id, node / r2r sub-communicators, local<->global
// rank maps and a schedule-id allocator split into an internal and an external
// half.  On one NVSwitch node the pair/even hierarchy of the reference collapses
// to a single node communicator, so only `node` (ranks of my host) and `r2r`
// (same local index on every host) are derived.
#pragma once
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "bootstrap/pmi.hpp"
#include "sched/sched.hpp"
#include "transport/atl.hpp"

namespace cclx {

namespace gpu {
class device_comm;
class bootstrap_if;
}
class topo_info;

class host_comm : public std::enable_shared_from_this<host_comm> {
public:
    // world communicator over a KVS rendezvous
    static std::shared_ptr<host_comm> create(int size, int rank, std::shared_ptr<kvs::ikvs> store);
    host_comm(std::shared_ptr<atl_comm> atl, std::shared_ptr<pmi> pm);
    ~host_comm();

    int rank() const { return atl_->rank(); }
    int size() const { return atl_->size(); }
    uint64_t id() const { return atl_->id(); }
    atl_comm& atl() { return *atl_; }
    std::shared_ptr<pmi> pm() { return pm_; }

    // schedule ids: external half for user operations, internal half for operations
    // the library issues itself (fusion, unordered coordination)
    uint64_t next_sched_id(bool internal = false);
    // id of the k-th match_id named by the coordinator of unordered collectives
    uint64_t unordered_sched_id(uint64_t k) const;
    // state the collective front-end keeps per communicator (unordered coordination)
    std::shared_ptr<void> frontend_state;
    std::shared_ptr<host_comm> split(int color, int key);
    std::shared_ptr<host_comm> node_comm();
    std::shared_ptr<host_comm> r2r_comm();
    int local_rank();
    int local_size();
    const std::vector<int>& host_index(); // host id of every rank

    sched_cache& cache() { return cache_; }

    // device side: created on demand (needs a CUDA device selected by the caller)
    gpu::device_comm* device();
    // scratch memory of the hierarchical (node / cross-node) device collectives, one slot per collective:
    // owned by the communicator, freed when its device state is released
    std::shared_ptr<void>& device_scratch(int which) { return dev_scratch_[which]; }
    bool has_device() const { return dev_ != nullptr; }
    void init_device();
    void release_device();

    // failure detection: heartbeat keys in the KVS, abort flag polled by device waits
    void abort();
    bool aborted() const { return aborted_; }

    // per-peer point-to-point sequence numbers (tags of send/recv)
    uint64_t p2p_send_seq(int peer) { return send_seq_[peer]++; }
    uint64_t p2p_recv_seq(int peer) { return recv_seq_[peer]++; }

private:
    void build_hosts();
    std::shared_ptr<atl_comm> atl_;
    std::shared_ptr<pmi> pm_;
    std::mutex mu_;
    uint64_t ext_sched_ = 0, int_sched_ = 0;
    std::shared_ptr<host_comm> node_, r2r_;
    std::vector<int> host_idx_;
    sched_cache cache_;
    std::shared_ptr<void> dev_scratch_[4]; // scratch of the hierarchical device collectives (released with the device state)
    std::unique_ptr<gpu::bootstrap_if> dev_bs_; // outlives dev_: later handle exchanges (buffer registration) use it
    std::unique_ptr<gpu::device_comm> dev_;
    std::unique_ptr<pmi> dev_pm_;
    bool aborted_ = false;
    std::vector<uint64_t> send_seq_, recv_seq_;
};

} // namespace cclx
