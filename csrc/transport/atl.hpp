// Abstract transport layer for CPU buffers: tagged non-blocking send / recv with
// N endpoints (one per worker), explicit progress, communicator split.
//
// Same contract as the reference's atl_base_comm (src/atl/atl_base_comm.hpp:32-281)
// and its 64-bit tag layout (src/comm/atl_tag.hpp:28-190): a message is matched
// by (source rank, tag) where tag = comm_id | sched_id | op_id.  Two transports sit
// behind it: this library's own `tcp` (a socket mesh on any host, with single-producer
// rings in POSIX shared memory and cross-memory rendezvous between ranks of one host),
// `ofi` (libfabric's tagged messages) and `mpi` (MPI point-to-point messages of an MPICH-ABI
// library); both libraries are opened with dlopen, and where one cannot be used on every rank
// `tcp` carries the traffic with a notice.
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace cclx {

class pmi;

struct atl_req {
    std::atomic<int> done{ 0 };
    size_t bytes = 0; // received size
    int error = 0; // set before `done` when the operation cannot complete: the peer's process is gone
    void reset() {
        done.store(0, std::memory_order_relaxed);
        bytes = 0;
        error = 0;
    }
    bool is_done() const { return done.load(std::memory_order_acquire) != 0; }
};

// tag = [comm_id:16][sched_id:24][op_id:24]
struct atl_tag {
    static constexpr uint64_t MAX_COMM = (1u << 16) - 1;
    static constexpr uint64_t MAX_SCHED = (1u << 24) - 1;
    static constexpr uint64_t MAX_OP = (1u << 24) - 1;
    static uint64_t make(uint64_t comm_id, uint64_t sched_id, uint64_t op_id) {
        return ((comm_id & MAX_COMM) << 48) | ((sched_id & MAX_SCHED) << 24) | (op_id & MAX_OP);
    }
    // reserved sched ids for point-to-point traffic (never cached, reference atl_tag.hpp:33-49)
    static constexpr uint64_t PT2PT_SCHED = MAX_SCHED;
    static constexpr uint64_t PT2PT_ACK_SCHED = MAX_SCHED - 1;
    static constexpr uint64_t INTERNAL_SCHED = MAX_SCHED - 2;
    // coordination messages of unordered collectives (op_id = coordination round)
    static constexpr uint64_t UNORDERED_SCHED = MAX_SCHED - 3;
    // the top of the external half of the schedule ids names operations by match_id
    static constexpr uint64_t UNORDERED_SPAN = 1u << 20;
};

// A registered memory region, as its owner describes it to a peer (plain data: it travels in a message).
// One-sided writes address it by offset.  Counterpart of the reference's atl_mr_t
// (src/atl/atl_def.h:160-175); here the key is the owner's pid, because between processes of one host
// the write is a cross-memory copy (process_vm_writev) that needs no pinning, and between hosts it is
// a message that the owner's progress engine applies to the region.
struct atl_mr {
    uint64_t addr = 0;
    uint64_t len = 0;
    int32_t pid = 0;
    int32_t owner = -1; // world rank
};

// process-wide mesh of connections among the ranks of one "world" (one KVS rendezvous)
class atl_transport {
public:
    virtual ~atl_transport() = default;
    virtual int world_rank() const = 0;
    virtual int world_size() const = 0;
    virtual int ep_count() const = 0;
    // `dst` / `src` are world ranks of this transport
    // `one_way`: the sender is not receiving from `dst` at the same time (a user's point-to-point stream).
    // Between processes of one host such messages keep to the rings, where the sender's copy-in and the
    // receiver's copy-out overlap on two cores (measured level with one cross-memory copy up to 512 KiB and
    // 1.4-1.6x faster at 1-2 MiB); exchanges inside collectives, where every rank copies in both directions
    // anyway, halve their copy work with the rendezvous (allreduce of 1-4 MiB: 10-25 % faster).
    virtual void send(int ep, const void* buf, size_t len, int dst, uint64_t tag, atl_req* req, bool one_way = false) = 0;
    virtual void recv(int ep, void* buf, size_t len, int src, uint64_t tag, atl_req* req) = 0;
    virtual bool probe(int ep, int src, uint64_t tag, size_t* len) = 0;
    virtual void poll(int ep) = 0;
    virtual bool same_host(int peer) const = 0;
    virtual const char* name() const = 0;
    // one-sided writes: register, tell the region to the writers by an ordinary message, write.
    // Writes of one rank to one region arrive in the order they were issued on one endpoint.
    virtual bool has_rma() const { return true; }
    virtual atl_mr mr_reg(void* buf, size_t len) = 0;
    virtual void mr_dereg(const atl_mr& mr) = 0;
    virtual void rma_write(int ep, const void* buf, size_t len, const atl_mr& mr, uint64_t offset, atl_req* req) = 0;
    std::atomic<uint64_t> rma_direct_writes{ 0 }, rma_message_writes{ 0 }, rndv_sends{ 0 }, peers_lost{ 0 };
    // statistics
    std::atomic<uint64_t> bytes_sent{ 0 }, bytes_received{ 0 }, msgs_sent{ 0 }, unexpected_msgs{ 0 };
};

std::shared_ptr<atl_transport> create_tcp_transport(pmi& pm, int ep_count);
// libfabric (opened at run time) behind the same interface; null with the reason in `why` when some rank
// cannot load the library
std::shared_ptr<atl_transport> create_ofi_transport(pmi& pm, int ep_count, std::string& why);
// an MPI library of the MPICH binary interface (opened at run time) behind the same interface; null with the
// reason in `why` when some rank cannot use it (no library, Open MPI, not started by the MPI launcher)
std::shared_ptr<atl_transport> create_mpi_transport(pmi& pm, int ep_count, std::string& why);

// A communicator's view of the transport: rank translation + comm id.
class atl_comm {
public:
    atl_comm(std::shared_ptr<atl_transport> tr, std::vector<int> world_ranks, int my_index, uint64_t comm_id);
    int rank() const { return rank_; }
    int size() const { return (int)ranks_.size(); }
    uint64_t id() const { return comm_id_; }
    int ep_count() const { return tr_->ep_count(); }
    int world_rank_of(int r) const { return ranks_[r]; }
    atl_transport& transport() { return *tr_; }
    std::shared_ptr<atl_transport> transport_ptr() { return tr_; }

    void send(int ep, const void* buf, size_t len, int dst, uint64_t tag, atl_req* req, bool one_way = false) {
        tr_->send(ep, buf, len, ranks_[dst], tag, req, one_way);
    }
    void recv(int ep, void* buf, size_t len, int src, uint64_t tag, atl_req* req) {
        tr_->recv(ep, buf, len, ranks_[src], tag, req);
    }
    void poll(int ep) { tr_->poll(ep); }
    void wait(int ep, atl_req* req);
    atl_mr mr_reg(void* buf, size_t len) { return tr_->mr_reg(buf, len); }
    void mr_dereg(const atl_mr& mr) { tr_->mr_dereg(mr); }
    void rma_write(int ep, const void* buf, size_t len, const atl_mr& mr, uint64_t offset, atl_req* req) {
        tr_->rma_write(ep, buf, len, mr, offset, req);
    }

    // blocking helpers used during setup (run on endpoint 0 with internal tags)
    void allgather(const void* send, void* recv, size_t bytes_per_rank);
    void barrier();
    // children created by split get ids that are unique inside the world
    std::shared_ptr<atl_comm> split(int color, int key);
    static uint64_t next_comm_id(); // process-wide counter
    static void bump_comm_id(uint64_t at_least);

private:
    std::shared_ptr<atl_transport> tr_;
    std::vector<int> ranks_;
    int rank_;
    uint64_t comm_id_;
    uint64_t internal_op_ = 0;
};

} // namespace cclx
