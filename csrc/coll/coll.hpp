// Collective front-end: parameter / attribute records, validation, the path
// decision (device kernels vs CPU scheduler), schedule creation with caching,
// fusion, partitioning among workers, start and completion events.
//
// Reference counterpart: ccl_coll_create and friends (src/coll/coll.cpp:96-378,
// :1055-1361 for the device fast path; src/coll/coll_param.cpp:103-800;
// src/coll/coll_check.cpp:27-142; src/parallelizer/parallelizer.cpp:31-753).
#pragma once
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "comm/host_comm.hpp"
#include "core/types.hpp"
#include "sched/sched.hpp"

namespace cclx {

struct coll_attr {
    int priority = 0;
    bool synchronous = false;
    bool to_cache = false;
    std::string match_id;
    reduction_fn_t reduction_fn = nullptr;
    // device path extras (no reference counterpart): fused epilogue of reductions
    bool do_scale = false;
    float scale = 1.0f;
    int out_dtype = -1; // -1: same as the input datatype
    std::string gpu_algo; // "" = automatic
    // the inter-node stage of a hierarchical device collective: CCL_<COLL>_SCALEOUT applies (reference
    // ccl_coll_param::is_scaleout, src/coll/coll_param.hpp:52-130)
    bool scaleout = false;
};

class event_impl {
public:
    virtual ~event_impl() = default;
    virtual void wait() = 0;
    virtual bool test() = 0;
    virtual bool cancel() { return false; }
    virtual void* native() { return nullptr; } // cudaEvent_t of device operations
};
typedef std::shared_ptr<event_impl> event_ptr;

struct coll_param {
    coll_type ctype = coll_allreduce;
    const void* send_buf = nullptr;
    void* recv_buf = nullptr;
    std::vector<void*> recv_bufs; // allgatherv vector form
    size_t count = 0; // allreduce/bcast/reduce: elements; allgather: send count; reduce_scatter: recv count; alltoall: per peer
    std::vector<size_t> send_counts, recv_counts; // vector collectives
    int dtype = dt_float32;
    int reduction = red_sum;
    int root = 0;
    int peer = -1;
    void* stream = nullptr; // cudaStream_t for device buffers, nullptr for host buffers
    bool device = false; // buffers are device memory (set when a device stream is passed)
    std::vector<event_ptr> deps;
};

// entry point used by the API layer
event_ptr coll_create(host_comm& comm, coll_param& p, const coll_attr& attr);

// Allreduce of several buffers as one operation (send[k] -> recv[k], counts[k] elements of `dtype`).  Device
// buffers of a single node travel as one fused sequence: pack kernel, one allreduce on a buffer of the
// symmetric heap, unpack kernel (gpu::launch_allreduce_fused).  Anything else is issued buffer by buffer;
// the returned event covers all of them.  Used by the fusion manager for device operations and by the
// torch backend's allreduce_coalesced.
event_ptr coll_allreduce_coalesced(host_comm& comm, const std::vector<const void*>& send, const std::vector<void*>& recv,
                                   const std::vector<size_t>& counts, int dtype, int reduction, const coll_attr& attr,
                                   void* stream, bool device);

// group API (reference src/coll/group/group.cpp:19-73): only send/recv may be
// issued between start and end; they are posted together at group_end
void group_start();
void group_end();
bool group_active();

void coll_validate(const host_comm& comm, const coll_param& p, const coll_attr& attr);
// true when recv aliases send at the position in-place collectives define
bool coll_is_inplace(const host_comm& comm, const coll_param& p);
std::string coll_cache_key(const host_comm& comm, const coll_param& p, const coll_attr& attr);
event_ptr make_completed_event();

// counters (observability)
struct coll_stats {
    uint64_t calls[coll_last] = {};
    uint64_t device_calls[coll_last] = {};
    uint64_t fused_ops = 0, fused_batches = 0;
    uint64_t cache_hits = 0;
    uint64_t postponed = 0; // operations parked until their match_id was named
};
coll_stats& stats();

} // namespace cclx
