#include "coll/coll.hpp"

#include <cuda_runtime.h>

#include <cstring>
#include <deque>
#include <list>
#include <map>
#include <mutex>
#include <sstream>

#include "coll/algorithms.hpp"
#include "coll/selection.hpp"
#include "core/datatype.hpp"
#include "core/env.hpp"
#include "core/log.hpp"
#include "core/trace.hpp"
#include "fusion/fusion.hpp"
#include "gpu/cuda_driver.hpp"
#include "gpu/device_comm.hpp"
#include "sched/entries.hpp"

namespace cclx {

coll_stats& stats() {
    static coll_stats s;
    return s;
}

// ---- events -----------------------------------------------------------------------------
namespace {

class completed_event : public event_impl {
public:
    void wait() override {}
    bool test() override { return true; }
};

// masters whose event was dropped before completion live here until they finish
// (reference: recycle_storage of the schedule cache)
std::mutex recycle_mu;
std::list<std::pair<std::unique_ptr<master_sched>, uint64_t>> recycle;

void purge_recycle() {
    std::lock_guard<std::mutex> lk(recycle_mu);
    for (auto it = recycle.begin(); it != recycle.end();) {
        if (it->first->ticket_retired(it->second))
            it = recycle.erase(it);
        else
            ++it;
    }
}

class host_event : public event_impl {
public:
    host_event(master_sched* m, uint64_t ticket, std::unique_ptr<master_sched> owned,
               std::shared_ptr<master_sched> cached = nullptr)
            : m_(m), ticket_(ticket), owned_(std::move(owned)), cached_(std::move(cached)) {}
    ~host_event() override {
        if (owned_ && !owned_->ticket_retired(ticket_)) {
            std::lock_guard<std::mutex> lk(recycle_mu);
            recycle.emplace_back(std::move(owned_), ticket_);
        }
    }
    void wait() override { executor::get().wait(m_, ticket_); }
    bool test() override {
        bool done = executor::get().test(m_, ticket_);
        if (done && m_->req().has_error())
            CCL_THROW("collective failed: ", m_->req().error());
        return done;
    }

private:
    master_sched* m_;
    uint64_t ticket_;
    std::unique_ptr<master_sched> owned_;
    std::shared_ptr<master_sched> cached_; // a cached schedule may leave the cache while this event lives
};

thread_local bool tl_no_fusion = false; // set while coll_allreduce_coalesced issues its buffers one by one

class cuda_event_impl : public event_impl {
public:
    cuda_event_impl(gpu::device_comm* dc, cudaStream_t st) : dc_(dc) {
        CUDA_CHECK(cudaSetDevice(dc->device_id()));
        CUDA_CHECK(cudaEventCreateWithFlags(&ev_, cudaEventDisableTiming));
        CUDA_CHECK(cudaEventRecord(ev_, st));
    }
    ~cuda_event_impl() override { cudaEventDestroy(ev_); }
    void wait() override {
        CUDA_CHECK(cudaEventSynchronize(ev_));
        dc_->check_status();
    }
    bool test() override {
        cudaError_t e = cudaEventQuery(ev_);
        if (e == cudaErrorNotReady)
            return false;
        CUDA_CHECK(e);
        dc_->check_status();
        return true;
    }
    void* native() override { return (void*)ev_; }

private:
    gpu::device_comm* dc_;
    cudaEvent_t ev_;
};

// placeholder returned for send/recv inside a group; bound at group_end
class group_event : public event_impl {
public:
    void bind(event_ptr e) { real_ = std::move(e); }
    void wait() override {
        CCL_THROW_IF_NOT(real_, "an operation issued inside a group can be waited only after group_end");
        real_->wait();
    }
    bool test() override { return real_ ? real_->test() : false; }
    void* native() override { return real_ ? real_->native() : nullptr; }

private:
    event_ptr real_;
};

struct group_item {
    host_comm* comm;
    coll_param param;
    coll_attr attr;
    std::shared_ptr<group_event> ev;
};
thread_local bool tl_group_active = false;
thread_local std::vector<group_item> tl_group;

size_t total(const std::vector<size_t>& v) {
    size_t s = 0;
    for (size_t x : v)
        s += x;
    return s;
}

std::vector<size_t> prefix(const std::vector<size_t>& v) {
    std::vector<size_t> o(v.size(), 0);
    for (size_t i = 1; i < v.size(); i++)
        o[i] = o[i - 1] + v[i - 1];
    return o;
}

// message size the selection tables are keyed by
size_t selection_bytes(const host_comm& comm, const coll_param& p) {
    const size_t esz = dtype_size(p.dtype);
    switch (p.ctype) {
        case coll_allgather: return p.count * esz * comm.size();
        case coll_allgatherv: return total(p.recv_counts) * esz;
        case coll_alltoall: return p.count * esz * comm.size();
        case coll_alltoallv: return total(p.send_counts) * esz;
        case coll_reduce_scatter: return p.count * esz * comm.size();
        case coll_barrier: return 0;
        default: return p.count * esz;
    }
}

} // namespace

event_ptr make_completed_event() {
    return std::make_shared<completed_event>();
}

// ---- validation -------------------------------------------------------------------------
void coll_validate(const host_comm& comm, const coll_param& p, const coll_attr& attr) {
    const int N = comm.size();
    if (p.ctype == coll_barrier)
        return;
    CCL_THROW_IF_NOT(datatype_table::get().exists(p.dtype), "unknown datatype ", p.dtype);
    const bool reduces = p.ctype == coll_allreduce || p.ctype == coll_reduce || p.ctype == coll_reduce_scatter;
    if (reduces) {
        CCL_THROW_IF_NOT(p.reduction >= red_sum && p.reduction <= red_custom, "invalid reduction ", p.reduction);
        if (p.reduction == red_custom)
            CCL_THROW_IF_NOT(attr.reduction_fn != nullptr, "custom reduction needs attr reduction_fn");
        if (p.dtype >= dt_custom_base)
            CCL_THROW_IF_NOT(p.reduction == red_custom, "custom datatypes can only be reduced with a custom reduction");
        if (p.reduction == red_custom)
            CCL_THROW_IF_NOT(!p.device, "custom reductions run on host buffers only");
    }
    switch (p.ctype) {
        case coll_allgatherv:
            CCL_THROW_IF_NOT((int)p.recv_counts.size() == N, "allgatherv: recv_counts needs ", N, " entries");
            CCL_THROW_IF_NOT(p.recv_counts[comm.rank()] == p.count, "allgatherv: send_count (", p.count,
                             ") differs from recv_counts[rank] (", p.recv_counts[comm.rank()], ")");
            if (!p.recv_bufs.empty())
                CCL_THROW_IF_NOT((int)p.recv_bufs.size() == N, "allgatherv: recv_bufs needs ", N, " entries");
            break;
        case coll_alltoallv:
            CCL_THROW_IF_NOT((int)p.send_counts.size() == N && (int)p.recv_counts.size() == N,
                             "alltoallv: send_counts and recv_counts need ", N, " entries");
            break;
        case coll_bcast:
        case coll_broadcast:
        case coll_reduce:
            CCL_THROW_IF_NOT(p.root >= 0 && p.root < N, "root ", p.root, " outside the communicator");
            break;
        case coll_send:
        case coll_recv:
            CCL_THROW_IF_NOT(p.peer >= 0 && p.peer < N && p.peer != comm.rank(), "invalid peer ", p.peer);
            break;
        default: break;
    }
    const size_t bytes = selection_bytes(comm, p);
    if (bytes == 0)
        return;
    const bool needs_send = p.ctype != coll_recv && p.ctype != coll_bcast;
    const bool needs_recv = p.ctype != coll_send && !(p.ctype == coll_reduce && comm.rank() != p.root);
    if (needs_send && p.ctype != coll_allgatherv && p.ctype != coll_allgather && p.ctype != coll_broadcast)
        CCL_THROW_IF_NOT(p.send_buf != nullptr, coll_name(p.ctype), ": send buffer is null");
    if (needs_recv && p.recv_bufs.empty())
        CCL_THROW_IF_NOT(p.recv_buf != nullptr, coll_name(p.ctype), ": recv buffer is null");
    // in-place aliasing rules (reference src/coll/coll_util.cpp:650-760)
    if (env_data::get().check_inplace_aliasing && p.send_buf && p.recv_buf && p.recv_bufs.empty()) {
        const size_t esz = dtype_size(p.dtype);
        const char* s = (const char*)p.send_buf;
        const char* r = (const char*)p.recv_buf;
        if (p.ctype == coll_allgatherv || p.ctype == coll_allgather) {
            std::vector<size_t> counts = p.recv_counts.empty() ? std::vector<size_t>(N, p.count) : p.recv_counts;
            const size_t off = prefix(counts)[comm.rank()] * esz;
            const size_t all = total(counts) * esz;
            const bool overlap = s < r + all && r < s + p.count * esz;
            if (overlap)
                CCL_THROW_IF_NOT(s == r + off, coll_name(p.ctype),
                                 ": send buffer overlaps recv buffer but is not at the in-place offset of this rank");
        }
        else if (p.ctype == coll_reduce_scatter) {
            const size_t off = (size_t)comm.rank() * p.count * esz;
            const bool overlap = r < s + p.count * N * esz && s < r + p.count * esz;
            if (overlap)
                CCL_THROW_IF_NOT(r == s + off,
                                 "reduce_scatter: recv buffer overlaps send buffer but is not at send + rank*recv_count");
        }
    }
}

bool coll_is_inplace(const host_comm& comm, const coll_param& p) {
    const size_t esz = dtype_size(p.dtype);
    switch (p.ctype) {
        case coll_allgather:
        case coll_allgatherv: {
            if (!p.send_buf)
                return true;
            std::vector<size_t> counts = p.recv_counts.empty() ? std::vector<size_t>(comm.size(), p.count) : p.recv_counts;
            return p.send_buf == (const char*)p.recv_buf + prefix(counts)[comm.rank()] * esz;
        }
        case coll_reduce_scatter: return p.recv_buf == (const char*)p.send_buf + (size_t)comm.rank() * p.count * esz;
        default: return p.send_buf == p.recv_buf;
    }
}

std::string coll_cache_key(const host_comm& comm, const coll_param& p, const coll_attr& attr) {
    std::ostringstream ss;
    ss << (int)p.ctype << '|' << p.send_buf << '|' << p.recv_buf << '|' << p.count << '|' << p.dtype << '|'
       << p.reduction << '|' << p.root << '|' << p.peer << '|' << (const void*)attr.reduction_fn << '|'
       << attr.priority;
    for (size_t c : p.send_counts)
        ss << ',' << c;
    ss << '|';
    for (size_t c : p.recv_counts)
        ss << ',' << c;
    ss << '|';
    for (void* b : p.recv_bufs)
        ss << ',' << b;
    if (env_data::get().cache_key == cache_key_t::match_id && !attr.match_id.empty())
        ss << "|m:" << attr.match_id;
    return ss.str();
}

// ---- CPU schedule construction --------------------------------------------------------------
namespace {

// `part` of `parts` (block-sliced collectives only): the schedule handles the part-th slice of every block
void build_cpu(sched& s, host_comm& comm, const coll_param& p, const coll_attr& attr, size_t off_elems,
               size_t count_elems, int part = 0, int parts = 1) {
    const int N = comm.size();
    const size_t esz = dtype_size(p.dtype);
    selector_param sp;
    sp.ctype = p.ctype;
    sp.comm_size = N;
    sp.vector_buf = !p.recv_bufs.empty();
    sp.custom_fn = attr.reduction_fn != nullptr;
    sp.scaleout = attr.scaleout;
    const char* sbuf = p.send_buf ? (const char*)p.send_buf + off_elems * esz : nullptr;
    char* rbuf = p.recv_buf ? (char*)p.recv_buf + off_elems * esz : nullptr;
    switch (p.ctype) {
        case coll_allreduce: {
            sp.count = count_elems;
            sp.bytes = count_elems * esz;
            const std::string a = algorithm_selector::get().select_cpu(sp);
            algo::buf_desc b{ sbuf, rbuf, count_elems, p.dtype, p.reduction, attr.reduction_fn };
            if (a == "ring")
                algo::allreduce_ring(s, b);
            else if (a == "recursive_doubling")
                algo::allreduce_recursive_doubling(s, b);
            else if (a == "rabenseifner")
                algo::allreduce_rabenseifner(s, b);
            else if (a == "nreduce")
                algo::allreduce_nreduce(s, b);
            else if (a == "2d")
                algo::allreduce_2d(s, b);
            else if (a == "double_tree")
                algo::allreduce_double_tree(s, b);
            else if (a == "ring_rma") {
                // a transport without one-sided writes (ofi) runs the two-sided ring
                if (comm.atl().transport().has_rma())
                    algo::allreduce_ring_rma(s, b);
                else
                    algo::allreduce_ring(s, b);
            }
            else
                CCL_THROW("allreduce: unknown algorithm ", a);
            break;
        }
        case coll_allgather:
        case coll_allgatherv: {
            std::vector<size_t> counts = p.ctype == coll_allgather ? std::vector<size_t>(N, p.count) : p.recv_counts;
            sp.bytes = total(counts) * esz;
            const std::string a = algorithm_selector::get().select_cpu(sp);
            if (!p.recv_bufs.empty()) {
                algo::allgatherv_naive_vec(s, p.send_buf, p.recv_bufs, counts, p.dtype);
                break;
            }
            std::vector<size_t> offs = prefix(counts);
            if (parts > 1) {
                // slice k of every rank's block, gathered into the matching places of recv
                std::vector<size_t> pc(N), po(N);
                for (int q = 0; q < N; q++) {
                    std::vector<size_t> c1, o1;
                    algo::block_partition(counts[q], parts, c1, o1);
                    pc[q] = c1[part];
                    po[q] = offs[q] + o1[part];
                }
                const char* src = p.send_buf ? (const char*)p.send_buf + (po[comm.rank()] - offs[comm.rank()]) * esz : nullptr;
                algo::allgatherv_ring(s, src, p.recv_buf, pc, po, p.dtype);
                break;
            }
            if (a == "ring")
                algo::allgatherv_ring(s, p.send_buf, p.recv_buf, counts, offs, p.dtype);
            else if (a == "multi_bcast")
                algo::allgatherv_multi_bcast(s, p.send_buf, p.recv_buf, counts, offs, p.dtype);
            else if (a == "flat")
                algo::allgatherv_flat(s, p.send_buf, p.recv_buf, counts, offs, p.dtype);
            else
                algo::allgatherv_naive(s, p.send_buf, p.recv_buf, counts, offs, p.dtype);
            break;
        }
        case coll_alltoall:
        case coll_alltoallv: {
            std::vector<size_t> sc = p.ctype == coll_alltoall ? std::vector<size_t>(N, p.count) : p.send_counts;
            std::vector<size_t> rc = p.ctype == coll_alltoall ? std::vector<size_t>(N, p.count) : p.recv_counts;
            sp.bytes = total(sc) * esz;
            const std::string a = algorithm_selector::get().select_cpu(sp);
            std::vector<size_t> so = prefix(sc), ro = prefix(rc);
            if (parts > 1) {
                for (int q = 0; q < N; q++) { // slice `part` of every block, on the send and on the recv side
                    std::vector<size_t> c1, o1;
                    algo::block_partition(sc[q], parts, c1, o1);
                    so[q] += o1[part];
                    sc[q] = c1[part];
                    algo::block_partition(rc[q], parts, c1, o1);
                    ro[q] += o1[part];
                    rc[q] = c1[part];
                }
            }
            if (a == "scatter")
                algo::alltoallv_scatter(s, p.send_buf, sc, so, p.recv_buf, rc, ro, p.dtype,
                                        env_data::get().alltoall_scatter_max_ops);
            else
                algo::alltoallv_naive(s, p.send_buf, sc, so, p.recv_buf, rc, ro, p.dtype);
            break;
        }
        case coll_barrier: {
            sp.bytes = 0;
            const std::string a = algorithm_selector::get().select_cpu(sp);
            if (a == "ring")
                algo::barrier_ring(s);
            else
                algo::barrier_dissemination(s);
            break;
        }
        case coll_bcast:
        case coll_broadcast: {
            sp.bytes = count_elems * esz;
            const std::string a = algorithm_selector::get().select_cpu(sp);
            // out-of-place form: the root's data travels from send_buf, lands in recv_buf everywhere
            if (p.ctype == coll_broadcast && comm.rank() == p.root && sbuf && sbuf != rbuf) {
                s.add<copy_entry>(sbuf, rbuf, count_elems * esz);
                s.add_barrier();
            }
            if (a == "naive")
                algo::bcast_naive(s, rbuf, count_elems * esz, p.root);
            else if (a == "ring")
                algo::bcast_ring(s, rbuf, count_elems, p.dtype, p.root);
            else if (a == "double_tree")
                algo::bcast_double_tree(s, rbuf, count_elems, p.dtype, p.root);
            else
                algo::bcast_tree(s, rbuf, count_elems * esz, p.root);
            break;
        }
        case coll_reduce: {
            sp.bytes = count_elems * esz;
            const std::string a = algorithm_selector::get().select_cpu(sp);
            algo::buf_desc b{ sbuf, comm.rank() == p.root ? rbuf : nullptr, count_elems, p.dtype, p.reduction,
                              attr.reduction_fn };
            if (a == "rabenseifner")
                algo::reduce_rabenseifner(s, b, p.root);
            else if (a == "ring")
                algo::reduce_ring(s, b, p.root);
            else if (a == "double_tree")
                algo::reduce_double_tree(s, b, p.root);
            else
                algo::reduce_tree(s, b, p.root);
            break;
        }
        case coll_reduce_scatter: {
            sp.bytes = p.count * esz * N;
            const std::string a = algorithm_selector::get().select_cpu(sp);
            algo::buf_desc b{ p.send_buf, p.recv_buf, p.count, p.dtype, p.reduction, attr.reduction_fn };
            if (a == "ring")
                algo::reduce_scatter_ring(s, b);
            else
                algo::reduce_scatter_naive(s, b);
            break;
        }
        case coll_send:
        case coll_recv: {
            // pieces of at most the large-message size, one tag each (reference parallelizer.cpp:326-333)
            const size_t big = std::max<size_t>(env_data::get().large_msg_size, 1);
            const size_t bytes = p.count * esz;
            size_t done = 0;
            uint64_t step = 0;
            do {
                const size_t n = std::min(big, bytes - done);
                if (p.ctype == coll_send)
                    algo::send_direct(s, (const char*)p.send_buf + done, n, p.peer, step);
                else
                    algo::recv_direct(s, (char*)p.recv_buf + done, n, p.peer, step);
                done += n;
                step++;
            } while (done < bytes);
            break;
        }
        default: CCL_THROW("unsupported collective ", (int)p.ctype);
    }
}

// How many partial schedules an operation is cut into (reference parallelizer.cpp:77-154, 224-330):
//  * allreduce / reduce / broadcast: one per worker once the message is long enough, and never fewer than
//    bytes / CCL_ATL_LARGE_MSG_SIZE (1 GiB), so that no single transport message exceeds that size;
//  * allgather(v): the ring form is cut per worker (part k gathers the k-th slice of every rank's block),
//    multi_bcast and flat already spread their peers over sub-schedules, direct / naive stay whole;
//  * alltoall(v): naive and scatter are cut into min(ranks, workers) parts (part k moves the k-th slice of
//    every block), in-place calls stay whole;
//  * reduce_scatter stays whole; send / recv are cut into pieces of at most the large-message size inside
//    their one schedule (build_cpu).
int part_count(const host_comm& comm, const coll_param& p, size_t bytes, const std::string& algo_name) {
    const int workers = executor::get().worker_count();
    const env_data& env = env_data::get();
    const bool is_bcast = p.ctype == coll_bcast || p.ctype == coll_broadcast;
    const bool reduce_like = p.ctype == coll_allreduce || p.ctype == coll_reduce || is_bcast;
    if (reduce_like) {
        const size_t esz = dtype_size(p.dtype);
        const size_t big = std::max<size_t>(env.large_msg_size, 1);
        size_t parts = 1;
        if (is_bcast && env.bcast_part_count > 0)
            // CCL_BCAST_PART_COUNT fixes the split of a broadcast
            parts = std::min<size_t>(std::min<size_t>(env.bcast_part_count, 64), std::max<size_t>(p.count, 1));
        else if (workers > 1 && p.count >= (size_t)workers * 64 && bytes > env.max_short_size &&
                 bytes >= (size_t)workers * env.min_chunk_size)
            // CCL_MAX_SHORT_SIZE keeps messages up to that size whole (reference parallelizer.cpp:224-235)
            parts = workers;
        const size_t need = (p.count * esz + big - 1) / big;
        parts = std::max(parts, std::min<size_t>(need, 1024));
        return (int)std::max<size_t>(1, std::min(parts, std::max<size_t>(p.count, 1)));
    }
    if (workers <= 1)
        return 1;
    if (p.ctype == coll_allgather || p.ctype == coll_allgatherv) {
        if (algo_name != "ring" || !p.recv_bufs.empty())
            return 1;
        size_t least = (size_t)-1;
        if (p.ctype == coll_allgather)
            least = p.count;
        else
            for (size_t c : p.recv_counts)
                least = std::min(least, c);
        if (bytes <= env.max_short_size || least < (size_t)workers * 64)
            return 1;
        return workers;
    }
    if (p.ctype == coll_alltoall || p.ctype == coll_alltoallv) {
        if (algo_name == "direct" || p.send_buf == p.recv_buf || !p.send_buf)
            return 1;
        // both sides of every block must cut it alike: the cut depends on the block sizes only when all of them
        // are long enough, which a rank can check for its own blocks; equal blocks (alltoall) always qualify
        if (p.ctype == coll_alltoallv)
            return 1;
        if (bytes <= env.max_short_size || p.count < (size_t)workers * 64)
            return 1;
        return std::min(comm.size(), workers);
    }
    return 1;
}

std::unique_ptr<master_sched> build_master(host_comm& comm, const coll_param& p, const coll_attr& attr,
                                           uint64_t sched_id) {
    std::unique_ptr<master_sched> m(new master_sched(&comm, sched_id));
    const env_data& env = env_data::get();
    static std::atomic<int> lifo_counter{ 0 };
    m->priority = env.priority_mode == priority_mode_t::lifo
                      ? lifo_counter.fetch_add(1)
                      : (env.priority_mode == priority_mode_t::direct ? attr.priority : 0);
    if (p.ctype == coll_barrier)
        m->priority = 1 << 30; // barriers drain first
    const size_t bytes = selection_bytes(comm, p);
    std::string algo_name;
    if (p.ctype != coll_barrier && p.ctype != coll_send && p.ctype != coll_recv) {
        selector_param sp;
        sp.ctype = p.ctype;
        sp.comm_size = comm.size();
        sp.vector_buf = !p.recv_bufs.empty();
        sp.custom_fn = attr.reduction_fn != nullptr;
        sp.scaleout = attr.scaleout;
        sp.count = p.count;
        sp.bytes = bytes;
        algo_name = algorithm_selector::get().select_cpu(sp);
    }
    const int parts = part_count(comm, p, bytes, algo_name);
    std::vector<size_t> cnt, off;
    algo::block_partition(p.count, parts, cnt, off);
    std::vector<std::function<bool()>> deps;
    for (auto& d : p.deps)
        if (d)
            deps.push_back([d] { return d->test(); });
    for (int i = 0; i < parts; i++) {
        sched* s = m->add_partial(i % executor::get().worker_count()); // more parts than workers: round robin
        if (!deps.empty()) {
            s->add<deps_entry>(deps);
            s->add_barrier();
        }
        if (parts == 1)
            build_cpu(*s, comm, p, attr, 0, p.count);
        else if (p.ctype == coll_allgather || p.ctype == coll_allgatherv || p.ctype == coll_alltoall)
            build_cpu(*s, comm, p, attr, 0, p.count, i, parts); // part i: the i-th slice of every block
        else
            build_cpu(*s, comm, p, attr, off[i], cnt[i]);
    }
    if (env.sched_dump) {
        std::string d;
        for (auto& s : m->partials())
            s->dump(d);
        LOG_INFO("built ", coll_name(p.ctype), ": ", d);
    }
    return m;
}

// host staging of device buffers (the node has no device communicator, or kernels are disabled)
event_ptr staged_device_coll(host_comm& comm, coll_param p, const coll_attr& attr);

// ---- device path ----------------------------------------------------------------------------
event_ptr device_coll(host_comm& comm, coll_param& p, const coll_attr& attr) {
    if (!comm.has_device()) {
        // first device operation: the heap is created on the device that owns the buffers
        const void* probe = p.send_buf ? p.send_buf : (p.recv_buf ? p.recv_buf : (p.recv_bufs.empty() ? nullptr : p.recv_bufs[0]));
        cudaPointerAttributes pa;
        if (probe && cudaPointerGetAttributes(&pa, probe) == cudaSuccess && pa.type == cudaMemoryTypeDevice)
            CUDA_CHECK(cudaSetDevice(pa.device));
        else
            (void)cudaGetLastError();
    }
    gpu::device_comm* dc = comm.device();
    cudaStream_t st = (cudaStream_t)p.stream;
    CUDA_CHECK(cudaSetDevice(dc->device_id()));
    const int N = comm.size(), r = comm.rank();
    const size_t esz = dtype_size(p.dtype);
    stats().device_calls[p.ctype]++;
    gpu::launch_opts o;
    o.scale = attr.scale;
    o.do_scale = attr.do_scale;
    const size_t sel_bytes = selection_bytes(comm, p);
    std::string forced = attr.gpu_algo.empty() ? algorithm_selector::get().forced_gpu(p.ctype, sel_bytes) : attr.gpu_algo;
    if (!forced.empty()) {
        o.algo = gpu::gpu_algo_from_name(forced);
        CCL_THROW_IF_NOT(o.algo >= 0, "unknown GPU algorithm ", forced);
    }
    const int out_dt = attr.out_dtype >= 0 ? attr.out_dtype : p.dtype;
    dev::rank_args ra;
    std::memset(&ra, 0, sizeof(ra));
    ra.send = p.send_buf;
    ra.recv = p.recv_buf;
    switch (p.ctype) {
        case coll_allreduce: gpu::launch_allreduce(*dc, &ra, p.count, p.dtype, out_dt, p.reduction, o, st); break;
        case coll_reduce_scatter:
            gpu::launch_reduce_scatter(*dc, &ra, p.count, p.dtype, out_dt, p.reduction, o, st);
            break;
        case coll_reduce: gpu::launch_reduce(*dc, &ra, p.count, p.dtype, out_dt, p.reduction, p.root, o, st); break;
        case coll_allgather:
        case coll_allgatherv: {
            std::vector<size_t> counts = p.ctype == coll_allgather ? std::vector<size_t>(N, p.count) : p.recv_counts;
            if (!p.recv_bufs.empty()) {
                // one destination buffer per rank: a broadcast per contributor
                for (int q = 0; q < N; q++) {
                    dev::rank_args b;
                    std::memset(&b, 0, sizeof(b));
                    b.send = q == r ? (p.send_buf ? p.send_buf : p.recv_bufs[q]) : nullptr;
                    b.recv = p.recv_bufs[q];
                    gpu::launch_broadcast(*dc, &b, counts[q] * esz, q, o, st);
                }
                break;
            }
            std::vector<size_t> offs = prefix(counts);
            for (int q = 0; q < N; q++) {
                ra.scount[q] = counts[q] * esz;
                ra.sdispl[q] = offs[q] * esz;
            }
            gpu::launch_allgatherv(*dc, &ra, o, st);
            break;
        }
        case coll_alltoall:
        case coll_alltoallv: {
            std::vector<size_t> sc = p.ctype == coll_alltoall ? std::vector<size_t>(N, p.count) : p.send_counts;
            std::vector<size_t> rc = p.ctype == coll_alltoall ? std::vector<size_t>(N, p.count) : p.recv_counts;
            std::vector<size_t> so = prefix(sc), ro = prefix(rc);
            for (int q = 0; q < N; q++) {
                ra.scount[q] = sc[q] * esz;
                ra.sdispl[q] = so[q] * esz;
                ra.rcount[q] = rc[q] * esz;
                ra.rdispl[q] = ro[q] * esz;
            }
            o.uniform = p.ctype == coll_alltoall;
            gpu::launch_alltoallv(*dc, &ra, o, st);
            break;
        }
        case coll_barrier: gpu::launch_barrier(*dc, st); break;
        case coll_bcast:
            ra.send = r == p.root ? p.recv_buf : nullptr;
            gpu::launch_broadcast(*dc, &ra, p.count * esz, p.root, o, st);
            break;
        case coll_broadcast:
            ra.send = r == p.root ? (p.send_buf ? p.send_buf : p.recv_buf) : nullptr;
            gpu::launch_broadcast(*dc, &ra, p.count * esz, p.root, o, st);
            break;
        case coll_send:
        case coll_recv: {
            dev::p2p_ops ops{};
            ops.n = 1;
            ops.op[0] = dev::p2p_op{ p.send_buf, p.recv_buf, p.count * esz, p.peer, p.ctype == coll_send ? 1 : 0 };
            gpu::launch_sendrecv(*dc, &ops, st);
            break;
        }
        default: CCL_THROW("unsupported device collective ", (int)p.ctype);
    }
    if (env_data::get().cuda_check_nan && p.recv_buf &&
        (p.ctype == coll_allreduce || p.ctype == coll_reduce_scatter || (p.ctype == coll_reduce && r == p.root)))
        gpu::launch_check_finite(*dc, p.recv_buf, p.count, out_dt, st);
    return std::make_shared<cuda_event_impl>(dc, st);
}

// Allreduce of device buffers across nodes, in three steps: reduce_scatter inside the node (device
// kernels over NVLink), allreduce of this rank's slice across the nodes (host path on the sub-communicator
// of equal local ranks, through pinned memory), all-gather inside the node.  The scheme of the reference's
// scale-out allreduce (src/coll/algorithms/allreduce/sycl/allreduce_sycl.cpp:170-384 with
// coll_util.cpp:553-642 for the host hop).  Needs the same number of ranks on every node and a count that
// splits evenly among them; otherwise the whole buffer takes the host path.
bool hier_allreduce_possible(host_comm& comm, const coll_param& p, const coll_attr& attr) {
    // CCL_TOPO_ALGO=0 switches the topology-aware (node / cross-node) composition off
    if (p.ctype != coll_allreduce || !env_data::get().cuda_kernels || !env_data::get().topo_algo ||
        attr.reduction_fn || attr.out_dtype >= 0 || attr.do_scale)
        return false;
    const int L = comm.local_size();
    if (L <= 0 || comm.size() % L != 0 || p.count % (size_t)L != 0 || p.count == 0)
        return false;
    const std::vector<int>& h = comm.host_index();
    std::vector<int> per_host;
    for (int v : h) {
        if ((size_t)v >= per_host.size())
            per_host.resize(v + 1, 0);
        per_host[v]++;
    }
    for (int c : per_host)
        if (c != L)
            return false;
    return true;
}

event_ptr hier_device_allreduce(host_comm& comm, coll_param& p, const coll_attr& attr) {
    auto node = comm.node_comm();
    auto r2r = comm.r2r_comm();
    const int L = node->size();
    const size_t esz = dtype_size(p.dtype);
    const size_t rc = p.count / (size_t)L, slice_bytes = rc * esz;
    cudaStream_t st = (cudaStream_t)p.stream;
    stats().device_calls[coll_allreduce]++;

    // scratch: this rank's slice on the device, its mirror in pinned host memory (kept by the communicator, grown on demand)
    struct scratch {
        cudaEvent_t last = nullptr; // recorded behind the last asynchronous use
        void* dev = nullptr;
        void* host = nullptr;
        size_t cap = 0;
        ~scratch() {
            if (dev)
                cudaFree(dev);
            if (host)
                cudaFreeHost(host);
            if (last)
                cudaEventDestroy(last);
        }
    };
    // the scratch belongs to the communicator (released with its device state); `last` orders a later call on
    // another stream behind the asynchronous tail of this one
    std::shared_ptr<void>& slot = comm.device_scratch(0);
    if (!slot)
        slot = std::make_shared<scratch>();
    scratch& sc = *std::static_pointer_cast<scratch>(slot);
    if (!sc.last)
        CUDA_CHECK(cudaEventCreateWithFlags(&sc.last, cudaEventDisableTiming));
    else
        CUDA_CHECK(cudaStreamWaitEvent(st, sc.last, 0));
    if (sc.cap < slice_bytes) {
        if (sc.dev)
            CUDA_CHECK(cudaFree(sc.dev));
        if (sc.host)
            CUDA_CHECK(cudaFreeHost(sc.host));
        sc.dev = sc.host = nullptr;
        sc.cap = 0;
        CUDA_CHECK(cudaMalloc(&sc.dev, slice_bytes));
        CUDA_CHECK(cudaMallocHost(&sc.host, slice_bytes));
        sc.cap = slice_bytes;
    }

    // The message travels in `chunks` parts (CCL_ALLREDUCE_PIPE_CHUNK_COUNT, as in the reference: 0 or 1 = one part):
    // the node-level reduce_scatter of every part is queued on the stream at once, each followed by the copy of
    // its slice to pinned memory; the host then takes the parts in order, so that the cross-node allreduce of part c
    // runs while the GPU still reduces parts c + 1 .., and the node allgather of part c while the network carries
    // part c + 1.  A part must split evenly among the node's ranks.
    size_t chunks = std::max<size_t>(1, env_data::get().allreduce_pipe_chunk_count);
    while (chunks > 1 && (p.count % (chunks * (size_t)L) != 0 || p.count / chunks < (size_t)L))
        chunks--;
    const size_t part = p.count / chunks; // elements of one part of the message
    const size_t prc = part / (size_t)L, pbytes = prc * esz; // my slice of one part
    coll_attr plain;
    std::vector<cudaEvent_t> staged(chunks, nullptr);
    std::vector<event_ptr> reduced(chunks);
    // 1. inside the node: my slice of the node-wide sum, part by part
    for (size_t c = 0; c < chunks; c++) {
        coll_param rs = p;
        rs.ctype = coll_reduce_scatter;
        rs.send_buf = (const char*)p.send_buf + c * part * esz;
        rs.count = prc;
        rs.recv_buf = (char*)sc.dev + c * pbytes;
        rs.deps.clear();
        reduced[c] = device_coll(*node, rs, plain);
        CUDA_CHECK(cudaMemcpyAsync((char*)sc.host + c * pbytes, (char*)sc.dev + c * pbytes, pbytes, cudaMemcpyDeviceToHost, st));
        CUDA_CHECK(cudaEventCreateWithFlags(&staged[c], cudaEventDisableTiming));
        CUDA_CHECK(cudaEventRecord(staged[c], st));
    }
    // in place is safe: part c of recv is written only after every part of send has been reduced (stream order)
    event_ptr done;
    for (size_t c = 0; c < chunks; c++) {
        // 2. across the nodes: same slice on the ranks with my local index
        reduced[c]->wait(); // reports a device-side failure of the node stage
        CUDA_CHECK(cudaEventSynchronize(staged[c]));
        CUDA_CHECK(cudaEventDestroy(staged[c]));
        if (r2r->size() > 1) {
            coll_param ar;
            ar.ctype = coll_allreduce;
            ar.send_buf = (char*)sc.host + c * pbytes;
            ar.recv_buf = (char*)sc.host + c * pbytes;
            ar.count = prc;
            ar.dtype = p.dtype;
            ar.reduction = p.reduction;
            ar.device = false;
            coll_attr host_attr;
            host_attr.scaleout = true; // CCL_ALLREDUCE_SCALEOUT chooses the inter-node algorithm
            coll_create(*r2r, ar, host_attr)->wait();
        }
        CUDA_CHECK(cudaMemcpyAsync((char*)sc.dev + c * pbytes, (char*)sc.host + c * pbytes, pbytes, cudaMemcpyHostToDevice, st));
        // 3. inside the node: everybody gets every slice of the part
        coll_param ag = p;
        ag.ctype = coll_allgather;
        ag.send_buf = (char*)sc.dev + c * pbytes;
        ag.recv_buf = (char*)p.recv_buf + c * part * esz;
        ag.count = prc;
        ag.deps.clear();
        done = device_coll(*node, ag, plain);
    }
    CUDA_CHECK(cudaEventRecord(sc.last, st)); // the allgather still reads sc.dev: the next user of the scratch waits for it
    return done;
}

// reduce_scatter on device buffers across nodes.  Send buffers are ordered by global rank, which the
// check below requires to be node-major (rank = node * L + local).  The blocks are regrouped by local
// rank, the node-level reduce_scatter leaves on local rank l the node's partial sums of the blocks of
// every rank with local index l, and those ranks finish with a reduce_scatter among themselves on the
// host path (CCL_REDUCE_SCATTER_SCALEOUT chooses its algorithm).  Per rank N * count elements cross
// NVLink once and M * count elements cross the network stage, instead of N * count through the host.
bool hier_reduce_scatter_possible(host_comm& comm, const coll_param& p, const coll_attr& attr) {
    if (p.ctype != coll_reduce_scatter || !env_data::get().cuda_kernels || !env_data::get().topo_algo ||
        attr.reduction_fn || attr.out_dtype >= 0 || attr.do_scale || p.count == 0 || p.reduction == red_custom)
        return false;
    const int L = comm.local_size();
    if (L <= 0 || comm.size() % L != 0)
        return false;
    const std::vector<int>& h = comm.host_index();
    for (int r = 0; r < comm.size(); r++)
        if (h[r] != r / L)
            return false;
    return true;
}

event_ptr hier_device_reduce_scatter(host_comm& comm, coll_param& p, const coll_attr& attr) {
    (void)attr;
    auto node = comm.node_comm();
    auto r2r = comm.r2r_comm();
    const int L = node->size(), M = r2r->size();
    const size_t esz = dtype_size(p.dtype);
    const size_t block = p.count * esz; // what one rank receives
    cudaStream_t st = (cudaStream_t)p.stream;
    stats().device_calls[coll_reduce_scatter]++;
    struct scratch {
        cudaEvent_t last = nullptr; // recorded behind the last asynchronous use
        void *grouped = nullptr, *slice = nullptr, *host_in = nullptr, *host_out = nullptr;
        size_t cap_grouped = 0, cap_slice = 0, cap_out = 0;
        static void grow_dev(void*& ptr, size_t& cap, size_t want) {
            if (cap >= want)
                return;
            if (ptr)
                CUDA_CHECK(cudaFree(ptr));
            ptr = nullptr;
            cap = 0;
            CUDA_CHECK(cudaMalloc(&ptr, want));
            cap = want;
        }
        ~scratch() {
            if (grouped)
                cudaFree(grouped);
            if (slice)
                cudaFree(slice);
            if (host_in)
                cudaFreeHost(host_in);
            if (host_out)
                cudaFreeHost(host_out);
        }
    };
    // the scratch belongs to the communicator (released with its device state); `last` orders a later call on
    // another stream behind the asynchronous tail of this one
    std::shared_ptr<void>& slot = comm.device_scratch(1);
    if (!slot)
        slot = std::make_shared<scratch>();
    scratch& sc = *std::static_pointer_cast<scratch>(slot);
    if (!sc.last)
        CUDA_CHECK(cudaEventCreateWithFlags(&sc.last, cudaEventDisableTiming));
    else
        CUDA_CHECK(cudaStreamWaitEvent(st, sc.last, 0));
    const size_t slice_bytes = (size_t)M * block;
    if (sc.cap_slice < slice_bytes) {
        if (sc.host_in)
            CUDA_CHECK(cudaFreeHost(sc.host_in));
        sc.host_in = nullptr;
        CUDA_CHECK(cudaMallocHost(&sc.host_in, slice_bytes));
    }
    scratch::grow_dev(sc.slice, sc.cap_slice, slice_bytes);
    if (sc.cap_out < block) {
        if (sc.host_out)
            CUDA_CHECK(cudaFreeHost(sc.host_out));
        sc.host_out = nullptr;
        sc.cap_out = 0;
        CUDA_CHECK(cudaMallocHost(&sc.host_out, block));
        sc.cap_out = block;
    }
    // 1. node-major -> local-rank-major (nothing to move when one of the two dimensions is 1)
    const void* grouped = p.send_buf;
    if (L > 1 && M > 1) {
        scratch::grow_dev(sc.grouped, sc.cap_grouped, (size_t)L * M * block);
        gpu::launch_transpose_blocks(p.send_buf, sc.grouped, M, L, block, st);
        grouped = sc.grouped;
    }
    // 2. inside the node: the partial sums of the M blocks that belong to my local index
    coll_param rs = p;
    rs.send_buf = grouped;
    rs.recv_buf = sc.slice;
    rs.count = (size_t)M * p.count;
    rs.deps.clear();
    coll_attr plain;
    device_coll(*node, rs, plain)->wait();
    CUDA_CHECK(cudaMemcpyAsync(sc.host_in, sc.slice, slice_bytes, cudaMemcpyDeviceToHost, st));
    CUDA_CHECK(cudaStreamSynchronize(st));
    // 3. among the ranks with my local index, one per node: block m goes to node m
    coll_param rx;
    rx.ctype = coll_reduce_scatter;
    rx.send_buf = sc.host_in;
    rx.recv_buf = sc.host_out;
    rx.count = p.count;
    rx.dtype = p.dtype;
    rx.reduction = p.reduction;
    rx.device = false;
    coll_attr host_attr;
    host_attr.scaleout = true;
    coll_create(*r2r, rx, host_attr)->wait();
    CUDA_CHECK(cudaMemcpyAsync(p.recv_buf, sc.host_out, block, cudaMemcpyHostToDevice, st));
    CUDA_CHECK(cudaStreamSynchronize(st)); // the pinned buffer is reused by the next call
    return make_completed_event();
}

// allgather of equal blocks on device buffers across nodes, on request (CCL_ALLGATHER=topo or
// CCL_ALLGATHERV=topo; the default stages the whole result through the host).  The mirror image of the
// reduce_scatter above: the ranks with my local index exchange their blocks on the host path (M blocks per
// rank instead of N), the node gathers the M-block slices on the device, and a block transpose turns
// the local-rank-major result into rank order.
bool hier_allgather_possible(host_comm& comm, const coll_param& p, const coll_attr& attr) {
    if ((p.ctype != coll_allgather && p.ctype != coll_allgatherv) || !env_data::get().cuda_kernels ||
        !env_data::get().topo_algo || attr.out_dtype >= 0 || !p.recv_bufs.empty() || p.count == 0)
        return false;
    if (p.ctype == coll_allgatherv)
        for (size_t c : p.recv_counts)
            if (c != p.count)
                return false;
    const size_t bytes = p.count * dtype_size(p.dtype) * (size_t)comm.size();
    if (!algorithm_selector::get().requested(p.ctype, bytes, "topo"))
        return false;
    const int L = comm.local_size();
    if (L <= 0 || comm.size() % L != 0)
        return false;
    const std::vector<int>& h = comm.host_index();
    for (int r = 0; r < comm.size(); r++)
        if (h[r] != r / L)
            return false;
    return true;
}

event_ptr hier_device_allgather(host_comm& comm, coll_param& p, const coll_attr& attr) {
    (void)attr;
    auto node = comm.node_comm();
    auto r2r = comm.r2r_comm();
    const int L = node->size(), M = r2r->size();
    const size_t esz = dtype_size(p.dtype);
    const size_t block = p.count * esz;
    const size_t slice_bytes = (size_t)M * block;
    cudaStream_t st = (cudaStream_t)p.stream;
    stats().device_calls[p.ctype]++;
    struct scratch {
        cudaEvent_t last = nullptr; // recorded behind the last asynchronous use
        void *host_in = nullptr, *host_out = nullptr, *slice = nullptr, *grouped = nullptr;
        size_t cap_in = 0, cap_out = 0, cap_slice = 0, cap_grouped = 0;
        static void grow_host(void*& ptr, size_t& cap, size_t want) {
            if (cap >= want)
                return;
            if (ptr)
                CUDA_CHECK(cudaFreeHost(ptr));
            ptr = nullptr;
            cap = 0;
            CUDA_CHECK(cudaMallocHost(&ptr, want));
            cap = want;
        }
        static void grow_dev(void*& ptr, size_t& cap, size_t want) {
            if (cap >= want)
                return;
            if (ptr)
                CUDA_CHECK(cudaFree(ptr));
            ptr = nullptr;
            cap = 0;
            CUDA_CHECK(cudaMalloc(&ptr, want));
            cap = want;
        }
        ~scratch() {
            if (host_in)
                cudaFreeHost(host_in);
            if (host_out)
                cudaFreeHost(host_out);
            if (slice)
                cudaFree(slice);
            if (grouped)
                cudaFree(grouped);
        }
    };
    // the scratch belongs to the communicator (released with its device state); `last` orders a later call on
    // another stream behind the asynchronous tail of this one
    std::shared_ptr<void>& slot = comm.device_scratch(2);
    if (!slot)
        slot = std::make_shared<scratch>();
    scratch& sc = *std::static_pointer_cast<scratch>(slot);
    if (!sc.last)
        CUDA_CHECK(cudaEventCreateWithFlags(&sc.last, cudaEventDisableTiming));
    else
        CUDA_CHECK(cudaStreamWaitEvent(st, sc.last, 0));
    scratch::grow_host(sc.host_in, sc.cap_in, block);
    scratch::grow_host(sc.host_out, sc.cap_out, slice_bytes);
    scratch::grow_dev(sc.slice, sc.cap_slice, slice_bytes);
    // 1. my block to the ranks with my local index, theirs to me (in place: my block sits inside recv)
    const void* mine = p.send_buf ? p.send_buf : (const char*)p.recv_buf + (size_t)comm.rank() * block;
    CUDA_CHECK(cudaMemcpyAsync(sc.host_in, mine, block, cudaMemcpyDeviceToHost, st));
    CUDA_CHECK(cudaStreamSynchronize(st));
    coll_param ag;
    ag.ctype = coll_allgather;
    ag.send_buf = sc.host_in;
    ag.recv_buf = sc.host_out;
    ag.count = p.count;
    ag.dtype = p.dtype;
    ag.device = false;
    coll_attr host_attr;
    host_attr.scaleout = true;
    coll_create(*r2r, ag, host_attr)->wait();
    CUDA_CHECK(cudaMemcpyAsync(sc.slice, sc.host_out, slice_bytes, cudaMemcpyHostToDevice, st));
    // 2. inside the node: everybody's slice, local-rank-major; 3. into rank order
    const bool regroup = L > 1 && M > 1;
    void* gathered = p.recv_buf;
    if (regroup) {
        scratch::grow_dev(sc.grouped, sc.cap_grouped, (size_t)L * slice_bytes);
        gathered = sc.grouped;
    }
    coll_param ng;
    ng.ctype = coll_allgather;
    ng.send_buf = sc.slice;
    ng.recv_buf = gathered;
    ng.count = (size_t)M * p.count;
    ng.dtype = p.dtype;
    ng.device = true;
    ng.stream = p.stream;
    coll_attr plain;
    event_ptr ev = device_coll(*node, ng, plain);
    if (regroup) {
        ev->wait();
        gpu::launch_transpose_blocks(sc.grouped, p.recv_buf, L, M, block, st);
    }
    CUDA_CHECK(cudaStreamSynchronize(st)); // scratch memory is reused by the next call
    return make_completed_event();
}

// broadcast / reduce of device buffers across nodes (rank = node * L + local on every node, L ranks each).
// broadcast: the root's buffer travels on the host path among the ranks that share the root's local index (one
// per node), then every node broadcasts it on the device from that rank.  reduce: every node reduces on the
// device to the rank with the root's local index, those ranks finish among themselves on the host path.  One rank
// per node stages through pinned memory instead of every rank (the reference composes its scale-out broadcast and
// reduce the same way: node stage, cross-node stage among equal local ranks; src/coll/algorithms/bcast.cpp:243,
// reduce.cpp:554).
bool hier_rooted_possible(host_comm& comm, const coll_param& p, const coll_attr& attr) {
    const bool bc = p.ctype == coll_bcast || p.ctype == coll_broadcast;
    if ((!bc && p.ctype != coll_reduce) || !env_data::get().cuda_kernels || !env_data::get().topo_algo || p.count == 0 ||
        attr.out_dtype >= 0 || attr.do_scale)
        return false;
    if (p.ctype == coll_reduce && (attr.reduction_fn || p.reduction == red_custom))
        return false;
    const int L = comm.local_size();
    if (L <= 0 || comm.size() % L != 0)
        return false;
    const std::vector<int>& h = comm.host_index();
    for (int r = 0; r < comm.size(); r++)
        if (h[r] != r / L)
            return false;
    return true;
}

namespace {
// the node stage runs kernels that wait for the rank with the data: the others enter it only once that rank is
// there too (it may have spent long on the network), so that their bounded device waits do not run out
void node_host_barrier(host_comm& node) {
    if (node.size() <= 1)
        return;
    coll_param b;
    b.ctype = coll_barrier;
    b.device = false;
    coll_attr a;
    coll_create(node, b, a)->wait();
}
} // namespace

event_ptr hier_device_broadcast(host_comm& comm, coll_param& p, const coll_attr& attr) {
    (void)attr;
    auto node = comm.node_comm();
    auto r2r = comm.r2r_comm();
    const int L = node->size();
    const int lroot = p.root % L, nroot = p.root / L;
    cudaStream_t st = (cudaStream_t)p.stream;
    stats().device_calls[p.ctype]++;
    const size_t bytes = p.count * dtype_size(p.dtype);
    if (comm.rank() == p.root && p.ctype == coll_broadcast && p.send_buf && p.send_buf != p.recv_buf)
        CUDA_CHECK(cudaMemcpyAsync(p.recv_buf, p.send_buf, bytes, cudaMemcpyDeviceToDevice, st));
    // 1. across the nodes, among the ranks with the root's local index
    if (node->rank() == lroot && r2r->size() > 1) {
        coll_param x;
        x.ctype = coll_bcast;
        x.recv_buf = p.recv_buf;
        x.count = p.count;
        x.dtype = p.dtype;
        x.root = nroot;
        x.device = true;
        x.stream = p.stream;
        coll_attr plain;
        staged_device_coll(*r2r, x, plain);
    }
    // 2. inside every node, from that rank
    node_host_barrier(*node);
    coll_param nb;
    nb.ctype = coll_bcast;
    nb.recv_buf = p.recv_buf;
    nb.count = p.count;
    nb.dtype = p.dtype;
    nb.root = lroot;
    nb.device = true;
    nb.stream = p.stream;
    coll_attr none;
    return device_coll(*node, nb, none);
}

event_ptr hier_device_reduce(host_comm& comm, coll_param& p, const coll_attr& attr) {
    (void)attr;
    auto node = comm.node_comm();
    auto r2r = comm.r2r_comm();
    const int L = node->size();
    const int lroot = p.root % L, nroot = p.root / L;
    cudaStream_t st = (cudaStream_t)p.stream;
    stats().device_calls[coll_reduce]++;
    const size_t bytes = p.count * dtype_size(p.dtype);
    struct scratch {
        cudaEvent_t last = nullptr;
        void* dev = nullptr;
        size_t cap = 0;
        ~scratch() {
            if (dev)
                cudaFree(dev);
            if (last)
                cudaEventDestroy(last);
        }
    };
    const bool holder = node->rank() == lroot; // receives its node's partial result
    void* partial = nullptr;
    if (holder && comm.rank() == p.root)
        partial = p.recv_buf;
    else if (holder) {
        std::shared_ptr<void>& slot = comm.device_scratch(3);
        if (!slot)
            slot = std::make_shared<scratch>();
        scratch& sc = *std::static_pointer_cast<scratch>(slot);
        if (!sc.last)
            CUDA_CHECK(cudaEventCreateWithFlags(&sc.last, cudaEventDisableTiming));
        else
            CUDA_CHECK(cudaStreamWaitEvent(st, sc.last, 0));
        if (sc.cap < bytes) {
            if (sc.dev)
                CUDA_CHECK(cudaFree(sc.dev));
            sc.dev = nullptr;
            sc.cap = 0;
            CUDA_CHECK(cudaMalloc(&sc.dev, bytes));
            sc.cap = bytes;
        }
        partial = sc.dev;
    }
    // 1. inside the node, to the rank with the root's local index
    coll_param nr = p;
    nr.ctype = coll_reduce;
    nr.recv_buf = partial;
    nr.root = lroot;
    nr.deps.clear();
    coll_attr plain;
    event_ptr ev = device_coll(*node, nr, plain);
    // 2. across the nodes, among those ranks, to the root's node (synchronous: it stages through pinned memory)
    if (holder && r2r->size() > 1) {
        ev->wait();
        coll_param x;
        x.ctype = coll_reduce;
        x.send_buf = partial;
        x.recv_buf = r2r->rank() == nroot ? partial : nullptr;
        x.count = p.count;
        x.dtype = p.dtype;
        x.reduction = p.reduction;
        x.root = nroot;
        x.device = true;
        x.stream = p.stream;
        coll_attr host_attr;
        host_attr.scaleout = true;
        return staged_device_coll(*r2r, x, host_attr);
    }
    return ev;
}

bool same_node(host_comm& comm) {
    const std::vector<int>& h = comm.host_index();
    for (int v : h)
        if (v != h[0])
            return false;
    return true;
}

event_ptr staged_device_coll(host_comm& comm, coll_param p, const coll_attr& attr) {
    // device -> pinned host, CPU collective, host -> device; synchronous
    cudaStream_t st = (cudaStream_t)p.stream;
    const int N = comm.size();
    const size_t esz = dtype_size(p.dtype);
    auto sz = [&](bool send) -> size_t {
        switch (p.ctype) {
            case coll_allgather: return (send ? p.count : p.count * N) * esz;
            case coll_allgatherv: return (send ? p.count : total(p.recv_counts)) * esz;
            case coll_alltoall: return p.count * N * esz;
            case coll_alltoallv: return total(send ? p.send_counts : p.recv_counts) * esz;
            case coll_reduce_scatter: return (send ? p.count * N : p.count) * esz;
            case coll_barrier: return 0;
            default: return p.count * esz;
        }
    };
    CCL_THROW_IF_NOT(p.recv_bufs.empty(), "vector buffers on device need the device communicator");
    const size_t sb = p.send_buf ? sz(true) : 0, rb = p.recv_buf ? sz(false) : 0;
    std::vector<char> hs(sb), hr(rb);
    const void* dsend = p.send_buf;
    void* drecv = p.recv_buf;
    if (sb)
        CUDA_CHECK(cudaMemcpyAsync(hs.data(), dsend, sb, cudaMemcpyDeviceToHost, st));
    if (rb && (p.ctype == coll_bcast || coll_is_inplace(comm, p)))
        CUDA_CHECK(cudaMemcpyAsync(hr.data(), drecv, rb, cudaMemcpyDeviceToHost, st));
    CUDA_CHECK(cudaStreamSynchronize(st));
    const bool inplace = dsend && drecv && coll_is_inplace(comm, p);
    coll_param h = p;
    h.device = false;
    h.stream = nullptr;
    h.recv_buf = rb ? hr.data() : nullptr;
    if (inplace) {
        size_t off = 0;
        if (p.ctype == coll_allgather || p.ctype == coll_allgatherv || p.ctype == coll_reduce_scatter)
            off = (const char*)dsend - (const char*)drecv;
        h.send_buf = hr.data() + off;
        if (p.ctype == coll_reduce_scatter) { // recv sits inside send
            h.send_buf = hs.data();
            h.recv_buf = hs.data() + ((const char*)drecv - (const char*)dsend);
        }
    }
    else
        h.send_buf = sb ? hs.data() : nullptr;
    coll_attr a = attr;
    a.synchronous = true;
    coll_create(comm, h, a);
    if (rb) {
        const void* src = (inplace && p.ctype == coll_reduce_scatter) ? h.recv_buf : hr.data();
        CUDA_CHECK(cudaMemcpyAsync(drecv, src, rb, cudaMemcpyHostToDevice, st));
        CUDA_CHECK(cudaStreamSynchronize(st));
    }
    return make_completed_event();
}

// ---- schedule: cached or new -----------------------------------------------------------------
constexpr uint64_t NO_SCHED_ID = ~0ull;

event_ptr start_sched(host_comm& comm, const coll_param& p, const coll_attr& attr, uint64_t fixed_id) {
    const env_data& env = env_data::get();
    const bool cacheable = attr.to_cache && p.ctype != coll_send && p.ctype != coll_recv && p.deps.empty() &&
                           (env.cache_key == cache_key_t::full || !attr.match_id.empty());
    if (p.ctype == coll_barrier && env.cache_flush)
        comm.cache().flush();
    master_sched* m = nullptr;
    std::unique_ptr<master_sched> owned;
    std::shared_ptr<master_sched> cached;
    uint64_t launch_id = executor::KEEP_ID;
    if (cacheable) {
        const std::string key = coll_cache_key(comm, p, attr);
        cached = comm.cache().find(key);
        m = cached.get();
        if (m) {
            stats().cache_hits++;
            // every call draws an id, hit or miss, so the ranks stay in step whatever their caches hold
            if (fixed_id == NO_SCHED_ID)
                launch_id = comm.next_sched_id();
        }
        else {
            auto fresh = build_master(comm, p, attr, fixed_id != NO_SCHED_ID ? fixed_id : comm.next_sched_id());
            cached = std::move(fresh);
            m = cached.get();
            comm.cache().insert(key, cached);
        }
    }
    else {
        uint64_t sid;
        if (fixed_id != NO_SCHED_ID)
            sid = fixed_id;
        else if (p.ctype == coll_send)
            sid = atl_tag::PT2PT_SCHED - 8 - (comm.p2p_send_seq(p.peer) & 0xff);
        else if (p.ctype == coll_recv)
            sid = atl_tag::PT2PT_SCHED - 8 - (comm.p2p_recv_seq(p.peer) & 0xff);
        else
            sid = comm.next_sched_id();
        owned = build_master(comm, p, attr, sid);
        m = owned.get();
    }
    const uint64_t ticket = executor::get().start(m, launch_id);
    return std::make_shared<host_event>(m, ticket, std::move(owned), std::move(cached));
}

// ---- unordered collectives -------------------------------------------------------------------
// With CCL_UNORDERED_COLL=1 operations that carry a match_id may be issued in a different order
// on every rank.  Rank 0 of the communicator names them: the k-th match_id it meets gets the k-th
// reserved schedule id, and coordination message k (a 256-byte record sent to every rank) tells
// the others.  A rank that issues a match_id it cannot name yet parks the operation behind a
// deferred event and posts a receive for the next coordination message; when the message arrives
// (on a worker thread) the parked operations of that match_id start, and another receive is
// posted while anything is still parked.  Messages that arrive for match_ids the rank has not
// issued yet are simply remembered.  Same role as the reference's ccl_unordered_coll_manager
// (src/unordered_coll/unordered_coll.cpp:96-300), which clones the communicator per match_id;
// here a schedule id inside the same communicator is enough because messages match by tag.
class deferred_event : public event_impl {
public:
    void bind(event_ptr e) {
        std::lock_guard<std::mutex> lk(mu_);
        real_ = std::move(e);
    }
    void fail(const std::string& why) {
        std::lock_guard<std::mutex> lk(mu_);
        error_ = why;
    }
    void wait() override {
        for (;;) {
            event_ptr r = current();
            if (r) {
                r->wait();
                return;
            }
            executor::get().progress();
        }
    }
    bool test() override {
        event_ptr r = current();
        if (r)
            return r->test();
        executor::get().progress();
        return false;
    }
    void* native() override { return nullptr; }

private:
    event_ptr current() {
        std::lock_guard<std::mutex> lk(mu_);
        if (!error_.empty())
            CCL_THROW("postponed operation failed: ", error_);
        return real_;
    }
    std::mutex mu_;
    event_ptr real_;
    std::string error_;
};

constexpr size_t UNORDERED_MSG_BYTES = 256;

struct unordered_state {
    struct parked {
        coll_param param;
        coll_attr attr;
        std::shared_ptr<deferred_event> ev;
    };
    struct round {
        char msg[UNORDERED_MSG_BYTES];
        std::unique_ptr<master_sched> m;
    };
    std::mutex mu;
    std::map<std::string, uint64_t> ids;
    std::map<std::string, std::vector<parked>> waiting;
    uint64_t rounds = 0; // coordination messages posted by this rank
    bool receiving = false;
    std::deque<std::unique_ptr<round>> live;
};

unordered_state& unordered_of(host_comm& comm) {
    static std::mutex create_mu;
    std::lock_guard<std::mutex> lk(create_mu);
    if (!comm.frontend_state)
        comm.frontend_state = std::make_shared<unordered_state>();
    return *static_cast<unordered_state*>(comm.frontend_state.get());
}

void unordered_post_round(host_comm& comm, unordered_state& st, const std::string* name);

// runs on a worker thread when coordination message k has arrived
void unordered_on_message(host_comm& comm, unordered_state& st, unordered_state::round* r, uint64_t k) {
    std::lock_guard<std::mutex> lk(st.mu);
    r->msg[UNORDERED_MSG_BYTES - 1] = 0;
    const std::string name(r->msg);
    const uint64_t sid = comm.unordered_sched_id(k);
    st.ids[name] = sid;
    st.receiving = false;
    auto it = st.waiting.find(name);
    if (it != st.waiting.end()) {
        // under the lock: a later operation with this match_id must not overtake the parked ones
        for (auto& w : it->second) {
            try {
                w.ev->bind(start_sched(comm, w.param, w.attr, sid));
            }
            catch (const std::exception& e) {
                w.ev->fail(e.what());
            }
        }
        st.waiting.erase(it);
    }
    if (!st.waiting.empty())
        unordered_post_round(comm, st, nullptr);
}

// st.mu is held.  name != nullptr: rank 0 announces it; otherwise post the receive of the next message
void unordered_post_round(host_comm& comm, unordered_state& st, const std::string* name) {
    // schedules of finished rounds are released a few rounds later, never from their own callback
    while (st.live.size() > 4 && st.live.front()->m->ticket_retired(1) && !st.live.front()->m->in_flight)
        st.live.pop_front();
    const uint64_t k = st.rounds++;
    std::unique_ptr<unordered_state::round> r(new unordered_state::round());
    std::memset(r->msg, 0, sizeof(r->msg));
    r->m.reset(new master_sched(&comm, atl_tag::UNORDERED_SCHED));
    r->m->priority = 1 << 29;
    sched* s = r->m->add_partial(0);
    if (name) {
        CCL_THROW_IF_NOT(name->size() < UNORDERED_MSG_BYTES, "match_id longer than ", UNORDERED_MSG_BYTES - 1,
                         " characters can not be used with unordered collectives");
        std::memcpy(r->msg, name->data(), name->size());
        for (int peer = 1; peer < comm.size(); peer++)
            s->add<send_entry>(r->msg, UNORDERED_MSG_BYTES, peer, k);
    }
    else {
        s->add<recv_entry>(r->msg, UNORDERED_MSG_BYTES, 0, k);
        unordered_state::round* raw = r.get();
        host_comm* c = &comm;
        unordered_state* stp = &st;
        r->m->user_complete = [c, stp, raw, k] { unordered_on_message(*c, *stp, raw, k); };
        st.receiving = true;
    }
    master_sched* m = r->m.get();
    st.live.push_back(std::move(r));
    executor::get().start(m);
}

event_ptr unordered_submit(host_comm& comm, const coll_param& p, const coll_attr& attr) {
    unordered_state& st = unordered_of(comm);
    std::lock_guard<std::mutex> lk(st.mu);
    auto it = st.ids.find(attr.match_id);
    if (it != st.ids.end())
        return start_sched(comm, p, attr, it->second);
    if (comm.rank() == 0) {
        const uint64_t sid = comm.unordered_sched_id(st.rounds);
        st.ids[attr.match_id] = sid;
        unordered_post_round(comm, st, &attr.match_id);
        return start_sched(comm, p, attr, sid);
    }
    auto ev = std::make_shared<deferred_event>();
    st.waiting[attr.match_id].push_back(unordered_state::parked{ p, attr, ev });
    stats().postponed++;
    if (!st.receiving)
        unordered_post_round(comm, st, nullptr);
    return ev;
}


} // namespace

// ---- entry point ----------------------------------------------------------------------------
event_ptr coll_create(host_comm& comm, coll_param& p, const coll_attr& attr) {
    const env_data& env = env_data::get();
    coll_validate(comm, p, attr);
    trace_range tr(1, coll_name(p.ctype), p.ctype == coll_barrier ? 0 : selection_bytes(comm, p));
    stats().calls[p.ctype]++;
    purge_recycle();

    // send/recv inside a group are posted at group_end
    if (tl_group_active) {
        CCL_THROW_IF_NOT(p.ctype == coll_send || p.ctype == coll_recv,
                         "only send and recv may be issued between group_start and group_end");
        auto ev = std::make_shared<group_event>();
        tl_group.push_back(group_item{ &comm, p, attr, ev });
        return ev;
    }

    const bool sync = attr.synchronous || env.op_sync || p.ctype == coll_barrier;
    const size_t esz = p.ctype == coll_barrier ? 0 : dtype_size(p.dtype);

    // ---- device buffers
    if (p.device) {
        for (auto& d : p.deps) // dependencies of a stream-ordered operation: wait on the host
            if (d)
                d->wait();
        event_ptr ev;
        if (env.fusion && !tl_no_fusion && env.cuda_kernels && same_node(comm) && comm.size() > 1) {
            // small allreduces of one stream are packed into one launch sequence; any other device operation of
            // this communicator first sends the waiting batch on its way (operation order)
            if (p.ctype == coll_allreduce && !sync && p.deps.empty()) {
                event_ptr fe = fusion_manager::get().try_add(comm, p, attr);
                if (fe)
                    return fe;
            }
            else
                fusion_manager::get().flush(&comm);
        }
        if (env.cuda_kernels && same_node(comm))
            ev = device_coll(comm, p, attr);
        else if (hier_allreduce_possible(comm, p, attr))
            ev = hier_device_allreduce(comm, p, attr);
        else if (hier_reduce_scatter_possible(comm, p, attr))
            ev = hier_device_reduce_scatter(comm, p, attr);
        else if (hier_allgather_possible(comm, p, attr))
            ev = hier_device_allgather(comm, p, attr);
        else if (hier_rooted_possible(comm, p, attr))
            ev = p.ctype == coll_reduce ? hier_device_reduce(comm, p, attr) : hier_device_broadcast(comm, p, attr);
        else
            ev = staged_device_coll(comm, p, attr);
        if (sync)
            ev->wait();
        return ev;
    }

    // ---- single rank: copy and complete (reference coll.cpp:96-130)
    if (comm.size() == 1) {
        for (auto& d : p.deps)
            if (d)
                d->wait();
        size_t bytes = 0;
        switch (p.ctype) {
            case coll_allgatherv: bytes = p.count * esz; break;
            case coll_alltoallv: bytes = p.send_counts[0] * esz; break;
            case coll_barrier: bytes = 0; break;
            default: bytes = p.count * esz;
        }
        void* dst = !p.recv_bufs.empty() ? p.recv_bufs[0] : p.recv_buf;
        if (bytes && p.send_buf && dst && p.send_buf != dst)
            std::memmove(dst, p.send_buf, bytes);
        return make_completed_event();
    }

    // ---- fusion of small allreduces; anything else first cuts the pending batch (operation order)
    if (env.fusion && !tl_no_fusion) {
        if (p.ctype == coll_allreduce && !sync) {
            event_ptr fe = fusion_manager::get().try_add(comm, p, attr);
            if (fe)
                return fe;
        }
        else
            fusion_manager::get().flush(&comm);
    }

    // ---- operations named by match_id may arrive in any order
    if (env.unordered_coll && !attr.match_id.empty() && p.ctype != coll_send && p.ctype != coll_recv) {
        event_ptr ev = unordered_submit(comm, p, attr);
        if (sync)
            ev->wait();
        return ev;
    }

    event_ptr ev = start_sched(comm, p, attr, NO_SCHED_ID);
    if (sync)
        ev->wait();
    return ev;
}

// ---- several buffers, one operation ----------------------------------------------------------------
namespace {
class multi_event : public event_impl {
public:
    explicit multi_event(std::vector<event_ptr> parts) : parts_(std::move(parts)) {}
    void wait() override {
        for (auto& e : parts_)
            e->wait();
    }
    bool test() override {
        for (auto& e : parts_)
            if (!e->test())
                return false;
        return true;
    }

private:
    std::vector<event_ptr> parts_;
};
} // namespace

event_ptr coll_allreduce_coalesced(host_comm& comm, const std::vector<const void*>& send, const std::vector<void*>& recv,
                                   const std::vector<size_t>& counts, int dtype, int reduction, const coll_attr& attr,
                                   void* stream, bool device) {
    const env_data& env = env_data::get();
    CCL_THROW_IF_NOT(send.size() == recv.size() && send.size() == counts.size(), "buffer and count lists differ in length");
    if (send.empty())
        return make_completed_event();
    const bool fused = device && env.cuda_kernels && same_node(comm) && comm.size() > 1 && attr.out_dtype < 0 &&
                       !attr.reduction_fn && reduction != red_custom && dtype <= dt_last_predefined && attr.gpu_algo.empty();
    if (fused) {
        if (!comm.has_device()) {
            cudaPointerAttributes pa;
            if (cudaPointerGetAttributes(&pa, recv[0]) == cudaSuccess && pa.type == cudaMemoryTypeDevice)
                CUDA_CHECK(cudaSetDevice(pa.device));
            else
                (void)cudaGetLastError();
        }
        gpu::device_comm* dc = comm.device();
        CUDA_CHECK(cudaSetDevice(dc->device_id()));
        stats().calls[coll_allreduce] += send.size();
        stats().device_calls[coll_allreduce] += send.size();
        gpu::launch_opts o;
        o.scale = attr.scale;
        o.do_scale = attr.do_scale;
        gpu::launch_allreduce_fused(*dc, send.data(), recv.data(), counts.data(), (int)send.size(), dtype, reduction, o,
                                    (cudaStream_t)stream);
        return std::make_shared<cuda_event_impl>(dc, (cudaStream_t)stream);
    }
    std::vector<event_ptr> parts;
    struct no_fusion_scope { // the buffers of one coalesced call are not queued again behind one another
        bool prev = tl_no_fusion;
        no_fusion_scope() { tl_no_fusion = true; }
        ~no_fusion_scope() { tl_no_fusion = prev; }
    } scope;
    for (size_t k = 0; k < send.size(); k++) {
        coll_param p;
        p.ctype = coll_allreduce;
        p.send_buf = send[k];
        p.recv_buf = recv[k];
        p.count = counts[k];
        p.dtype = dtype;
        p.reduction = reduction;
        p.stream = stream;
        p.device = device;
        parts.push_back(coll_create(comm, p, attr));
    }
    return std::make_shared<multi_event>(std::move(parts));
}

// ---- group ------------------------------------------------------------------------------------
void group_start() {
    CCL_THROW_IF_NOT(!tl_group_active, "group_start called twice");
    tl_group_active = true;
    tl_group.clear();
}

bool group_active() {
    return tl_group_active;
}

void group_end() {
    CCL_THROW_IF_NOT(tl_group_active, "group_end without group_start");
    tl_group_active = false;
    std::vector<group_item> items;
    items.swap(tl_group);
    // device operations of one communicator and stream go out together, in as few launches as possible
    std::vector<bool> done(items.size(), false);
    for (size_t i = 0; i < items.size(); i++) {
        if (done[i])
            continue;
        group_item& it = items[i];
        if (!it.param.device || !env_data::get().cuda_kernels || !same_node(*it.comm)) {
            it.ev->bind(coll_create(*it.comm, it.param, it.attr));
            done[i] = true;
            continue;
        }
        gpu::device_comm* dc = it.comm->device();
        cudaStream_t st = (cudaStream_t)it.param.stream;
        std::vector<size_t> batch;
        dev::p2p_ops ops{};
        auto flush = [&] {
            if (ops.n == 0)
                return;
            CUDA_CHECK(cudaSetDevice(dc->device_id()));
            gpu::launch_sendrecv(*dc, &ops, st);
            auto ev = std::make_shared<cuda_event_impl>(dc, st);
            for (size_t k : batch) {
                items[k].ev->bind(ev);
                done[k] = true;
            }
            batch.clear();
            ops = dev::p2p_ops{};
        };
        for (size_t k = i; k < items.size(); k++) {
            group_item& g = items[k];
            if (done[k] || g.comm != it.comm || g.param.stream != it.param.stream || !g.param.device)
                continue;
            const int is_send = g.param.ctype == coll_send ? 1 : 0;
            bool clash = ops.n == dev::P2P_MAX_OPS;
            for (int q = 0; q < ops.n && !clash; q++)
                clash = ops.op[q].peer == g.param.peer && ops.op[q].is_send == is_send;
            if (clash)
                flush();
            ops.op[ops.n++] = dev::p2p_op{ g.param.send_buf, g.param.recv_buf,
                                           g.param.count * dtype_size(g.param.dtype), g.param.peer, is_send };
            batch.push_back(k);
            stats().calls[g.param.ctype]++;
            stats().device_calls[g.param.ctype]++;
        }
        flush();
    }
}

} // namespace cclx
