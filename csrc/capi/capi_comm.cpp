// Flat C API over KVS, communicators, collectives (host and device buffers) and events.
#include <cstring>
#include <memory>

#include "bootstrap/kvs.hpp"
#include "capi/capi_common.hpp"
#include "coll/algorithms.hpp"
#include "coll/coll.hpp"
#include "coll/selection.hpp"
#include "bootstrap/launcher.hpp"
#include "comm/host_comm.hpp"
#include "core/comp.hpp"
#include "core/datatype.hpp"
#include "core/env.hpp"
#include "core/log.hpp"
#include "fusion/fusion.hpp"
#include "gpu/device_comm.hpp"
#include "bootstrap/elastic.hpp"
#include "topo/numa.hpp"
#include "topo/topo.hpp"

using namespace cclx;

namespace {
struct kvs_handle {
    std::shared_ptr<kvs::internal_kvs> k;
};
struct comm_handle {
    std::shared_ptr<host_comm> c;
};
struct event_handle {
    event_ptr e;
};
} // namespace

// ---- kvs ---------------------------------------------------------------------------------------
CCLX_API void* cclx_kvs_create_main(const char* ip_port) {
    kvs_handle* h = nullptr;
    capi::guard([&] {
        env_data::get();
        h = new kvs_handle{ kvs::internal_kvs::create_main(ip_port ? ip_port : "") };
    });
    return h;
}

CCLX_API void* cclx_kvs_create_peer(const char* addr) {
    kvs_handle* h = nullptr;
    capi::guard([&] {
        env_data::get();
        h = new kvs_handle{ kvs::internal_kvs::create_peer(kvs::address::from_string(addr)) };
    });
    return h;
}

CCLX_API int cclx_kvs_address(void* h, char* out, size_t cap) {
    return capi::guard([&] {
        std::string s = ((kvs_handle*)h)->k->get_address().str();
        CCL_THROW_IF_NOT(s.size() + 1 <= cap, "address buffer too small");
        std::memcpy(out, s.c_str(), s.size() + 1);
    });
}

CCLX_API int cclx_kvs_set(void* h, const char* key, const void* val, size_t len) {
    return capi::guard([&] { ((kvs_handle*)h)->k->raw().set(key, val, len); });
}

// returns the value length or -1; copies at most cap bytes
CCLX_API long long cclx_kvs_get(void* h, const char* key, void* out, size_t cap, int timeout_ms) {
    long long n = -1;
    capi::guard([&] {
        kvs::bytes b;
        if (timeout_ms < 0) {
            if (!((kvs_handle*)h)->k->raw().try_get(key, b))
                return;
        }
        else
            b = ((kvs_handle*)h)->k->raw().get(key, timeout_ms);
        std::memcpy(out, b.data(), std::min(cap, b.size()));
        n = (long long)b.size();
    });
    return n;
}

CCLX_API long long cclx_kvs_add(void* h, const char* key, long long delta) {
    long long v = 0;
    capi::guard([&] { v = ((kvs_handle*)h)->k->raw().add(key, delta); });
    return v;
}

CCLX_API long long cclx_kvs_count(void* h, const char* prefix) {
    long long v = -1;
    capi::guard([&] { v = (long long)((kvs_handle*)h)->k->raw().count(prefix); });
    return v;
}

CCLX_API int cclx_kvs_del(void* h, const char* key) {
    return capi::guard([&] { ((kvs_handle*)h)->k->raw().del(key); });
}

CCLX_API int cclx_kvs_barrier(void* h, const char* name, int participants, int timeout_ms) {
    return capi::guard([&] { ((kvs_handle*)h)->k->raw().barrier(name, (uint32_t)participants, timeout_ms); });
}

CCLX_API int cclx_kvs_destroy(void* h) {
    return capi::guard([&] { delete (kvs_handle*)h; });
}

// ---- elastic membership ------------------------------------------------------------------------
struct elastic_handle {
    std::unique_ptr<elastic_group> g;
};

CCLX_API void* cclx_elastic_create(void* kvs_h, const char* pod_id, int heartbeat_ms, int dead_after_ms, int min_size) {
    elastic_handle* h = nullptr;
    capi::guard([&] {
        h = new elastic_handle{ std::unique_ptr<elastic_group>(
            new elastic_group(((kvs_handle*)kvs_h)->k, pod_id, heartbeat_ms, dead_after_ms)) };
        h->g->set_min_size((size_t)std::max(min_size, 1));
    });
    return h;
}
// callback: int (*fn)(size_t live_pods) returning 0 wait, 1 run, 2 finalize (nullptr restores the default)
CCLX_API int cclx_elastic_set_resize_fn(void* h, int (*fn)(size_t)) {
    return capi::guard([&] {
        if (fn)
            ((elastic_handle*)h)->g->set_resize_fn([fn](size_t n) { return (resize_action)fn(n); });
        else
            ((elastic_handle*)h)->g->set_resize_fn(nullptr);
    });
}
// out: rank, size, generation; members as a comma separated list in `members` (cap bytes)
CCLX_API int cclx_elastic_form(void* h, int timeout_ms, long long* out3, char* members, size_t cap) {
    return capi::guard([&] {
        elastic_group::view v = ((elastic_handle*)h)->g->form(timeout_ms);
        out3[0] = v.rank;
        out3[1] = v.size;
        out3[2] = (long long)v.generation;
        std::string list;
        for (auto& m : v.members)
            list += (list.empty() ? "" : ",") + m;
        CCL_THROW_IF_NOT(list.size() + 1 <= cap, "member list buffer too small");
        std::memcpy(members, list.c_str(), list.size() + 1);
    });
}
// Test hook: `fn(generation)` runs inside form() after this pod published its member list and before it reads
// the others' (tests/test_elastic.py lets a third pod register in that window).
CCLX_API int cclx_elastic_set_window_hook(void* h, void (*fn)(unsigned long long)) {
    return capi::guard([&] {
        auto* e = (elastic_handle*)h;
        if (fn)
            e->g->set_window_hook([fn](uint64_t g) { fn((unsigned long long)g); });
        else
            e->g->set_window_hook(nullptr);
    });
}

CCLX_API int cclx_elastic_changed(void* h) {
    int r = -1;
    capi::guard([&] { r = ((elastic_handle*)h)->g->changed() ? 1 : 0; });
    return r;
}
CCLX_API int cclx_elastic_leave(void* h) {
    return capi::guard([&] { ((elastic_handle*)h)->g->leave(); });
}
CCLX_API int cclx_elastic_destroy(void* h) {
    return capi::guard([&] { delete (elastic_handle*)h; });
}
// communicator of the current generation (bootstraps through the generation's key prefix)
CCLX_API void* cclx_elastic_comm_create(void* h) {
    comm_handle* c = nullptr;
    capi::guard([&] {
        elastic_group& g = *((elastic_handle*)h)->g;
        c = new comm_handle{ host_comm::create(g.current().size, g.current().rank, g.generation_store()) };
    });
    return c;
}

// ---- communicator ------------------------------------------------------------------------------
CCLX_API void* cclx_comm_create(int size, int rank, void* kvs_h) {
    comm_handle* h = nullptr;
    capi::guard([&] { h = new comm_handle{ host_comm::create(size, rank, ((kvs_handle*)kvs_h)->k) }; });
    return h;
}

// rank, size and store from the process launcher (PMI-1 or torchrun-style variables)
CCLX_API void* cclx_comm_create_from_launcher() {
    comm_handle* h = nullptr;
    capi::guard([&] {
        env_data::get();
        launcher_world w = bootstrap_from_launcher();
        h = new comm_handle{ host_comm::create(w.size, w.rank, w.store) };
    });
    return h;
}

CCLX_API void* cclx_comm_split(void* c, int color, int key) {
    comm_handle* h = nullptr;
    capi::guard([&] { h = new comm_handle{ ((comm_handle*)c)->c->split(color, key) }; });
    return h;
}

CCLX_API void* cclx_comm_node(void* c) {
    comm_handle* h = nullptr;
    capi::guard([&] { h = new comm_handle{ ((comm_handle*)c)->c->node_comm() }; });
    return h;
}

CCLX_API void* cclx_comm_r2r(void* c) {
    comm_handle* h = nullptr;
    capi::guard([&] { h = new comm_handle{ ((comm_handle*)c)->c->r2r_comm() }; });
    return h;
}

// neighbours of `rank` in double-tree number `which` (0 / 1): out = { parent, left, right, root }
CCLX_API int cclx_bin_tree(int size, int rank, int which, int root, int* out) {
    return capi::guard([&] {
        cclx::algo::bin_tree t(size, rank, which, root);
        out[0] = t.parent;
        out[1] = t.left;
        out[2] = t.right;
        out[3] = t.root_rank;
    });
}

CCLX_API int cclx_comm_rank(void* c) {
    return ((comm_handle*)c)->c->rank();
}
CCLX_API int cclx_comm_size(void* c) {
    return ((comm_handle*)c)->c->size();
}
// name of the transport that carries the communicator's host traffic ("tcp", "ofi:<provider>")
CCLX_API const char* cclx_comm_transport_name(void* c) {
    return ((comm_handle*)c)->c->atl().transport().name();
}
// transport counters of the communicator's world: 0 messages sent, 1 bytes sent, 2 bytes received,
// 3 unexpected messages, 4 one-sided writes done as cross-memory copies, 5 one-sided writes sent as messages,
// 6 long messages sent by rendezvous (read out of this process by the receiver)
CCLX_API long long cclx_comm_transport_stat(void* c, int which) {
    atl_transport& t = ((comm_handle*)c)->c->atl().transport();
    switch (which) {
        case 0: return (long long)t.msgs_sent.load();
        case 1: return (long long)t.bytes_sent.load();
        case 2: return (long long)t.bytes_received.load();
        case 3: return (long long)t.unexpected_msgs.load();
        case 4: return (long long)t.rma_direct_writes.load();
        case 5: return (long long)t.rma_message_writes.load();
        case 6: return (long long)t.rndv_sends.load();
        default: return -1;
    }
}
CCLX_API long long cclx_comm_id(void* c) {
    return (long long)((comm_handle*)c)->c->id();
}
CCLX_API int cclx_comm_local_rank(void* c) {
    int v = -1;
    capi::guard([&] { v = ((comm_handle*)c)->c->local_rank(); });
    return v;
}
CCLX_API int cclx_comm_local_size(void* c) {
    int v = -1;
    capi::guard([&] { v = ((comm_handle*)c)->c->local_size(); });
    return v;
}

// device communicator of this node (created on first use, collective); not owned by the caller
CCLX_API void* cclx_comm_device(void* c) {
    gpu::device_comm* d = nullptr;
    capi::guard([&] { d = ((comm_handle*)c)->c->device(); });
    return d;
}

CCLX_API int cclx_comm_release_device(void* c) {
    return capi::guard([&] { ((comm_handle*)c)->c->release_device(); });
}

CCLX_API int cclx_comm_abort(void* c) {
    return capi::guard([&] { ((comm_handle*)c)->c->abort(); });
}

CCLX_API int cclx_comm_heartbeat(void* c) {
    return capi::guard([&] { ((comm_handle*)c)->c->pm()->heartbeat(); });
}

CCLX_API int cclx_comm_peer_alive(void* c, int peer, int max_age_ms) {
    int v = -1;
    capi::guard([&] { v = ((comm_handle*)c)->c->pm()->peer_alive(peer, max_age_ms) ? 1 : 0; });
    return v;
}

CCLX_API int cclx_comm_destroy(void* c) {
    return capi::guard([&] { delete (comm_handle*)c; });
}

CCLX_API long long cclx_comm_cache_size(void* c) {
    return (long long)((comm_handle*)c)->c->cache().size();
}

// ---- collectives -------------------------------------------------------------------------------
struct cclx_coll_desc {
    int ctype;
    const void* send_buf;
    void* recv_buf;
    size_t count;
    int dtype;
    int reduction;
    int root;
    int peer;
    const size_t* send_counts; // world entries or null
    const size_t* recv_counts;
    void* const* recv_bufs; // world entries or null (allgatherv vector form)
    void* stream; // cudaStream_t when device != 0
    int device;
    // attributes
    int priority;
    int synchronous;
    int to_cache;
    const char* match_id;
    void* reduction_fn;
    int do_scale;
    float scale;
    int out_dtype;
    const char* gpu_algo;
    // dependencies
    void* const* deps;
    int n_deps;
};

CCLX_API void* cclx_coll(void* c, const cclx_coll_desc* d) {
    event_handle* h = nullptr;
    capi::guard([&] {
        host_comm& comm = *((comm_handle*)c)->c;
        const int N = comm.size();
        coll_param p;
        p.ctype = (coll_type)d->ctype;
        p.send_buf = d->send_buf;
        p.recv_buf = d->recv_buf;
        p.count = d->count;
        p.dtype = d->dtype;
        p.reduction = d->reduction;
        p.root = d->root;
        p.peer = d->peer;
        if (d->send_counts)
            p.send_counts.assign(d->send_counts, d->send_counts + N);
        if (d->recv_counts)
            p.recv_counts.assign(d->recv_counts, d->recv_counts + N);
        if (d->recv_bufs)
            p.recv_bufs.assign(d->recv_bufs, d->recv_bufs + N);
        p.stream = d->stream;
        p.device = d->device != 0;
        for (int i = 0; i < d->n_deps; i++)
            if (d->deps[i])
                p.deps.push_back(((event_handle*)d->deps[i])->e);
        coll_attr a;
        a.priority = d->priority;
        a.synchronous = d->synchronous != 0;
        a.to_cache = d->to_cache != 0;
        if (d->match_id)
            a.match_id = d->match_id;
        a.reduction_fn = (reduction_fn_t)d->reduction_fn;
        a.do_scale = d->do_scale != 0;
        a.scale = d->scale;
        a.out_dtype = d->out_dtype;
        if (d->gpu_algo)
            a.gpu_algo = d->gpu_algo;
        h = new event_handle{ coll_create(comm, p, a) };
    });
    return h;
}

CCLX_API int cclx_event_wait(void* e) {
    return capi::guard([&] { ((event_handle*)e)->e->wait(); });
}
// 1 complete, 0 pending, -1 error
CCLX_API int cclx_event_test(void* e) {
    int v = -1;
    capi::guard([&] { v = ((event_handle*)e)->e->test() ? 1 : 0; });
    return v;
}
CCLX_API void* cclx_event_native(void* e) {
    return ((event_handle*)e)->e->native();
}
CCLX_API int cclx_event_destroy(void* e) {
    return capi::guard([&] { delete (event_handle*)e; });
}

CCLX_API int cclx_group_start() {
    return capi::guard([] { group_start(); });
}
CCLX_API int cclx_group_end() {
    return capi::guard([] { group_end(); });
}
CCLX_API int cclx_fusion_flush() {
    return capi::guard([] { fusion_manager::get().flush(nullptr); });
}

// ---- misc ---------------------------------------------------------------------------------------
CCLX_API int cclx_datatype_create(size_t size) {
    int v = -1;
    capi::guard([&] { v = datatype_table::get().create(size); });
    return v;
}
CCLX_API int cclx_datatype_free(int idx) {
    return capi::guard([&] { datatype_table::get().free(idx); });
}
CCLX_API long long cclx_datatype_size(int idx) {
    long long v = -1;
    capi::guard([&] { v = (long long)dtype_size(idx); });
    return v;
}

CCLX_API int cclx_comp_reduce(const void* in, size_t count, void* inout, int dtype, int op) {
    return capi::guard([&] { comp_reduce(in, count, inout, dtype, op); });
}
CCLX_API const char* cclx_comp_impl(int which) {
    return which == 0 ? comp_bf16_impl_name() : comp_fp16_impl_name();
}

// name of the CPU algorithm the selector picks
CCLX_API int cclx_select_cpu_algo(int ctype, size_t bytes, int comm_size, int scaleout, char* out, size_t cap) {
    return capi::guard([&] {
        selector_param sp;
        sp.ctype = (coll_type)ctype;
        sp.bytes = bytes;
        sp.count = bytes;
        sp.comm_size = comm_size;
        sp.scaleout = scaleout != 0;
        std::string a = algorithm_selector::get().select_cpu(sp);
        CCL_THROW_IF_NOT(a.size() + 1 <= cap, "buffer too small");
        std::memcpy(out, a.c_str(), a.size() + 1);
    });
}
CCLX_API int cclx_selector_reload() {
    return capi::guard([] {
        env_data::reload();
        algorithm_selector::get().reload();
    });
}
CCLX_API int cclx_parse_algo_spec(int ctype, const char* spec) {
    return capi::guard(
        [&] { algorithm_selector::parse(spec, algorithm_selector::known_cpu_algos((coll_type)ctype)); });
}

// stats: which = 0 calls, 1 device calls, 2 fused ops, 3 fused batches, 4 cache hits, 5 postponed
CCLX_API long long cclx_stats(int which, int ctype) {
    coll_stats& s = stats();
    switch (which) {
        case 0: return (long long)s.calls[ctype];
        case 1: return (long long)s.device_calls[ctype];
        case 2: return (long long)s.fused_ops;
        case 3: return (long long)s.fused_batches;
        case 4: return (long long)s.cache_hits;
        case 5: return (long long)s.postponed;
        default: return -1;
    }
}

CCLX_API int cclx_topo_describe(char* out, size_t cap) {
    return capi::guard([&] {
        std::string s = topo_info::local().describe();
        CCL_THROW_IF_NOT(s.size() + 1 <= cap, "buffer too small");
        std::memcpy(out, s.c_str(), s.size() + 1);
    });
}

// NUMA helpers.  `sys_root` empty = this machine's sysfs.  Lists are returned as int arrays; the
// return value is the number of entries (or -1).
CCLX_API int cclx_numa_query(const char* sys_root, int what, int arg, const char* text, int* out, int cap) {
    int n = -1;
    int rc = capi::guard([&] {
        numa_info custom(sys_root && sys_root[0] ? sys_root : "/sys");
        const numa_info& ni = custom;
        std::vector<int> v;
        switch (what) {
            case 0: v = { ni.node_count() }; break;
            case 1: v = ni.cpus_of_node(arg); break;
            case 2: v = { ni.node_of_cpu(arg) }; break;
            case 3: v = { ni.node_of_pci(text ? text : "") }; break;
            case 4: v = numa_info::parse_cpulist(text ? text : ""); break;
            case 5: v = ni.allowed_cpus(); break;
            default: CCL_THROW("unknown numa query ", what);
        }
        n = (int)std::min<size_t>(v.size(), (size_t)cap);
        for (int k = 0; k < n; k++)
            out[k] = v[k];
    });
    return rc == 0 ? n : -1;
}

CCLX_API int cclx_numa_auto_worker_cpus(const int* cpus, int ncpus, int local_rank, int local_size, int workers,
                                        int* out) {
    std::vector<int> v = numa_info::auto_worker_cpus(std::vector<int>(cpus, cpus + ncpus), local_rank, local_size,
                                                     workers);
    for (size_t k = 0; k < v.size(); k++)
        out[k] = v[k];
    return (int)v.size();
}

// binds the calling thread's memory to `node`, allocates and touches a buffer there, restores the policy
CCLX_API int cclx_numa_selftest(int node, size_t bytes) {
    return capi::guard([&] {
        const numa_info& ni = numa_info::get();
        ni.bind_thread_memory(node);
        void* p = ni.alloc_on_node(bytes, node);
        CCL_THROW_IF_NOT(p, "allocation failed");
        std::memset(p, 1, bytes);
        ni.free_on_node(p, bytes);
        ni.bind_thread_memory(-1);
    });
}

CCLX_API int cclx_env_size(const char* text, size_t* out) {
    return env_to_size(text, *out) ? 0 : -1;
}
