// Implementation of the public ccl:: API on top of the internal layers.
// Dispatch structure follows the reference glue (src/ccl_api_functions.cpp:44-1290):
// every free function fills an internal parameter record and forwards to the
// collective front-end; kvs / communicator / event handles wrap shared objects.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "bootstrap/kvs.hpp"
#include "coll/coll.hpp"
#include "coll/selection.hpp"
#include "bootstrap/launcher.hpp"
#include "comm/host_comm.hpp"
#include "core/datatype.hpp"
#include "core/env.hpp"
#include "core/log.hpp"
#include "oneapi/ccl.hpp"

namespace ccl {
namespace v1 {

const init_attr default_init_attr{};
const kvs_attr default_kvs_attr{};
const comm_attr default_comm_attr{};
const comm_split_attr default_comm_split_attr{};
const allgather_attr default_allgather_attr{};
const allgatherv_attr default_allgatherv_attr{};
const allreduce_attr default_allreduce_attr{};
const alltoall_attr default_alltoall_attr{};
const alltoallv_attr default_alltoallv_attr{};
const barrier_attr default_barrier_attr{};
const broadcast_attr default_broadcast_attr{};
const reduce_attr default_reduce_attr{};
const reduce_scatter_attr default_reduce_scatter_attr{};
const pt2pt_attr default_pt2pt_attr{};

namespace {

// translate internal failures into the public exception type
template <class F>
auto guarded(F&& f) -> decltype(f()) {
    try {
        return f();
    }
    catch (const ccl::v1::exception&) {
        throw;
    }
    catch (const std::exception& e) {
        throw ccl::v1::exception(e.what());
    }
}

// user-supplied store behind the internal interface (reference users_kvs.cpp)
class users_kvs : public cclx::kvs::ikvs {
public:
    explicit users_kvs(std::shared_ptr<kvs_interface> u) : u_(std::move(u)) {}
    void set(const std::string& key, const cclx::kvs::bytes& val) override {
        // values of a user store are text (the reference requires NUL-terminated data): hex-encode
        static const char* hex = "0123456789abcdef";
        std::vector<char> enc;
        enc.reserve(val.size() * 2 + 1);
        for (unsigned char c : val) {
            enc.push_back(hex[c >> 4]);
            enc.push_back(hex[c & 15]);
        }
        enc.push_back('\0');
        u_->set(key, enc);
    }
    bool try_get(const std::string& key, cclx::kvs::bytes& out) override {
        std::vector<char> enc = u_->get(key);
        if (enc.empty())
            return false;
        out.clear();
        auto nib = [](char c) { return c <= '9' ? c - '0' : c - 'a' + 10; };
        for (size_t i = 0; i + 1 < enc.size() && enc[i] != '\0'; i += 2)
            out.push_back((char)((nib(enc[i]) << 4) | nib(enc[i + 1])));
        return true;
    }
    cclx::kvs::address get_address() const override {
        char buf[64];
        std::snprintf(buf, sizeof(buf), "user_%p", (void*)u_.get());
        return cclx::kvs::address::from_string(buf);
    }

private:
    std::shared_ptr<kvs_interface> u_;
};

std::shared_ptr<cclx::kvs::ikvs> to_internal(const std::shared_ptr<kvs_interface>& k) {
    if (auto own = std::dynamic_pointer_cast<kvs>(k))
        return own->impl();
    return std::make_shared<users_kvs>(k);
}

cclx::coll_attr to_attr(const operation_attr& a) {
    cclx::coll_attr o;
    o.priority = (int)a.priority;
    o.synchronous = a.synchronous;
    o.to_cache = a.to_cache;
    o.match_id = a.match_id;
    o.reduction_fn = (cclx::reduction_fn_t)a.fn;
    o.do_scale = a.do_scale;
    o.scale = a.scale;
    o.out_dtype = a.out_dtype;
    o.gpu_algo = a.algorithm;
    return o;
}

void fill_common(cclx::coll_param& p, const stream* s, const vector_class<event>& deps) {
    if (s && s->is_device()) {
        p.stream = (void*)s->get_native();
        p.device = true;
    }
    for (auto& d : deps)
        if (d)
            p.deps.push_back(d.impl());
}

event run(const communicator& comm, cclx::coll_param& p, const operation_attr& attr) {
    if (comm.is_stub())
        return event(cclx::make_completed_event());
    return guarded([&] {
        CCL_THROW_IF_NOT(comm.impl() != nullptr, "communicator is not initialised");
        cclx::coll_attr a = to_attr(attr);
        return event(cclx::coll_create(*comm.impl(), p, a));
    });
}

std::once_flag init_once;

} // namespace

// ---- environment ----------------------------------------------------------------------------
void init(const init_attr&) {
    std::call_once(init_once, [] {
        cclx::env_data::get();
        cclx::algorithm_selector::get();
    });
}

library_version get_library_version() {
    library_version v;
    v.major = CCL_MAJOR_VERSION;
    v.minor = CCL_MINOR_VERSION;
    v.update = CCL_UPDATE_VERSION;
    v.product_status = CCL_PRODUCT_STATUS;
    v.build_date = __DATE__;
    v.full = "oneccl-b200 2021.14 (sm_100a, CUDA)";
    v.cl_backend_name = "cuda";
    return v;
}

datatype register_datatype(const datatype_attr& attr) {
    return guarded([&] {
        // workers must not look at the table while it changes (reference exec.cpp:180-208)
        cclx::executor::get().lock_workers();
        int idx;
        try {
            idx = cclx::datatype_table::get().create(attr.get<datatype_attr_id::size>());
        }
        catch (...) {
            cclx::executor::get().unlock_workers();
            throw;
        }
        cclx::executor::get().unlock_workers();
        return (datatype)idx;
    });
}

void deregister_datatype(datatype dtype) {
    guarded([&] {
        cclx::executor::get().lock_workers();
        try {
            cclx::datatype_table::get().free((int)dtype);
        }
        catch (...) {
            cclx::executor::get().unlock_workers();
            throw;
        }
        cclx::executor::get().unlock_workers();
        return 0;
    });
}

size_t get_datatype_size(datatype dtype) {
    return guarded([&] { return cclx::dtype_size((int)dtype); });
}

// ---- kvs ------------------------------------------------------------------------------------
kvs::kvs(std::shared_ptr<cclx::kvs::ikvs> impl) : impl_(std::move(impl)) {}
kvs::~kvs() = default;

kvs::address_type kvs::get_address() const {
    address_type a;
    a.fill(0);
    if (!impl_)
        return a; // stub backend
    cclx::kvs::address in = impl_->get_address();
    std::memcpy(a.data(), in.data, address_max_size);
    return a;
}

vector_class<char> kvs::get(const string_class& key) {
    return guarded([&] {
        cclx::kvs::bytes out;
        if (!impl_ || !impl_->try_get("USER_DATA/" + key, out))
            return vector_class<char>();
        return out;
    });
}

void kvs::set(const string_class& key, const vector_class<char>& data) {
    guarded([&] {
        if (impl_)
            impl_->set("USER_DATA/" + key, data);
        return 0;
    });
}

shared_ptr_class<kvs> create_main_kvs(const kvs_attr& attr) {
    return guarded([&] {
        init();
        if (cclx::env_data::get().backend == cclx::backend_t::stub)
            return std::make_shared<kvs>(nullptr);
        std::string ip_port = attr.is_valid<kvs_attr_id::ip_port>() ? attr.get<kvs_attr_id::ip_port>() : "";
        return std::make_shared<kvs>(cclx::kvs::internal_kvs::create_main(ip_port));
    });
}

shared_ptr_class<kvs> create_kvs(const kvs::address_type& addr, const kvs_attr&) {
    return guarded([&] {
        init();
        if (cclx::env_data::get().backend == cclx::backend_t::stub)
            return std::make_shared<kvs>(nullptr);
        cclx::kvs::address a;
        std::memcpy(a.data, addr.data(), kvs::address_max_size);
        return std::make_shared<kvs>(cclx::kvs::internal_kvs::create_peer(a));
    });
}

// ---- device objects ---------------------------------------------------------------------------
device create_device() {
    return device(-1);
}
context create_context() {
    return context();
}
stream create_stream() {
    return stream();
}

namespace {
class wrapped_cuda_event : public cclx::event_impl {
public:
    explicit wrapped_cuda_event(CUevent_st* e) : e_(e) {}
    void wait() override;
    bool test() override;
    void* native() override { return e_; }

private:
    CUevent_st* e_;
};
} // namespace

void wrapped_cuda_event_sync(CUevent_st* e) {
    cudaError_t r = cudaEventSynchronize((cudaEvent_t)e);
    CCL_THROW_IF_NOT(r == cudaSuccess, "cudaEventSynchronize failed: ", cudaGetErrorString(r));
}
bool wrapped_cuda_event_query(CUevent_st* e) {
    cudaError_t r = cudaEventQuery((cudaEvent_t)e);
    if (r == cudaErrorNotReady)
        return false;
    CCL_THROW_IF_NOT(r == cudaSuccess, "cudaEventQuery failed: ", cudaGetErrorString(r));
    return true;
}
namespace {
void wrapped_cuda_event::wait() {
    wrapped_cuda_event_sync(e_);
}
bool wrapped_cuda_event::test() {
    return wrapped_cuda_event_query(e_);
}
} // namespace

event create_event(CUevent_st* native_event) {
    return event(std::make_shared<wrapped_cuda_event>(native_event));
}

void event::wait() {
    guarded([&] {
        if (impl_)
            impl_->wait();
        return 0;
    });
}
bool event::test() {
    return guarded([&] { return impl_ ? impl_->test() : true; });
}
bool event::cancel() {
    // operations can not be withdrawn once posted (the reference leaves cancel unimplemented too)
    return false;
}
CUevent_st* event::get_native() const {
    return impl_ ? (CUevent_st*)impl_->native() : nullptr;
}

// ---- communicator -----------------------------------------------------------------------------
int communicator::rank() const {
    return impl_ ? impl_->rank() : stub_rank_;
}
int communicator::size() const {
    return impl_ ? impl_->size() : (stub_size_ > 0 ? stub_size_ : 1);
}
device communicator::get_device() const {
    return device(-1);
}
context communicator::get_context() const {
    return context();
}
communicator communicator::split(const comm_split_attr& attr) {
    return split_communicator(*this, attr);
}

communicator split_communicator(const communicator& comm, const comm_split_attr& attr) {
    return guarded([&] {
        CCL_THROW_IF_NOT(attr.is_valid<comm_split_attr_id::color>(), "split needs the color attribute");
        return communicator(comm.impl()->split(attr.get<comm_split_attr_id::color>(), comm.rank()));
    });
}

communicator create_communicator(int size, int rank, shared_ptr_class<kvs_interface> k, const comm_attr&) {
    return guarded([&] {
        init();
        if (cclx::env_data::get().backend == cclx::backend_t::stub)
            return communicator(size, rank);
        CCL_THROW_IF_NOT(k != nullptr, "kvs is null");
        return communicator(cclx::host_comm::create(size, rank, to_internal(k)));
    });
}

communicator create_communicator(int size, int rank, const device& dev, const context&,
                                 shared_ptr_class<kvs_interface> k, const comm_attr& attr) {
    (void)dev;
    return create_communicator(size, rank, k, attr);
}

vector_class<communicator> create_communicators(int size, const vector_class<int>& local_ranks,
                                                shared_ptr_class<kvs_interface> k, const comm_attr& attr) {
    // one rank per process (reference limitation: "multiple ranks within single process" is unsupported)
    if (local_ranks.size() != 1)
        throw unimplemented("one process drives one rank: pass exactly one local rank");
    vector_class<communicator> v;
    v.push_back(create_communicator(size, local_ranks[0], k, attr));
    return v;
}

} // namespace v1

namespace preview {

communicator create_communicator(const comm_attr&) {
    return v1::guarded([&] {
        v1::init();
        cclx::launcher_world w = cclx::bootstrap_from_launcher();
        if (cclx::env_data::get().backend == cclx::backend_t::stub)
            return communicator(w.size, w.rank);
        return communicator(cclx::host_comm::create(w.size, w.rank, w.store));
    });
}

vector_class<communicator> split_communicators(const vector_class<pair_class<communicator, comm_split_attr>>& attrs) {
    vector_class<communicator> out;
    for (auto& p : attrs)
        out.push_back(v1::split_communicator(p.first, p.second));
    return out;
}

namespace {
event coalesced(const vector_class<void*>& bufs, const vector_class<size_t>& counts, datatype dtype, reduction rtype,
                const communicator& comm, const stream* s, const allreduce_attr& attr) {
    if (comm.is_stub())
        return event(cclx::make_completed_event());
    return v1::guarded([&] {
        CCL_THROW_IF_NOT(comm.impl() != nullptr, "communicator is not initialised");
        cclx::coll_attr a = v1::to_attr(attr);
        std::vector<const void*> send(bufs.begin(), bufs.end());
        const bool device = s && s->is_device();
        return event(cclx::coll_allreduce_coalesced(*comm.impl(), send, bufs, counts, (int)dtype, (int)rtype, a,
                                                    device ? (void*)s->get_native() : nullptr, device));
    });
}
} // namespace

event allreduce_coalesced(const vector_class<void*>& bufs, const vector_class<size_t>& counts, datatype dtype,
                          reduction rtype, const communicator& comm, const stream& s, const allreduce_attr& attr) {
    return coalesced(bufs, counts, dtype, rtype, comm, &s, attr);
}
event allreduce_coalesced(const vector_class<void*>& bufs, const vector_class<size_t>& counts, datatype dtype,
                          reduction rtype, const communicator& comm, const allreduce_attr& attr) {
    return coalesced(bufs, counts, dtype, rtype, comm, nullptr, attr);
}

} // namespace preview

namespace v1 {

void group_start() {
    guarded([] {
        cclx::group_start();
        return 0;
    });
}
void group_end() {
    guarded([] {
        cclx::group_end();
        return 0;
    });
}

// ---- operations -------------------------------------------------------------------------------
#define STREAM_PAIR(NAME, PARAMS_DECL, ATTR_T, BODY) \
    event NAME(PARAMS_DECL, const communicator& comm, const stream& s, const ATTR_T& attr, \
               const vector_class<event>& deps) { \
        const stream* sp = &s; \
        BODY \
    } \
    event NAME(PARAMS_DECL, const communicator& comm, const ATTR_T& attr, const vector_class<event>& deps) { \
        const stream* sp = nullptr; \
        BODY \
    }

#define P1 const void *send_buf, void *recv_buf, size_t count, datatype dtype
STREAM_PAIR(allgather, P1, allgather_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_allgather;
    p.send_buf = send_buf;
    p.recv_buf = recv_buf;
    p.count = count;
    p.dtype = (int)dtype;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
#undef P1

#define P2 const void *send_buf, size_t send_count, void *recv_buf, const vector_class<size_t>&recv_counts, datatype dtype
STREAM_PAIR(allgatherv, P2, allgatherv_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_allgatherv;
    p.send_buf = send_buf;
    p.recv_buf = recv_buf;
    p.count = send_count;
    p.recv_counts = recv_counts;
    p.dtype = (int)dtype;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
#undef P2

#define P3 const void *send_buf, size_t send_count, const vector_class<void*>&recv_bufs, const vector_class<size_t>&recv_counts, datatype dtype
STREAM_PAIR(allgatherv, P3, allgatherv_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_allgatherv;
    p.send_buf = send_buf;
    p.recv_bufs = recv_bufs;
    p.count = send_count;
    p.recv_counts = recv_counts;
    p.dtype = (int)dtype;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
#undef P3

#define P4 const void *send_buf, void *recv_buf, size_t count, datatype dtype, reduction rtype
STREAM_PAIR(allreduce, P4, allreduce_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_allreduce;
    p.send_buf = send_buf;
    p.recv_buf = recv_buf;
    p.count = count;
    p.dtype = (int)dtype;
    p.reduction = (int)rtype;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
STREAM_PAIR(reduce_scatter, P4, reduce_scatter_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_reduce_scatter;
    p.send_buf = send_buf;
    p.recv_buf = recv_buf;
    p.count = count;
    p.dtype = (int)dtype;
    p.reduction = (int)rtype;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
#undef P4

#define P5 const void *send_buf, void *recv_buf, size_t count, datatype dtype
STREAM_PAIR(alltoall, P5, alltoall_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_alltoall;
    p.send_buf = send_buf;
    p.recv_buf = recv_buf;
    p.count = count;
    p.dtype = (int)dtype;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
#undef P5

#define P6 const void *send_buf, const vector_class<size_t>&send_counts, void *recv_buf, const vector_class<size_t>&recv_counts, datatype dtype
STREAM_PAIR(alltoallv, P6, alltoallv_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_alltoallv;
    p.send_buf = send_buf;
    p.recv_buf = recv_buf;
    p.send_counts = send_counts;
    p.recv_counts = recv_counts;
    p.dtype = (int)dtype;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
#undef P6

event barrier(const communicator& comm, const stream& s, const barrier_attr& attr, const vector_class<event>& deps) {
    cclx::coll_param p;
    p.ctype = cclx::coll_barrier;
    fill_common(p, &s, deps);
    return run(comm, p, attr);
}
event barrier(const communicator& comm, const barrier_attr& attr, const vector_class<event>& deps) {
    cclx::coll_param p;
    p.ctype = cclx::coll_barrier;
    fill_common(p, nullptr, deps);
    return run(comm, p, attr);
}

#define P7 void *buf, size_t count, datatype dtype, int root
STREAM_PAIR(broadcast, P7, broadcast_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_bcast;
    p.send_buf = buf;
    p.recv_buf = buf;
    p.count = count;
    p.dtype = (int)dtype;
    p.root = root;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
#undef P7

#define P8 void *send_buf, void *recv_buf, size_t count, datatype dtype, int root
STREAM_PAIR(broadcast, P8, broadcast_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_broadcast;
    p.send_buf = send_buf;
    p.recv_buf = recv_buf;
    p.count = count;
    p.dtype = (int)dtype;
    p.root = root;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
#undef P8

#define P9 const void *send_buf, void *recv_buf, size_t count, datatype dtype, reduction rtype, int root
STREAM_PAIR(reduce, P9, reduce_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_reduce;
    p.send_buf = send_buf;
    p.recv_buf = recv_buf;
    p.count = count;
    p.dtype = (int)dtype;
    p.reduction = (int)rtype;
    p.root = root;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
#undef P9

#define P10 void *buf, size_t count, datatype dtype, int peer
STREAM_PAIR(send, P10, pt2pt_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_send;
    p.send_buf = buf;
    p.count = count;
    p.dtype = (int)dtype;
    p.peer = peer;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
STREAM_PAIR(recv, P10, pt2pt_attr, {
    cclx::coll_param p;
    p.ctype = cclx::coll_recv;
    p.recv_buf = buf;
    p.count = count;
    p.dtype = (int)dtype;
    p.peer = peer;
    fill_common(p, sp, deps);
    return run(comm, p, attr);
})
#undef P10
#undef STREAM_PAIR

} // namespace v1
} // namespace ccl
