// Public C++ API (specification 1.0 surface of oneCCL) for the B200-native library.
//
// Source compatible with programs written against the reference headers
// (include/oneapi/ccl/api_functions.hpp:48-2062, types.hpp:41-123,
// coll_attr_ids.hpp:29-93, kvs.hpp:38-72, communicator.hpp:43-140,
// stream.hpp:41-107, event.hpp:34-102): ccl::init, create_main_kvs / create_kvs,
// create_communicator, create_stream, the twelve operations with their overload
// sets (void* + datatype, typed pointers, with and without stream, vector
// forms), operation attributes set through attr.set<attr_id>(value), custom
// datatypes, group_start / group_end.
//
// The classes are thin handles over shared implementation objects instead of
// the reference's PIMPL + policy machinery.  A stream wraps a cudaStream_t:
// operations given such a stream treat their buffers as device memory and run
// on the GPU kernels; without a stream the CPU scheduler path is used.
#pragma once
#include <array>
#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

#define CCL_MAJOR_VERSION 2021
#define CCL_MINOR_VERSION 14
#define CCL_UPDATE_VERSION 0
#define CCL_PRODUCT_STATUS "b200"
#define CCL_API __attribute__((visibility("default")))

struct CUstream_st;
struct CUevent_st;

namespace cclx {
class host_comm;
class event_impl;
namespace kvs {
class ikvs;
}
} // namespace cclx

namespace ccl {

template <class T>
using vector_class = std::vector<T>;
template <class A, class B>
using pair_class = std::pair<A, B>;
template <class T>
using shared_ptr_class = std::shared_ptr<T>;
template <class T>
using reference_wrapper_class = std::reference_wrapper<T>;
using string_class = std::string;
template <class T, size_t N>
using array_class = std::array<T, N>;

namespace v1 {

// ---- exceptions ---------------------------------------------------------------------
class exception : public std::runtime_error {
public:
    explicit exception(const std::string& what) : std::runtime_error(what) {}
};
class invalid_argument : public exception {
    using exception::exception;
};
class unimplemented : public exception {
    using exception::exception;
};
class unsupported : public exception {
    using exception::exception;
};

// ---- scalar types -------------------------------------------------------------------
enum class reduction : int { sum = 0, prod, min, max, custom };

enum class datatype : int {
    int8 = 0,
    uint8,
    int16,
    uint16,
    int32,
    uint32,
    int64,
    uint64,
    float16,
    float32,
    float64,
    bfloat16
};

// 16-bit floats travel as opaque 16-bit patterns (reference lp_types.hpp:27-67)
struct float16 {
    uint16_t data;
};
struct bfloat16 {
    uint16_t data;
};

typedef struct {
    unsigned int major;
    unsigned int minor;
    unsigned int update;
    const char* product_status;
    const char* build_date;
    const char* full;
    string_class cl_backend_name;
} library_version;

typedef struct {
    const char* match_id;
    const size_t offset;
} fn_context;

typedef void (*reduction_fn)(const void* in_buf, size_t in_count, void* inout_buf, size_t* out_count, datatype dtype,
                             const fn_context* context);

template <class T>
struct native_type_info {
    static constexpr bool supported = false;
};
#define CCL_NATIVE_TYPE(T, DT) \
    template <> \
    struct native_type_info<T> { \
        static constexpr bool supported = true; \
        static constexpr datatype dtype = datatype::DT; \
    };
CCL_NATIVE_TYPE(int8_t, int8)
CCL_NATIVE_TYPE(uint8_t, uint8)
CCL_NATIVE_TYPE(int16_t, int16)
CCL_NATIVE_TYPE(uint16_t, uint16)
CCL_NATIVE_TYPE(int32_t, int32)
CCL_NATIVE_TYPE(uint32_t, uint32)
CCL_NATIVE_TYPE(int64_t, int64)
CCL_NATIVE_TYPE(uint64_t, uint64)
CCL_NATIVE_TYPE(float16, float16)
CCL_NATIVE_TYPE(float, float32)
CCL_NATIVE_TYPE(double, float64)
CCL_NATIVE_TYPE(bfloat16, bfloat16)
#undef CCL_NATIVE_TYPE

template <class T>
constexpr bool is_native_type_supported() {
    return native_type_info<typename std::remove_cv<T>::type>::supported;
}

// ---- attribute ids ------------------------------------------------------------------
enum class init_attr_id : int { version };
enum class kvs_attr_id : int { version, ip_port };
enum class comm_attr_id : int { version };
enum class comm_split_attr_id : int { version, color, group };
enum class split_group : int { cluster };
enum class datatype_attr_id : int { version, size };
enum class stream_attr_id : int { version, native_handle };
enum class operation_attr_id : int { version, priority, to_cache, synchronous, match_id, last_value };
enum class allgather_attr_id : int { op_id_offset = 5 };
enum class allgatherv_attr_id : int { op_id_offset = 5 };
enum class allreduce_attr_id : int { op_id_offset = 5, reduction_fn = op_id_offset };
enum class alltoall_attr_id : int { op_id_offset = 5 };
enum class alltoallv_attr_id : int { op_id_offset = 5 };
enum class barrier_attr_id : int { op_id_offset = 5 };
enum class broadcast_attr_id : int { op_id_offset = 5 };
enum class reduce_attr_id : int { op_id_offset = 5, reduction_fn = op_id_offset };
enum class reduce_scatter_attr_id : int { op_id_offset = 5, reduction_fn = op_id_offset };
enum class pt2pt_attr_id : int { op_id_offset = 5, group_id = op_id_offset };
// B200 extension: fused epilogue of device reductions (scale, output datatype) and forced kernel
enum class device_attr_ext_id : int { scale, out_dtype, algorithm };

// ---- attributes ---------------------------------------------------------------------
class init_attr {};
class comm_attr {};

class kvs_attr {
public:
    template <kvs_attr_id id, class V>
    V set(const V& v) {
        static_assert(id == kvs_attr_id::ip_port, "unknown kvs attribute");
        string_class old = ip_port_;
        ip_port_ = v;
        return V(old);
    }
    template <kvs_attr_id id>
    const string_class& get() const {
        return ip_port_;
    }
    template <kvs_attr_id id>
    bool is_valid() const noexcept {
        return id == kvs_attr_id::ip_port ? !ip_port_.empty() : false;
    }

private:
    string_class ip_port_;
};

class comm_split_attr {
public:
    template <comm_split_attr_id id, class V>
    V set(const V& v) {
        if (id == comm_split_attr_id::color) {
            color_ = (int)v;
            has_color_ = true;
        }
        return v;
    }
    template <comm_split_attr_id id>
    int get() const {
        return color_;
    }
    template <comm_split_attr_id id>
    bool is_valid() const noexcept {
        return id == comm_split_attr_id::color ? has_color_ : false;
    }

private:
    int color_ = 0;
    bool has_color_ = false;
};

class datatype_attr {
public:
    template <datatype_attr_id id, class V>
    V set(const V& v) {
        static_assert(id == datatype_attr_id::size, "unknown datatype attribute");
        size_t old = size_;
        size_ = (size_t)v;
        return (V)old;
    }
    template <datatype_attr_id id>
    size_t get() const {
        return size_;
    }

private:
    size_t size_ = 1;
};

// common operation attributes + the per-operation extras
class operation_attr {
public:
    template <operation_attr_id id, class V>
    void set(const V& v) {
        set_common(id, v);
    }
    template <operation_attr_id id>
    auto get() const -> typename std::conditional<id == operation_attr_id::match_id, const string_class&,
                                                  typename std::conditional<id == operation_attr_id::priority,
                                                                            size_t, bool>::type>::type {
        return get_common<id>();
    }
    // extension setters (device path)
    template <device_attr_ext_id id, class V>
    void set(const V& v) {
        set_ext(id, v);
    }

    size_t priority = 0;
    bool to_cache = false;
    bool synchronous = false;
    string_class match_id;
    reduction_fn fn = nullptr;
    int group_id = 0;
    bool do_scale = false;
    float scale = 1.0f;
    int out_dtype = -1;
    string_class algorithm;

protected:
    void set_common(operation_attr_id id, size_t v) {
        if (id == operation_attr_id::priority)
            priority = v;
        else if (id == operation_attr_id::to_cache)
            to_cache = v != 0;
        else if (id == operation_attr_id::synchronous)
            synchronous = v != 0;
    }
    void set_common(operation_attr_id id, int v) { set_common(id, (size_t)v); }
    void set_common(operation_attr_id id, bool v) { set_common(id, (size_t)v); }
    void set_common(operation_attr_id id, const string_class& v) {
        if (id == operation_attr_id::match_id)
            match_id = v;
    }
    void set_common(operation_attr_id id, const char* v) { set_common(id, string_class(v)); }
    void set_ext(device_attr_ext_id id, float v) {
        if (id == device_attr_ext_id::scale) {
            scale = v;
            do_scale = true;
        }
    }
    void set_ext(device_attr_ext_id id, double v) { set_ext(id, (float)v); }
    void set_ext(device_attr_ext_id id, datatype v) {
        if (id == device_attr_ext_id::out_dtype)
            out_dtype = (int)v;
    }
    void set_ext(device_attr_ext_id id, const string_class& v) {
        if (id == device_attr_ext_id::algorithm)
            algorithm = v;
    }
    void set_ext(device_attr_ext_id id, const char* v) { set_ext(id, string_class(v)); }
    template <operation_attr_id id>
    typename std::enable_if<id == operation_attr_id::match_id, const string_class&>::type get_common() const {
        return match_id;
    }
    template <operation_attr_id id>
    typename std::enable_if<id == operation_attr_id::priority, size_t>::type get_common() const {
        return priority;
    }
    template <operation_attr_id id>
    typename std::enable_if<id == operation_attr_id::to_cache || id == operation_attr_id::synchronous, bool>::type
    get_common() const {
        return id == operation_attr_id::to_cache ? to_cache : synchronous;
    }
};

#define CCL_DECLARE_OP_ATTR(NAME, IDTYPE, HAS_FN) \
    class NAME : public operation_attr { \
    public: \
        using operation_attr::set; \
        using operation_attr::get; \
        template <IDTYPE id, class V> \
        void set(const V& v) { \
            set_specific(v); \
        } \
\
    private: \
        void set_specific(reduction_fn f) { \
            static_assert(HAS_FN || true, ""); \
            fn = f; \
        } \
        void set_specific(int g) { group_id = g; } \
    };
CCL_DECLARE_OP_ATTR(allgather_attr, allgather_attr_id, false)
CCL_DECLARE_OP_ATTR(allgatherv_attr, allgatherv_attr_id, false)
CCL_DECLARE_OP_ATTR(allreduce_attr, allreduce_attr_id, true)
CCL_DECLARE_OP_ATTR(alltoall_attr, alltoall_attr_id, false)
CCL_DECLARE_OP_ATTR(alltoallv_attr, alltoallv_attr_id, false)
CCL_DECLARE_OP_ATTR(barrier_attr, barrier_attr_id, false)
CCL_DECLARE_OP_ATTR(broadcast_attr, broadcast_attr_id, false)
CCL_DECLARE_OP_ATTR(reduce_attr, reduce_attr_id, true)
CCL_DECLARE_OP_ATTR(reduce_scatter_attr, reduce_scatter_attr_id, true)
CCL_DECLARE_OP_ATTR(pt2pt_attr, pt2pt_attr_id, false)
#undef CCL_DECLARE_OP_ATTR

CCL_API extern const init_attr default_init_attr;
CCL_API extern const kvs_attr default_kvs_attr;
CCL_API extern const comm_attr default_comm_attr;
CCL_API extern const comm_split_attr default_comm_split_attr;
CCL_API extern const allgather_attr default_allgather_attr;
CCL_API extern const allgatherv_attr default_allgatherv_attr;
CCL_API extern const allreduce_attr default_allreduce_attr;
CCL_API extern const alltoall_attr default_alltoall_attr;
CCL_API extern const alltoallv_attr default_alltoallv_attr;
CCL_API extern const barrier_attr default_barrier_attr;
CCL_API extern const broadcast_attr default_broadcast_attr;
CCL_API extern const reduce_attr default_reduce_attr;
CCL_API extern const reduce_scatter_attr default_reduce_scatter_attr;
CCL_API extern const pt2pt_attr default_pt2pt_attr;

template <class attr_id, attr_id id, class V>
struct attr_value_pair {
    V value;
};
template <kvs_attr_id id, class V>
attr_value_pair<kvs_attr_id, id, V> attr_val(V v) {
    return { v };
}
template <operation_attr_id id, class V>
attr_value_pair<operation_attr_id, id, V> attr_val(V v) {
    return { v };
}
template <allreduce_attr_id id, class V>
attr_value_pair<allreduce_attr_id, id, V> attr_val(V v) {
    return { v };
}
template <reduce_attr_id id, class V>
attr_value_pair<reduce_attr_id, id, V> attr_val(V v) {
    return { v };
}
template <reduce_scatter_attr_id id, class V>
attr_value_pair<reduce_scatter_attr_id, id, V> attr_val(V v) {
    return { v };
}
template <comm_split_attr_id id, class V>
attr_value_pair<comm_split_attr_id, id, V> attr_val(V v) {
    return { v };
}
template <datatype_attr_id id, class V>
attr_value_pair<datatype_attr_id, id, V> attr_val(V v) {
    return { v };
}

namespace detail {
template <class A>
void apply_attr(A&) {}
template <class A, class attr_id, attr_id id, class V, class... Rest>
void apply_attr(A& a, const attr_value_pair<attr_id, id, V>& p, const Rest&... rest) {
    a.template set<id>(p.value);
    apply_attr(a, rest...);
}
} // namespace detail

// ---- kvs ----------------------------------------------------------------------------
class kvs_interface {
public:
    virtual ~kvs_interface() = default;
    virtual vector_class<char> get(const string_class& key) = 0;
    virtual void set(const string_class& key, const vector_class<char>& data) = 0;
};

class CCL_API kvs final : public kvs_interface {
public:
    static constexpr size_t address_max_size = 256;
    using address_type = array_class<char, address_max_size>;
    ~kvs() override;
    address_type get_address() const;
    vector_class<char> get(const string_class& key) override;
    void set(const string_class& key, const vector_class<char>& data) override;
    // internal
    std::shared_ptr<cclx::kvs::ikvs> impl() const { return impl_; }
    explicit kvs(std::shared_ptr<cclx::kvs::ikvs> impl);

private:
    std::shared_ptr<cclx::kvs::ikvs> impl_;
};

// ---- device / context / stream / event --------------------------------------------------
class CCL_API device {
public:
    explicit device(int index = -1) : index_(index) {}
    int get_native() const { return index_; }

private:
    int index_;
};

class CCL_API context {
public:
    context() = default;
    void* get_native() const { return nullptr; }
};

class CCL_API stream {
public:
    stream() = default; // host stream: operations use the CPU path
    explicit stream(CUstream_st* s) : native_(s), is_device_(true) {}
    CUstream_st* get_native() const { return native_; }
    bool is_device() const { return is_device_; }

private:
    CUstream_st* native_ = nullptr;
    bool is_device_ = false;
};

class CCL_API event {
public:
    event() = default;
    explicit event(std::shared_ptr<cclx::event_impl> impl) : impl_(std::move(impl)) {}
    void wait();
    bool test();
    bool cancel();
    // cudaEvent_t of a device operation, nullptr for host operations
    CUevent_st* get_native() const;
    explicit operator bool() const { return (bool)impl_; }
    std::shared_ptr<cclx::event_impl> impl() const { return impl_; }

private:
    std::shared_ptr<cclx::event_impl> impl_;
};

// ---- communicator -----------------------------------------------------------------------
class CCL_API communicator {
public:
    communicator() = default;
    explicit communicator(std::shared_ptr<cclx::host_comm> impl) : impl_(std::move(impl)) {}
    // stub backend (CCL_BACKEND=stub): every operation completes without communicating
    communicator(int stub_size, int stub_rank) : stub_size_(stub_size), stub_rank_(stub_rank) {}
    bool is_stub() const { return stub_size_ > 0; }
    int rank() const;
    int size() const;
    communicator split(const comm_split_attr& attr);
    device get_device() const;
    context get_context() const;
    std::shared_ptr<cclx::host_comm> impl() const { return impl_; }

private:
    std::shared_ptr<cclx::host_comm> impl_;
    int stub_size_ = 0, stub_rank_ = 0;
};

// ---- environment ------------------------------------------------------------------------
CCL_API void init(const init_attr& attr = default_init_attr);
CCL_API library_version get_library_version();
CCL_API datatype register_datatype(const datatype_attr& attr);
CCL_API void deregister_datatype(datatype dtype);
CCL_API size_t get_datatype_size(datatype dtype);

template <class... Avs>
init_attr create_init_attr(Avs&&...) {
    return init_attr();
}
template <class... Avs>
kvs_attr create_kvs_attr(Avs&&... avs) {
    kvs_attr a;
    detail::apply_attr(a, avs...);
    return a;
}
template <class... Avs>
comm_attr create_comm_attr(Avs&&...) {
    return comm_attr();
}
template <class... Avs>
comm_split_attr create_comm_split_attr(Avs&&... avs) {
    comm_split_attr a;
    detail::apply_attr(a, avs...);
    return a;
}
template <class... Avs>
datatype_attr create_datatype_attr(Avs&&... avs) {
    datatype_attr a;
    detail::apply_attr(a, avs...);
    return a;
}
template <class Attr, class... Avs>
Attr create_operation_attr(Avs&&... avs) {
    Attr a;
    detail::apply_attr(a, avs...);
    return a;
}

CCL_API shared_ptr_class<kvs> create_main_kvs(const kvs_attr& attr = default_kvs_attr);
CCL_API shared_ptr_class<kvs> create_kvs(const kvs::address_type& addr, const kvs_attr& attr = default_kvs_attr);

CCL_API device create_device();
inline device create_device(int cuda_device_index) {
    return device(cuda_device_index);
}
CCL_API context create_context();
CCL_API stream create_stream();
inline stream create_stream(CUstream_st* native_stream) {
    return stream(native_stream);
}
CCL_API event create_event(CUevent_st* native_event);

CCL_API communicator create_communicator(int size, int rank, shared_ptr_class<kvs_interface> kvs,
                                         const comm_attr& attr = default_comm_attr);
CCL_API communicator create_communicator(int size, int rank, const device& dev, const context& ctx,
                                         shared_ptr_class<kvs_interface> kvs,
                                         const comm_attr& attr = default_comm_attr);
CCL_API vector_class<communicator> create_communicators(int size, const vector_class<int>& local_ranks,
                                                        shared_ptr_class<kvs_interface> kvs,
                                                        const comm_attr& attr = default_comm_attr);
CCL_API communicator split_communicator(const communicator& comm, const comm_split_attr& attr);

CCL_API void group_start();
CCL_API void group_end();

// ---- operations: untyped forms --------------------------------------------------------------
#define CCL_DEPS const vector_class<event>& deps = {}

CCL_API event allgather(const void* send_buf, void* recv_buf, size_t count, datatype dtype, const communicator& comm,
                        const stream& stream, const allgather_attr& attr = default_allgather_attr, CCL_DEPS);
CCL_API event allgather(const void* send_buf, void* recv_buf, size_t count, datatype dtype, const communicator& comm,
                        const allgather_attr& attr = default_allgather_attr, CCL_DEPS);

CCL_API event allgatherv(const void* send_buf, size_t send_count, void* recv_buf,
                         const vector_class<size_t>& recv_counts, datatype dtype, const communicator& comm,
                         const stream& stream, const allgatherv_attr& attr = default_allgatherv_attr, CCL_DEPS);
CCL_API event allgatherv(const void* send_buf, size_t send_count, void* recv_buf,
                         const vector_class<size_t>& recv_counts, datatype dtype, const communicator& comm,
                         const allgatherv_attr& attr = default_allgatherv_attr, CCL_DEPS);
CCL_API event allgatherv(const void* send_buf, size_t send_count, const vector_class<void*>& recv_bufs,
                         const vector_class<size_t>& recv_counts, datatype dtype, const communicator& comm,
                         const stream& stream, const allgatherv_attr& attr = default_allgatherv_attr, CCL_DEPS);
CCL_API event allgatherv(const void* send_buf, size_t send_count, const vector_class<void*>& recv_bufs,
                         const vector_class<size_t>& recv_counts, datatype dtype, const communicator& comm,
                         const allgatherv_attr& attr = default_allgatherv_attr, CCL_DEPS);

CCL_API event allreduce(const void* send_buf, void* recv_buf, size_t count, datatype dtype, reduction rtype,
                        const communicator& comm, const stream& stream,
                        const allreduce_attr& attr = default_allreduce_attr, CCL_DEPS);
CCL_API event allreduce(const void* send_buf, void* recv_buf, size_t count, datatype dtype, reduction rtype,
                        const communicator& comm, const allreduce_attr& attr = default_allreduce_attr, CCL_DEPS);

CCL_API event alltoall(const void* send_buf, void* recv_buf, size_t count, datatype dtype, const communicator& comm,
                       const stream& stream, const alltoall_attr& attr = default_alltoall_attr, CCL_DEPS);
CCL_API event alltoall(const void* send_buf, void* recv_buf, size_t count, datatype dtype, const communicator& comm,
                       const alltoall_attr& attr = default_alltoall_attr, CCL_DEPS);

CCL_API event alltoallv(const void* send_buf, const vector_class<size_t>& send_counts, void* recv_buf,
                        const vector_class<size_t>& recv_counts, datatype dtype, const communicator& comm,
                        const stream& stream, const alltoallv_attr& attr = default_alltoallv_attr, CCL_DEPS);
CCL_API event alltoallv(const void* send_buf, const vector_class<size_t>& send_counts, void* recv_buf,
                        const vector_class<size_t>& recv_counts, datatype dtype, const communicator& comm,
                        const alltoallv_attr& attr = default_alltoallv_attr, CCL_DEPS);

CCL_API event barrier(const communicator& comm, const stream& stream,
                      const barrier_attr& attr = default_barrier_attr, CCL_DEPS);
CCL_API event barrier(const communicator& comm, const barrier_attr& attr = default_barrier_attr, CCL_DEPS);

// in-place form
CCL_API event broadcast(void* buf, size_t count, datatype dtype, int root, const communicator& comm,
                        const stream& stream, const broadcast_attr& attr = default_broadcast_attr, CCL_DEPS);
CCL_API event broadcast(void* buf, size_t count, datatype dtype, int root, const communicator& comm,
                        const broadcast_attr& attr = default_broadcast_attr, CCL_DEPS);
// out-of-place form
CCL_API event broadcast(void* send_buf, void* recv_buf, size_t count, datatype dtype, int root,
                        const communicator& comm, const stream& stream,
                        const broadcast_attr& attr = default_broadcast_attr, CCL_DEPS);
CCL_API event broadcast(void* send_buf, void* recv_buf, size_t count, datatype dtype, int root,
                        const communicator& comm, const broadcast_attr& attr = default_broadcast_attr, CCL_DEPS);

CCL_API event reduce(const void* send_buf, void* recv_buf, size_t count, datatype dtype, reduction rtype, int root,
                     const communicator& comm, const stream& stream, const reduce_attr& attr = default_reduce_attr,
                     CCL_DEPS);
CCL_API event reduce(const void* send_buf, void* recv_buf, size_t count, datatype dtype, reduction rtype, int root,
                     const communicator& comm, const reduce_attr& attr = default_reduce_attr, CCL_DEPS);

CCL_API event reduce_scatter(const void* send_buf, void* recv_buf, size_t recv_count, datatype dtype,
                             reduction rtype, const communicator& comm, const stream& stream,
                             const reduce_scatter_attr& attr = default_reduce_scatter_attr, CCL_DEPS);
CCL_API event reduce_scatter(const void* send_buf, void* recv_buf, size_t recv_count, datatype dtype,
                             reduction rtype, const communicator& comm,
                             const reduce_scatter_attr& attr = default_reduce_scatter_attr, CCL_DEPS);

CCL_API event send(void* buf, size_t count, datatype dtype, int peer, const communicator& comm, const stream& stream,
                   const pt2pt_attr& attr = default_pt2pt_attr, CCL_DEPS);
CCL_API event send(void* buf, size_t count, datatype dtype, int peer, const communicator& comm,
                   const pt2pt_attr& attr = default_pt2pt_attr, CCL_DEPS);
CCL_API event recv(void* buf, size_t count, datatype dtype, int peer, const communicator& comm, const stream& stream,
                   const pt2pt_attr& attr = default_pt2pt_attr, CCL_DEPS);
CCL_API event recv(void* buf, size_t count, datatype dtype, int peer, const communicator& comm,
                   const pt2pt_attr& attr = default_pt2pt_attr, CCL_DEPS);

// ---- operations: type-safe forms ------------------------------------------------------------
#define CCL_TYPED template <class T, class = typename std::enable_if<is_native_type_supported<T>(), event>::type>
#define CCL_DT native_type_info<typename std::remove_cv<T>::type>::dtype

CCL_TYPED event allgather(const T* send_buf, T* recv_buf, size_t count, const communicator& comm, const stream& s,
                          const allgather_attr& attr = default_allgather_attr, CCL_DEPS) {
    return allgather((const void*)send_buf, (void*)recv_buf, count, CCL_DT, comm, s, attr, deps);
}
CCL_TYPED event allgather(const T* send_buf, T* recv_buf, size_t count, const communicator& comm,
                          const allgather_attr& attr = default_allgather_attr, CCL_DEPS) {
    return allgather((const void*)send_buf, (void*)recv_buf, count, CCL_DT, comm, attr, deps);
}
CCL_TYPED event allgatherv(const T* send_buf, size_t send_count, T* recv_buf, const vector_class<size_t>& recv_counts,
                           const communicator& comm, const stream& s,
                           const allgatherv_attr& attr = default_allgatherv_attr, CCL_DEPS) {
    return allgatherv((const void*)send_buf, send_count, (void*)recv_buf, recv_counts, CCL_DT, comm, s, attr, deps);
}
CCL_TYPED event allgatherv(const T* send_buf, size_t send_count, T* recv_buf, const vector_class<size_t>& recv_counts,
                           const communicator& comm, const allgatherv_attr& attr = default_allgatherv_attr,
                           CCL_DEPS) {
    return allgatherv((const void*)send_buf, send_count, (void*)recv_buf, recv_counts, CCL_DT, comm, attr, deps);
}
CCL_TYPED event allgatherv(const T* send_buf, size_t send_count, vector_class<T*>& recv_bufs,
                           const vector_class<size_t>& recv_counts, const communicator& comm, const stream& s,
                           const allgatherv_attr& attr = default_allgatherv_attr, CCL_DEPS) {
    vector_class<void*> v(recv_bufs.begin(), recv_bufs.end());
    return allgatherv((const void*)send_buf, send_count, v, recv_counts, CCL_DT, comm, s, attr, deps);
}
CCL_TYPED event allgatherv(const T* send_buf, size_t send_count, vector_class<T*>& recv_bufs,
                           const vector_class<size_t>& recv_counts, const communicator& comm,
                           const allgatherv_attr& attr = default_allgatherv_attr, CCL_DEPS) {
    vector_class<void*> v(recv_bufs.begin(), recv_bufs.end());
    return allgatherv((const void*)send_buf, send_count, v, recv_counts, CCL_DT, comm, attr, deps);
}
CCL_TYPED event allreduce(const T* send_buf, T* recv_buf, size_t count, reduction rtype, const communicator& comm,
                          const stream& s, const allreduce_attr& attr = default_allreduce_attr, CCL_DEPS) {
    return allreduce((const void*)send_buf, (void*)recv_buf, count, CCL_DT, rtype, comm, s, attr, deps);
}
CCL_TYPED event allreduce(const T* send_buf, T* recv_buf, size_t count, reduction rtype, const communicator& comm,
                          const allreduce_attr& attr = default_allreduce_attr, CCL_DEPS) {
    return allreduce((const void*)send_buf, (void*)recv_buf, count, CCL_DT, rtype, comm, attr, deps);
}
CCL_TYPED event alltoall(const T* send_buf, T* recv_buf, size_t count, const communicator& comm, const stream& s,
                         const alltoall_attr& attr = default_alltoall_attr, CCL_DEPS) {
    return alltoall((const void*)send_buf, (void*)recv_buf, count, CCL_DT, comm, s, attr, deps);
}
CCL_TYPED event alltoall(const T* send_buf, T* recv_buf, size_t count, const communicator& comm,
                         const alltoall_attr& attr = default_alltoall_attr, CCL_DEPS) {
    return alltoall((const void*)send_buf, (void*)recv_buf, count, CCL_DT, comm, attr, deps);
}
CCL_TYPED event alltoallv(const T* send_buf, const vector_class<size_t>& send_counts, T* recv_buf,
                          const vector_class<size_t>& recv_counts, const communicator& comm, const stream& s,
                          const alltoallv_attr& attr = default_alltoallv_attr, CCL_DEPS) {
    return alltoallv((const void*)send_buf, send_counts, (void*)recv_buf, recv_counts, CCL_DT, comm, s, attr, deps);
}
CCL_TYPED event alltoallv(const T* send_buf, const vector_class<size_t>& send_counts, T* recv_buf,
                          const vector_class<size_t>& recv_counts, const communicator& comm,
                          const alltoallv_attr& attr = default_alltoallv_attr, CCL_DEPS) {
    return alltoallv((const void*)send_buf, send_counts, (void*)recv_buf, recv_counts, CCL_DT, comm, attr, deps);
}
CCL_TYPED event broadcast(T* buf, size_t count, int root, const communicator& comm, const stream& s,
                          const broadcast_attr& attr = default_broadcast_attr, CCL_DEPS) {
    return broadcast((void*)buf, count, CCL_DT, root, comm, s, attr, deps);
}
CCL_TYPED event broadcast(T* buf, size_t count, int root, const communicator& comm,
                          const broadcast_attr& attr = default_broadcast_attr, CCL_DEPS) {
    return broadcast((void*)buf, count, CCL_DT, root, comm, attr, deps);
}
CCL_TYPED event broadcast(T* send_buf, T* recv_buf, size_t count, int root, const communicator& comm,
                          const stream& s, const broadcast_attr& attr = default_broadcast_attr, CCL_DEPS) {
    return broadcast((void*)send_buf, (void*)recv_buf, count, CCL_DT, root, comm, s, attr, deps);
}
CCL_TYPED event broadcast(T* send_buf, T* recv_buf, size_t count, int root, const communicator& comm,
                          const broadcast_attr& attr = default_broadcast_attr, CCL_DEPS) {
    return broadcast((void*)send_buf, (void*)recv_buf, count, CCL_DT, root, comm, attr, deps);
}
CCL_TYPED event reduce(const T* send_buf, T* recv_buf, size_t count, reduction rtype, int root,
                       const communicator& comm, const stream& s, const reduce_attr& attr = default_reduce_attr,
                       CCL_DEPS) {
    return reduce((const void*)send_buf, (void*)recv_buf, count, CCL_DT, rtype, root, comm, s, attr, deps);
}
CCL_TYPED event reduce(const T* send_buf, T* recv_buf, size_t count, reduction rtype, int root,
                       const communicator& comm, const reduce_attr& attr = default_reduce_attr, CCL_DEPS) {
    return reduce((const void*)send_buf, (void*)recv_buf, count, CCL_DT, rtype, root, comm, attr, deps);
}
CCL_TYPED event reduce_scatter(const T* send_buf, T* recv_buf, size_t recv_count, reduction rtype,
                               const communicator& comm, const stream& s,
                               const reduce_scatter_attr& attr = default_reduce_scatter_attr, CCL_DEPS) {
    return reduce_scatter((const void*)send_buf, (void*)recv_buf, recv_count, CCL_DT, rtype, comm, s, attr, deps);
}
CCL_TYPED event reduce_scatter(const T* send_buf, T* recv_buf, size_t recv_count, reduction rtype,
                               const communicator& comm,
                               const reduce_scatter_attr& attr = default_reduce_scatter_attr, CCL_DEPS) {
    return reduce_scatter((const void*)send_buf, (void*)recv_buf, recv_count, CCL_DT, rtype, comm, attr, deps);
}
CCL_TYPED event send(T* buf, size_t count, int peer, const communicator& comm, const stream& s,
                     const pt2pt_attr& attr = default_pt2pt_attr, CCL_DEPS) {
    return send((void*)buf, count, CCL_DT, peer, comm, s, attr, deps);
}
CCL_TYPED event send(T* buf, size_t count, int peer, const communicator& comm,
                     const pt2pt_attr& attr = default_pt2pt_attr, CCL_DEPS) {
    return send((void*)buf, count, CCL_DT, peer, comm, attr, deps);
}
CCL_TYPED event recv(T* buf, size_t count, int peer, const communicator& comm, const stream& s,
                     const pt2pt_attr& attr = default_pt2pt_attr, CCL_DEPS) {
    return recv((void*)buf, count, CCL_DT, peer, comm, s, attr, deps);
}
CCL_TYPED event recv(T* buf, size_t count, int peer, const communicator& comm,
                     const pt2pt_attr& attr = default_pt2pt_attr, CCL_DEPS) {
    return recv((void*)buf, count, CCL_DT, peer, comm, attr, deps);
}

#undef CCL_TYPED
#undef CCL_DT
#undef CCL_DEPS

} // namespace v1

using namespace v1;

// Functions the reference keeps in ccl::preview (include/oneapi/ccl/api_functions.hpp:242-254,328-379).
namespace preview {

// A communicator whose size, rank and key-value store come from the process launcher: a PMI-1 process
// manager (Hydra's mpiexec: PMI_FD / PMI_PORT), or torchrun-style variables (RANK, WORLD_SIZE, MASTER_ADDR,
// MASTER_PORT); a process that no launcher started gets a communicator of size 1.
CCL_API communicator create_communicator(const comm_attr& attr = default_comm_attr);

template <class... Avs>
comm_split_attr create_comm_split_attr(Avs&&... avs) {
    return v1::create_comm_split_attr(std::forward<Avs>(avs)...);
}

// one split per (communicator, attribute) pair
CCL_API vector_class<communicator> split_communicators(
    const vector_class<pair_class<communicator, comm_split_attr>>& attrs);

// Extension (no counterpart in the oneCCL specification): in-place allreduce of several buffers of one
// datatype as ONE operation.  Device buffers of a single node are packed into a buffer of the symmetric heap by
// one kernel, reduced by one zero-copy allreduce and unpacked by one kernel, on the given stream; host buffers
// are issued one by one.  The event covers every buffer.  What CCL_FUSION=1 does behind the ordinary allreduce,
// without the queueing.
CCL_API event allreduce_coalesced(const vector_class<void*>& bufs, const vector_class<size_t>& counts, datatype dtype,
                                  reduction rtype, const communicator& comm, const stream& s,
                                  const allreduce_attr& attr = default_allreduce_attr);
CCL_API event allreduce_coalesced(const vector_class<void*>& bufs, const vector_class<size_t>& counts, datatype dtype,
                                  reduction rtype, const communicator& comm,
                                  const allreduce_attr& attr = default_allreduce_attr);

} // namespace preview

} // namespace ccl
