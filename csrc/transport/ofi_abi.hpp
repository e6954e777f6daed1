// The part of the libfabric 1.x binary interface that the OFI transport uses, declared here so that the
// library needs no libfabric headers to build and no libfabric to load (the shared object is opened at run
// time, like the reference does: src/common/api_wrapper/ofi_api_wrapper.cpp:26-84).  libfabric objects are
// structures that start with a `fid` and carry tables of function pointers; the "functions" of its API are
// inline calls through those tables.  Only the members up to the last one used matter for the layout, but the
// tables are declared in full up to that point; structures that the provider allocates (fi_info and its
// attribute blocks) are declared completely because fi_dupinfo / fi_getinfo hand them back filled in.
#pragma once
#include <stddef.h>
#include <stdint.h>
#include <sys/types.h>
#include <sys/uio.h>

namespace cclx {
namespace ofi {

typedef uint64_t fi_addr_t;
constexpr uint64_t ADDR_UNSPEC = (uint64_t)-1;
constexpr uint32_t make_version(uint32_t major, uint32_t minor) {
    return (major << 16) | minor;
}

// capability / flag bits
constexpr uint64_t CAP_MSG = 1ull << 1, CAP_TAGGED = 1ull << 3, CAP_RECV = 1ull << 10, CAP_SEND = 1ull << 11;
constexpr uint64_t FLAG_PEEK = 1ull << 19, CAP_DIRECTED_RECV = 1ull << 59, CAP_LOCAL_COMM = 1ull << 51,
                   CAP_REMOTE_COMM = 1ull << 52;
constexpr uint64_t MODE_CONTEXT = 1ull << 59, MODE_CONTEXT2 = 1ull << 52;
constexpr uint64_t ORDER_SAS = 1ull << 8;
// enums (values of the C enums)
enum { EP_UNSPEC = 0, EP_MSG, EP_DGRAM, EP_RDM };
enum { AV_UNSPEC = 0, AV_MAP, AV_TABLE };
enum { PROGRESS_UNSPEC = 0, PROGRESS_AUTO, PROGRESS_MANUAL };
enum { THREAD_UNSPEC = 0, THREAD_SAFE, THREAD_FID, THREAD_DOMAIN, THREAD_COMPLETION, THREAD_ENDPOINT };
enum { RM_UNSPEC = 0, RM_DISABLED, RM_ENABLED };
enum { CQ_FORMAT_UNSPEC = 0, CQ_FORMAT_CONTEXT, CQ_FORMAT_MSG, CQ_FORMAT_DATA, CQ_FORMAT_TAGGED };
enum { WAIT_NONE = 0 };
enum { CTRL_ENABLE = 6 }; // control command that activates an endpoint
// error numbers (libfabric returns negative errno values)
constexpr int E_AGAIN = 11, E_NOMSG = 42, E_CANCELED = 125, E_AVAIL = 259, E_TRUNC = 265;

struct fid;
struct fid_fabric;
struct fid_domain;
struct fid_ep;
struct fid_cq;
struct fid_av;
struct fi_info;

struct fi_ops {
    size_t size;
    int (*close)(fid*);
    int (*bind)(fid*, fid* bfid, uint64_t flags);
    int (*control)(fid*, int command, void* arg);
    int (*ops_open)(fid*, const char*, uint64_t, void**, void*);
    int (*tostr)(const fid*, char*, size_t);
    int (*ops_set)(fid*, const char*, uint64_t, void*, void*);
};
struct fid {
    size_t fclass;
    void* context;
    fi_ops* ops;
};

struct fi_tx_attr {
    uint64_t caps, mode, op_flags, msg_order, comp_order;
    size_t inject_size, size, iov_limit, rma_iov_limit;
    uint32_t tclass;
};
struct fi_rx_attr {
    uint64_t caps, mode, op_flags, msg_order, comp_order;
    size_t total_buffered_recv, size, iov_limit;
};
struct fi_ep_attr {
    int type;
    uint32_t protocol, protocol_version;
    size_t max_msg_size, msg_prefix_size, max_order_raw_size, max_order_war_size, max_order_waw_size;
    uint64_t mem_tag_format;
    size_t tx_ctx_cnt, rx_ctx_cnt, auth_key_size;
    uint8_t* auth_key;
};
struct fi_domain_attr {
    fid_domain* domain;
    char* name;
    int threading, control_progress, data_progress, resource_mgmt, av_type, mr_mode;
    size_t mr_key_size, cq_data_size, cq_cnt, ep_cnt, tx_ctx_cnt, rx_ctx_cnt, max_ep_tx_ctx, max_ep_rx_ctx,
        max_ep_stx_ctx, max_ep_srx_ctx, cntr_cnt, mr_iov_limit;
    uint64_t caps, mode;
    uint8_t* auth_key;
    size_t auth_key_size, max_err_data, mr_cnt;
    uint32_t tclass;
    size_t max_ep_auth_key;
};
struct fi_fabric_attr {
    fid_fabric* fabric;
    char* name;
    char* prov_name;
    uint32_t prov_version, api_version;
};
struct fi_info {
    fi_info* next;
    uint64_t caps, mode;
    uint32_t addr_format;
    size_t src_addrlen, dest_addrlen;
    void* src_addr;
    void* dest_addr;
    fid* handle;
    fi_tx_attr* tx_attr;
    fi_rx_attr* rx_attr;
    fi_ep_attr* ep_attr;
    fi_domain_attr* domain_attr;
    fi_fabric_attr* fabric_attr;
    void* nic;
};

struct fi_ops_fabric {
    size_t size;
    int (*domain)(fid_fabric*, fi_info*, fid_domain**, void* context);
    // passive_ep, eq_open, wait_open, trywait, domain2 follow (unused)
};
struct fid_fabric {
    fid f;
    fi_ops_fabric* ops;
    uint32_t api_version;
};

struct fi_av_attr {
    int type;
    int rx_ctx_bits;
    size_t count, ep_per_node;
    const char* name;
    void* map_addr;
    uint64_t flags;
};
struct fi_cq_attr {
    size_t size;
    uint64_t flags;
    int format;
    int wait_obj;
    int signaling_vector;
    int wait_cond;
    void* wait_set;
};
struct fi_ops_domain {
    size_t size;
    int (*av_open)(fid_domain*, fi_av_attr*, fid_av**, void* context);
    int (*cq_open)(fid_domain*, fi_cq_attr*, fid_cq**, void* context);
    int (*endpoint)(fid_domain*, fi_info*, fid_ep**, void* context);
    // scalable_ep, cntr_open, poll_open, stx_ctx, srx_ctx, query_atomic, query_collective, endpoint2 follow
};
struct fid_domain {
    fid f;
    fi_ops_domain* ops;
    void* mr;
};

struct fi_ops_av {
    size_t size;
    int (*insert)(fid_av*, const void* addr, size_t count, fi_addr_t* fi_addr, uint64_t flags, void* context);
    // insertsvc, insertsym, remove, lookup, straddr, ... follow
};
struct fid_av {
    fid f;
    fi_ops_av* ops;
};

struct fi_cq_tagged_entry {
    void* op_context;
    uint64_t flags;
    size_t len;
    void* buf;
    uint64_t data;
    uint64_t tag;
};
struct fi_cq_err_entry {
    void* op_context;
    uint64_t flags;
    size_t len;
    void* buf;
    uint64_t data;
    uint64_t tag;
    size_t olen;
    int err;
    int prov_errno;
    void* err_data;
    size_t err_data_size;
    fi_addr_t src_addr;
};
struct fi_ops_cq {
    size_t size;
    ssize_t (*read)(fid_cq*, void* buf, size_t count);
    ssize_t (*readfrom)(fid_cq*, void* buf, size_t count, fi_addr_t* src);
    ssize_t (*readerr)(fid_cq*, fi_cq_err_entry* buf, uint64_t flags);
    // sread, sreadfrom, signal, strerror follow
};
struct fid_cq {
    fid f;
    fi_ops_cq* ops;
};

struct fi_ops_cm {
    size_t size;
    int (*setname)(fid*, void* addr, size_t addrlen);
    int (*getname)(fid*, void* addr, size_t* addrlen);
    // getpeer, connect, listen, accept, reject, shutdown, join follow
};
struct fi_msg_tagged {
    const iovec* msg_iov;
    void** desc;
    size_t iov_count;
    fi_addr_t addr;
    uint64_t tag;
    uint64_t ignore;
    void* context;
    uint64_t data;
};
struct fi_ops_tagged {
    size_t size;
    ssize_t (*recv)(fid_ep*, void* buf, size_t len, void* desc, fi_addr_t src, uint64_t tag, uint64_t ignore,
                    void* context);
    ssize_t (*recvv)(fid_ep*, const iovec*, void** desc, size_t count, fi_addr_t src, uint64_t tag, uint64_t ignore,
                     void* context);
    ssize_t (*recvmsg)(fid_ep*, const fi_msg_tagged* msg, uint64_t flags);
    ssize_t (*send)(fid_ep*, const void* buf, size_t len, void* desc, fi_addr_t dest, uint64_t tag, void* context);
    // sendv, sendmsg, inject, senddata, injectdata follow
};
struct fi_ops_ep {
    size_t size;
    ssize_t (*cancel)(fid*, void* context);
    // getopt, setopt, tx_ctx, rx_ctx, rx_size_left, tx_size_left follow
};
struct fid_ep {
    fid f;
    fi_ops_ep* ops;
    fi_ops_cm* cm;
    void* msg;
    void* rma;
    fi_ops_tagged* tagged;
    void* atomic;
    void* collective;
};

// space the provider may use per operation in flight (FI_CONTEXT / FI_CONTEXT2 modes)
struct op_context {
    void* internal[8];
};

// the exported functions, resolved with dlsym
struct library {
    int (*getinfo)(uint32_t version, const char* node, const char* service, uint64_t flags, const fi_info* hints,
                   fi_info** info) = nullptr;
    void (*freeinfo)(fi_info*) = nullptr;
    fi_info* (*dupinfo)(const fi_info*) = nullptr;
    int (*fabric)(fi_fabric_attr*, fid_fabric**, void* context) = nullptr;
    const char* (*strerror)(int) = nullptr;
    uint32_t (*version)() = nullptr;
    void* handle = nullptr;
    const char* path = "";
};

} // namespace ofi
} // namespace cclx
