// Shared pieces of the launch translation units: datatype / reduction dispatch
// and the real-vs-emulated launch helper.
#pragma once
#include <algorithm>
#include <map>
#include <mutex>
#include <utility>

#include "core/env.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"
#include "gpu/device/collectives.cuh"
#include "gpu/buffer_exchange.hpp"
#include "gpu/device_comm.hpp"

namespace cclx {
namespace gpu {

#define CCLX_DISPATCH_DTYPE(dt, T, ...)                                  \
    switch (dt) {                                                        \
        case dt_int8: { typedef signed char T; __VA_ARGS__; } break;     \
        case dt_uint8: { typedef unsigned char T; __VA_ARGS__; } break;  \
        case dt_int16: { typedef short T; __VA_ARGS__; } break;          \
        case dt_uint16: { typedef unsigned short T; __VA_ARGS__; } break; \
        case dt_int32: { typedef int T; __VA_ARGS__; } break;            \
        case dt_uint32: { typedef unsigned int T; __VA_ARGS__; } break;  \
        case dt_int64: { typedef long long T; __VA_ARGS__; } break;      \
        case dt_uint64: { typedef unsigned long long T; __VA_ARGS__; } break; \
        case dt_float16: { typedef __half T; __VA_ARGS__; } break;       \
        case dt_float32: { typedef float T; __VA_ARGS__; } break;        \
        case dt_float64: { typedef double T; __VA_ARGS__; } break;       \
        case dt_bfloat16: { typedef __nv_bfloat16 T; __VA_ARGS__; } break; \
        default: CCL_THROW("datatype ", dt, " is not supported by the GPU reduction kernels"); \
    }

#define CCLX_DISPATCH_OP(op, OP, ...)                                   \
    switch (op) {                                                       \
        case red_sum: { typedef dev::op_sum OP; __VA_ARGS__; } break;   \
        case red_prod: { typedef dev::op_prod OP; __VA_ARGS__; } break; \
        case red_min: { typedef dev::op_min OP; __VA_ARGS__; } break;   \
        case red_max: { typedef dev::op_max OP; __VA_ARGS__; } break;   \
        default: CCL_THROW("reduction ", op, " is not supported on GPU buffers"); \
    }

// Reductions: every same-type pair for the four built-in ops, plus the
// widening / narrowing sum pairs used by mixed-precision data parallelism.
// F is a generic lambda called as F(Tin{}, Tout{}, Op{}).
template <class F>
void dispatch_reduce_types(int dt_in, int dt_out, int op, F&& f) {
    if (dt_in == dt_out) {
        CCLX_DISPATCH_DTYPE(dt_in, T, CCLX_DISPATCH_OP(op, OP, f(T(), T(), OP())));
        return;
    }
    CCL_THROW_IF_NOT(op == red_sum, "mixed-precision reductions support sum only");
    if (dt_in == dt_bfloat16 && dt_out == dt_float32)
        f(__nv_bfloat16(), float(), dev::op_sum());
    else if (dt_in == dt_float16 && dt_out == dt_float32)
        f(__half(), float(), dev::op_sum());
    else if (dt_in == dt_float32 && dt_out == dt_bfloat16)
        f(float(), __nv_bfloat16(), dev::op_sum());
    else
        CCL_THROW("unsupported datatype pair ", dt_in, " -> ", dt_out);
}

inline bool nvls_type_ok(int dt, int op) {
    return op == red_sum && (dt == dt_float32 || dt == dt_bfloat16 || dt == dt_float16);
}

inline int pick_blocks(const device_comm& dc, size_t units, size_t units_per_block, int requested) {
    int cap = dc.max_blocks();
    if (requested > 0)
        return std::max(1, std::min(requested, cap));
    size_t want = (units + units_per_block - 1) / std::max<size_t>(units_per_block, 1);
    return (int)std::max<size_t>(1, std::min<size_t>(want, (size_t)cap));
}

// Where the send (or recv) buffers of a collective live, for the zero-copy kernels: the same offset of
// the symmetric heap on every rank, or the same offset of one registered allocation on every rank.
struct zc_view {
    bool ok = false;
    bool registered = false; // peers are reached through per-rank pointers (not heap base + one offset)
    size_t off = 0; // heap offset, or offset inside the registration
    int id = -1;
    bool shared = false; // the per-rank pointers came from the automatic buffer exchange: ptr[]
    char* ptr[dev::MAX_RANKS] = {};
};

inline zc_view zero_copy_view(const device_comm& dc, const dev::rank_args* ra, bool recv_side, size_t bytes) {
    zc_view v;
    const int entries = dc.emulated() ? dc.world() : 1;
    bool heap = true, reg = true;
    size_t hoff = 0, roff = 0;
    int rid = -1;
    for (int e = 0; e < entries; e++) {
        const void* p = recv_side ? (const void*)ra[e].recv : ra[e].send;
        const int owner = dc.emulated() ? e : dc.rank();
        if (!p)
            return v;
        if (heap) {
            const size_t o = dc.symm_offset(p, owner);
            if (o == (size_t)-1 || (o & 15) || (e > 0 && o != hoff))
                heap = false;
            hoff = o;
        }
        if (reg) {
            int id = -1;
            size_t o = 0;
            if (!dc.find_user(p, bytes, owner, id, o) || (((uintptr_t)p) & 15) || (e > 0 && (id != rid || o != roff)))
                reg = false;
            rid = id;
            roff = o;
        }
    }
    if (heap) {
        v.ok = true;
        v.off = hoff;
    }
    else if (reg) {
        v.ok = true;
        v.registered = true;
        v.off = roff;
        v.id = rid;
    }
    return v;
}

// rank q's buffer of a registered / automatically shared view, as mapped in this process
inline char* view_ptr(const device_comm& dc, const zc_view& v, int q) {
    return v.shared ? v.ptr[q] : dc.user_base(v.id, q) + v.off;
}

// Both sides of a collective at once.  Small messages decide locally (symmetric heap or explicit
// registration, as zero_copy_view).  From CCL_CUDA_AUTO_REGISTER_MIN_BYTES on, in multi-process mode, the
// ranks tell one another where their buffers live (buffer_exchange): ordinary cudaMalloc memory, e.g. a
// torch tensor, then takes the zero-copy kernels as well, offsets may differ between ranks, and all ranks
// reach the same verdict (zero-copy only if every rank's buffer can be shared).  The sizes are the same on
// every rank, so either all ranks enter the exchange or none does.
// `allow_exchange` = false keeps the local decision for large messages too (a caller that would rather stage an
// ordinary buffer than share it; it must decide that from values that are equal on every rank).
inline void zero_copy_views(device_comm& dc, const dev::rank_args* ra, bool want_in, size_t in_bytes, bool want_out,
                            size_t out_bytes, zc_view& vin, zc_view& vout, bool allow_exchange = true) {
    if (want_in)
        vin = zero_copy_view(dc, ra, false, in_bytes);
    if (want_out)
        vout = zero_copy_view(dc, ra, true, out_bytes);
    buffer_exchange* bx = dc.exchange();
    const size_t big = std::max(want_in ? in_bytes : 0, want_out ? out_bytes : 0);
    if (dc.emulated() || !bx || !allow_exchange || big < env_data::get().auto_register_min)
        return;
    shared_view in, out;
    bx->exchange(want_in ? ra[0].send : nullptr, in_bytes, want_out ? ra[0].recv : nullptr, out_bytes, in, out);
    auto apply = [&](const shared_view& sv, zc_view& v) {
        v = zc_view();
        if (!sv.ok)
            return;
        v.ok = true;
        if (sv.heap_equal) {
            v.off = sv.heap_off;
            return;
        }
        v.registered = v.shared = true;
        for (int q = 0; q < dc.world(); q++)
            v.ptr[q] = sv.ptr[q];
    };
    if (want_in)
        apply(in, vin);
    if (want_out)
        apply(out, vout);
}

// peers' addresses of a registered buffer into the argument block
inline void fill_registered(const device_comm& dc, dev::coll_args& a, const zc_view& v, bool recv_side) {
    for (int q = 0; q < dc.world(); q++) {
        if (recv_side)
            a.reg_out[q] = view_ptr(dc, v, q);
        else
            a.reg_in[q] = view_ptr(dc, v, q);
    }
    a.flags |= recv_side ? dev::CF_REG_OUT : dev::CF_REG_IN;
}

// Fill the mode-dependent part of coll_args.  In emulation mode the per-rank
// table is uploaded to the device (the stream is drained first because an
// earlier launch may still read the previous table).
inline void prepare_args(device_comm& dc, dev::coll_args& a, const dev::rank_args* ra, cudaStream_t st) {
    a.sig_skew = dc.test_sig_skew;
    if (dc.emulated()) {
        CUDA_CHECK(cudaStreamSynchronize(st));
        CUDA_CHECK(cudaMemcpy(dc.emu_args_dev(), ra, dc.world() * sizeof(dev::rank_args), cudaMemcpyHostToDevice));
        a.emu = 1;
        a.emu_tab = dc.emu_args_dev();
        a.r0 = ra[0];
    }
    else {
        a.emu = 0;
        a.emu_tab = nullptr;
        a.r0 = ra[0];
    }
}

// Blocks of one kernel that can be resident at the same time on an otherwise idle GPU (occupancy of the
// kernel at this block size x SMs), looked up once per (kernel, block size).  Blocks of a collective kernel
// wait for the block of the same index on every peer, so a grid above this number could leave a block
// waiting for a peer's block that is queued behind it: launch_kernel refuses such a grid.  (The
// reference states the same rule for its SYCL kernels: threads <= hardware threads, else deadlock,
// src/coll/algorithms/allreduce/sycl/allreduce_small_sycl_impl.hpp:170-182.)
template <class K>
int resident_blocks(const device_comm& dc, K kernel, int threads) {
    static std::mutex mu;
    static std::map<std::pair<const void*, int>, int> cache;
    std::lock_guard<std::mutex> g(mu);
    const auto key = std::make_pair((const void*)kernel, threads * 64 + dc.device_id());
    auto it = cache.find(key);
    if (it != cache.end())
        return it->second;
    int per_sm = 0;
    CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0));
    const int n = per_sm * dc.sm_count();
    cache[key] = n;
    return n;
}

template <class K, class... Args>
void launch_kernel(device_comm& dc, K kernel, int blocks, int threads, cudaStream_t st, Args... args) {
    dc.check_status();
    if (dc.emulated()) {
        void* argv[] = { (void*)&args... };
        dim3 grid(blocks, dc.world());
        CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3(threads), argv, 0, st));
    }
    else {
        const int cap = resident_blocks(dc, kernel, threads);
        CCL_THROW_IF_NOT(blocks <= cap, "a collective kernel was asked for ", blocks, " blocks of ", threads,
                         " threads but only ", cap, " can be resident at once");
        kernel<<<blocks, threads, 0, st>>>(args...);
        CUDA_CHECK(cudaGetLastError());
    }
}

} // namespace gpu
} // namespace cclx
