// Device-side building blocks shared by every collective kernel:
//  * comm_dev       : what a kernel needs to know about one rank (peer-mapped
//                     flag arenas / staging / heap, NVLS multicast window,
//                     status words), resident in device memory.
//  * peer_barrier   : bounded cross-GPU barrier on monotonic epoch flags.  It
//                     plays the role of the reference's comm_barrier
//                     (src/coll/algorithms/utils/sycl_kernels.hpp:103-146), but
//                     with release/acquire at system scope on per-block slots
//                     and a time limit after which the kernel reports an error
//                     status instead of spinning forever.
//  * 16-byte pack helpers and typed accumulate ops (bf16/fp16 accumulate in
//                     fp32, like the reference's bf16 kernels: src/kernels/bf16.h:18-66).
//
// A kernel can run in two modes.  Real mode: one process per GPU, the table has
// one entry.  Emulation mode: all ranks live on one GPU, the launch is
// cooperative with gridDim.y == world and blockIdx.y selects the rank; this is
// how multi-rank logic is exercised on a single device.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gpu/device/layout.hpp"

namespace cclx {
namespace dev {

// ---- memory-model helpers -------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// 16-byte load that never hits a stale L1 line (peer / staging data written by other GPUs)
__device__ __forceinline__ uint4 ld_cv16(const void* p) {
    return __ldcv(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void st16(void* p, const uint4& v) {
    *reinterpret_cast<uint4*>(p) = v;
}

// ---- NVLS multimem ----------------------------------------------------------
__device__ __forceinline__ void multimem_st16(void* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x),
                 "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
template <class T>
__device__ __forceinline__ uint4 multimem_ld_reduce_add16(const void* mc);
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add16<float>(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add16<__nv_bfloat16>(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add16<__half>(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}

// ---- per-kernel synchronisation state ---------------------------------------
struct block_sync {
    uint32_t epoch; // value of the last barrier this comm completed before this kernel
    uint32_t gen; // staging generation used by this kernel (0/1)
    uint32_t used; // barriers executed so far by this kernel
    bool ok;
};

__device__ __forceinline__ void sync_begin(const comm_dev& c, block_sync& s) {
    s.epoch = ld_volatile_u32(c.state + STATE_EPOCH);
    s.gen = ld_volatile_u32(c.state + STATE_GEN) & 1u;
    s.used = 0;
    s.ok = true;
}

// Called by every block exactly once at the end of a kernel.  The last block of
// this rank to finish publishes the new epoch / generation for the next kernel.
// `nblocks` is the number of blocks of this rank (gridDim.x), `nbarriers` the
// number of peer_barrier calls every block of this kernel makes.
__device__ __forceinline__ void sync_end(const comm_dev& c, uint32_t nblocks, uint32_t nbarriers,
                                         uint32_t advance_gen) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        uint32_t done = atomicAdd(c.state + STATE_DONE, 1u);
        if (done == nblocks - 1) {
            c.state[STATE_EPOCH] += nbarriers;
            c.state[STATE_GEN] += advance_gen;
            __threadfence();
            c.state[STATE_DONE] = 0;
        }
    }
}

__device__ __forceinline__ void report(const comm_dev& c, uint32_t code, uint32_t peer, uint32_t detail) {
    if (c.status[0] == ST_OK) {
        c.status[1] = blockIdx.x;
        c.status[2] = peer;
        c.status[3] = detail;
        __threadfence_system();
        c.status[0] = code;
    }
}

// Spin until *p reaches `target` (wrap-safe), the abort flag is raised or the
// time limit passes.  Returns false on timeout/abort after recording the status.
__device__ __forceinline__ bool wait_flag_sys(const comm_dev& c, const uint32_t* p, uint32_t target,
                                              uint32_t peer, uint32_t code) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0;; it++) {
        uint32_t v = ld_acquire_sys(p);
        if ((int32_t)(v - target) >= 0)
            return true;
        if ((it & 0x3ff) == 0x3ff) {
            unsigned long long now = globaltimer_ns();
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > c.timeout_ns) {
                report(c, code, peer, target);
                return false;
            }
            if (*c.abort_flag) {
                report(c, ST_ABORTED, peer, target);
                return false;
            }
        }
    }
}

// Cross-GPU barrier among the blocks with the same blockIdx.x on every rank.
// All threads of the block must call it.  Writes made by any thread of the
// block before the call are visible to the peers' threads after their call
// returns (bar.sync + release.sys / acquire.sys + bar.sync).
//
// `sig` (non-zero; used by the first barrier of a kernel) is a hash of the arguments that must be
// equal on every rank because the kernel applies them to the peers' memory (buffer kind, heap offsets,
// count).  Every rank leaves its value in the peers' signature words before it raises its flag and
// compares the peers' values with its own once their flags have arrived; a difference ends the kernel
// with ST_ARG_MISMATCH before any data is touched.  The slot is chosen by the barrier's epoch, so a
// peer that is already in its next kernel writes another slot.
__device__ __forceinline__ bool peer_barrier(const comm_dev& c, block_sync& s, uint32_t sig = 0) {
    __shared__ int bar_fail;
    if (threadIdx.x == 0)
        bar_fail = 0;
    __syncthreads();
    s.used++;
    const uint32_t target = s.epoch + s.used;
    if (s.ok && threadIdx.x < (unsigned)c.world) {
        const int p = threadIdx.x;
        const bool check = sig != 0 && s.used == 1; // every block checks: all of them write the same word
        const int slot = SIG_BASE_WORD + (int)(target % SIG_SLOTS) * MAX_RANKS;
        if (check)
            c.p2p_flags[p][slot + c.rank] = sig;
        // the release store is the only system-scope fence of the barrier: it orders the
        // block's earlier writes (made visible to this thread by bar.sync) before the flag
        st_release_sys(c.flags[p] + blockIdx.x * MAX_RANKS + c.rank, target);
        if (!wait_flag_sys(c, c.flags[c.rank] + blockIdx.x * MAX_RANKS + p, target, p, ST_BARRIER_TIMEOUT))
            bar_fail = 1;
        else if (check) {
            const uint32_t theirs = ld_volatile_u32(c.p2p_flags[c.rank] + slot + p);
            if (theirs != sig) {
                report(c, ST_ARG_MISMATCH, p, theirs);
                bar_fail = 1;
            }
        }
    }
    __syncthreads();
    if (bar_fail)
        s.ok = false;
    return s.ok;
}

// Hash of the arguments of a zero-copy collective that every rank must pass alike (never zero).
__device__ __forceinline__ uint32_t arg_signature(uint32_t kind, size_t in_off, size_t out_off, size_t count,
                                                  uint32_t flags) {
    unsigned long long h = 0x9E3779B97F4A7C15ull * (kind + 1);
    h = (h ^ (unsigned long long)in_off) * 0xBF58476D1CE4E5B9ull;
    h = (h ^ (unsigned long long)out_off) * 0x94D049BB133111EBull;
    h = (h ^ (unsigned long long)count) * 0xBF58476D1CE4E5B9ull;
    h = (h ^ flags) * 0x94D049BB133111EBull;
    const uint32_t r = (uint32_t)(h >> 32) ^ (uint32_t)h;
    return r ? r : 1u;
}

// ---- typed packs --------------------------------------------------------------
template <class T>
struct acc_of {
    typedef T type;
};
template <>
struct acc_of<__nv_bfloat16> {
    typedef float type;
};
template <>
struct acc_of<__half> {
    typedef float type;
};

template <class A, class T>
__device__ __forceinline__ A to_acc(T v) {
    return (A)v;
}
template <>
__device__ __forceinline__ float to_acc<float, __nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float to_acc<float, __half>(__half v) {
    return __half2float(v);
}

template <class T, class A>
__device__ __forceinline__ T from_acc(A v) {
    return (T)v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, float>(float v) {
    return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_acc<__half, float>(float v) {
    return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, double>(double v) {
    return __float2bfloat16_rn((float)v);
}
template <>
__device__ __forceinline__ __half from_acc<__half, double>(double v) {
    return __float2half_rn((float)v);
}

struct op_sum {
    template <class A>
    static __device__ __forceinline__ A apply(A a, A b) {
        return a + b;
    }
};
struct op_prod {
    template <class A>
    static __device__ __forceinline__ A apply(A a, A b) {
        return a * b;
    }
};
struct op_min {
    template <class A>
    static __device__ __forceinline__ A apply(A a, A b) {
        return b < a ? b : a;
    }
};
struct op_max {
    template <class A>
    static __device__ __forceinline__ A apply(A a, A b) {
        return a < b ? b : a;
    }
};

template <class T>
struct pack_traits {
    static constexpr int N = 16 / (int)sizeof(T);
};

template <class T, class A>
__device__ __forceinline__ void unpack16(const uint4& v, A (&a)[pack_traits<T>::N]) {
    const T* t = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int k = 0; k < pack_traits<T>::N; k++)
        a[k] = to_acc<A, T>(t[k]);
}
template <class T, class A, class Op>
__device__ __forceinline__ void accum16(const uint4& v, A (&a)[pack_traits<T>::N]) {
    const T* t = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int k = 0; k < pack_traits<T>::N; k++)
        a[k] = Op::apply(a[k], to_acc<A, T>(t[k]));
}

// scale is applied only to floating accumulators
template <class A>
__device__ __forceinline__ A apply_scale(A a, float) {
    return a;
}
template <>
__device__ __forceinline__ float apply_scale<float>(float a, float s) {
    return a * s;
}
template <>
__device__ __forceinline__ double apply_scale<double>(double a, float s) {
    return a * (double)s;
}

// Store N accumulators as N contiguous Tout values at dst (dst is aligned to
// min(16, N*sizeof(Tout)) bytes by construction of the callers).
template <class Tout, class A, int N>
__device__ __forceinline__ void store_out(Tout* dst, const A (&a)[N], float scale, bool do_scale) {
    constexpr int BYTES = N * (int)sizeof(Tout);
    static_assert(BYTES % 16 == 0 || BYTES < 16, "pack size");
    if constexpr (BYTES >= 16) {
        constexpr int PER = 16 / (int)sizeof(Tout);
#pragma unroll
        for (int q = 0; q < BYTES / 16; q++) {
            uint4 o;
            Tout* t = reinterpret_cast<Tout*>(&o);
#pragma unroll
            for (int k = 0; k < PER; k++) {
                A v = a[q * PER + k];
                t[k] = from_acc<Tout, A>(do_scale ? apply_scale<A>(v, scale) : v);
            }
            reinterpret_cast<uint4*>(dst)[q] = o;
        }
    }
    else {
#pragma unroll
        for (int k = 0; k < N; k++) {
            A v = a[k];
            dst[k] = from_acc<Tout, A>(do_scale ? apply_scale<A>(v, scale) : v);
        }
    }
}

// Block-cooperative byte copy.  Uses 16-byte accesses when both pointers are
// 16-byte aligned, 4-byte when 4-byte aligned, bytes otherwise.  `volatile_src`
// selects loads that bypass L1 (data written by another GPU).
template <bool VOLATILE_SRC>
__device__ __forceinline__ void threads_copy(void* dst, const void* src, size_t bytes, size_t tid, size_t nt);

template <bool VOLATILE_SRC>
__device__ __forceinline__ void block_copy(void* dst, const void* src, size_t bytes) {
    threads_copy<VOLATILE_SRC>(dst, src, bytes, threadIdx.x, blockDim.x);
}

// The same copy by a subset of the block: `nt` threads numbered `tid` = 0 .. nt - 1.
template <bool VOLATILE_SRC>
__device__ __forceinline__ void threads_copy(void* dst, const void* src, size_t bytes, size_t tid, size_t nt) {
    const uintptr_t d = (uintptr_t)dst, s = (uintptr_t)src;
    if (((d | s) & 15) == 0) {
        const size_t nv = bytes >> 4;
        const uint4* sv = reinterpret_cast<const uint4*>(src);
        uint4* dv = reinterpret_cast<uint4*>(dst);
        size_t i = tid;
        if (VOLATILE_SRC) { // a source behind NVLink: more loads in flight per thread
            for (; i + 7 * nt < nv; i += 8 * nt) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; u++)
                    v[u] = __ldcv(sv + i + u * nt);
#pragma unroll
                for (int u = 0; u < 8; u++)
                    dv[i + u * nt] = v[u];
            }
        }
        for (; i + 3 * nt < nv; i += 4 * nt) {
            uint4 a, b, c2, e;
            if (VOLATILE_SRC) {
                a = __ldcv(sv + i);
                b = __ldcv(sv + i + nt);
                c2 = __ldcv(sv + i + 2 * nt);
                e = __ldcv(sv + i + 3 * nt);
            }
            else {
                a = sv[i];
                b = sv[i + nt];
                c2 = sv[i + 2 * nt];
                e = sv[i + 3 * nt];
            }
            dv[i] = a;
            dv[i + nt] = b;
            dv[i + 2 * nt] = c2;
            dv[i + 3 * nt] = e;
        }
        for (; i < nv; i += nt)
            dv[i] = VOLATILE_SRC ? __ldcv(sv + i) : sv[i];
        const size_t done = nv << 4;
        const unsigned char* sb = reinterpret_cast<const unsigned char*>(src) + done;
        unsigned char* db = reinterpret_cast<unsigned char*>(dst) + done;
        for (size_t k = tid; k < bytes - done; k += nt)
            db[k] = VOLATILE_SRC ? __ldcv(sb + k) : sb[k];
    }
    else if (((d | s) & 3) == 0) {
        const size_t nw = bytes >> 2;
        const uint32_t* sw = reinterpret_cast<const uint32_t*>(src);
        uint32_t* dw = reinterpret_cast<uint32_t*>(dst);
        for (size_t i = tid; i < nw; i += nt)
            dw[i] = VOLATILE_SRC ? __ldcv(sw + i) : sw[i];
        const size_t done = nw << 2;
        const unsigned char* sb = reinterpret_cast<const unsigned char*>(src) + done;
        unsigned char* db = reinterpret_cast<unsigned char*>(dst) + done;
        for (size_t k = tid; k < bytes - done; k += nt)
            db[k] = VOLATILE_SRC ? __ldcv(sb + k) : sb[k];
    }
    else {
        const unsigned char* sb = reinterpret_cast<const unsigned char*>(src);
        unsigned char* db = reinterpret_cast<unsigned char*>(dst);
        for (size_t k = tid; k < bytes; k += nt)
            db[k] = VOLATILE_SRC ? __ldcv(sb + k) : sb[k];
    }
}

// Named barriers (ids 1 .. 15; 0 is __syncthreads): `count` threads in total, those that call arrive do not
// wait.  When a barrier completes, the memory accesses that its participants made before are performed
// with respect to all of them.
__device__ __forceinline__ void named_bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_bar_arrive(int id, int count) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Split [0, n) units into `parts` nearly equal contiguous ranges.
__device__ __host__ __forceinline__ void split_range(size_t n, int parts, int idx, size_t& lo, size_t& hi) {
    size_t base = n / parts, rem = n % parts;
    lo = (size_t)idx * base + ((size_t)idx < rem ? (size_t)idx : rem);
    hi = lo + base + ((size_t)idx < rem ? 1 : 0);
}

} // namespace dev
} // namespace cclx
