// Collective kernels for one NVSwitch node: every kernel moves data with plain
// peer loads/stores (or NVLS multimem) issued from inside the kernel and
// synchronises with peer_barrier; no host round trip inside a collective.
//
// What they replace in the reference:
//   allreduce_oneshot   <- reduce_sum "read_all" (allreduce_small_sycl_impl.hpp:23-113),
//                          allreduce_kernel (src/kernels/kernels.cl:190-217)
//   allreduce_twoshot   <- reduce_sum_general + copy (allreduce_small_sycl_rw_kernel.hpp:43-94),
//                          allreduce_large_read_write_* (allreduce_large_sycl_impl.hpp:23-230)
//   allreduce_pipelined <- allreduce_large_impl, the chunk pipeline (allreduce_large_sycl_impl.hpp:234-684)
//   allreduce_symm      <- same two-shot on registered (IPC) user buffers, no tmp copy
//   reduce_scatter_pipelined <- reduce_scatter_large_impl (reduce_scatter_large_sycl_impl.hpp:76-304)
//   reduce_scatter      <- reduce_scatter_small/large_impl, reduce_monolithic_* (kernels.cl:269-421)
//   allgatherv          <- gather / read_write, write_monolithic_* (kernels.cl:424-560)
//   alltoallv, alltoall_symm <- alltoallv_kernel_* (kernels.cl:110-116)
//   broadcast / reduce  <- ze_copy_entry fan-out, ze_onesided_reduce
// Design differences: push-style (remote stores, local reduction) so that a
// collective costs one NVLink one-way trip plus one flag; two staging
// generations instead of a trailing barrier; fused scale + output cast in the
// reduction epilogue; bf16/fp16 accumulate in fp32.
#pragma once
#include "gpu/device/coll_args.hpp"
#include "gpu/device/common.cuh"

namespace cclx {
namespace dev {

__device__ __forceinline__ size_t round_up16(size_t b) {
    return (b + 15) & ~(size_t)15;
}

// Load pack `i` (16 bytes) of a T array of `count` elements; zero-fill past the end.
template <class T>
__device__ __forceinline__ uint4 load_pack(const T* base, size_t i, size_t count, bool vec) {
    constexpr int N = pack_traits<T>::N;
    const size_t e0 = i * N;
    if (vec && e0 + N <= count)
        return *reinterpret_cast<const uint4*>(base + e0);
    uint4 v = make_uint4(0, 0, 0, 0);
    T* t = reinterpret_cast<T*>(&v);
#pragma unroll
    for (int k = 0; k < N; k++)
        if (e0 + k < count)
            t[k] = base[e0 + k];
    return v;
}

// Store N accumulators as elements [i*N, i*N+N) of a Tout array of `count` elements.
template <class Tout, class A, int N>
__device__ __forceinline__ void store_pack(Tout* base, size_t i, size_t count, bool vec, const A (&a)[N],
                                           float scale, bool do_scale) {
    const size_t e0 = i * N;
    if (vec && e0 + N <= count) {
        store_out<Tout, A, N>(base + e0, a, scale, do_scale);
    }
    else {
#pragma unroll
        for (int k = 0; k < N; k++)
            if (e0 + k < count) {
                A v = a[k];
                base[e0 + k] = from_acc<Tout, A>(do_scale ? apply_scale<A>(v, scale) : v);
            }
    }
}

template <class Tout, int N>
__device__ __forceinline__ bool out_vec_ok(const Tout* p) {
    constexpr int B = N * (int)sizeof(Tout) >= 16 ? 16 : N * (int)sizeof(Tout);
    return (((uintptr_t)p) & (B - 1)) == 0;
}

#define CCLX_KERNEL_PROLOGUE()                                   \
    const int er = a.emu ? (int)blockIdx.y : 0;                  \
    const comm_dev& c = tab[er];                                 \
    const rank_args& ra = a.emu ? a.emu_tab[er] : a.r0;          \
    block_sync s;                                                \
    sync_begin(c, s);                                            \
    const size_t tid = threadIdx.x, nt = blockDim.x;             \
    (void)tid;                                                   \
    (void)nt;                                                    \
    (void)ra

// rank p's send / recv buffer of a zero-copy operation: an offset into the symmetric heap, or the
// address of p's registered allocation as mapped in this process
__device__ __forceinline__ const char* peer_in(const comm_dev& c, const coll_args& a, int p) {
    return (a.flags & CF_REG_IN) ? a.reg_in[p] : c.heap[p] + a.in_off;
}
__device__ __forceinline__ char* peer_out(const comm_dev& c, const coll_args& a, int p) {
    return (a.flags & CF_REG_OUT) ? a.reg_out[p] : c.heap[p] + a.out_off;
}

// What every rank must pass alike to one collective kernel: the kernel itself (`kind`), the element
// count, and for the zero-copy forms the buffer kind and the offsets that are applied to the peers'
// memory.  `sig_skew` is a test hook that makes one emulated rank disagree.
__device__ __forceinline__ uint32_t kernel_signature(uint32_t kind, const coll_args& a, const comm_dev& c) {
    const uint32_t f = (uint32_t)a.flags & (CF_SYMM_IN | CF_SYMM_OUT | CF_NVLS | CF_REG_IN | CF_REG_OUT);
    const bool zc = f & (CF_SYMM_IN | CF_SYMM_OUT | CF_REG_IN | CF_REG_OUT);
    uint32_t sg = arg_signature(kind, zc ? a.in_off : 0, zc ? a.out_off : 0, a.count, f);
    if (a.sig_skew == c.rank + 1)
        sg ^= 0x5a5a5a5au;
    return sg ? sg : 1u;
}

// ---------------------------------------------------------------------------
// one-shot allreduce: push my data into slot[rank] of everybody's staging,
// one barrier, reduce the `world` slots locally.
// staging need: world * round_up16(count * sizeof(T)) <= staging_bytes
// ---------------------------------------------------------------------------
template <class T, class Tout, class Op>
__global__ void __launch_bounds__(1024) allreduce_oneshot_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(1, a, c);
    typedef typename acc_of<T>::type A;
    constexpr int N = pack_traits<T>::N;
    const T* send = reinterpret_cast<const T*>(ra.send);
    Tout* recv = reinterpret_cast<Tout*>(ra.recv);
    const size_t count = a.count;
    const size_t slot = round_up16(count * sizeof(T));
    const size_t npacks = slot >> 4;
    size_t lo, hi;
    split_range(npacks, gridDim.x, blockIdx.x, lo, hi);
    const bool vin = (((uintptr_t)send) & 15) == 0;
    const bool vout = out_vec_ok<Tout, N>(recv);
    const size_t goff = (size_t)s.gen * c.staging_bytes + (size_t)c.rank * slot;
    const bool nvls = (a.flags & CF_NVLS) != 0;

    for (size_t i = lo + tid; i < hi; i += nt) {
        uint4 v = load_pack<T>(send, i, count, vin);
        if (nvls) {
            multimem_st16(c.mc_staging + goff + (i << 4), v);
        }
        else {
#pragma unroll 4
            for (int p = 0; p < c.world; p++)
                st16(c.staging[p] + goff + (i << 4), v);
        }
    }
    if (peer_barrier(c, s, sig)) {
        const char* mine = c.staging[c.rank] + (size_t)s.gen * c.staging_bytes;
        for (size_t i = lo + tid; i < hi; i += nt) {
            A acc[N];
            unpack16<T, A>(ld_cv16(mine + (i << 4)), acc);
            for (int p = 1; p < c.world; p++)
                accum16<T, A, Op>(ld_cv16(mine + (size_t)p * slot + (i << 4)), acc);
            store_pack<Tout, A, N>(recv, i, count, vout, acc, a.scale, a.do_scale != 0);
        }
    }
    sync_end(c, gridDim.x, 1, true);
}

// ---------------------------------------------------------------------------
// two-shot allreduce through staging: push my contribution to slice q into
// slot[rank] at rank q; barrier; reduce my slice, write it to my recv and push
// it into everybody's OUT region; barrier; copy the other slices from OUT.
// staging need: world*slice_cap*16 + npacks*N*sizeof(Tout) <= staging_bytes
// ---------------------------------------------------------------------------
template <class T, class Tout, class Op>
__global__ void __launch_bounds__(1024) allreduce_twoshot_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(2, a, c);
    typedef typename acc_of<T>::type A;
    constexpr int N = pack_traits<T>::N;
    constexpr size_t RAWP = (size_t)N * sizeof(Tout); // bytes of one reduced pack
    constexpr size_t OUTP = RAWP < 16 ? 16 : RAWP; // staged in whole 16-byte units
    constexpr int ON = (int)(OUTP / sizeof(Tout));
    static_assert(RAWP >= 16 || RAWP == 8, "unexpected output pack size");
    const T* send = reinterpret_cast<const T*>(ra.send);
    Tout* recv = reinterpret_cast<Tout*>(ra.recv);
    const size_t count = a.count;
    const size_t npacks = round_up16(count * sizeof(T)) >> 4;
    const int W = c.world;
    const size_t slice_cap = (npacks + W - 1) / W; // packs per slot
    const size_t in_bytes = (size_t)W * slice_cap * 16;
    const size_t gbase = (size_t)s.gen * c.staging_bytes;
    const bool vin = (((uintptr_t)send) & 15) == 0;
    const bool vout = out_vec_ok<Tout, N>(recv);

    // phase 1: scatter my contributions
    for (int k = 1; k < W; k++) {
        const int q = (c.rank + k) % W;
        size_t qlo, qhi, lo, hi;
        split_range(npacks, W, q, qlo, qhi);
        split_range(qhi - qlo, gridDim.x, blockIdx.x, lo, hi);
        char* dst = c.staging[q] + gbase + (size_t)c.rank * slice_cap * 16;
        for (size_t i = lo + tid; i < hi; i += nt)
            st16(dst + (i << 4), load_pack<T>(send, qlo + i, count, vin));
    }
    bool ok = peer_barrier(c, s, sig);
    // phase 2: reduce my slice and broadcast the result
    size_t mlo, mhi, lo, hi;
    split_range(npacks, W, c.rank, mlo, mhi);
    split_range(mhi - mlo, gridDim.x, blockIdx.x, lo, hi);
    if (ok) {
        const char* mine = c.staging[c.rank] + gbase;
        for (size_t i = lo + tid; i < hi; i += nt) {
            A acc[N];
            // fixed rank order so that the rounding is reproducible
            bool first = true;
            for (int p = 0; p < W; p++) {
                uint4 v = (p == c.rank) ? load_pack<T>(send, mlo + i, count, vin)
                                        : ld_cv16(mine + (size_t)p * slice_cap * 16 + (i << 4));
                if (first) {
                    unpack16<T, A>(v, acc);
                    first = false;
                }
                else
                    accum16<T, A, Op>(v, acc);
            }
            store_pack<Tout, A, N>(recv, mlo + i, count, vout, acc, a.scale, a.do_scale != 0);
            // reduced pack in output precision, pushed to the peers' OUT region
            alignas(16) Tout o[ON] = {};
#pragma unroll
            for (int k = 0; k < N; k++)
                o[k] = from_acc<Tout, A>(a.do_scale ? apply_scale<A>(acc[k], a.scale) : acc[k]);
            for (int k = 1; k < W; k++) {
                const int p = (c.rank + k) % W;
                char* dst = c.staging[p] + gbase + in_bytes + (mlo + i) * OUTP;
#pragma unroll
                for (int q = 0; q < (int)(OUTP / 16); q++)
                    st16(dst + q * 16, reinterpret_cast<const uint4*>(o)[q]);
            }
        }
    }
    ok = peer_barrier(c, s, sig);
    // phase 3: collect the other slices
    if (ok) {
        const char* outr = c.staging[c.rank] + gbase + in_bytes;
        for (int k = 1; k < W; k++) {
            const int q = (c.rank + k) % W;
            size_t qlo, qhi, l2, h2;
            split_range(npacks, W, q, qlo, qhi);
            split_range(qhi - qlo, gridDim.x, blockIdx.x, l2, h2);
            for (size_t i = l2 + tid; i < h2; i += nt) {
                const size_t e0 = (qlo + i) * N;
                const char* src = outr + (qlo + i) * OUTP;
                alignas(16) Tout o[ON];
#pragma unroll
                for (int q2 = 0; q2 < (int)(OUTP / 16); q2++)
                    reinterpret_cast<uint4*>(o)[q2] = ld_cv16(src + q2 * 16);
                if (vout && e0 + N <= count) {
                    if constexpr (RAWP >= 16) {
#pragma unroll
                        for (int q2 = 0; q2 < (int)(OUTP / 16); q2++)
                            reinterpret_cast<uint4*>(recv + e0)[q2] = reinterpret_cast<const uint4*>(o)[q2];
                    }
                    else
                        *reinterpret_cast<uint2*>(recv + e0) = *reinterpret_cast<const uint2*>(o);
                }
                else {
#pragma unroll
                    for (int k2 = 0; k2 < N; k2++)
                        if (e0 + k2 < count)
                            recv[e0 + k2] = o[k2];
                }
            }
        }
    }
    sync_end(c, gridDim.x, 2, true);
}

// ---------------------------------------------------------------------------
// pipelined allreduce through staging for large messages in ordinary (not
// registered) buffers.  The message is cut into chunks; one staging generation
// holds IN[2] and OUT[2] chunk buffers.  Iteration j of every block does
//   A: copy its piece of chunk j   from send   into this rank's IN[j&1]
//   B: reduce its share of chunk j-1 across the ranks (multimem.ld_reduce on
//      the multicast window, or loads from every peer) and write the result
//      into every rank's OUT[(j-1)&1] (multimem.st, or stores to every peer)
//   C: copy its piece of chunk j-2 from OUT[(j-2)&1] into recv
// and ends with one cross-GPU barrier, so the local copies of the neighbouring
// chunks run under the NVLink traffic of the current one.  A chunk is divided
// first among the blocks and then, inside a block's piece, among the ranks, so
// that all data dependencies stay between blocks of equal index and the
// per-block barrier is enough.  Same role as the three-stage pipeline of the
// reference's allreduce_large_impl
// (src/coll/algorithms/allreduce/sycl/allreduce_large_sycl_impl.hpp:234-684).
// a.stride = packs per chunk (a multiple of gridDim.x * world).
// staging need: 2*chunk*16 + 2*chunk*N*sizeof(Tout) <= staging_bytes
// ---------------------------------------------------------------------------
template <class T, class Tout, class Op, bool NVLS>
__global__ void __launch_bounds__(1024) allreduce_pipelined_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(3, a, c);
    typedef typename acc_of<T>::type A;
    constexpr int N = pack_traits<T>::N;
    constexpr size_t RAWP = (size_t)N * sizeof(Tout); // bytes of one reduced pack
    constexpr size_t OUTP = RAWP < 16 ? 16 : RAWP; // staged in whole 16-byte units
    constexpr int OQ = (int)(OUTP / 16);
    constexpr int ON = (int)(OUTP / sizeof(Tout));
    static_assert(RAWP >= 16 || RAWP == 8, "unexpected output pack size");
    const T* send = reinterpret_cast<const T*>(ra.send);
    Tout* recv = reinterpret_cast<Tout*>(ra.recv);
    const size_t count = a.count;
    const size_t npacks = round_up16(count * sizeof(T)) >> 4;
    const int W = c.world;
    const size_t cp = a.stride;
    const size_t nchunks = (npacks + cp - 1) / cp;
    const size_t piece = cp / gridDim.x;
    const size_t sub = piece / W;
    const size_t gbase = (size_t)s.gen * c.staging_bytes;
    const size_t out_base = gbase + 2 * cp * 16;
    const bool vin = (((uintptr_t)send) & 15) == 0;
    const bool vout = out_vec_ok<Tout, N>(recv);
    const bool scale = a.do_scale != 0;
    char* my_stage = c.staging[c.rank];
    bool ok = true;
    // with several chunks in flight the block splits into a reducing half and a copying half, so that
    // the local copies of chunks j and j-2 really run while chunk j-1 is on the wire
    const bool split = nchunks >= 2 && nt >= 64;
    const size_t half = nt / 2;
    const bool do_red = !split || tid < half, do_copy = !split || tid >= half;
    const size_t rt = tid, rnt = split ? half : nt;
    const size_t ct = split ? tid - half : tid, cnt = split ? nt - half : nt;

    for (size_t j = 0; j < nchunks + 2; j++) {
        if (j < nchunks && do_copy) { // A
            const size_t p0 = j * cp + blockIdx.x * piece;
            char* dst = my_stage + gbase + (j & 1) * cp * 16 + blockIdx.x * piece * 16;
            const size_t n = p0 < npacks ? min(piece, npacks - p0) : 0;
            size_t i = ct;
            for (; i + 3 * cnt < n; i += 4 * cnt) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; u++)
                    v[u] = load_pack<T>(send, p0 + i + u * cnt, count, vin);
#pragma unroll
                for (int u = 0; u < 4; u++)
                    st16(dst + ((i + u * cnt) << 4), v[u]);
            }
            for (; i < n; i += cnt)
                st16(dst + (i << 4), load_pack<T>(send, p0 + i, count, vin));
        }
        if (j >= 1 && j <= nchunks && ok && do_red) { // B
            const size_t jj = j - 1;
            const size_t q0 = blockIdx.x * piece + (size_t)c.rank * sub; // first pack of my share inside the chunk
            const size_t p0 = jj * cp + q0;
            const size_t n = p0 < npacks ? min(sub, npacks - p0) : 0;
            const size_t in_off = gbase + (jj & 1) * cp * 16 + q0 * 16;
            const size_t o_off = out_base + (jj & 1) * cp * OUTP + q0 * OUTP;
            auto finish = [&](size_t i, A(&acc)[N]) {
                alignas(16) Tout o[ON] = {};
#pragma unroll
                for (int k = 0; k < N; k++)
                    o[k] = from_acc<Tout, A>(scale ? apply_scale<A>(acc[k], a.scale) : acc[k]);
                if (NVLS) {
#pragma unroll
                    for (int q = 0; q < OQ; q++)
                        multimem_st16(c.mc_staging + o_off + i * OUTP + q * 16, reinterpret_cast<const uint4*>(o)[q]);
                }
                else {
                    for (int k = 0; k < W; k++) {
                        char* dst = c.staging[(c.rank + k) % W] + o_off + i * OUTP;
#pragma unroll
                        for (int q = 0; q < OQ; q++)
                            st16(dst + q * 16, reinterpret_cast<const uint4*>(o)[q]);
                    }
                }
            };
            if constexpr (NVLS) {
                size_t i = rt;
                for (; i + 3 * rnt < n; i += 4 * rnt) { // four switch round trips in flight per thread
                    uint4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        v[u] = multimem_ld_reduce_add16<T>(c.mc_staging + in_off + ((i + u * rnt) << 4));
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        A au[N];
                        unpack16<T, A>(v[u], au);
                        finish(i + u * rnt, au);
                    }
                }
                for (; i < n; i += rnt) {
                    A a0[N];
                    unpack16<T, A>(multimem_ld_reduce_add16<T>(c.mc_staging + in_off + (i << 4)), a0);
                    finish(i, a0);
                }
            }
            else {
                for (size_t i = rt; i < n; i += rnt) {
                    uint4 v[MAX_RANKS];
                    for (int p = 0; p < W; p++) // fixed rank order: reproducible rounding
                        v[p] = ld_cv16(c.staging[p] + in_off + (i << 4));
                    A acc[N];
                    unpack16<T, A>(v[0], acc);
                    for (int p = 1; p < W; p++)
                        accum16<T, A, Op>(v[p], acc);
                    finish(i, acc);
                }
            }
        }
        if (j >= 2 && ok && do_copy) { // C
            const size_t jj = j - 2;
            const size_t p0 = jj * cp + blockIdx.x * piece;
            const size_t n = p0 < npacks ? min(piece, npacks - p0) : 0;
            const char* src = my_stage + out_base + (jj & 1) * cp * OUTP + blockIdx.x * piece * OUTP;
            auto put = [&](size_t i, const uint4(&raw)[OQ]) {
                const size_t e0 = (p0 + i) * N;
                const Tout* o = reinterpret_cast<const Tout*>(raw);
                if (vout && e0 + N <= count) {
                    if constexpr (RAWP >= 16) {
#pragma unroll
                        for (int q = 0; q < OQ; q++)
                            reinterpret_cast<uint4*>(recv + e0)[q] = raw[q];
                    }
                    else
                        *reinterpret_cast<uint2*>(recv + e0) = *reinterpret_cast<const uint2*>(raw);
                }
                else {
#pragma unroll
                    for (int k2 = 0; k2 < N; k2++)
                        if (e0 + k2 < count)
                            recv[e0 + k2] = o[k2];
                }
            };
            size_t i = ct;
            for (; i + 3 * cnt < n; i += 4 * cnt) { // four loads in flight per thread
                uint4 raw[4][OQ];
#pragma unroll
                for (int u = 0; u < 4; u++)
#pragma unroll
                    for (int q = 0; q < OQ; q++)
                        raw[u][q] = ld_cv16(src + (i + u * cnt) * OUTP + q * 16);
#pragma unroll
                for (int u = 0; u < 4; u++)
                    put(i + u * cnt, raw[u]);
            }
            for (; i < n; i += cnt) {
                uint4 raw[OQ];
#pragma unroll
                for (int q = 0; q < OQ; q++)
                    raw[q] = ld_cv16(src + i * OUTP + q * 16);
                put(i, raw);
            }
        }
        if (j <= nchunks)
            ok = peer_barrier(c, s, sig);
    }
    sync_end(c, gridDim.x, (uint32_t)(nchunks + 1), true);
}

// ---------------------------------------------------------------------------
// Inner loops of the zero-copy peer-load kernels for a world size known at compile time (2, 4, 8): the
// per-peer values stay in registers (a loop over a run-time world size indexes its array dynamically, which
// puts it into local memory), the peer pointers are read through constant indices, and every thread keeps
// eight 16-byte loads in flight (8 / WT packs of WT peers each).
// ---------------------------------------------------------------------------
template <int WT>
struct p2p_unroll {
    static constexpr int U = WT >= 8 ? 1 : 8 / WT;
};

// allreduce: packs [i, end) of my slice, stride nt: load from every peer, reduce, store to every peer
template <class T, class A, class Op, int N, int WT>
__device__ __forceinline__ void ar_p2p_loop(const comm_dev& c, const coll_args& a, size_t i, size_t end, size_t nt,
                                            bool scale) {
    constexpr int U = p2p_unroll<WT>::U;
    auto finish = [&](size_t at, const uint4 (&v)[WT]) {
        A acc[N];
        unpack16<T, A>(v[0], acc);
#pragma unroll
        for (int p = 1; p < WT; p++)
            accum16<T, A, Op>(v[p], acc);
        uint4 o;
        T* t = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int k = 0; k < N; k++)
            t[k] = from_acc<T, A>(scale ? apply_scale<A>(acc[k], a.scale) : acc[k]);
#pragma unroll
        for (int k = 0; k < WT; k++)
            st16(peer_out(c, a, (c.rank + k) % WT) + (at << 4), o);
    };
    for (; i + (U - 1) * nt < end; i += U * nt) {
        uint4 v[U][WT];
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int p = 0; p < WT; p++)
                v[u][p] = ld_cv16(peer_in(c, a, p) + ((i + u * nt) << 4));
#pragma unroll
        for (int u = 0; u < U; u++)
            finish(i + u * nt, v[u]);
    }
    for (; i < end; i += nt) {
        uint4 v[WT];
#pragma unroll
        for (int p = 0; p < WT; p++)
            v[p] = ld_cv16(peer_in(c, a, p) + (i << 4));
        finish(i, v);
    }
}

// reduce_scatter: packs [i, end) of my block (byte offset blk in every peer's input), result to recv
template <class T, class A, class Op, int N, int WT>
__device__ __forceinline__ size_t rs_p2p_loop(const comm_dev& c, const coll_args& a, size_t blk, T* recv, size_t rc,
                                              bool vout, size_t i, size_t end, size_t nt) {
    constexpr int U = p2p_unroll<WT>::U;
    for (; i + (U - 1) * nt < end; i += U * nt) {
        uint4 v[U][WT];
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int p = 0; p < WT; p++)
                v[u][p] = ld_cv16(peer_in(c, a, p) + blk + ((i + u * nt) << 4));
#pragma unroll
        for (int u = 0; u < U; u++) {
            A acc[N];
            unpack16<T, A>(v[u][0], acc);
#pragma unroll
            for (int p = 1; p < WT; p++)
                accum16<T, A, Op>(v[u][p], acc);
            store_pack<T, A, N>(recv, i + u * nt, rc, vout, acc, a.scale, a.do_scale != 0);
        }
    }
    return i; // the caller's one-pack loop takes the rest
}

// alltoall: packs [i, end) of every block: block q of my send buffer goes to rank q, at my place (doff)
template <int WT>
__device__ __forceinline__ size_t a2a_p2p_loop(const comm_dev& c, const coll_args& a, const char* send, size_t b,
                                               size_t doff, size_t i, size_t end, size_t nt) {
    constexpr int U = p2p_unroll<WT>::U;
    for (; i + (U - 1) * nt < end; i += U * nt) {
        uint4 v[U][WT];
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int k = 0; k < WT; k++)
                v[u][k] = *reinterpret_cast<const uint4*>(send + (size_t)((c.rank + k) % WT) * b + ((i + u * nt) << 4));
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int k = 0; k < WT; k++)
                st16(peer_out(c, a, (c.rank + k) % WT) + doff + ((i + u * nt) << 4), v[u][k]);
    }
    return i;
}

// ---------------------------------------------------------------------------
// two-shot allreduce on symmetric (registered) buffers, no staging copy.
// P2P form: read my slice from every peer, reduce, write it to every peer.
// NVLS form (sum of f32/bf16/f16): multimem.ld_reduce + multimem.st, the
// switch does the reduction and the broadcast.
// The tail that does not fill a 16-byte pack is read before and written after
// the second barrier so that in-place calls do not race.
// ---------------------------------------------------------------------------
// U = 16-byte packs in flight per thread of the NVLS form: 4 for a grid as wide as the GPU, 8 for the
// narrow grids that leave most SMs to a concurrent compute kernel (gradient buckets during backward).
template <class T, class Op, bool NVLS, int UNROLL = 4>
__global__ void __launch_bounds__(1024) allreduce_symm_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(4, a, c);
    typedef typename acc_of<T>::type A;
    constexpr int N = pack_traits<T>::N;
    const int W = c.world;
    const size_t count = a.count;
    const size_t full = count / N; // whole packs
    const size_t tail = count - full * N;
    size_t mlo, mhi, lo, hi;
    split_range(full, W, c.rank, mlo, mhi);
    split_range(mhi - mlo, gridDim.x, blockIdx.x, lo, hi);
    const bool scale = a.do_scale != 0;

    bool ok = peer_barrier(c, s, sig);
    A tail_acc = A();
    if (ok) {
        if (NVLS) {
            const char* in = c.mc_heap + a.in_off;
            char* out = c.mc_heap + a.out_off;
            size_t i = mlo + lo + tid;
            const size_t end = mlo + hi;
            // several packs in flight per thread keep enough bytes on the wire for the switch round trip
            constexpr int U = UNROLL;
            auto rescale = [&](uint4& v) {
                A t0[N];
                unpack16<T, A>(v, t0);
                T* o0 = reinterpret_cast<T*>(&v);
#pragma unroll
                for (int k = 0; k < N; k++)
                    o0[k] = from_acc<T, A>(apply_scale<A>(t0[k], a.scale));
            };
            for (; i + (U - 1) * nt < end; i += U * nt) {
                uint4 v[U];
#pragma unroll
                for (int u = 0; u < U; u++)
                    v[u] = multimem_ld_reduce_add16<T>(in + ((i + u * nt) << 4));
                if (scale) {
#pragma unroll
                    for (int u = 0; u < U; u++)
                        rescale(v[u]);
                }
#pragma unroll
                for (int u = 0; u < U; u++)
                    multimem_st16(out + ((i + u * nt) << 4), v[u]);
            }
            for (; i < end; i += nt) {
                uint4 v0 = multimem_ld_reduce_add16<T>(in + (i << 4));
                if (scale)
                    rescale(v0);
                multimem_st16(out + (i << 4), v0);
            }
        }
        else {
            // two packs x world loads in flight per thread
            auto reduce_one = [&](size_t i, const uint4 (&v)[MAX_RANKS]) {
                A acc[N];
                unpack16<T, A>(v[0], acc);
                for (int p = 1; p < W; p++)
                    accum16<T, A, Op>(v[p], acc);
                uint4 o;
                T* t = reinterpret_cast<T*>(&o);
#pragma unroll
                for (int k = 0; k < N; k++)
                    t[k] = from_acc<T, A>(scale ? apply_scale<A>(acc[k], a.scale) : acc[k]);
                for (int k = 0; k < W; k++) {
                    const int p = (c.rank + k) % W;
                    st16(peer_out(c, a, p) + (i << 4), o);
                }
            };
            size_t i = mlo + lo + tid;
            const size_t end = mlo + hi;
            if (W == 8)
                ar_p2p_loop<T, A, Op, N, 8>(c, a, i, end, nt, scale);
            else if (W == 4)
                ar_p2p_loop<T, A, Op, N, 4>(c, a, i, end, nt, scale);
            else if (W == 2)
                ar_p2p_loop<T, A, Op, N, 2>(c, a, i, end, nt, scale);
            else {
                for (; i + nt < end; i += 2 * nt) {
                    uint4 v0[MAX_RANKS], v1[MAX_RANKS];
                    for (int p = 0; p < W; p++) {
                        v0[p] = ld_cv16(peer_in(c, a, p) + (i << 4));
                        v1[p] = ld_cv16(peer_in(c, a, p) + ((i + nt) << 4));
                    }
                    reduce_one(i, v0);
                    reduce_one(i + nt, v1);
                }
                for (; i < end; i += nt) {
                    uint4 v0[MAX_RANKS];
                    for (int p = 0; p < W; p++)
                        v0[p] = ld_cv16(peer_in(c, a, p) + (i << 4));
                    reduce_one(i, v0);
                }
            }
        }
        if (blockIdx.x == 0 && tid < tail) {
            const size_t e = full * N + tid;
            tail_acc = to_acc<A, T>(__ldcv(reinterpret_cast<const T*>(peer_in(c, a, 0)) + e));
            for (int p = 1; p < W; p++)
                tail_acc = Op::apply(tail_acc,
                                     to_acc<A, T>(__ldcv(reinterpret_cast<const T*>(peer_in(c, a, p)) + e)));
        }
    }
    ok = peer_barrier(c, s, sig);
    if (ok && blockIdx.x == 0 && tid < tail) {
        const size_t e = full * N + tid;
        reinterpret_cast<T*>(peer_out(c, a, c.rank))[e] =
            from_acc<T, A>(scale ? apply_scale<A>(tail_acc, a.scale) : tail_acc);
    }
    // nobody reads a peer's input after the second barrier, so the next
    // operation on the stream may overwrite it
    sync_end(c, gridDim.x, 2, false);
}

// ---------------------------------------------------------------------------
// reduce_scatter: recv[i] = op_p send_p[rank*rc + i]; push block q to rank q.
// staging need: world * round_up16(rc*sizeof(T)) <= staging_bytes
// ---------------------------------------------------------------------------
template <class T, class Tout, class Op>
__global__ void __launch_bounds__(1024) reduce_scatter_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(5, a, c);
    typedef typename acc_of<T>::type A;
    constexpr int N = pack_traits<T>::N;
    const T* send = reinterpret_cast<const T*>(ra.send);
    Tout* recv = reinterpret_cast<Tout*>(ra.recv);
    const size_t rc = a.count; // elements per rank
    const int W = c.world;
    const size_t slot = round_up16(rc * sizeof(T));
    const size_t npacks = slot >> 4;
    size_t lo, hi;
    split_range(npacks, gridDim.x, blockIdx.x, lo, hi);
    const size_t gbase = (size_t)s.gen * c.staging_bytes;
    const bool vout = out_vec_ok<Tout, N>(recv);

    // the loads for all peers are in flight together, then the stores
    for (size_t i = lo + tid; i < hi; i += nt) {
        uint4 v[MAX_RANKS];
        for (int k = 1; k < W; k++) {
            const T* blk = send + (size_t)((c.rank + k) % W) * a.stride;
            v[k] = load_pack<T>(blk, i, rc, (((uintptr_t)blk) & 15) == 0);
        }
        for (int k = 1; k < W; k++)
            st16(c.staging[(c.rank + k) % W] + gbase + (size_t)c.rank * slot + (i << 4), v[k]);
    }
    if (peer_barrier(c, s, sig)) {
        const char* mine = c.staging[c.rank] + gbase;
        const T* own = send + (size_t)c.rank * a.stride;
        const bool vown = (((uintptr_t)own) & 15) == 0;
        for (size_t i = lo + tid; i < hi; i += nt) {
            A acc[N];
            bool first = true;
            for (int p = 0; p < W; p++) {
                uint4 v = (p == c.rank) ? load_pack<T>(own, i, rc, vown)
                                        : ld_cv16(mine + (size_t)p * slot + (i << 4));
                if (first) {
                    unpack16<T, A>(v, acc);
                    first = false;
                }
                else
                    accum16<T, A, Op>(v, acc);
            }
            store_pack<Tout, A, N>(recv, i, rc, vout, acc, a.scale, a.do_scale != 0);
        }
    }
    sync_end(c, gridDim.x, 1, true);
}

// ---------------------------------------------------------------------------
// pipelined reduce_scatter through staging for large ordinary send buffers: chunk j holds, for every
// destination rank q, packs [j*cs, (j+1)*cs) of block q.  Iteration j of every block
//   A: copies its piece of every slab of chunk j from send into this rank's IN[j&1]   (copying half)
//   B: reduces its piece of MY slab of chunk j-1 across the ranks (multimem.ld_reduce, or loads from
//      every peer) straight into recv                                                  (reducing half)
// followed by one cross-GPU barrier; pieces are cut by block index first, so the per-block barrier
// covers every dependency.  a.stride = elements between blocks of send, a.in_off = cs (packs per slab).
// staging need: 2 * world * cs * 16 <= staging_bytes
// ---------------------------------------------------------------------------
template <class T, class Tout, class Op, bool NVLS>
__global__ void __launch_bounds__(1024) reduce_scatter_pipelined_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(6, a, c);
    typedef typename acc_of<T>::type A;
    constexpr int N = pack_traits<T>::N;
    const T* send = reinterpret_cast<const T*>(ra.send);
    Tout* recv = reinterpret_cast<Tout*>(ra.recv);
    const size_t rc = a.count;
    const int W = c.world;
    const size_t rpacks = round_up16(rc * sizeof(T)) >> 4;
    const size_t cs = a.in_off;
    const size_t nchunks = (rpacks + cs - 1) / cs;
    const size_t piece = cs / gridDim.x;
    const size_t gbase = (size_t)s.gen * c.staging_bytes;
    const bool vout = out_vec_ok<Tout, N>(recv);
    char* my_stage = c.staging[c.rank];
    bool ok = true;
    const bool split = nchunks >= 2 && nt >= 64;
    const size_t half = nt / 2;
    const bool do_red = !split || tid < half, do_copy = !split || tid >= half;
    const size_t rt = tid, rnt = split ? half : nt;
    const size_t ct = split ? tid - half : tid, cnt = split ? nt - half : nt;

    for (size_t j = 0; j <= nchunks; j++) {
        if (j < nchunks && do_copy) { // A
            const size_t p0 = j * cs + blockIdx.x * piece;
            const size_t n = p0 < rpacks ? min(piece, rpacks - p0) : 0;
            char* dst0 = my_stage + gbase + (j & 1) * (size_t)W * cs * 16 + blockIdx.x * piece * 16;
            for (int q = 0; q < W; q++) {
                const T* blk = send + (size_t)q * a.stride;
                const bool vin = (((uintptr_t)blk) & 15) == 0;
                char* dst = dst0 + (size_t)q * cs * 16;
                size_t i = ct;
                for (; i + 3 * cnt < n; i += 4 * cnt) {
                    uint4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        v[u] = load_pack<T>(blk, p0 + i + u * cnt, rc, vin);
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        st16(dst + ((i + u * cnt) << 4), v[u]);
                }
                for (; i < n; i += cnt)
                    st16(dst + (i << 4), load_pack<T>(blk, p0 + i, rc, vin));
            }
        }
        if (j >= 1 && ok && do_red) { // B
            const size_t jj = j - 1;
            const size_t p0 = jj * cs + blockIdx.x * piece;
            const size_t n = p0 < rpacks ? min(piece, rpacks - p0) : 0;
            const size_t off = gbase + (jj & 1) * (size_t)W * cs * 16 + ((size_t)c.rank * cs + blockIdx.x * piece) * 16;
            if constexpr (NVLS) {
                size_t i = rt;
                for (; i + 3 * rnt < n; i += 4 * rnt) {
                    uint4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        v[u] = multimem_ld_reduce_add16<T>(c.mc_staging + off + ((i + u * rnt) << 4));
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        A acc[N];
                        unpack16<T, A>(v[u], acc);
                        store_pack<Tout, A, N>(recv, p0 + i + u * rnt, rc, vout, acc, a.scale, a.do_scale != 0);
                    }
                }
                for (; i < n; i += rnt) {
                    A acc[N];
                    unpack16<T, A>(multimem_ld_reduce_add16<T>(c.mc_staging + off + (i << 4)), acc);
                    store_pack<Tout, A, N>(recv, p0 + i, rc, vout, acc, a.scale, a.do_scale != 0);
                }
            }
            else {
                for (size_t i = rt; i < n; i += rnt) {
                    uint4 v[MAX_RANKS];
                    for (int p = 0; p < W; p++) // fixed rank order: reproducible rounding
                        v[p] = ld_cv16(c.staging[p] + off + (i << 4));
                    A acc[N];
                    unpack16<T, A>(v[0], acc);
                    for (int p = 1; p < W; p++)
                        accum16<T, A, Op>(v[p], acc);
                    store_pack<Tout, A, N>(recv, p0 + i, rc, vout, acc, a.scale, a.do_scale != 0);
                }
            }
        }
        if (j < nchunks)
            ok = peer_barrier(c, s, sig);
    }
    sync_end(c, gridDim.x, (uint32_t)nchunks, true);
}

// reduce_scatter on symmetric send buffers: pull my block from every peer
// (NVLS: one multimem.ld_reduce), write locally.  recv is an ordinary pointer.
template <class T, class Op, bool NVLS>
__global__ void __launch_bounds__(1024) reduce_scatter_symm_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(7, a, c);
    typedef typename acc_of<T>::type A;
    constexpr int N = pack_traits<T>::N;
    T* recv = reinterpret_cast<T*>(ra.recv);
    const size_t rc = a.count;
    const int W = c.world;
    const size_t blk = (size_t)c.rank * rc * sizeof(T); // my block inside every peer's send
    const bool aligned = ((((uintptr_t)peer_in(c, a, 0)) + blk) & 15) == 0;
    const size_t full = aligned ? rc / N : 0;
    const bool vout = (((uintptr_t)recv) & 15) == 0;
    size_t lo, hi;
    split_range(full, gridDim.x, blockIdx.x, lo, hi);
    bool ok = peer_barrier(c, s, sig);
    if (ok) {
        size_t i = lo + tid;
        if (NVLS) {
            // four in-switch reductions in flight per thread: the round trip through the switch is long
            constexpr int U = 4;
            const char* src = c.mc_heap + a.in_off + blk;
            for (; i + (U - 1) * nt < hi; i += U * nt) {
                uint4 v[U];
#pragma unroll
                for (int u = 0; u < U; u++)
                    v[u] = multimem_ld_reduce_add16<T>(src + ((i + u * nt) << 4));
#pragma unroll
                for (int u = 0; u < U; u++) {
                    A acc[N];
                    unpack16<T, A>(v[u], acc);
                    store_pack<T, A, N>(recv, i + u * nt, rc, vout, acc, a.scale, a.do_scale != 0);
                }
            }
        }
        else {
            // eight peer loads in flight per thread, in registers for the usual world sizes
            if (W == 8)
                i = rs_p2p_loop<T, A, Op, N, 8>(c, a, blk, recv, rc, vout, i, hi, nt);
            else if (W == 4)
                i = rs_p2p_loop<T, A, Op, N, 4>(c, a, blk, recv, rc, vout, i, hi, nt);
            else if (W == 2)
                i = rs_p2p_loop<T, A, Op, N, 2>(c, a, blk, recv, rc, vout, i, hi, nt);
            for (; i + nt < hi; i += 2 * nt) {
                uint4 v0[MAX_RANKS], v1[MAX_RANKS];
                for (int p = 0; p < W; p++) {
                    v0[p] = ld_cv16(peer_in(c, a, p) + blk + (i << 4));
                    v1[p] = ld_cv16(peer_in(c, a, p) + blk + ((i + nt) << 4));
                }
                A acc0[N], acc1[N];
                unpack16<T, A>(v0[0], acc0);
                unpack16<T, A>(v1[0], acc1);
                for (int p = 1; p < W; p++) {
                    accum16<T, A, Op>(v0[p], acc0);
                    accum16<T, A, Op>(v1[p], acc1);
                }
                store_pack<T, A, N>(recv, i, rc, vout, acc0, a.scale, a.do_scale != 0);
                store_pack<T, A, N>(recv, i + nt, rc, vout, acc1, a.scale, a.do_scale != 0);
            }
        }
        for (; i < hi; i += nt) {
            A acc[N];
            if (NVLS) {
                unpack16<T, A>(multimem_ld_reduce_add16<T>(c.mc_heap + a.in_off + blk + (i << 4)), acc);
            }
            else {
                unpack16<T, A>(ld_cv16(peer_in(c, a, 0) + blk + (i << 4)), acc);
                for (int p = 1; p < W; p++)
                    accum16<T, A, Op>(ld_cv16(peer_in(c, a, p) + blk + (i << 4)), acc);
            }
            store_pack<T, A, N>(recv, i, rc, vout, acc, a.scale, a.do_scale != 0);
        }
        // elements outside whole aligned packs
        for (size_t e = full * N + (size_t)blockIdx.x * nt + tid; e < rc; e += (size_t)gridDim.x * nt) {
            A acc = to_acc<A, T>(__ldcv(reinterpret_cast<const T*>(peer_in(c, a, 0) + blk) + e));
            for (int p = 1; p < W; p++)
                acc = Op::apply(acc, to_acc<A, T>(__ldcv(reinterpret_cast<const T*>(peer_in(c, a, p) + blk) + e)));
            recv[e] = from_acc<T, A>(a.do_scale ? apply_scale<A>(acc, a.scale) : acc);
        }
    }
    peer_barrier(c, s, sig); // peers may still read my send buffer until here
    sync_end(c, gridDim.x, 2, false);
}

// ---------------------------------------------------------------------------
// allgatherv (byte oriented): rank p contributes scount[p] bytes placed at
// sdispl[p] of every recv buffer.  `send` may be nullptr / equal to
// recv+sdispl[rank] (in-place).
//  PUSH (small): write my block into slot[rank] of every staging, barrier, copy out.
//  PULL (large): copy my block to my staging, barrier, read every peer's staging.
// staging need: push: sum of blocks rounded per slot; pull: own block.
// ---------------------------------------------------------------------------
template <bool PUSH>
__global__ void __launch_bounds__(1024) allgatherv_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(8, a, c);
    const int W = c.world;
    const size_t gbase = (size_t)s.gen * c.staging_bytes;
    char* recv = reinterpret_cast<char*>(ra.recv);
    const char* send = ra.send ? reinterpret_cast<const char*>(ra.send) : recv + ra.sdispl[c.rank];
    const size_t mybytes = ra.scount[c.rank];
    size_t lo, hi;
    if (PUSH) {
        // slot offsets: prefix of rounded sizes (identical on every rank)
        size_t myoff = 0;
        for (int p = 0; p < c.rank; p++)
            myoff += round_up16(ra.scount[p]);
        split_range((mybytes + 15) >> 4, gridDim.x, blockIdx.x, lo, hi);
        const size_t blo = lo << 4, bhi = (hi << 4) < mybytes ? (hi << 4) : mybytes;
        const bool nvls = (a.flags & CF_NVLS) != 0;
        const bool uniform = (a.flags & CF_UNIFORM) != 0;
        if (bhi > blo) {
            // read once, store to every peer (one multimem.st reaches all of them)
            const unsigned char* sb = reinterpret_cast<const unsigned char*>(send);
            const bool vin = (((uintptr_t)send) & 15) == 0;
            for (size_t i = lo + tid; i < hi; i += nt) {
                const uint4 v = load_pack<unsigned char>(sb, i, mybytes, vin);
                if (nvls)
                    multimem_st16(c.mc_staging + gbase + myoff + (i << 4), v);
                else
                    for (int k = 1; k < W; k++)
                        st16(c.staging[(c.rank + k) % W] + gbase + myoff + (i << 4), v);
            }
            if (send != recv + ra.sdispl[c.rank])
                block_copy<false>(recv + ra.sdispl[c.rank] + blo, send + blo, bhi - blo);
        }
        if (peer_barrier(c, s, sig)) {
            if (uniform) {
                // equal aligned blocks: one pass with the loads of all peers in flight together
                const char* st = c.staging[c.rank] + gbase;
                for (size_t i = lo + tid; i < hi; i += nt) {
                    uint4 v[MAX_RANKS];
                    for (int k = 1; k < W; k++)
                        v[k] = ld_cv16(st + (size_t)((c.rank + k) % W) * mybytes + (i << 4));
                    for (int k = 1; k < W; k++)
                        *reinterpret_cast<uint4*>(recv + (size_t)((c.rank + k) % W) * mybytes + (i << 4)) = v[k];
                }
            }
            else {
                size_t off = 0;
                for (int p = 0; p < W; p++) {
                    const size_t pb = ra.scount[p];
                    if (p != c.rank) {
                        split_range((pb + 15) >> 4, gridDim.x, blockIdx.x, lo, hi);
                        const size_t l = lo << 4, h = (hi << 4) < pb ? (hi << 4) : pb;
                        if (h > l)
                            block_copy<true>(recv + ra.sdispl[p] + l, c.staging[c.rank] + gbase + off + l, h - l);
                    }
                    off += round_up16(pb);
                }
            }
        }
        sync_end(c, gridDim.x, 1, true);
    }
    else {
        split_range((mybytes + 15) >> 4, gridDim.x, blockIdx.x, lo, hi);
        const size_t blo = lo << 4, bhi = (hi << 4) < mybytes ? (hi << 4) : mybytes;
        if (bhi > blo) {
            block_copy<false>(c.staging[c.rank] + gbase + blo, send + blo, bhi - blo);
            if (send != recv + ra.sdispl[c.rank])
                block_copy<false>(recv + ra.sdispl[c.rank] + blo, send + blo, bhi - blo);
        }
        if (peer_barrier(c, s, sig)) {
            for (int k = 1; k < W; k++) {
                const int p = (c.rank + k) % W;
                const size_t pb = ra.scount[p];
                split_range((pb + 15) >> 4, gridDim.x, blockIdx.x, lo, hi);
                const size_t l = lo << 4, h = (hi << 4) < pb ? (hi << 4) : pb;
                if (h > l)
                    block_copy<true>(recv + ra.sdispl[p] + l, c.staging[p] + gbase + l, h - l);
            }
        }
        sync_end(c, gridDim.x, 1, true);
    }
}

// allgather into a symmetric recv buffer: every rank stores its block straight
// into all peers' recv (multimem.st when NVLS), no staging.
template <bool NVLS>
__global__ void __launch_bounds__(1024) allgather_symm_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(9, a, c);
    const int W = c.world;
    const size_t bytes = a.count; // bytes per rank, multiple of 16, 16-byte aligned offsets
    const char* send = ra.send ? reinterpret_cast<const char*>(ra.send)
                               : peer_out(c, a, c.rank) + (size_t)c.rank * bytes;
    const size_t doff = (size_t)c.rank * bytes; // place of my block inside every recv buffer
    size_t lo, hi;
    split_range(bytes >> 4, gridDim.x, blockIdx.x, lo, hi);
    // peers must have finished reading the previous contents of recv
    bool ok = peer_barrier(c, s, sig);
    if (ok) {
        const bool vin = (((uintptr_t)send) & 15) == 0;
        size_t i = lo + tid;
        if (vin) {
            // four local loads in flight per thread before their stores go out
            constexpr int U = 4;
            for (; i + (U - 1) * nt < hi; i += U * nt) {
                uint4 v[U];
#pragma unroll
                for (int u = 0; u < U; u++)
                    v[u] = *reinterpret_cast<const uint4*>(send + ((i + u * nt) << 4));
#pragma unroll
                for (int u = 0; u < U; u++) {
                    if (NVLS) {
                        multimem_st16(c.mc_heap + a.out_off + doff + ((i + u * nt) << 4), v[u]);
                    }
                    else {
                        for (int k = 0; k < W; k++)
                            st16(peer_out(c, a, (c.rank + k) % W) + doff + ((i + u * nt) << 4), v[u]);
                    }
                }
            }
        }
        for (; i < hi; i += nt) {
            uint4 v = load_pack<unsigned char>(reinterpret_cast<const unsigned char*>(send), i, bytes, vin);
            if (NVLS) {
                multimem_st16(c.mc_heap + a.out_off + doff + (i << 4), v);
            }
            else {
                for (int k = 0; k < W; k++) {
                    const int p = (c.rank + k) % W;
                    st16(peer_out(c, a, p) + doff + (i << 4), v);
                }
            }
        }
    }
    peer_barrier(c, s, sig);
    sync_end(c, gridDim.x, 2, false);
}

// ---------------------------------------------------------------------------
// alltoallv (byte oriented).  Every rank owns a slot of slot_bytes =
// staging_bytes / world in each peer's staging.  Rank r writes the block for q
// into slot[r] at rank q; after the barrier q copies slot[p] to recv+rdispl[p].
// Blocks larger than a slot take several rounds inside the kernel.  Whether
// another round is needed is agreed on the device: every rank pushes a "more"
// word to all peers before the round's barrier and ORs the words it received,
// so no rank needs the job-wide maximum block size on the host.
// ---------------------------------------------------------------------------
static __global__ void __launch_bounds__(1024) alltoallv_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(10, a, c);
    const int W = c.world;
    const size_t slot = (c.staging_bytes / W) & ~(size_t)15;
    const char* send = reinterpret_cast<const char*>(ra.send);
    char* recv = reinterpret_cast<char*>(ra.recv);
    __shared__ int more_s;
    uint32_t rounds = 0;
    size_t lo, hi;
    for (;;) {
        const size_t round_off = (size_t)rounds * slot;
        const uint32_t g = (s.gen + rounds) & 1u;
        const size_t gbase = (size_t)g * c.staging_bytes;
        bool more = false;
        const bool uniform = (a.flags & CF_UNIFORM) != 0;
        if (uniform) {
            // equal aligned blocks: the loads for all peers are in flight together
            const size_t b = ra.scount[0];
            size_t rb = b > round_off ? b - round_off : 0;
            if (rb > slot) {
                rb = slot;
                more = true;
            }
            split_range(rb >> 4, gridDim.x, blockIdx.x, lo, hi);
            for (size_t i = lo + tid; i < hi; i += nt) {
                uint4 v[MAX_RANKS];
                for (int k = 0; k < W; k++)
                    v[k] = *reinterpret_cast<const uint4*>(send + (size_t)((c.rank + k) % W) * b + round_off + (i << 4));
                *reinterpret_cast<uint4*>(recv + (size_t)c.rank * b + round_off + (i << 4)) = v[0];
                for (int k = 1; k < W; k++)
                    st16(c.staging[(c.rank + k) % W] + gbase + (size_t)c.rank * slot + (i << 4), v[k]);
            }
        }
        else
            for (int k = 0; k < W; k++) {
                const int q = (c.rank + k) % W;
                size_t b = ra.scount[q] > round_off ? ra.scount[q] - round_off : 0;
                if (b > slot) {
                    b = slot;
                    more = true;
                }
                if (ra.rcount[q] > round_off + slot)
                    more = true;
                split_range((b + 15) >> 4, gridDim.x, blockIdx.x, lo, hi);
                const size_t l = lo << 4, h = (hi << 4) < b ? (hi << 4) : b;
                if (h > l) {
                    const char* src = send + ra.sdispl[q] + round_off + l;
                    if (q == c.rank)
                        block_copy<false>(recv + ra.rdispl[q] + round_off + l, src, h - l);
                    else
                        block_copy<false>(c.staging[q] + gbase + (size_t)c.rank * slot + l, src, h - l);
                }
            }
        const size_t hdr = ((size_t)g * MAX_BLOCKS + blockIdx.x) * MAX_RANKS;
        if (tid < (size_t)W)
            c.aux[tid][hdr + c.rank] = more ? 1u : 0u;
        if (!peer_barrier(c, s, sig)) {
            rounds++;
            break;
        }
        if (uniform) {
            const size_t b = ra.scount[0];
            size_t rb = b > round_off ? b - round_off : 0;
            rb = rb > slot ? slot : rb;
            split_range(rb >> 4, gridDim.x, blockIdx.x, lo, hi);
            const char* st = c.staging[c.rank] + gbase;
            for (size_t i = lo + tid; i < hi; i += nt) {
                uint4 v[MAX_RANKS];
                for (int k = 1; k < W; k++)
                    v[k] = ld_cv16(st + (size_t)((c.rank + k) % W) * slot + (i << 4));
                for (int k = 1; k < W; k++)
                    *reinterpret_cast<uint4*>(recv + (size_t)((c.rank + k) % W) * b + round_off + (i << 4)) = v[k];
            }
        }
        else
            for (int k = 1; k < W; k++) {
                const int p = (c.rank + k) % W;
                size_t b = ra.rcount[p] > round_off ? ra.rcount[p] - round_off : 0;
                if (b > slot)
                    b = slot;
                split_range((b + 15) >> 4, gridDim.x, blockIdx.x, lo, hi);
                const size_t l = lo << 4, h = (hi << 4) < b ? (hi << 4) : b;
                if (h > l)
                    block_copy<true>(recv + ra.rdispl[p] + round_off + l,
                                     c.staging[c.rank] + gbase + (size_t)p * slot + l, h - l);
            }
        if (tid == 0) {
            uint32_t m = 0;
            for (int p = 0; p < W; p++)
                m |= ld_volatile_u32(c.aux[c.rank] + hdr + p);
            more_s = (int)m;
        }
        __syncthreads();
        const int again = more_s;
        rounds++;
        __syncthreads();
        if (!again)
            break;
    }
    sync_end(c, gridDim.x, rounds, rounds);
}

// alltoall with equal blocks into a symmetric recv buffer: every rank stores block q of its send
// buffer straight into rank q's recv (at the place of the sender), no staging and no second copy.
// a.count = bytes per peer (multiple of 16); send is 16-byte aligned and distinct from recv.
static __global__ void __launch_bounds__(1024) alltoall_symm_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(11, a, c);
    const int W = c.world;
    const size_t b = a.count;
    const char* send = reinterpret_cast<const char*>(ra.send);
    size_t lo, hi;
    split_range(b >> 4, gridDim.x, blockIdx.x, lo, hi);
    // peers must have finished reading the previous contents of recv
    bool ok = peer_barrier(c, s, sig);
    if (ok) {
        const size_t doff = (size_t)c.rank * b;
        size_t i = lo + tid;
        if (W == 8)
            i = a2a_p2p_loop<8>(c, a, send, b, doff, i, hi, nt);
        else if (W == 4)
            i = a2a_p2p_loop<4>(c, a, send, b, doff, i, hi, nt);
        else if (W == 2)
            i = a2a_p2p_loop<2>(c, a, send, b, doff, i, hi, nt);
        for (; i < hi; i += nt) {
            uint4 v[MAX_RANKS];
            for (int k = 0; k < W; k++)
                v[k] = *reinterpret_cast<const uint4*>(send + (size_t)((c.rank + k) % W) * b + (i << 4));
            for (int k = 0; k < W; k++)
                st16(peer_out(c, a, (c.rank + k) % W) + doff + (i << 4), v[k]);
        }
    }
    peer_barrier(c, s, sig);
    sync_end(c, gridDim.x, 2, false);
}

// ---------------------------------------------------------------------------
// broadcast (byte oriented, <= staging_bytes per launch): root pushes into
// every staging (multimem.st when NVLS), barrier, the others copy out.
// ---------------------------------------------------------------------------
static __global__ void __launch_bounds__(1024) broadcast_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(12, a, c);
    const int W = c.world;
    const size_t bytes = a.count;
    const size_t gbase = (size_t)s.gen * c.staging_bytes;
    const char* send = reinterpret_cast<const char*>(ra.send);
    char* recv = reinterpret_cast<char*>(ra.recv);
    size_t lo, hi;
    split_range((bytes + 15) >> 4, gridDim.x, blockIdx.x, lo, hi);
    const size_t l = lo << 4, h = (hi << 4) < bytes ? (hi << 4) : bytes;
    if (c.rank == a.root && h > l) {
        if ((a.flags & CF_NVLS) && ((((uintptr_t)send) & 15) == 0)) {
            for (size_t i = lo + tid; i < hi; i += nt)
                multimem_st16(c.mc_staging + gbase + (i << 4),
                              load_pack<unsigned char>(reinterpret_cast<const unsigned char*>(send), i, bytes, true));
        }
        else {
            for (int k = 1; k < W; k++) {
                const int p = (c.rank + k) % W;
                block_copy<false>(c.staging[p] + gbase + l, send + l, h - l);
            }
        }
        if (recv != send)
            block_copy<false>(recv + l, send + l, h - l);
    }
    if (peer_barrier(c, s, sig)) {
        if (c.rank != a.root && h > l)
            block_copy<true>(recv + l, c.staging[c.rank] + gbase + l, h - l);
    }
    sync_end(c, gridDim.x, 1, true);
}

// ---------------------------------------------------------------------------
// reduce to root: every rank pushes its buffer into slot[rank] at the root.
// staging need at root: world * round_up16(count*sizeof(T))
// ---------------------------------------------------------------------------
template <class T, class Tout, class Op>
__global__ void __launch_bounds__(1024) reduce_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(13, a, c);
    typedef typename acc_of<T>::type A;
    constexpr int N = pack_traits<T>::N;
    const T* send = reinterpret_cast<const T*>(ra.send);
    Tout* recv = reinterpret_cast<Tout*>(ra.recv);
    const size_t count = a.count;
    const int W = c.world;
    const size_t slot = round_up16(count * sizeof(T));
    const size_t npacks = slot >> 4;
    size_t lo, hi;
    split_range(npacks, gridDim.x, blockIdx.x, lo, hi);
    const size_t gbase = (size_t)s.gen * c.staging_bytes;
    const bool vin = (((uintptr_t)send) & 15) == 0;
    if (c.rank != a.root) {
        char* dst = c.staging[a.root] + gbase + (size_t)c.rank * slot;
        for (size_t i = lo + tid; i < hi; i += nt)
            st16(dst + (i << 4), load_pack<T>(send, i, count, vin));
    }
    if (peer_barrier(c, s, sig) && c.rank == a.root) {
        const bool vout = out_vec_ok<Tout, N>(recv);
        const char* mine = c.staging[c.rank] + gbase;
        for (size_t i = lo + tid; i < hi; i += nt) {
            A acc[N];
            bool first = true;
            for (int p = 0; p < W; p++) {
                uint4 v = (p == c.rank) ? load_pack<T>(send, i, count, vin)
                                        : ld_cv16(mine + (size_t)p * slot + (i << 4));
                if (first) {
                    unpack16<T, A>(v, acc);
                    first = false;
                }
                else
                    accum16<T, A, Op>(v, acc);
            }
            store_pack<Tout, A, N>(recv, i, count, vout, acc, a.scale, a.do_scale != 0);
        }
    }
    sync_end(c, gridDim.x, 1, true);
}

// barrier only
static __global__ void __launch_bounds__(64) barrier_kernel(const comm_dev* tab, coll_args a) {
    CCLX_KERNEL_PROLOGUE();
    const uint32_t sig = kernel_signature(14, a, c);
    peer_barrier(c, s, sig);
    sync_end(c, gridDim.x, 1, false);
}

// ---------------------------------------------------------------------------
// point-to-point.  Every ordered pair owns one data slot (at the receiver,
// written by the sender's stores; or, in pull mode, at the sender, read by the
// receiver's loads), cut into lanes: independent chains of chunks, each with a ring of P2P_STAGES
// buffers of P2P_CHUNK_BYTES and its own pair of counters, so no grid-wide
// synchronisation is needed and a message of any size is one launch.
// p2p flag area of rank x (peer-mapped), in words:
//   ready[(p*P2P_LANES)+l] : chunks that sender p has put into lane l of x's slot[p] so far
//   ack  [(q*P2P_LANES)+l] : chunks of x's messages to q that q has drained from lane l so far
// Chunk number n of a lane (counted over the life of the communicator) uses stage n % P2P_STAGES.
// send: wait ack >= n + 1 - P2P_STAGES on my side, push, fence, set ready = n + 1 at the peer.
// recv: wait ready >= n + 1 on my side, copy out, set ack = n + 1 at the peer.
// Chunk k of a message goes through lane k % nl, where nl = min(chunks, lanes in use) depends on the byte
// count alone, so the two sides agree on it without talking.  How many blocks serve the lanes is each
// side's own choice (block b takes lanes b, b + nb, ... one after the other, in rising order): a launch
// keeps all its blocks resident at once, whatever the number of operations in it, and because both
// sides walk the lanes in the same order the lowest unfinished lane of a message is always being
// served on both sides.  One launch serves a list of operations (blockIdx.z), which is how send/recv
// issued inside a group run side by side without ordering deadlocks.
//
// Inside a block, warp 0 does the waiting and the signalling and the other warps copy, so that the
// system-scope fence in front of a flag (a round trip over NVLink for the sender) overlaps the copy of
// the next chunk:
//   control: wait(j + 1); arrive GO[j + 1]; sync DONE[j]; release flag(j)
//   copiers: sync GO[j]; copy item j; arrive DONE[j]
// GO and DONE alternate between two named barriers each; the control warp reaches GO[j + 2] only after
// DONE[j] completed, so a barrier is never entered for a later phase while an earlier one is open.
// ---------------------------------------------------------------------------
static __global__ void __launch_bounds__(1024)
    sendrecv_kernel(const comm_dev* tab, p2p_layout L, p2p_ops r0, const p2p_ops* emu_tab, int emu) {
    const int er = emu ? (int)blockIdx.y : 0;
    const comm_dev& c = tab[er];
    const p2p_ops& ops = emu ? emu_tab[er] : r0;
    const int oi = blockIdx.z;
    if (oi >= ops.n)
        return;
    const p2p_op op = ops.op[oi];
    const int peer = op.peer;
    if (peer < 0)
        return;
    // a zero-byte message still synchronises the pair once
    const size_t nchunks = op.bytes ? (op.bytes + P2P_CHUNK_BYTES - 1) / P2P_CHUNK_BYTES : 1;
    const int nl = nchunks < (size_t)L.lanes ? (int)nchunks : L.lanes;
    const int nb = nl < (int)gridDim.x ? nl : (int)gridDim.x;
    const int b = blockIdx.x;
    if (b >= nb)
        return;
    __shared__ volatile int fail;
    __shared__ volatile uint32_t stage_of[2];
    if (threadIdx.x == 0)
        fail = 0;
    __syncthreads();
    const int nthr = blockDim.x;
    enum { BAR_GO = 1, BAR_DONE = 3 };
    if (threadIdx.x < 32) {
        uint32_t* prev_signal = nullptr;
        uint32_t prev_value = 0;
        uint32_t j = 0;
        for (int ln = b; ln < nl; ln += nb) {
            const uint32_t mine = (uint32_t)((nchunks - ln + nl - 1) / nl); // chunks of this lane
            uint32_t* seqw = c.p2p_seq + ((op.is_send ? 0 : MAX_RANKS) + peer) * P2P_LANES + ln;
            const uint32_t* ack = c.p2p_flags[c.rank] + P2P_ACK_BASE + peer * P2P_LANES + ln;
            const uint32_t* ready = c.p2p_flags[c.rank] + peer * P2P_LANES + ln;
            uint32_t* signal = op.is_send ? c.p2p_flags[peer] + c.rank * P2P_LANES + ln
                                          : c.p2p_flags[peer] + P2P_ACK_BASE + c.rank * P2P_LANES + ln;
            const uint32_t n0 = *seqw;
            for (uint32_t i = 0; i < mine; i++, j++) {
                const uint32_t n = n0 + i;
                if (threadIdx.x == 0) { // item j may start: its stage is free (send) or filled (recv)
                    const bool ok = op.is_send ? wait_flag_sys(c, ack, n + 1 - P2P_STAGES, peer, ST_FLAG_TIMEOUT)
                                               : wait_flag_sys(c, ready, n + 1, peer, ST_FLAG_TIMEOUT);
                    if (!ok)
                        fail = 1;
                    stage_of[j & 1] = n % P2P_STAGES;
                }
                __syncwarp();
                named_bar_arrive(BAR_GO + (j & 1), nthr);
                if (fail)
                    return; // the copiers leave at the barrier just released
                if (prev_signal) { // the item before has been copied: tell the peer
                    named_bar_sync(BAR_DONE + ((j - 1) & 1), nthr);
                    if (threadIdx.x == 0)
                        st_release_sys(prev_signal, prev_value);
                }
                prev_signal = signal;
                prev_value = n + 1;
            }
            if (threadIdx.x == 0)
                *seqw = n0 + mine;
        }
        if (prev_signal) {
            named_bar_sync(BAR_DONE + ((j - 1) & 1), nthr);
            if (threadIdx.x == 0)
                st_release_sys(prev_signal, prev_value);
        }
        return;
    }
    // the ring of the pair: in the receiver's area (the sender stores across NVLink) or, in pull mode, in the
    // sender's (the receiver loads across NVLink)
    const int owner = (op.is_send != 0) == (L.pull != 0) ? c.rank : peer;
    char* slot = L.data[owner] + (size_t)(owner == c.rank ? peer : c.rank) * L.slot_bytes;
    const size_t wt = threadIdx.x - 32, wn = nthr - 32;
    uint32_t j = 0;
    for (int ln = b; ln < nl; ln += nb) {
        const uint32_t mine = (uint32_t)((nchunks - ln + nl - 1) / nl);
        char* ring = slot + (size_t)ln * P2P_STAGES * P2P_CHUNK_BYTES;
        for (uint32_t i = 0; i < mine; i++, j++) {
            const size_t l = ((size_t)ln + (size_t)i * nl) * P2P_CHUNK_BYTES;
            const size_t len = op.bytes - l < P2P_CHUNK_BYTES ? op.bytes - l : P2P_CHUNK_BYTES;
            named_bar_sync(BAR_GO + (j & 1), nthr);
            if (fail)
                return;
            char* stage = ring + (size_t)stage_of[j & 1] * P2P_CHUNK_BYTES;
            if (len) {
                if (op.is_send)
                    threads_copy<false>(stage, reinterpret_cast<const char*>(op.send) + l, len, wt, wn);
                else
                    threads_copy<true>(reinterpret_cast<char*>(op.recv) + l, stage, len, wt, wn);
            }
            named_bar_arrive(BAR_DONE + (j & 1), nthr);
        }
    }
}

// A barrier whose flag nobody sets: used by the failure-detection test to let
// a wait run out and check that the status word reports it while the context
// stays usable.  It waits on a private word of this rank's p2p flag area.
static __global__ void __launch_bounds__(64) wait_unset_flag_kernel(const comm_dev* tab, coll_args a) {
    const int er = a.emu ? (int)blockIdx.y : 0;
    const comm_dev& c = tab[er];
    if (threadIdx.x == 0) {
        uint32_t* word = c.p2p_flags[c.rank] + P2P_SPARE_WORD; // never written by anyone
        wait_flag_sys(c, word, 1u, (uint32_t)c.rank, ST_FLAG_TIMEOUT);
    }
}

// ---------------------------------------------------------------------------
// local helpers: out = op(a, b) (reduce_local_* of kernels.cl:219-246),
// pack / unpack of a tensor list into one fused buffer (fusion copy entries,
// src/fusion/fusion.cpp:283-362) driven by a pointer table.
// ---------------------------------------------------------------------------
template <class T, class Op>
__global__ void __launch_bounds__(1024) reduce_local_kernel(const T* in, T* inout, size_t count) {
    typedef typename acc_of<T>::type A;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        inout[i] = from_acc<T, A>(Op::apply(to_acc<A, T>(inout[i]), to_acc<A, T>(in[i])));
}

struct pack_table {
    const void* const* ptrs; // device array of n tensor pointers
    const size_t* offs; // device array of n byte offsets into the fused buffer (16-byte aligned)
    const size_t* lens; // device array of n tensor sizes in bytes
    int n;
};

template <bool UNPACK>
__global__ void __launch_bounds__(512) pack_kernel(pack_table t, char* fused) {
    // blockIdx.y walks tensors, blockIdx.x strides inside one tensor
    for (int k = blockIdx.y; k < t.n; k += gridDim.y) {
        const size_t bytes = t.lens[k];
        size_t lo, hi;
        split_range((bytes + 15) >> 4, gridDim.x, blockIdx.x, lo, hi);
        const size_t l = lo << 4, h = (hi << 4) < bytes ? (hi << 4) : bytes;
        if (h <= l)
            continue;
        char* user = const_cast<char*>(reinterpret_cast<const char*>(t.ptrs[k]));
        if (UNPACK)
            block_copy<false>(user + l, fused + t.offs[k] + l, h - l);
        else
            block_copy<false>(fused + t.offs[k] + l, user + l, h - l);
    }
}

} // namespace dev
} // namespace cclx
