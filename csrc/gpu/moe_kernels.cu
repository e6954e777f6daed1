// Expert-parallel helpers around the all-to-all: row gather in dispatch order
// and the combine step (un-permute + weighted sum of the top-k expert outputs).
//
// The reference offers alltoallv (src/coll/algorithms/alltoallv.cpp:112-751,
// alltoallv_kernel_* in src/kernels/kernels.cl:110-116) and leaves routing to the
// application; here the two memory-bound passes next to the exchange are
// kernels of the library so that the MoE layer is: route -> gather -> alltoallv
// -> expert FFN (tcgen05 GEMMs) -> alltoallv -> combine.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <vector>

#include "capi/capi_common.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"

namespace {

// out[i, :] = x[src_row[i], :]      (bf16 rows of `hidden` elements, hidden % 8 == 0)
__global__ void __launch_bounds__(256) gather_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const long long* __restrict__ src_row,
                                                          __nv_bfloat16* __restrict__ out, size_t n_rows,
                                                          int hidden) {
    const int packs = hidden / 8;
    for (size_t r = blockIdx.x; r < n_rows; r += gridDim.x) {
        const uint4* s = reinterpret_cast<const uint4*>(x + (size_t)src_row[r] * hidden);
        uint4* d = reinterpret_cast<uint4*>(out + r * hidden);
        for (int i = threadIdx.x; i < packs; i += blockDim.x)
            d[i] = s[i];
    }
}

// out[t, :] = sum_k w[t, k] * y[pos[t, k], :]   (fp32 accumulate, bf16 out)
__global__ void __launch_bounds__(256) combine_rows_kernel(const __nv_bfloat16* __restrict__ y,
                                                           const long long* __restrict__ pos,
                                                           const float* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ out, size_t n_tokens, int topk,
                                                           int hidden) {
    const int packs = hidden / 8;
    for (size_t t = blockIdx.x; t < n_tokens; t += gridDim.x) {
        for (int i = threadIdx.x; i < packs; i += blockDim.x) {
            float acc[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
            for (int k = 0; k < topk; k++) {
                const float wk = w[t * topk + k];
                uint4 v = reinterpret_cast<const uint4*>(y + (size_t)pos[t * topk + k] * hidden)[i];
                const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
                for (int e = 0; e < 8; e++)
                    acc[e] += wk * __bfloat162float(h[e]);
            }
            uint4 o;
            __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
            for (int e = 0; e < 8; e++)
                oh[e] = __float2bfloat16_rn(acc[e]);
            reinterpret_cast<uint4*>(out + t * hidden)[i] = o;
        }
    }
}

int blocks_for(size_t rows) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    size_t cap = (size_t)sms * 8;
    return (int)(rows < cap ? (rows ? rows : 1) : cap);
}

} // namespace

CCLX_API int cclx_moe_gather_rows(const void* x, const long long* src_row, void* out, size_t n_rows, int hidden,
                                  void* stream) {
    return cclx::capi::guard([&] {
        CCL_THROW_IF_NOT(hidden % 8 == 0, "hidden size must be a multiple of 8");
        if (n_rows == 0)
            return;
        gather_rows_kernel<<<blocks_for(n_rows), 256, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)x, src_row, (__nv_bfloat16*)out, n_rows, hidden);
        CUDA_CHECK(cudaGetLastError());
    });
}

CCLX_API int cclx_moe_combine(const void* y, const long long* pos, const float* w, void* out, size_t n_tokens,
                              int topk, int hidden, void* stream) {
    return cclx::capi::guard([&] {
        CCL_THROW_IF_NOT(hidden % 8 == 0, "hidden size must be a multiple of 8");
        if (n_tokens == 0)
            return;
        combine_rows_kernel<<<blocks_for(n_tokens), 256, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)y, pos, w, (__nv_bfloat16*)out, n_tokens, topk, hidden);
        CUDA_CHECK(cudaGetLastError());
    });
}

// ---------------------------------------------------------------------------------------------
// Routing on the device: top-k experts per token with softmax weights over the chosen logits, the number of
// (token, slot) items per expert, and a permutation that groups the items by expert (with its inverse).  Two
// small kernels replace topk / softmax / bincount / argsort / scatter of an eager implementation (six launches
// and a sort).  Inside an expert's group the items stand in the order the atomics grant, which no consumer
// depends on: the combine step finds every item through `pos`, and an expert's rows are computed independently
// of their place.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int ROUTE_MAX_EXPERTS = 64;
constexpr int ROUTE_MAX_TOPK = 8;

__global__ void __launch_bounds__(256)
    route_topk_kernel(const float* __restrict__ logits, int n_tokens, int n_experts, int topk, long long* __restrict__ idx,
                      float* __restrict__ wts, unsigned long long* __restrict__ counts) {
    __shared__ unsigned int hist[ROUTE_MAX_EXPERTS];
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x)
        hist[e] = 0;
    __syncthreads();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n_tokens) {
        const float* row = logits + (size_t)t * n_experts;
        int best[ROUTE_MAX_TOPK];
        float val[ROUTE_MAX_TOPK];
        for (int s = 0; s < topk; s++) {
            // largest logit not taken yet; ties go to the lower expert index (as torch.topk on a sorted scan would)
            int be = -1;
            float bv = 0.f;
            for (int e = 0; e < n_experts; e++) {
                bool taken = false;
                for (int q = 0; q < s; q++)
                    taken |= best[q] == e;
                const float v = row[e];
                if (!taken && (be < 0 || v > bv)) {
                    be = e;
                    bv = v;
                }
            }
            best[s] = be;
            val[s] = bv;
        }
        float sum = 0.f;
        const float vmax = val[0]; // the first pick is the maximum
        for (int s = 0; s < topk; s++) {
            val[s] = __expf(val[s] - vmax);
            sum += val[s];
        }
        for (int s = 0; s < topk; s++) {
            idx[(size_t)t * topk + s] = best[s];
            wts[(size_t)t * topk + s] = val[s] / sum;
            atomicAdd(&hist[best[s]], 1u);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x)
        if (hist[e])
            atomicAdd(&counts[e], (unsigned long long)hist[e]);
}

// cursor[e] starts at zero; item i = token * topk + slot lands at offset(expert) + ticket.  Tickets are drawn in
// shared memory first and every block asks the global counters once per expert (a million items on eight
// global counters would serialise on them).
__global__ void __launch_bounds__(256)
    route_place_kernel(const long long* __restrict__ idx, size_t n_items, int n_experts,
                       const unsigned long long* __restrict__ counts, unsigned int* __restrict__ cursor,
                       long long* __restrict__ order, long long* __restrict__ pos) {
    __shared__ unsigned long long offs[ROUTE_MAX_EXPERTS];
    __shared__ unsigned int local_n[ROUTE_MAX_EXPERTS], base[ROUTE_MAX_EXPERTS];
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x)
        local_n[e] = 0;
    if (threadIdx.x == 0) {
        unsigned long long acc = 0;
        for (int e = 0; e < n_experts; e++) {
            offs[e] = acc;
            acc += counts[e];
        }
    }
    __syncthreads();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    int e = -1;
    unsigned int ticket = 0;
    if (i < n_items) {
        e = (int)idx[i];
        ticket = atomicAdd(&local_n[e], 1u);
    }
    __syncthreads();
    for (int x = threadIdx.x; x < n_experts; x += blockDim.x)
        base[x] = local_n[x] ? atomicAdd(&cursor[x], local_n[x]) : 0u;
    __syncthreads();
    if (e >= 0) {
        const unsigned long long p = offs[e] + base[e] + ticket;
        order[p] = (long long)i;
        pos[i] = (long long)p;
    }
}
} // namespace

// logits [n_tokens, n_experts] fp32 -> idx [n_tokens, topk] (int64), wts [n_tokens, topk] (fp32),
// counts [n_experts] (int64), order / pos [n_tokens * topk] (int64).  scratch: n_experts 32-bit words.
CCLX_API int cclx_moe_route(const float* logits, int n_tokens, int n_experts, int topk, long long* idx, float* wts,
                            long long* counts, long long* order, long long* pos, void* scratch, void* stream) {
    return cclx::capi::guard([&] {
        CCL_THROW_IF_NOT(n_experts >= 1 && n_experts <= ROUTE_MAX_EXPERTS, "routing supports up to ", ROUTE_MAX_EXPERTS,
                         " experts");
        CCL_THROW_IF_NOT(topk >= 1 && topk <= ROUTE_MAX_TOPK && topk <= n_experts, "top-k must be between 1 and min(",
                         ROUTE_MAX_TOPK, ", experts)");
        cudaStream_t st = (cudaStream_t)stream;
        CUDA_CHECK(cudaMemsetAsync(counts, 0, sizeof(long long) * n_experts, st));
        CUDA_CHECK(cudaMemsetAsync(scratch, 0, sizeof(unsigned int) * n_experts, st));
        if (n_tokens == 0)
            return;
        route_topk_kernel<<<(n_tokens + 255) / 256, 256, 0, st>>>(logits, n_tokens, n_experts, topk, idx, wts,
                                                                  (unsigned long long*)counts);
        CUDA_CHECK(cudaGetLastError());
        const size_t n_items = (size_t)n_tokens * topk;
        route_place_kernel<<<(unsigned)((n_items + 255) / 256), 256, 0, st>>>(
            idx, n_items, n_experts, (const unsigned long long*)counts, (unsigned int*)scratch, order, pos);
        CUDA_CHECK(cudaGetLastError());
    });
}

// ---------------------------------------------------------------------------------------------
// Fused dispatch and combine over peer memory: the all-to-all of an expert-parallel layer without
// staging buffers, send-side row gather or receive-side copies.
//
//   dispatch: every rank tells every peer how many rows it sends to each expert (a W x W table in
//             symmetric memory, written redundantly per block so that the per-block barrier is
//             enough), derives where its rows start inside each expert's receive buffer (ranks in
//             order), and stores row `order[i] / topk` of x straight into the owner's buffer.
//   combine : after the expert FFN wrote its output rows (same layout as the receive buffer) every
//             rank pulls the rows of its tokens from the owners with peer loads and forms the
//             weighted sum in fp32.
//
// The reference leaves both steps to alltoallv (src/coll/algorithms/alltoallv.cpp:112-751) around
// user kernels; on NVSwitch the rows can go directly where they are needed.
// ---------------------------------------------------------------------------------------------
#include "gpu/device/common.cuh"
#include "gpu/device_comm.hpp"

namespace {

using namespace cclx;
using namespace cclx::dev;

struct moe_rank_args {
    const __nv_bfloat16* x; // dispatch: [tokens, hidden] input rows | combine: unused
    const long long* order; // dispatch: (token, slot) pairs sorted by expert, as token * topk + slot
    const long long* send_counts; // dispatch: rows for every expert [world]
    const long long* expert; // combine: expert of every (token, slot) [tokens * topk]
    const long long* pos; // combine: place of (token, slot) in `order`
    const float* weight; // combine: routing weights [tokens * topk]
    __nv_bfloat16* out; // combine: [tokens, hidden]
    int* meta; // [0, W) first row of my block inside expert e's buffer, [W, 2W) prefix of send_counts,
               // [2W] rows this rank's expert received, [2W+1] 1 if some buffer overflowed
};

struct moe_args {
    moe_rank_args r0;
    const moe_rank_args* emu_tab;
    int emu;
    int topk;
    int hidden;
    size_t n_items; // tokens * topk
    size_t cap_rows; // rows of the receive / output buffers
    size_t buf_off; // heap offset of the receive buffer (dispatch) or of the expert output (combine)
    size_t cnt_off; // heap offset of the int32 table [blocks][W][W]
};

__global__ void __launch_bounds__(512) moe_dispatch_kernel(const comm_dev* tab, moe_args a) {
    const int er = a.emu ? (int)blockIdx.y : 0;
    const comm_dev& c = tab[er];
    const moe_rank_args& ra = a.emu ? a.emu_tab[er] : a.r0;
    block_sync s;
    sync_begin(c, s);
    const int W = c.world;
    __shared__ int s_dst[MAX_RANKS], s_pre[MAX_RANKS + 1], s_over;
    // my counts into every rank's table, slot of this block
    const size_t blk_words = (size_t)blockIdx.x * W * W;
    for (int i = threadIdx.x; i < W * W; i += blockDim.x) {
        const int p = i / W, e = i % W;
        int* t = reinterpret_cast<int*>(c.heap[p] + a.cnt_off) + blk_words;
        t[c.rank * W + e] = (int)ra.send_counts[e];
    }
    bool ok = peer_barrier(c, s);
    if (threadIdx.x == 0) {
        const int* t = reinterpret_cast<const int*>(c.heap[c.rank] + a.cnt_off) + blk_words;
        int over = 0, pre = 0, recv = 0;
        for (int e = 0; e < W; e++) {
            int off = 0, tot = 0;
            for (int q = 0; q < W; q++) {
                const int v = __ldcv(t + q * W + e);
                if (q < c.rank)
                    off += v;
                tot += v;
            }
            s_dst[e] = off;
            s_pre[e] = pre;
            pre += (int)ra.send_counts[e];
            over |= tot > (long long)a.cap_rows ? 1 : 0;
            if (e == c.rank)
                recv = tot;
        }
        s_pre[W] = pre;
        s_over = over;
        if (blockIdx.x == 0) {
            for (int e = 0; e < W; e++) {
                ra.meta[e] = s_dst[e];
                ra.meta[W + e] = s_pre[e];
            }
            ra.meta[2 * W] = recv;
            ra.meta[2 * W + 1] = over;
        }
    }
    __syncthreads();
    if (ok && !s_over) {
        // one warp per row
        const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
        const size_t warp = (size_t)blockIdx.x * wpb + (threadIdx.x >> 5), nwarps = (size_t)gridDim.x * wpb;
        const int packs = a.hidden / 8;
        for (size_t i = warp; i < a.n_items; i += nwarps) {
            int e = 0;
            while (e + 1 < W && (long long)i >= s_pre[e + 1])
                e++;
            const size_t row = (size_t)s_dst[e] + (i - (size_t)s_pre[e]);
            const uint4* src = reinterpret_cast<const uint4*>(ra.x + (size_t)(ra.order[i] / a.topk) * a.hidden);
            char* dst = c.heap[e] + a.buf_off + row * (size_t)a.hidden * 2;
            for (int k = lane; k < packs; k += 32)
                st16(dst + (size_t)k * 16, src[k]);
        }
    }
    peer_barrier(c, s);
    sync_end(c, gridDim.x, 2, false);
}

__global__ void __launch_bounds__(512) moe_combine_kernel(const comm_dev* tab, moe_args a) {
    const int er = a.emu ? (int)blockIdx.y : 0;
    const comm_dev& c = tab[er];
    const moe_rank_args& ra = a.emu ? a.emu_tab[er] : a.r0;
    block_sync s;
    sync_begin(c, s);
    const int W = c.world;
    // every owner has finished its expert FFN (this launch is ordered after it on each rank's stream)
    bool ok = peer_barrier(c, s);
    if (ok) {
        const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
        const size_t warp = (size_t)blockIdx.x * wpb + (threadIdx.x >> 5), nwarps = (size_t)gridDim.x * wpb;
        const int packs = a.hidden / 8;
        const size_t tokens = a.n_items / a.topk;
        for (size_t t = warp; t < tokens; t += nwarps) {
            for (int k0 = lane; k0 < packs; k0 += 32) {
                float acc[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
                for (int sl = 0; sl < a.topk; sl++) {
                    const size_t f = t * a.topk + sl;
                    const int e = (int)ra.expert[f];
                    const size_t row = (size_t)ra.meta[e] + ((size_t)ra.pos[f] - (size_t)ra.meta[W + e]);
                    const float w = ra.weight[f];
                    const uint4 v = ld_cv16(c.heap[e] + a.buf_off + row * (size_t)a.hidden * 2 + (size_t)k0 * 16);
                    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        acc[q] = fmaf(w, __bfloat162float(h[q]), acc[q]);
                }
                uint4 o;
                __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
                for (int q = 0; q < 8; q++)
                    oh[q] = __float2bfloat16_rn(acc[q]);
                reinterpret_cast<uint4*>(ra.out + t * a.hidden)[k0] = o;
            }
        }
    }
    // nobody may overwrite its output rows (the next layer's FFN) before every reader is done
    peer_barrier(c, s);
    sync_end(c, gridDim.x, 2, false);
}

void launch_moe(gpu::device_comm& dc, bool dispatch, moe_args& a, const moe_rank_args* ra, int blocks,
                cudaStream_t st) {
    dc.check_status();
    blocks = blocks > 0 ? std::min(blocks, dc.max_blocks()) : std::min(dc.max_blocks(), 128);
    a.r0 = ra[0];
    if (dc.emulated()) {
        static_assert(sizeof(moe_rank_args) <= sizeof(dev::rank_args), "argument block too large");
        CUDA_CHECK(cudaStreamSynchronize(st));
        CUDA_CHECK(cudaMemcpy(dc.emu_args_dev(), ra, dc.world() * sizeof(moe_rank_args), cudaMemcpyHostToDevice));
        a.emu = 1;
        a.emu_tab = reinterpret_cast<const moe_rank_args*>(dc.emu_args_dev());
        const comm_dev* tab = dc.table();
        void* argv[] = { (void*)&tab, (void*)&a };
        dim3 grid(blocks, dc.world());
        CUDA_CHECK(cudaLaunchCooperativeKernel(dispatch ? (const void*)moe_dispatch_kernel : (const void*)moe_combine_kernel,
                                               grid, dim3(512), argv, 0, st));
    }
    else {
        a.emu = 0;
        a.emu_tab = nullptr;
        if (dispatch)
            moe_dispatch_kernel<<<blocks, 512, 0, st>>>(dc.table(), a);
        else
            moe_combine_kernel<<<blocks, 512, 0, st>>>(dc.table(), a);
        CUDA_CHECK(cudaGetLastError());
    }
}

} // namespace

// Arrays hold one pointer per entry: one entry in real mode, `world` entries in emulation mode.
// `recv_buf` / `cnt_table` are this rank's (entry 0's) symmetric allocations: [cap_rows, hidden] bf16 and
// at least 256 * world * world int32.  meta: 2 * world + 2 int32 per entry.
CCLX_API int cclx_moe_dispatch(void* h, const void* const* x, const long long* const* order,
                               const long long* const* send_counts, int* const* meta, size_t n_items, int topk,
                               int hidden, const void* recv_buf, size_t cap_rows, const void* cnt_table, int blocks,
                               void* stream) {
    return cclx::capi::guard([&] {
        gpu::device_comm* dc = (gpu::device_comm*)h;
        CCL_THROW_IF_NOT(hidden % 8 == 0 && topk >= 1, "hidden size must be a multiple of 8");
        const int entries = dc->emulated() ? dc->world() : 1;
        const int owner = dc->emulated() ? 0 : dc->rank();
        moe_args a{};
        a.topk = topk;
        a.hidden = hidden;
        a.n_items = n_items;
        a.cap_rows = cap_rows;
        a.buf_off = dc->symm_offset(recv_buf, owner);
        a.cnt_off = dc->symm_offset(cnt_table, owner);
        CCL_THROW_IF_NOT(a.buf_off != (size_t)-1 && a.cnt_off != (size_t)-1 && (a.buf_off & 15) == 0,
                         "the receive buffer and the count table must come from the symmetric heap");
        std::vector<moe_rank_args> ra(entries);
        for (int e = 0; e < entries; e++) {
            ra[e] = moe_rank_args{};
            ra[e].x = (const __nv_bfloat16*)x[e];
            ra[e].order = order[e];
            ra[e].send_counts = send_counts[e];
            ra[e].meta = meta[e];
        }
        launch_moe(*dc, true, a, ra.data(), blocks, (cudaStream_t)stream);
    });
}

CCLX_API int cclx_moe_combine_peer(void* h, const long long* const* expert, const long long* const* pos,
                                   const float* const* weight, void* const* out, int* const* meta, size_t n_items,
                                   int topk, int hidden, const void* expert_out, int blocks, void* stream) {
    return cclx::capi::guard([&] {
        gpu::device_comm* dc = (gpu::device_comm*)h;
        CCL_THROW_IF_NOT(hidden % 8 == 0 && topk >= 1, "hidden size must be a multiple of 8");
        const int entries = dc->emulated() ? dc->world() : 1;
        const int owner = dc->emulated() ? 0 : dc->rank();
        moe_args a{};
        a.topk = topk;
        a.hidden = hidden;
        a.n_items = n_items;
        a.buf_off = dc->symm_offset(expert_out, owner);
        CCL_THROW_IF_NOT(a.buf_off != (size_t)-1 && (a.buf_off & 15) == 0,
                         "the expert output must come from the symmetric heap");
        std::vector<moe_rank_args> ra(entries);
        for (int e = 0; e < entries; e++) {
            ra[e] = moe_rank_args{};
            ra[e].expert = expert[e];
            ra[e].pos = pos[e];
            ra[e].weight = weight[e];
            ra[e].out = (__nv_bfloat16*)out[e];
            ra[e].meta = meta[e];
        }
        launch_moe(*dc, false, a, ra.data(), blocks, (cudaStream_t)stream);
    });
}
