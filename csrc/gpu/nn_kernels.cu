// Memory-bound layer kernels of the transformer blocks used by the data-parallel training path:
// LayerNorm forward / backward (input gradient plus the weight and bias gradients in the same pass),
// column sums for bias gradients, and the strided copies that assemble a packed QKV gradient.
// The reference is a communication library and has no such kernels; they exist because the training
// step that the gradient allreduce overlaps with is otherwise dominated by framework kernels that
// re-read activations several times.  All math in fp32, bf16 storage.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

#include "capi/capi_common.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"

namespace {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One warp per row, V 16-byte packs per lane (row length D = 256 * V).  Lane l holds packs l, l+32, ...
template <int V>
__device__ __forceinline__ void load_row(const __nv_bfloat16* row, int lane, float (&x)[V * 8]) {
    const uint4* p = reinterpret_cast<const uint4*>(row);
#pragma unroll
    for (int v = 0; v < V; v++) {
        const uint4 u = p[lane + v * 32];
        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
        for (int e = 0; e < 8; e++)
            x[v * 8 + e] = __bfloat162float(h[e]);
    }
}

template <int V>
__device__ __forceinline__ void store_row(__nv_bfloat16* row, int lane, const float (&x)[V * 8]) {
    uint4* p = reinterpret_cast<uint4*>(row);
#pragma unroll
    for (int v = 0; v < V; v++) {
        uint4 u;
        __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(&u);
#pragma unroll
        for (int e = 0; e < 8; e++)
            h[e] = __float2bfloat16_rn(x[v * 8 + e]);
        p[lane + v * 32] = u;
    }
}

// y = (x - mean) * rstd * w + b ; optionally x = x + residual first (the sum is written to `sum_out`)
template <int V>
__global__ void __launch_bounds__(256) ln_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                                     const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                                                     __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ sum_out,
                                                     float* __restrict__ mean, float* __restrict__ rstd, size_t rows,
                                                     float eps) {
    constexpr int D = V * 256;
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    float wv[V * 8], bv[V * 8];
    load_row<V>(w, lane, wv);
    load_row<V>(b, lane, bv);
    for (size_t r = (size_t)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += (size_t)gridDim.x * wpb) {
        float xv[V * 8];
        load_row<V>(x + r * D, lane, xv);
        if (res) {
            float rv[V * 8];
            load_row<V>(res + r * D, lane, rv);
#pragma unroll
            for (int i = 0; i < V * 8; i++)
                xv[i] = __bfloat162float(__float2bfloat16_rn(xv[i] + rv[i])); // the sum lives in bf16
            store_row<V>(sum_out + r * D, lane, xv);
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < V * 8; i++)
            s += xv[i];
        const float m = warp_sum_f(s) * (1.0f / D);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < V * 8; i++) {
            const float d = xv[i] - m;
            q += d * d;
        }
        const float rs = rsqrtf(warp_sum_f(q) * (1.0f / D) + eps);
#pragma unroll
        for (int i = 0; i < V * 8; i++)
            xv[i] = (xv[i] - m) * rs * wv[i] + bv[i];
        store_row<V>(y + r * D, lane, xv);
        if (lane == 0) {
            mean[r] = m;
            rstd[r] = rs;
        }
    }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * w;  partial dgamma / dbeta per block.
// `dres` (optional) is added to dx: the gradient that reached the residual branch.
template <int V>
__global__ void __launch_bounds__(256) ln_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                     const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean,
                                                     const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dres,
                                                     __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, size_t rows) {
    constexpr int D = V * 256;
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5, warp = threadIdx.x >> 5;
    float wv[V * 8], dg[V * 8], db[V * 8];
    load_row<V>(w, lane, wv);
#pragma unroll
    for (int i = 0; i < V * 8; i++)
        dg[i] = db[i] = 0.f;
    for (size_t r = (size_t)blockIdx.x * wpb + warp; r < rows; r += (size_t)gridDim.x * wpb) {
        float xv[V * 8], gv[V * 8];
        load_row<V>(x + r * D, lane, xv);
        load_row<V>(dy + r * D, lane, gv);
        const float m = mean[r], rs = rstd[r];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < V * 8; i++) {
            const float xh = (xv[i] - m) * rs;
            db[i] += gv[i];
            dg[i] += gv[i] * xh;
            const float g = gv[i] * wv[i];
            s1 += g;
            s2 += g * xh;
            xv[i] = xh;
            gv[i] = g;
        }
        s1 = warp_sum_f(s1) * (1.0f / D);
        s2 = warp_sum_f(s2) * (1.0f / D);
#pragma unroll
        for (int i = 0; i < V * 8; i++)
            gv[i] = rs * (gv[i] - s1 - xv[i] * s2);
        if (dres) {
            load_row<V>(dres + r * D, lane, xv);
#pragma unroll
            for (int i = 0; i < V * 8; i++)
                gv[i] += xv[i];
        }
        store_row<V>(dx + r * D, lane, gv);
    }
    // block partials: warps add into shared memory one after the other (fixed order), then one row out
    __shared__ float sh[2][D];
    for (int k = 0; k < wpb; k++) {
        if (warp == k) {
#pragma unroll
            for (int v = 0; v < V; v++)
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const int col = (lane + v * 32) * 8 + e;
                    sh[0][col] = (k == 0 ? 0.f : sh[0][col]) + dg[v * 8 + e];
                    sh[1][col] = (k == 0 ? 0.f : sh[1][col]) + db[v * 8 + e];
                }
        }
        __syncthreads();
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        partial[((size_t)blockIdx.x * 2 + 0) * D + c] = sh[0][c];
        partial[((size_t)blockIdx.x * 2 + 1) * D + c] = sh[1][c];
    }
}

// out[c] = sum over `n` partial rows (fixed order per column); two outputs interleaved as in ln_bwd_kernel.
// A block owns 32 columns of one output: 8 row groups add their share of the partial rows, a fixed tree
// in shared memory joins them.  grid = (D / 32, 2).
__global__ void __launch_bounds__(256) ln_bwd_final_kernel(const float* __restrict__ partial, int n, int D,
                                                           __nv_bfloat16* __restrict__ dgamma, __nv_bfloat16* __restrict__ dbeta) {
    const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane, which = blockIdx.y;
    float a = 0.f;
    if (c < D)
        for (int k = grp; k < n; k += 8)
            a += partial[((size_t)k * 2 + which) * D + c];
    __shared__ float sh[8][32];
    sh[grp][lane] = a;
    __syncthreads();
    if (grp == 0 && c < D) {
        float s = 0.f;
#pragma unroll
        for (int g = 0; g < 8; g++)
            s += sh[g][lane];
        (which == 0 ? dgamma : dbeta)[c] = __float2bfloat16_rn(s);
    }
}

} // namespace

namespace {

// column sums of a [rows, N] bf16 matrix (bias gradient): partial[chunk][N], then a fixed-order sum by the last block.
// One warp covers 256 columns (a 16-byte pack per lane); grid = (N / 256, chunks).
__global__ void __launch_bounds__(256) colsum_kernel(const __nv_bfloat16* __restrict__ dy, size_t rows, int N,
                                                     float* __restrict__ partial, unsigned* __restrict__ counters,
                                                     __nv_bfloat16* __restrict__ out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int col = (blockIdx.x * 32 + lane) * 8;
    float acc[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
    if (col < N) {
        const size_t per = (rows + gridDim.y - 1) / gridDim.y;
        const size_t r0 = (size_t)blockIdx.y * per, r1 = min(rows, r0 + per);
        size_t r = r0 + warp;
        for (; r + 3 * wpb < r1; r += 4 * wpb) { // four rows in flight per lane
            uint4 u[4];
#pragma unroll
            for (int k = 0; k < 4; k++)
                u[k] = *reinterpret_cast<const uint4*>(dy + (r + (size_t)k * wpb) * N + col);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u[k]);
#pragma unroll
                for (int e = 0; e < 8; e++)
                    acc[e] += __bfloat162float(h[e]);
            }
        }
        for (; r < r1; r += wpb) {
            const uint4 u = *reinterpret_cast<const uint4*>(dy + r * N + col);
            const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
            for (int e = 0; e < 8; e++)
                acc[e] += __bfloat162float(h[e]);
        }
    }
    __shared__ float sh[8][256];
    __shared__ int last;
#pragma unroll
    for (int e = 0; e < 8; e++)
        sh[warp][lane * 8 + e] = acc[e];
    __syncthreads();
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < N) {
        float s = 0.f;
        for (int k = 0; k < wpb; k++)
            s += sh[k][threadIdx.x];
        partial[(size_t)blockIdx.y * N + c] = s;
    }
    // the block that finishes last for this column tile adds the chunks in index order (the result does
    // not depend on which block that is) and re-arms the counter for the next call
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0)
        last = atomicAdd(counters + blockIdx.x, 1u) == gridDim.y - 1 ? 1 : 0;
    __syncthreads();
    if (last) {
        __threadfence();
        if (c < N) {
            float s = 0.f;
            for (unsigned k = 0; k < gridDim.y; k++)
                s += __ldcg(partial + (size_t)k * N + c);
            out[c] = __float2bfloat16_rn(s);
        }
        if (threadIdx.x == 0)
            counters[blockIdx.x] = 0;
    }
}

// dst[b, s, h, :] = src[b, s, h, :] for head rows of `dh` elements (dh % 8 == 0) with arbitrary element
// strides of the three outer dimensions on both sides: assembles a packed QKV gradient from the three
// attention gradients without a concatenation pass per tensor.
struct head_copy_args {
    const __nv_bfloat16* src[3];
    long long sb[3], ss[3], sh[3]; // source strides of (batch, sequence, head)
    __nv_bfloat16* dst[3];
    long long db, ds, dh_stride; // destination strides (the same for the three parts)
    int B, S, H, dh;
};

__global__ void __launch_bounds__(256) head_copy_kernel(head_copy_args a) {
    const int ppr = a.dh / 8; // packs per head row
    const size_t total = (size_t)a.B * a.S * a.H * ppr;
    const int part = blockIdx.y;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int p = (int)(i % ppr);
        size_t t = i / ppr;
        const int h = (int)(t % a.H);
        t /= a.H;
        const int s = (int)(t % a.S);
        const int b = (int)(t / a.S);
        const uint4 v = *reinterpret_cast<const uint4*>(a.src[part] + b * a.sb[part] + s * a.ss[part] + h * a.sh[part] + p * 8);
        *reinterpret_cast<uint4*>(a.dst[part] + b * a.db + s * a.ds + h * a.dh_stride + p * 8) = v;
    }
}

int sm_count_now() {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms;
}

} // namespace

// ---- C entry points -----------------------------------------------------------------------------
// D must be 256, 512, 768 or 1024.  mean / rstd: fp32 [rows].  res / sum_out may be null (no residual).
CCLX_API int cclx_layer_norm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* sum_out,
                                 float* mean, float* rstd, size_t rows, int D, float eps, void* stream) {
    return cclx::capi::guard([&] {
        CCL_THROW_IF_NOT(D % 256 == 0 && D >= 256 && D <= 1024, "fused LayerNorm supports 256, 512, 768 and 1024 columns");
        CCL_THROW_IF_NOT((res == nullptr) == (sum_out == nullptr), "residual input and sum output go together");
        if (rows == 0)
            return;
        const int blocks = (int)std::min<size_t>((rows + 7) / 8, (size_t)sm_count_now() * 4);
        cudaStream_t st = (cudaStream_t)stream;
#define LN_FWD(V)                                                                                                          \
    ln_fwd_kernel<V><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, \
                                             (const __nv_bfloat16*)b, (__nv_bfloat16*)y, (__nv_bfloat16*)sum_out, mean,   \
                                             rstd, rows, eps)
        switch (D / 256) {
            case 1: LN_FWD(1); break;
            case 2: LN_FWD(2); break;
            case 3: LN_FWD(3); break;
            default: LN_FWD(4); break;
        }
#undef LN_FWD
        CUDA_CHECK(cudaGetLastError());
    });
}

// workspace: fp32 [cclx_layer_norm_bwd_blocks(rows) * 2 * D].  dres may be null.
CCLX_API int cclx_layer_norm_bwd_blocks(size_t rows) {
    return (int)std::min<size_t>((rows + 7) / 8, (size_t)sm_count_now());
}

CCLX_API int cclx_layer_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                 const void* dres, void* dx, void* dgamma, void* dbeta, float* workspace, size_t rows, int D,
                                 void* stream) {
    return cclx::capi::guard([&] {
        CCL_THROW_IF_NOT(D % 256 == 0 && D >= 256 && D <= 1024, "fused LayerNorm supports 256, 512, 768 and 1024 columns");
        if (rows == 0)
            return;
        const int blocks = cclx_layer_norm_bwd_blocks(rows);
        cudaStream_t st = (cudaStream_t)stream;
#define LN_BWD(V)                                                                                                      \
    ln_bwd_kernel<V><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, \
                                             mean, rstd, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, workspace, rows)
        switch (D / 256) {
            case 1: LN_BWD(1); break;
            case 2: LN_BWD(2); break;
            case 3: LN_BWD(3); break;
            default: LN_BWD(4); break;
        }
#undef LN_BWD
        CUDA_CHECK(cudaGetLastError());
        ln_bwd_final_kernel<<<dim3((D + 31) / 32, 2), 256, 0, st>>>(workspace, blocks, D, (__nv_bfloat16*)dgamma,
                                                                   (__nv_bfloat16*)dbeta);
        CUDA_CHECK(cudaGetLastError());
    });
}

// workspace: fp32 [64 * N]; counters: (N + 255) / 256 zero-initialised words that the kernel leaves zero
CCLX_API int cclx_colsum_bf16(const void* dy, size_t rows, int N, void* out, float* workspace, unsigned* counters,
                              void* stream) {
    return cclx::capi::guard([&] {
        CCL_THROW_IF_NOT(N % 8 == 0, "column count must be a multiple of 8");
        if (rows == 0 || N == 0)
            return;
        const int chunks = (int)std::min<size_t>(64, (rows + 31) / 32);
        colsum_kernel<<<dim3((N + 255) / 256, chunks), 256, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)dy, rows, N, workspace, counters, (__nv_bfloat16*)out);
        CUDA_CHECK(cudaGetLastError());
    });
}

// three [B, H, S, dh]-indexed sources with element strides (sb, ss, sh) each -> three destinations sharing one
// set of strides; strides: 9 source values (b, s, h per part) then 3 destination values.
CCLX_API int cclx_head_copy3(const void* const* src, void* const* dst, const long long* strides, int B, int S, int H, int dh,
                             void* stream) {
    return cclx::capi::guard([&] {
        CCL_THROW_IF_NOT(dh % 8 == 0, "head size must be a multiple of 8");
        head_copy_args a;
        for (int p = 0; p < 3; p++) {
            a.src[p] = (const __nv_bfloat16*)src[p];
            a.dst[p] = (__nv_bfloat16*)dst[p];
            a.sb[p] = strides[p * 3 + 0];
            a.ss[p] = strides[p * 3 + 1];
            a.sh[p] = strides[p * 3 + 2];
            CCL_THROW_IF_NOT(((uintptr_t)src[p] & 15) == 0 && ((uintptr_t)dst[p] & 15) == 0 && a.sb[p] % 8 == 0 &&
                                 a.ss[p] % 8 == 0 && a.sh[p] % 8 == 0,
                             "head copy needs 16-byte aligned rows");
        }
        a.db = strides[9];
        a.ds = strides[10];
        a.dh_stride = strides[11];
        CCL_THROW_IF_NOT(a.db % 8 == 0 && a.ds % 8 == 0 && a.dh_stride % 8 == 0, "head copy needs 16-byte aligned rows");
        a.B = B;
        a.S = S;
        a.H = H;
        a.dh = dh;
        const size_t total = (size_t)B * S * H * (dh / 8);
        const int blocks = (int)std::min<size_t>((total + 255) / 256, (size_t)sm_count_now() * 8);
        head_copy_kernel<<<dim3(blocks, 3), 256, 0, (cudaStream_t)stream>>>(a);
        CUDA_CHECK(cudaGetLastError());
    });
}
