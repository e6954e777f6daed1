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
