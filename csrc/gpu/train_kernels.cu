// Device kernels of the data-parallel training step that sit next to the
// gradient allreduce: squared-norm of the reduced gradient bucket, fused AdamW
// on flat buffers (fp32 master weights, bf16 model weights written in the same
// pass, gradient read in the bucket's own dtype, clipping factor taken from
// the device-resident norm), and a fused softmax cross-entropy that turns the
// bf16 logits into their gradient in place.
//
// The reference library stops at the collective; these kernels are what makes
// "allreduce fused with 1/world scale and cast" end to end: the bucket stays
// bf16 on the wire and is widened exactly once, inside the optimizer.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "capi/capi_common.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

template <class T>
__device__ __forceinline__ float ldf(const T* p, size_t i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, size_t i) {
    return p[i];
}
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) {
    return __bfloat162float(p[i]);
}

// Squared L2 norm in two deterministic stages (every rank of a data-parallel job must get
// the same bits, otherwise the clipping factor and then the replicas drift apart):
// stage 1: block b writes sum of its grid-stride share of g^2 to partial[b];
// stage 2: one block adds the partials in a fixed tree order and accumulates into out[0].
constexpr int SQN_MAX_BLOCKS = 1024;

template <class T>
__device__ __forceinline__ float sq_pack(const uint4& u) {
    const T* h = reinterpret_cast<const T*>(&u);
    float a = 0.f;
#pragma unroll
    for (int k = 0; k < (int)(16 / sizeof(T)); k++) {
        const float v = ldf<T>(h, k);
        a = fmaf(v, v, a);
    }
    return a;
}

template <class T>
__global__ void __launch_bounds__(512) sq_norm_partial_kernel(const T* g, size_t n, float* partial) {
    constexpr size_t N = 16 / sizeof(T);
    float acc = 0.f;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    // 16-byte loads, four of them in flight per thread; the order of the additions depends on n,
    // the grid and the alignment of g only
    const size_t nv = ((((uintptr_t)g) & 15) == 0) ? n / N : 0;
    const uint4* gv = reinterpret_cast<const uint4*>(g);
    size_t i = gtid;
    for (; i + 3 * stride < nv; i += 4 * stride) {
        const uint4 a = gv[i], b = gv[i + stride], c = gv[i + 2 * stride], d = gv[i + 3 * stride];
        acc += (sq_pack<T>(a) + sq_pack<T>(b)) + (sq_pack<T>(c) + sq_pack<T>(d));
    }
    for (; i < nv; i += stride)
        acc += sq_pack<T>(gv[i]);
    for (size_t e = nv * N + gtid; e < n; e += stride) {
        const float v = ldf<T>(g, e);
        acc = fmaf(v, v, acc);
    }
    __shared__ float part[16];
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0)
        part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0)
            partial[blockIdx.x] = v;
    }
}

__global__ void __launch_bounds__(SQN_MAX_BLOCKS) sq_norm_final_kernel(const float* partial, int n, float* out) {
    __shared__ float sh[SQN_MAX_BLOCKS];
    sh[threadIdx.x] = (int)threadIdx.x < n ? partial[threadIdx.x] : 0.f;
    __syncthreads();
    for (int s = SQN_MAX_BLOCKS / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s)
            sh[threadIdx.x] += sh[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0)
        out[0] += sh[0];
}

__global__ void bump_step_kernel(int* step) {
    *step += 1;
}

struct adamw_args {
    float lr, beta1, beta2, eps, weight_decay;
    float bias1, bias2; // 1 - beta^t
    float grad_scale; // multiplies the gradient (1/world when the allreduce did not scale)
    float max_norm; // <= 0: no clipping
    size_t n_decay; // elements [0, n_decay) get weight decay
};

// one pass: read grad (T) + master/m/v (fp32), write master/m/v and the bf16 model copy
template <class T>
__global__ void __launch_bounds__(512)
    adamw_flat_kernel(float* __restrict__ master, const T* __restrict__ grad, float* __restrict__ m,
                      float* __restrict__ v, __nv_bfloat16* __restrict__ model, size_t n, adamw_args a,
                      const float* __restrict__ sq_norm, const int* __restrict__ step_dev) {
    if (step_dev) { // step number kept on the device: the launch can be replayed from a CUDA graph
        const float t = (float)*step_dev;
        a.bias1 = 1.f - powf(a.beta1, t);
        a.bias2 = 1.f - powf(a.beta2, t);
    }
    float clip = 1.f;
    if (a.max_norm > 0.f && sq_norm) {
        const float norm = sqrtf(*sq_norm) * a.grad_scale;
        clip = fminf(1.f, a.max_norm / (norm + 1e-6f));
    }
    const float gs = a.grad_scale * clip;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float g = ldf<T>(grad, i) * gs;
        float p = master[i];
        float mi = m[i] * a.beta1 + (1.f - a.beta1) * g;
        float vi = v[i] * a.beta2 + (1.f - a.beta2) * g * g;
        const float wd = i < a.n_decay ? a.weight_decay : 0.f;
        p -= a.lr * (wd * p + (mi / a.bias1) / (sqrtf(vi / a.bias2) + a.eps));
        master[i] = p;
        m[i] = mi;
        v[i] = vi;
        if (model)
            model[i] = __float2bfloat16_rn(p);
    }
}

// One block per row of logits [rows, vocab] (bf16, row pitch ld).  Computes
// loss_row = logsumexp - logit[target] and overwrites the row with
// (softmax - onehot) * grad_scale, all math in fp32.  Rows whose target is
// negative (ignore) produce zero loss and zero gradient.  Columns
// [vocab, vocab + pad_cols) are alignment padding and receive zeros.
__global__ void __launch_bounds__(1024)
    softmax_xent_kernel(__nv_bfloat16* logits, const long long* targets, float* loss_rows, int vocab, size_t ld,
                        float grad_scale, int pad_cols) {
    const size_t row = blockIdx.x;
    __nv_bfloat16* x = logits + row * ld;
    const long long tgt = targets[row];
    __shared__ float red[32];
    __shared__ float s_max, s_sum;
    const int nv = vocab / 8; // whole 16-byte packs (row start is 16-byte aligned when ld % 8 == 0)
    const bool vec = (ld % 8 == 0) && ((((uintptr_t)logits) & 15) == 0);

    float mx = -INFINITY;
    if (vec) {
        const uint4* xv = reinterpret_cast<const uint4*>(x);
        for (int i = threadIdx.x; i < nv; i += blockDim.x) {
            uint4 u = xv[i];
            const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
            for (int k = 0; k < 8; k++)
                mx = fmaxf(mx, __bfloat162float(h[k]));
        }
        for (int i = nv * 8 + threadIdx.x; i < vocab; i += blockDim.x)
            mx = fmaxf(mx, __bfloat162float(x[i]));
    }
    else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x)
            mx = fmaxf(mx, __bfloat162float(x[i]));
    }
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : -INFINITY;
        v = warp_max(v);
        if (threadIdx.x == 0)
            s_max = v;
    }
    __syncthreads();
    mx = s_max;

    float sum = 0.f;
    if (vec) {
        const uint4* xv = reinterpret_cast<const uint4*>(x);
        for (int i = threadIdx.x; i < nv; i += blockDim.x) {
            uint4 u = xv[i];
            const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u);
#pragma unroll
            for (int k = 0; k < 8; k++)
                sum += __expf(__bfloat162float(h[k]) - mx);
        }
        for (int i = nv * 8 + threadIdx.x; i < vocab; i += blockDim.x)
            sum += __expf(__bfloat162float(x[i]) - mx);
    }
    else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x)
            sum += __expf(__bfloat162float(x[i]) - mx);
    }
    sum = warp_sum(sum);
    __syncthreads();
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0)
            s_sum = v;
    }
    __syncthreads();
    sum = s_sum;
    const bool ignore = tgt < 0 || tgt >= vocab;
    if (threadIdx.x == 0)
        loss_rows[row] = ignore ? 0.f : (logf(sum) + mx - __bfloat162float(x[tgt]));
    __syncthreads(); // x[tgt] is read before any thread overwrites the row
    const float inv = ignore ? 0.f : grad_scale / sum;
    // alignment padding behind the vocabulary takes no part in the softmax: zero gradient
    for (int i = vocab + threadIdx.x; i < vocab + pad_cols; i += blockDim.x)
        x[i] = __float2bfloat16_rn(0.f);
    if (vec) {
        uint4* xv = reinterpret_cast<uint4*>(x);
        for (int i = threadIdx.x; i < nv; i += blockDim.x) {
            uint4 u = xv[i];
            __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(&u);
#pragma unroll
            for (int k = 0; k < 8; k++) {
                float p = __expf(__bfloat162float(h[k]) - mx) * inv;
                if ((long long)(i * 8 + k) == tgt)
                    p -= grad_scale;
                h[k] = __float2bfloat16_rn(p);
            }
            xv[i] = u;
        }
        for (int i = nv * 8 + threadIdx.x; i < vocab; i += blockDim.x) {
            float p = __expf(__bfloat162float(x[i]) - mx) * inv;
            if (i == tgt)
                p -= grad_scale;
            x[i] = __float2bfloat16_rn(p);
        }
    }
    else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            float p = __expf(__bfloat162float(x[i]) - mx) * inv;
            if (!ignore && i == tgt)
                p -= grad_scale;
            x[i] = __float2bfloat16_rn(p);
        }
    }
}

// Same contract as softmax_xent_kernel for rows that fit the register file: every thread keeps up
// to PPT 16-byte packs of the row in registers, so the row is read from memory once.  The exponentials
// are computed once (fp32, summed in fp32) and parked in the same registers as bf16 until the
// normaliser is known; the gradient is bf16 anyway, the second rounding costs at most one more ulp.
// Needs vocab % 8 == 0 columns handled as packs plus a scalar tail, ld % 8 == 0 and a 16-byte aligned base.
template <int PPT>
__global__ void __launch_bounds__(1024)
    softmax_xent_regs_kernel(__nv_bfloat16* logits, const long long* targets, float* loss_rows, int vocab, size_t ld,
                             float grad_scale, int pad_cols) {
    constexpr float LOG2E = 1.4426950408889634f;
    const size_t row = blockIdx.x;
    __nv_bfloat16* x = logits + row * ld;
    const long long tgt = targets[row];
    __shared__ float red[32];
    __shared__ float s_max, s_sum, s_tgt;
    const int nv = vocab / 8;
    uint4* xv = reinterpret_cast<uint4*>(x);
    const int tail = nv * 8 + (int)threadIdx.x; // at most 7 leftover columns, one per thread
    const bool has_tail = tail < vocab;

    uint4 u[PPT];
#pragma unroll
    for (int j = 0; j < PPT; j++) {
        const int i = (int)threadIdx.x + j * 1024;
        u[j] = i < nv ? xv[i] : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u); // -inf pairs
    }
    float xt = has_tail ? __bfloat162float(x[tail]) : -INFINITY;
    if (threadIdx.x == 0)
        s_tgt = (tgt >= 0 && tgt < vocab) ? __bfloat162float(x[tgt]) : 0.f;

    float mx = xt;
#pragma unroll
    for (int j = 0; j < PPT; j++) {
        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&u[j]);
#pragma unroll
        for (int k = 0; k < 8; k++)
            mx = fmaxf(mx, __bfloat162float(h[k]));
    }
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = warp_max(red[threadIdx.x]);
        if (threadIdx.x == 0)
            s_max = v;
    }
    __syncthreads();
    mx = s_max;
    const float ms = mx * LOG2E;

    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PPT; j++) {
        __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(&u[j]);
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const float e = exp2f(fmaf(__bfloat162float(h[k]), LOG2E, -ms)); // exp2(-inf) = 0 for the filler
            sum += e;
            h[k] = __float2bfloat16_rn(e);
        }
    }
    const float et = has_tail ? exp2f(fmaf(xt, LOG2E, -ms)) : 0.f;
    sum += et;
    sum = warp_sum(sum);
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = warp_sum(red[threadIdx.x]);
        if (threadIdx.x == 0)
            s_sum = v;
    }
    __syncthreads();
    sum = s_sum;
    const bool ignore = tgt < 0 || tgt >= vocab;
    if (threadIdx.x == 0)
        loss_rows[row] = ignore ? 0.f : (logf(sum) + mx - s_tgt);
    const float inv = ignore ? 0.f : grad_scale / sum;
    for (int i = vocab + threadIdx.x; i < vocab + pad_cols; i += blockDim.x)
        x[i] = __float2bfloat16_rn(0.f);
#pragma unroll
    for (int j = 0; j < PPT; j++) {
        const int i = (int)threadIdx.x + j * 1024;
        if (i < nv) {
            __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(&u[j]);
#pragma unroll
            for (int k = 0; k < 8; k++) {
                float p = __bfloat162float(h[k]) * inv;
                if (!ignore && (long long)i * 8 + k == tgt)
                    p -= grad_scale;
                h[k] = __float2bfloat16_rn(p);
            }
            xv[i] = u[j];
        }
    }
    if (has_tail) {
        float p = et * inv;
        if (!ignore && tail == tgt)
            p -= grad_scale;
        x[tail] = __float2bfloat16_rn(p);
    }
}

void launch_softmax_xent(__nv_bfloat16* logits, const long long* targets, float* loss_rows, size_t rows, int vocab,
                         size_t ld, float grad_scale, int pad_cols, cudaStream_t st) {
    const bool vec = (ld % 8 == 0) && ((((uintptr_t)logits) & 15) == 0);
    const int nv = vocab / 8;
    if (vec && nv <= 4 * 1024)
        softmax_xent_regs_kernel<4><<<(unsigned)rows, 1024, 0, st>>>(logits, targets, loss_rows, vocab, ld, grad_scale,
                                                                    pad_cols);
    else if (vec && nv <= 7 * 1024)
        softmax_xent_regs_kernel<7><<<(unsigned)rows, 1024, 0, st>>>(logits, targets, loss_rows, vocab, ld, grad_scale,
                                                                    pad_cols);
    else
        softmax_xent_kernel<<<(unsigned)rows, 1024, 0, st>>>(logits, targets, loss_rows, vocab, ld, grad_scale,
                                                            pad_cols);
    CUDA_CHECK(cudaGetLastError());
}

int grid_for(size_t n, int threads) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    size_t want = (n + threads - 1) / threads;
    size_t cap = (size_t)sms * 4;
    return (int)(want < cap ? (want ? want : 1) : cap);
}

} // namespace

// dt: 9 = float32, 11 = bfloat16 (ccl datatype codes).  out[0] += sum(g^2).
// `partials`: caller-provided scratch of at least 1024 floats.
CCLX_API int cclx_sq_norm(const void* g, size_t n, int dt, float* out, float* partials, void* stream) {
    return cclx::capi::guard([&] {
        if (n == 0)
            return;
        CCL_THROW_IF_NOT(partials != nullptr, "sq_norm needs a partials buffer of 1024 floats");
        // the grid depends on n only, so that every rank adds in the same order
        size_t want = (n + 512 * 32 - 1) / (512 * 32);
        const int blocks = (int)(want < 1 ? 1 : (want > (size_t)SQN_MAX_BLOCKS ? SQN_MAX_BLOCKS : want));
        if (dt == 11)
            sq_norm_partial_kernel<__nv_bfloat16><<<blocks, 512, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)g, n,
                                                                                           partials);
        else if (dt == 9)
            sq_norm_partial_kernel<float><<<blocks, 512, 0, (cudaStream_t)stream>>>((const float*)g, n, partials);
        else
            CCL_THROW("sq_norm supports float32 and bfloat16 gradients");
        CUDA_CHECK(cudaGetLastError());
        sq_norm_final_kernel<<<1, SQN_MAX_BLOCKS, 0, (cudaStream_t)stream>>>(partials, blocks, out);
        CUDA_CHECK(cudaGetLastError());
    });
}

// `step_dev` (optional): device word holding the step number.  When given, the launch first adds one to
// it and the update takes its bias corrections from it instead of `step`, so that the same launch
// sequence can be replayed from a CUDA graph.
CCLX_API int cclx_adamw_flat(float* master, const void* grad, int grad_dt, float* m, float* v, void* model_bf16,
                             size_t n, size_t n_decay, float lr, float beta1, float beta2, float eps,
                             float weight_decay, int step, float grad_scale, float max_norm, const float* sq_norm,
                             int* step_dev, void* stream) {
    return cclx::capi::guard([&] {
        if (n == 0)
            return;
        if (step_dev) {
            bump_step_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(step_dev);
            CUDA_CHECK(cudaGetLastError());
        }
        adamw_args a;
        a.lr = lr;
        a.beta1 = beta1;
        a.beta2 = beta2;
        a.eps = eps;
        a.weight_decay = weight_decay;
        a.bias1 = 1.f - powf(beta1, (float)step);
        a.bias2 = 1.f - powf(beta2, (float)step);
        a.grad_scale = grad_scale;
        a.max_norm = max_norm;
        a.n_decay = n_decay;
        const int blocks = grid_for(n, 512);
        if (grad_dt == 11)
            adamw_flat_kernel<__nv_bfloat16><<<blocks, 512, 0, (cudaStream_t)stream>>>(
                master, (const __nv_bfloat16*)grad, m, v, (__nv_bfloat16*)model_bf16, n, a, sq_norm, step_dev);
        else if (grad_dt == 9)
            adamw_flat_kernel<float><<<blocks, 512, 0, (cudaStream_t)stream>>>(master, (const float*)grad, m, v,
                                                                               (__nv_bfloat16*)model_bf16, n, a, sq_norm, step_dev);
        else
            CCL_THROW("adamw_flat supports float32 and bfloat16 gradients");
        CUDA_CHECK(cudaGetLastError());
    });
}

CCLX_API int cclx_softmax_xent(void* logits_bf16, const long long* targets, float* loss_rows, size_t rows, int vocab,
                               size_t ld, float grad_scale, int pad_cols, void* stream) {
    return cclx::capi::guard([&] {
        if (rows == 0)
            return;
        launch_softmax_xent((__nv_bfloat16*)logits_bf16, targets, loss_rows, rows, vocab, ld, grad_scale, pad_cols,
                            (cudaStream_t)stream);
    });
}

// ---------------------------------------------------------------------------------------------
// Mean cross-entropy without any allocation (declared and documented in gpu/xent_noalloc.h).
// The per-row losses of the regular kernel go to a fixed device array that is part of this
// library image; a one-block kernel then averages them into the caller's float.
// ---------------------------------------------------------------------------------------------
#include "gpu/xent_noalloc.h"

#include <mutex>

namespace {

// scratch: one loss per row.  Lives in every device's copy of this module until the process ends.
static __device__ __align__(256) float xent_row_scratch[CCLX_XENT_NOALLOC_MAX_ROWS];

// out[0] = sum(rows[0..n)) / n, fixed summation order (one block, strided partials, tree in shared memory)
__global__ void __launch_bounds__(1024) mean_rows_kernel(const float* rows, size_t n, float* out) {
    __shared__ float part[1024];
    float acc = 0.f;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x)
        acc += rows[i];
    part[threadIdx.x] = acc;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s)
            part[threadIdx.x] += part[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0)
        out[0] = part[0] / (float)n;
}

constexpr int XENT_MAX_DEVICES = 64;
std::mutex xent_setup_mu;
float* xent_scratch_addr[XENT_MAX_DEVICES] = {};

// Device address of the scratch array on the current device.  In host code the array's name
// is only a handle for the runtime, never an address a kernel may use: ask the runtime once
// per device, with that device current.
float* xent_scratch_for_current_device() {
    int dev = -1;
    CUDA_CHECK(cudaGetDevice(&dev));
    CCL_THROW_IF_NOT(dev >= 0 && dev < XENT_MAX_DEVICES, "device index ", dev, " out of range");
    std::lock_guard<std::mutex> lk(xent_setup_mu);
    if (!xent_scratch_addr[dev]) {
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, xent_row_scratch);
        CCL_THROW_IF_NOT(e == cudaSuccess && p != nullptr, "cudaGetSymbolAddress(xent_row_scratch) failed: ",
                         cudaGetErrorString(e));
        xent_scratch_addr[dev] = p;
    }
    return xent_scratch_addr[dev];
}

} // namespace

CCLX_API int cclx_softmax_xent_mean_noalloc(void* logits_bf16, const long long* targets, float* mean_loss, size_t rows,
                                            int vocab, size_t ld, float grad_scale, int pad_cols, void* stream) {
    return cclx::capi::guard([&] {
        CCL_THROW_IF_NOT(rows <= (size_t)CCLX_XENT_NOALLOC_MAX_ROWS, "softmax_xent_mean_noalloc: ", rows,
                         " rows exceed the built-in scratch of ", CCLX_XENT_NOALLOC_MAX_ROWS,
                         " rows; split the batch or use cclx_softmax_xent with a caller-provided buffer");
        CCL_THROW_IF_NOT(logits_bf16 && targets && mean_loss, "softmax_xent_mean_noalloc: null pointer argument");
        CCL_THROW_IF_NOT(vocab > 0 && (size_t)(vocab + pad_cols) <= ld, "softmax_xent_mean_noalloc: bad row layout");
        if (rows == 0)
            return;
        float* scratch = xent_scratch_for_current_device();
        cudaStream_t st = (cudaStream_t)stream;
        launch_softmax_xent((__nv_bfloat16*)logits_bf16, targets, scratch, rows, vocab, ld, grad_scale, pad_cols, st);
        mean_rows_kernel<<<1, 1024, 0, st>>>(scratch, rows, mean_loss);
        CUDA_CHECK(cudaGetLastError());
    });
}
