// Host interface of the fused GEMM + collective kernels (see fused_gemm.cuh).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace cclx {
namespace gpu {

class device_comm;

// C[M,N] = act(A[M,K] * B[N,K]^T), bf16 in/out, fp32 accumulate, single GPU.
// `err` points at 4 zero-initialised device words that receive an error code.
void gemm_bf16_plain(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int ctas,
                     uint32_t* err, cudaStream_t st);

// the same product on CTA pairs (tcgen05.mma.cta_group::2, 256 x 256 tiles); `clusters` 0 = one pair per two SMs
void gemm_bf16_2sm(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int clusters,
                   uint32_t* err, cudaStream_t st, const int* rows_dev = nullptr);

struct fused_plan; // opaque

// mode 1: all-gather(X rows) -> GEMM.  M = total rows (world * rows per rank).
// mode 2: GEMM -> reduce-scatter over rows.  Output rows per rank = M / world.
// Collective in real mode: allocates symmetric buffers and flag words.
fused_plan* fused_plan_create(device_comm& dc, int mode, int M, int N, int K, int epilogue, int n_comm, int ctas);
void fused_plan_destroy(fused_plan* p);
// mode 1: pointer to the [M/world, K] slot of (emulated) rank r where that rank writes its shard of X
void* fused_plan_x_shard(fused_plan* p, int r);
// mode 1: the whole gathered X [M,K] of rank r (valid after a run)
void* fused_plan_x_full(fused_plan* p, int r);
// arrays have one entry in real mode and world entries in emulation mode.
// mode 1: A ignored (X comes from the shards), B = weights [N,K], C = [M,N]
// mode 2: A = [M,K] local activations, B = weights [N,K], C = [M/world, N] reduced output
void fused_plan_run(fused_plan* p, const void* const* A, const void* const* B, void* const* C, cudaStream_t st);
// error words of (emulated) rank r: 0 = ok
uint32_t fused_plan_error(fused_plan* p, int r);

} // namespace gpu
} // namespace cclx
