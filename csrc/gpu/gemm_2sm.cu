// bf16 GEMM on CTA pairs: C[M,N] = A[M,K] * B[N,K]^T with tcgen05.mma.cta_group::2.
//
// Two CTAs of a cluster share one 256 x 256 output tile.  Each stages its own 128 rows of A and its
// own 128-row half of the B tile (32 KB per 64-deep K step instead of the 48 KB a single CTA needs
// for 128 x 256), which is what the L2 -> shared-memory path can sustain at full tensor rate.  The
// even CTA issues the MMAs for both; each CTA's tensor memory holds its 128 accumulator rows and its
// own epilogue warps drain them.  Tiles are visited in column groups of 8 so that the clusters of
// one wave work on a near-square patch of C and re-use A and B from the L2.
//
// Roles per CTA (192 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only), warps 2-5
// epilogue (TMEM -> registers -> bf16 -> padded shared-memory transpose -> coalesced stores).
// Every mbarrier wait is bounded; the cluster barriers at start and end are reached on every path.
// The reference library has no GEMM: this kernel serves the tensor-parallel and expert-parallel layers.
#include <algorithm>
#include <cstring>

#include "core/env.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"
#include "gpu/fused_gemm.cuh"
#include "gpu/fused_gemm.hpp"

namespace cclx {
namespace gpu {

constexpr int G2_STAGES = 6;
constexpr int G2_BN = 256; // tile columns
constexpr int G2_HALF = 128; // rows of A and rows of B staged per CTA
constexpr int G2_STAGE_A = G2_HALF * GEMM_BK * 2;
constexpr int G2_STAGE_B = G2_HALF * GEMM_BK * 2;
constexpr int G2_RING = G2_STAGES * (G2_STAGE_A + G2_STAGE_B);
constexpr int G2_EPI = 4 * 32 * GEMM_EPI_ROW_BYTES;
constexpr int G2_SMEM = 1024 + G2_RING + G2_EPI + 256;
constexpr int G2_GROUP_N = 8; // tile columns per raster group

struct gemm2_params {
    CUtensorMap tmA; // [M,K], box 64 x 128
    CUtensorMap tmB; // [N,K], box 64 x 128
    __nv_bfloat16* C;
    uint32_t* err;
    int M, N, K, epilogue;
    unsigned long long timeout_ns;
    const int* rows; // optional device word: only the first min(M, *rows) rows of A are multiplied
};

namespace {

__device__ __forceinline__ void g2_fail(const gemm2_params& P, volatile int* abort_flag, uint32_t code, uint32_t detail) {
    *abort_flag = 1;
    if (P.err && P.err[0] == GE_OK) {
        P.err[1] = blockIdx.x;
        P.err[2] = detail;
        __threadfence();
        P.err[0] = code;
    }
}

// tile index -> (row block of 256, column block of 256), column groups of G2_GROUP_N
__device__ __forceinline__ void g2_tile(int t, int tiles_m, int tiles_n, int& mi, int& ni) {
    const int per_group = G2_GROUP_N * tiles_m;
    const int grp = t / per_group, in = t % per_group;
    const int width = min(G2_GROUP_N, tiles_n - grp * G2_GROUP_N);
    mi = in / width;
    ni = grp * G2_GROUP_N + in % width;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    gemm2sm_kernel(const __grid_constant__ gemm2_params P) {
    using namespace sm100;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + G2_STAGES * G2_STAGE_A;
    uint8_t* sEpi = smem + G2_RING;
    uint64_t* bars = (uint64_t*)(smem + G2_RING + G2_EPI);
    uint64_t* full = bars; // [STAGES]  used in the leader: bytes of both CTAs
    uint64_t* empty = bars + G2_STAGES; // [STAGES]  per CTA, signalled by the MMA commit
    uint64_t* tfull = bars + 2 * G2_STAGES; // [2] per CTA
    uint64_t* tempty = bars + 2 * G2_STAGES + 2; // [2] used in the leader: 4 warps x 2 CTAs
    uint32_t* tmem_holder = (uint32_t*)(bars + 2 * G2_STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cr = cluster_ctarank(); // 0 = leader
    const bool leader = cr == 0;
    const int n_clusters = gridDim.x >> 1, cluster = blockIdx.x >> 1;
    // the row count may live on the device (rows that a kernel in front of this one delivered): every thread
    // reads the same word, so all roles walk the same tiles
    const int M = P.rows ? max(0, min(P.M, *P.rows)) : P.M;
    const int tiles_m = (M + 255) / 256, tiles_n = (P.N + G2_BN - 1) / G2_BN;
    const int total_tiles = tiles_m * tiles_n;
    const int KB = (P.K + GEMM_BK - 1) / GEMM_BK;
    const unsigned long long limit = P.timeout_ns;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < G2_STAGES; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], 8);
        }
        mbar_fence_init();
        tma_prefetch_desc(&P.tmA);
        tma_prefetch_desc(&P.tmB);
    }
    if (warp == 2) {
        tmem_alloc_2sm(tmem_holder, 512);
        tc_fence_before_sync();
    }
    __syncthreads();
    cluster_sync_all(); // the peer's barriers exist before anything is signalled across the pair
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int t = cluster; t < total_tiles && !*abort_flag; t += n_clusters) {
                int mi, ni;
                g2_tile(t, tiles_m, tiles_n, mi, ni);
                for (int kb = 0; kb < KB; kb++, it++) {
                    const uint32_t st = it % G2_STAGES, ph = (it / G2_STAGES) & 1;
                    if (!mbar_wait(&empty[st], ph ^ 1, abort_flag, limit)) {
                        g2_fail(P, abort_flag, GE_MBAR_TIMEOUT, 2);
                        break;
                    }
                    if (leader)
                        mbar_expect_tx(&full[st], 2 * (G2_STAGE_A + G2_STAGE_B));
                    tma_load_2d_2sm(sA + st * G2_STAGE_A, &P.tmA, kb * GEMM_BK, mi * 256 + (int)cr * G2_HALF, &full[st]);
                    tma_load_2d_2sm(sB + st * G2_STAGE_B, &P.tmB, kb * GEMM_BK, ni * G2_BN + (int)cr * G2_HALF,
                                    &full[st]);
                }
            }
            if (leader) { // copies of both CTAs still in flight must land before the pair may exit
                const uint32_t first = it > (uint32_t)G2_STAGES ? it - G2_STAGES : 0;
                for (uint32_t i = first; i < it; i++)
                    mbar_wait(&full[i % G2_STAGES], (i / G2_STAGES) & 1, abort_flag, limit);
            }
        }
        __syncwarp();
    }
    else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = make_idesc_bf16(256, G2_BN);
            uint32_t it = 0, tc = 0;
            for (int t = cluster; t < total_tiles && !*abort_flag; t += n_clusters, tc++) {
                const uint32_t acc = tc & 1, aph = (tc >> 1) & 1;
                if (!mbar_wait(&tempty[acc], aph ^ 1, abort_flag, limit)) {
                    g2_fail(P, abort_flag, GE_MBAR_TIMEOUT, 3);
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * G2_BN;
                bool bad = false;
                for (int kb = 0; kb < KB; kb++, it++) {
                    const uint32_t st = it % G2_STAGES, ph = (it / G2_STAGES) & 1;
                    if (!mbar_wait(&full[st], ph, abort_flag, limit)) {
                        g2_fail(P, abort_flag, GE_MBAR_TIMEOUT, 4);
                        bad = true;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(sA + st * G2_STAGE_A);
                    const uint32_t b_addr = smem_u32(sB + st * G2_STAGE_B);
#pragma unroll
                    for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; k++)
                        umma_bf16_2sm(d_tmem, make_smem_desc_sw128(a_addr + k * GEMM_UMMA_K * 2),
                                      make_smem_desc_sw128(b_addr + k * GEMM_UMMA_K * 2), idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit_2sm(&empty[st], 3); // both CTAs may refill the stage once these MMAs have read it
                }
                if (bad)
                    break;
                umma_commit_2sm(&tfull[acc], 3); // accumulator complete in both CTAs
            }
        }
        __syncwarp();
    }
    else {
        const int q = warp & 3; // TMEM lane quarter this warp may read
        uint8_t* stage = sEpi + (warp - 2) * 32 * GEMM_EPI_ROW_BYTES;
        const uint32_t tempty_leader = smem_u32(&tempty[0]) & PEER_BIT_MASK;
        uint32_t tc = 0;
        for (int t = cluster; t < total_tiles && !*abort_flag; t += n_clusters, tc++) {
            int mi, ni;
            g2_tile(t, tiles_m, tiles_n, mi, ni);
            const uint32_t acc = tc & 1, aph = (tc >> 1) & 1;
            if (!mbar_wait(&tfull[acc], aph, abort_flag, limit)) {
                if (lane == 0)
                    g2_fail(P, abort_flag, GE_MBAR_TIMEOUT, 5);
                break;
            }
            tc_fence_after_sync();
            const int row0 = mi * 256 + (int)cr * G2_HALF + q * 32;
#pragma unroll 1
            for (int c = 0; c < G2_BN / GEMM_EPI_COLS; c++) {
                uint32_t r0[32], r1[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * G2_BN + c * GEMM_EPI_COLS;
                tmem_ld_32x32(taddr, r0);
                tmem_ld_32x32(taddr + 32, r1);
                tmem_ld_wait();
                if (c == G2_BN / GEMM_EPI_COLS - 1) {
                    // all reads of this accumulator are done: hand it back to the leader's MMA warp
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive_cluster(tempty_leader + acc * 8);
                }
                uint32_t packed[32];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    float a0 = __uint_as_float(r0[2 * i]), a1 = __uint_as_float(r0[2 * i + 1]);
                    float b0 = __uint_as_float(r1[2 * i]), b1 = __uint_as_float(r1[2 * i + 1]);
                    if (P.epilogue == EPI_SILU) {
                        a0 = silu_f(a0);
                        a1 = silu_f(a1);
                        b0 = silu_f(b0);
                        b1 = silu_f(b1);
                    }
                    __nv_bfloat162 lo = __floats2bfloat162_rn(a0, a1);
                    __nv_bfloat162 hi = __floats2bfloat162_rn(b0, b1);
                    packed[i] = *reinterpret_cast<uint32_t*>(&lo);
                    packed[16 + i] = *reinterpret_cast<uint32_t*>(&hi);
                }
                uint8_t* myrow = stage + lane * GEMM_EPI_ROW_BYTES;
#pragma unroll
                for (int v = 0; v < 8; v++)
                    *reinterpret_cast<uint4*>(myrow + v * 16) =
                        make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
                __syncwarp();
                const int gcol = ni * G2_BN + c * GEMM_EPI_COLS + (lane & 7) * 8;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int rr = i * 4 + (lane >> 3);
                    const int grow = row0 + rr;
                    if (grow < M && gcol < P.N) {
                        uint4 v = *reinterpret_cast<const uint4*>(stage + rr * GEMM_EPI_ROW_BYTES + (lane & 7) * 16);
                        *reinterpret_cast<uint4*>(P.C + (size_t)grow * P.N + gcol) = v;
                    }
                }
                __syncwarp();
            }
        }
    }

    // converge: nobody leaves while the partner may still read its shared memory or signal its barriers
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc_2sm(tmem_base, 512);
    }
}

} // namespace

CUtensorMap make_bf16_kmajor_map(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

void gemm_bf16_2sm(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int clusters,
                   uint32_t* err, cudaStream_t st, const int* rows_dev) {
    CCL_THROW_IF_NOT(M > 0 && N > 0 && K > 0 && N % 8 == 0 && K % 8 == 0, "unsupported GEMM shape ", M, "x", N, "x", K);
    int dev_now = 0;
    CUDA_CHECK(cudaGetDevice(&dev_now));
    static bool attr_done[64] = {}; // the attribute is per device
    if (dev_now >= 64 || !attr_done[dev_now]) {
        CUDA_CHECK(cudaFuncSetAttribute(gemm2sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM));
        if (dev_now < 64)
            attr_done[dev_now] = true;
    }
    gemm2_params P;
    std::memset(&P, 0, sizeof(P));
    P.tmA = make_bf16_kmajor_map(A, M, K, G2_HALF);
    P.tmB = make_bf16_kmajor_map(B, N, K, G2_HALF);
    P.C = (__nv_bfloat16*)C;
    P.err = err;
    P.M = M;
    P.N = N;
    P.K = K;
    P.epilogue = epilogue;
    P.rows = rows_dev;
    P.timeout_ns = (unsigned long long)env_data::get().wait_timeout_ms * 1000000ull;
    int dev = 0, sms = 0;
    CUDA_CHECK(cudaGetDevice(&dev));
    CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int tiles = ((M + 255) / 256) * ((N + G2_BN - 1) / G2_BN);
    int nc = clusters > 0 ? clusters : sms / 2;
    nc = std::max(1, std::min(nc, tiles));
    // the cluster shape is a compile-time attribute of the kernel; the grid must be a multiple of it
    gemm2sm_kernel<<<dim3(2 * nc), GEMM_THREADS, G2_SMEM, st>>>(P);
    CUDA_CHECK(cudaGetLastError());
}

} // namespace gpu
} // namespace cclx
