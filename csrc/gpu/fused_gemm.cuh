// Persistent warp-specialised bf16 GEMM for sm_100a with the collective fused in:
//
//   GM_PLAIN : C[M,N] = A[M,K] * B[N,K]^T                      (local)
//   GM_AG    : all-gather(X over rows) -> GEMM: dedicated copy CTAs pull the
//              peers' row shards of X into this GPU's copy with bulk async
//              copies and publish one flag per 128-row block; the TMA producer
//              of a GEMM CTA waits for the block's flag before loading the A
//              tile, so math on early shards overlaps the transfer of late ones.
//   GM_RS    : GEMM -> reduce-scatter(over rows): the epilogue stores each
//              bf16 partial tile straight into the owning rank's slot (peer
//              stores), bumps a per-tile counter there, and after its GEMM
//              tiles every CTA reduces the tiles it owns (fp32 sum of `world`
//              partials) as soon as their counters are complete.
//              Ring form (rs_ring): every rank visits the owners in the order r+1, r+2, ..., r; the
//              epilogue adds the partial sum that rank r+1 produced for the same tile one step
//              earlier and passes the result on to rank r-1, so the last step writes the finished
//              rows and nothing is left to reduce after the GEMM.
//
// Mainloop: TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast) fills a
// 4-stage shared-memory ring; one elected thread issues tcgen05.mma
// (cta_group::1, M=128, N=BN, K=16) accumulating into TMEM; two TMEM
// accumulators let the epilogue of tile i overlap the mainloop of tile i+1.
// Epilogue: tcgen05.ld -> registers -> (SiLU) -> bf16 -> padded shared-memory
// transpose -> 128-byte coalesced global stores.
// Every wait (mbarrier, flag) is bounded; on a timeout the CTA records an error
// code, drains its own copies, frees its TMEM and returns.
//
// The reference has no counterpart kernel: it offers allgatherv / reduce_scatter
// (src/coll/algorithms/allgatherv/sycl/allgatherv_sycl.cpp:22-160,
// src/coll/algorithms/reduce_scatter/sycl/reduce_scatter_sycl.cpp:27-143) and
// leaves the GEMM to the user.
#pragma once
#include <cuda.h>

#include "gpu/device/common.cuh"
#include "gpu/device/sm100_ptx.cuh"

namespace cclx {
namespace gpu {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_UMMA_K = 16;
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_THREADS = 192; // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr int GEMM_EMU_MAX = 4;
constexpr int GEMM_EPI_COLS = 64; // columns per epilogue chunk
constexpr int GEMM_EPI_ROW_BYTES = GEMM_EPI_COLS * 2 + 16; // padded bf16 row in shared memory
constexpr int COPY_PIECE = 32768;
constexpr int COPY_NBUF = 6;
constexpr int COPY_AHEAD = 4;

enum { GM_PLAIN = 0, GM_AG = 1, GM_RS = 2 };
enum { EPI_NONE = 0, EPI_SILU = 1 };
enum { PLAN_SEQ = 0, PLAN_DONE = 1, PLAN_WORDS = 4 };
enum : uint32_t { GE_OK = 0, GE_MBAR_TIMEOUT = 101, GE_FLAG_TIMEOUT = 102, GE_BARRIER = 103 };

struct alignas(64) fused_rank {
    CUtensorMap tmA; // [M,K] bf16, box 64 x 128 (AG: over this rank's gathered copy of X)
    CUtensorMap tmB; // [N,K] bf16, box 64 x BN
    __nv_bfloat16* C; // PLAIN/AG: [M,N] output; RS: reduced [M/world, N] output
    uint32_t* plan_state; // PLAN_WORDS local words (call sequence, finished-CTA counter)
    uint32_t* err; // 4 local words: code, block, detail, detail
};

struct fused_params {
    fused_rank r[GEMM_EMU_MAX];
    int M, N, K;
    int mode, epilogue, emu, world;
    int n_comm; // GM_AG: number of copy CTAs (the last n_comm blocks of the grid)
    int rs_ring; // GM_RS: partial sums travel rank r -> r-1 inside the epilogue (no reduction pass at the end)
    size_t x_off; // GM_AG: heap offset of the gathered X [M,K]
    size_t part_off; // GM_RS: heap offset of the partial slots [world][M/world][N]
    uint32_t flag_off; // first auxiliary flag word of this plan
    unsigned long long timeout_ns;
};

template <int BN>
struct gemm_smem {
    static constexpr int A_STAGE = GEMM_BM * GEMM_BK * 2;
    static constexpr int B_STAGE = BN * GEMM_BK * 2;
    static constexpr int EPI_BYTES = 4 * 32 * GEMM_EPI_ROW_BYTES;
    static constexpr int RING = GEMM_STAGES * (A_STAGE + B_STAGE);
    static constexpr int COPY_RING = COPY_NBUF * COPY_PIECE;
    static constexpr int DATA = (RING + EPI_BYTES) > COPY_RING ? (RING + EPI_BYTES) : COPY_RING;
    static constexpr int TOTAL = 1024 /* alignment slack */ + DATA + 256 /* barriers */;
};

__device__ __forceinline__ float silu_f(float x) {
    return x / (1.0f + __expf(-x));
}

__device__ __forceinline__ void gemm_fail(const fused_rank& fr, volatile int* abort_flag, uint32_t code,
                                          uint32_t detail) {
    *abort_flag = 1;
    if (fr.err[0] == GE_OK) {
        fr.err[1] = blockIdx.x;
        fr.err[2] = detail;
        __threadfence();
        fr.err[0] = code;
    }
}

// wait until *flag >= target (wrap-safe); scope selects gpu / sys acquire
template <bool SYS>
__device__ __forceinline__ bool wait_word(const uint32_t* flag, uint32_t target, volatile int* abort_flag,
                                          unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0;; it++) {
        uint32_t v = SYS ? dev::ld_acquire_sys(flag) : dev::ld_acquire_gpu(flag);
        if ((int32_t)(v - target) >= 0)
            return true;
        if ((it & 0xff) == 0xff) {
            if (*abort_flag)
                return false;
            unsigned long long now = sm100::gtimer();
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > limit_ns)
                return false;
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    fused_gemm_kernel(const dev::comm_dev* tab, const __grid_constant__ fused_params P) {
    using namespace sm100;
    typedef gemm_smem<BN> L;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + GEMM_STAGES * L::A_STAGE;
    uint8_t* sEpi = smem + L::RING;
    uint64_t* bars = (uint64_t*)(smem + L::DATA);
    uint64_t* full = bars; // [STAGES]
    uint64_t* empty = bars + GEMM_STAGES; // [STAGES]
    uint64_t* tfull = bars + 2 * GEMM_STAGES; // [2]
    uint64_t* tempty = bars + 2 * GEMM_STAGES + 2; // [2]
    uint64_t* cbar = bars + 2 * GEMM_STAGES + 4; // [COPY_NBUF] copy CTAs only
    uint32_t* tmem_holder = (uint32_t*)(bars + 2 * GEMM_STAGES + 4 + COPY_NBUF);
    volatile int* abort_flag = (volatile int*)(tmem_holder + 1);

    const int er = P.emu ? (int)blockIdx.y : 0;
    const fused_rank& fr = P.r[er];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = P.world;
    const bool fused = P.mode != GM_PLAIN;
    const dev::comm_dev* cp = fused ? tab + er : nullptr;
    const int rank = fused ? cp->rank : 0;
    const int G = (int)gridDim.x - P.n_comm; // GEMM CTAs
    const bool is_copy_cta = (int)blockIdx.x >= G;
    const int tiles_m = (P.M + GEMM_BM - 1) / GEMM_BM;
    const int tiles_n = (P.N + BN - 1) / BN;
    const int total_tiles = tiles_m * tiles_n;
    const int tiles_m_per = fused ? tiles_m / W : tiles_m;
    const int KB = (P.K + GEMM_BK - 1) / GEMM_BK;
    const unsigned long long limit = P.timeout_ns;
    const uint32_t seq = fused ? dev::ld_volatile_u32(fr.plan_state + PLAN_SEQ) + 1 : 1;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < GEMM_STAGES; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], 4);
        }
        for (int i = 0; i < COPY_NBUF; i++)
            mbar_init(&cbar[i], 1);
        mbar_fence_init();
        tma_prefetch_desc(&fr.tmA);
        tma_prefetch_desc(&fr.tmB);
    }
    if (warp == 2 && !is_copy_cta) {
        tmem_alloc(tmem_holder, 512);
        tc_fence_before_sync();
    }
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = is_copy_cta ? 0u : *tmem_holder;

    // ------------------------------------------------------------------ copy CTAs (GM_AG)
    if (is_copy_cta) {
        dev::block_sync s;
        dev::sync_begin(*cp, s);
        // every peer has written its shard (stream order on its side) once it reaches this barrier
        bool ok = dev::peer_barrier(*cp, s);
        if (ok && threadIdx.x == 0) {
            const int cid = (int)blockIdx.x - G;
            const size_t chunk_bytes = (size_t)GEMM_BM * P.K * 2;
            const int n_remote = (W - 1) * tiles_m_per;
            uint32_t ld_cnt = 0, st_cnt = 0;
            uint8_t* ring = smem;
            for (int ci = cid; ci < n_remote && !*abort_flag; ci += P.n_comm) {
                const int src = (rank + 1 + ci / tiles_m_per) % W;
                const int mi = src * tiles_m_per + ci % tiles_m_per;
                const size_t off = P.x_off + (size_t)mi * chunk_bytes;
                const char* gsrc = cp->heap[src] + off;
                char* gdst = cp->heap[rank] + off;
                size_t rows_left = (size_t)P.M - (size_t)mi * GEMM_BM;
                const size_t bytes = (rows_left < (size_t)GEMM_BM ? rows_left : (size_t)GEMM_BM) * P.K * 2;
                const int np = (int)((bytes + COPY_PIECE - 1) / COPY_PIECE);
                for (int j = 0; j < np + COPY_AHEAD; j++) {
                    if (j < np) {
                        const uint32_t slot = ld_cnt % COPY_NBUF;
                        if (ld_cnt >= (uint32_t)COPY_NBUF)
                            bulk_wait_read<COPY_NBUF - 1 - COPY_AHEAD>();
                        const size_t o = (size_t)j * COPY_PIECE;
                        const uint32_t n = (uint32_t)((bytes - o) < (size_t)COPY_PIECE ? (bytes - o) : COPY_PIECE);
                        mbar_expect_tx(&cbar[slot], n);
                        bulk_g2s(ring + (size_t)slot * COPY_PIECE, gsrc + o, n, &cbar[slot]);
                        ld_cnt++;
                    }
                    const int k = j - COPY_AHEAD;
                    if (k >= 0) {
                        const uint32_t slot = st_cnt % COPY_NBUF;
                        if (!mbar_wait(&cbar[slot], (st_cnt / COPY_NBUF) & 1, abort_flag, limit)) {
                            gemm_fail(fr, abort_flag, GE_MBAR_TIMEOUT, 1);
                            break;
                        }
                        const size_t o = (size_t)k * COPY_PIECE;
                        const uint32_t n = (uint32_t)((bytes - o) < (size_t)COPY_PIECE ? (bytes - o) : COPY_PIECE);
                        bulk_s2g(gdst + o, ring + (size_t)slot * COPY_PIECE, n);
                        bulk_commit();
                        st_cnt++;
                    }
                }
                bulk_wait_all<0>();
                fence_proxy_async();
                __threadfence();
                dev::st_release_gpu(cp->aux[rank] + P.flag_off + mi, seq);
            }
            // loads that were issued but never consumed (abort path): wait for them to land
            while (st_cnt < ld_cnt) {
                mbar_wait(&cbar[st_cnt % COPY_NBUF], (st_cnt / COPY_NBUF) & 1, abort_flag, limit);
                st_cnt++;
            }
            bulk_wait_all<0>();
        }
        __syncthreads();
        // peers may overwrite their shard (next call) only after everybody has read it
        dev::peer_barrier(*cp, s);
        // epoch accounting for the barrier slots used by the copy CTAs
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            uint32_t done = atomicAdd(cp->state + dev::STATE_DONE, 1u);
            if (done == (uint32_t)P.n_comm - 1) {
                cp->state[dev::STATE_EPOCH] += 2;
                __threadfence();
                cp->state[dev::STATE_DONE] = 0;
            }
        }
    }
    else {
        // -------------------------------------------------------------- GEMM CTAs
        const int g = blockIdx.x;
        dev::block_sync s;
        if (P.mode == GM_RS) {
            // the owners' partial slots are free again once every rank entered this call
            dev::sync_begin(*cp, s);
            if (!dev::peer_barrier(*cp, s))
                gemm_fail(fr, abort_flag, GE_BARRIER, 0);
        }
        // tile order: AG starts with the local shard, RS ends with it
        const int m_rot = P.mode == GM_AG ? rank * tiles_m_per : (P.mode == GM_RS ? ((rank + 1) % W) * tiles_m_per : 0);

        if (warp == 0) {
            if (lane == 0) {
                uint32_t it = 0;
                for (int t = g; t < total_tiles && !*abort_flag; t += G) {
                    const int mi = (t / tiles_n + m_rot) % tiles_m;
                    const int ni = t % tiles_n;
                    if (P.mode == GM_AG && mi / tiles_m_per != rank) {
                        if (!wait_word<false>(cp->aux[rank] + P.flag_off + mi, seq, abort_flag, limit)) {
                            gemm_fail(fr, abort_flag, GE_FLAG_TIMEOUT, (uint32_t)mi);
                            break;
                        }
                        fence_proxy_async();
                    }
                    for (int kb = 0; kb < KB; kb++, it++) {
                        const uint32_t st = it % GEMM_STAGES, ph = (it / GEMM_STAGES) & 1;
                        if (!mbar_wait(&empty[st], ph ^ 1, abort_flag, limit)) {
                            gemm_fail(fr, abort_flag, GE_MBAR_TIMEOUT, 2);
                            break;
                        }
                        mbar_expect_tx(&full[st], L::A_STAGE + L::B_STAGE);
                        tma_load_2d(sA + st * L::A_STAGE, &fr.tmA, kb * GEMM_BK, mi * GEMM_BM, &full[st]);
                        tma_load_2d(sB + st * L::B_STAGE, &fr.tmB, kb * GEMM_BK, ni * BN, &full[st]);
                    }
                }
                // own copies still in flight must land before the CTA may exit
                const uint32_t first = it > (uint32_t)GEMM_STAGES ? it - GEMM_STAGES : 0;
                for (uint32_t i = first; i < it; i++)
                    mbar_wait(&full[i % GEMM_STAGES], (i / GEMM_STAGES) & 1, abort_flag, limit);
            }
            __syncwarp();
        }
        else if (warp == 1) {
            if (lane == 0) {
                constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN);
                uint32_t it = 0, tc = 0;
                for (int t = g; t < total_tiles && !*abort_flag; t += G, tc++) {
                    const uint32_t acc = tc & 1, aph = (tc >> 1) & 1;
                    if (!mbar_wait(&tempty[acc], aph ^ 1, abort_flag, limit)) {
                        gemm_fail(fr, abort_flag, GE_MBAR_TIMEOUT, 3);
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    bool bad = false;
                    for (int kb = 0; kb < KB; kb++, it++) {
                        const uint32_t st = it % GEMM_STAGES, ph = (it / GEMM_STAGES) & 1;
                        if (!mbar_wait(&full[st], ph, abort_flag, limit)) {
                            gemm_fail(fr, abort_flag, GE_MBAR_TIMEOUT, 4);
                            bad = true;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t a_addr = smem_u32(sA + st * L::A_STAGE);
                        const uint32_t b_addr = smem_u32(sB + st * L::B_STAGE);
#pragma unroll
                        for (int k = 0; k < GEMM_BK / GEMM_UMMA_K; k++) {
                            umma_bf16(d_tmem, make_smem_desc_sw128(a_addr + k * GEMM_UMMA_K * 2),
                                      make_smem_desc_sw128(b_addr + k * GEMM_UMMA_K * 2), idesc,
                                      (kb | k) != 0 ? 1u : 0u);
                        }
                        umma_commit(&empty[st]); // the stage is free once these MMAs have read it
                    }
                    if (bad)
                        break;
                    umma_commit(&tfull[acc]); // accumulator complete
                }
            }
            __syncwarp();
        }
        else {
            const int q = warp & 3; // TMEM lane quarter this warp may read
            uint8_t* stage = sEpi + (warp - 2) * 32 * GEMM_EPI_ROW_BYTES;
            uint32_t tc = 0;
            const int M_per = P.M / W;
            for (int t = g; t < total_tiles && !*abort_flag; t += G, tc++) {
                const int mi = (t / tiles_n + m_rot) % tiles_m;
                const int ni = t % tiles_n;
                const uint32_t acc = tc & 1, aph = (tc >> 1) & 1;
                if (!mbar_wait(&tfull[acc], aph, abort_flag, limit)) {
                    if (lane == 0)
                        gemm_fail(fr, abort_flag, GE_MBAR_TIMEOUT, 5);
                    break;
                }
                tc_fence_after_sync();
                // destination of this tile
                __nv_bfloat16* cbase;
                size_t ldc = (size_t)P.N;
                int row0 = mi * GEMM_BM + q * 32; // first row handled by this warp
                int row_limit = P.M;
                int owner = 0, mb_local = 0;
                const __nv_bfloat16* incoming = nullptr; // ring: partial sum of the previous rank for this tile
                bool ring_final = false;
                if (P.mode == GM_RS) {
                    owner = mi / tiles_m_per;
                    mb_local = mi % tiles_m_per;
                    row0 = mb_local * GEMM_BM + q * 32;
                    row_limit = M_per;
                    if (P.rs_ring) {
                        const int step = (owner - rank - 1 + W) % W; // 0 .. W-1, my own rows come last
                        const size_t slot = (size_t)owner * M_per * P.N; // inbox region of this owner's rows
                        if (step > 0) {
                            const uint32_t* f = cp->aux[rank] + P.flag_off + ((size_t)owner * tiles_m_per + mb_local) * tiles_n + ni;
                            bool got = true;
                            if (lane == 0)
                                got = wait_word<true>(f, seq * 4u, abort_flag, limit);
                            got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
                            if (!got) {
                                if (lane == 0)
                                    gemm_fail(fr, abort_flag, GE_FLAG_TIMEOUT, (uint32_t)mi);
                                break;
                            }
                            incoming = (const __nv_bfloat16*)(cp->heap[rank] + P.part_off) + slot;
                        }
                        ring_final = step == W - 1;
                        if (ring_final)
                            cbase = fr.C;
                        else
                            cbase = (__nv_bfloat16*)(cp->heap[(rank + W - 1) % W] + P.part_off) + slot;
                    }
                    else
                        cbase = (__nv_bfloat16*)(cp->heap[owner] + P.part_off) + (size_t)rank * M_per * P.N;
                }
                else
                    cbase = fr.C;
#pragma unroll 1
                for (int c = 0; c < BN / GEMM_EPI_COLS; c++) {
                    uint32_t r0[32], r1[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c * GEMM_EPI_COLS;
                    tmem_ld_32x32(taddr, r0);
                    tmem_ld_32x32(taddr + 32, r1);
                    tmem_ld_wait();
                    if (c == BN / GEMM_EPI_COLS - 1) {
                        // all TMEM reads of this accumulator are done: hand it back to the MMA warp
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0)
                            mbar_arrive(&tempty[acc]);
                    }
                    if (incoming) {
                        // my row of the incoming partial tile: 64 bf16 = eight 16-byte loads
                        const int irow = row0 + lane;
                        const int icol = ni * BN + c * GEMM_EPI_COLS;
                        const __nv_bfloat16* src = incoming + (size_t)irow * P.N + icol;
                        uint4 inc[8];
#pragma unroll
                        for (int v = 0; v < 8; v++)
                            inc[v] = (irow < row_limit && icol + v * 8 < P.N) ? dev::ld_cv16(src + v * 8) : make_uint4(0, 0, 0, 0);
#pragma unroll
                        for (int v = 0; v < 4; v++) {
                            const __nv_bfloat16* h0 = reinterpret_cast<const __nv_bfloat16*>(&inc[v]);
                            const __nv_bfloat16* h1 = reinterpret_cast<const __nv_bfloat16*>(&inc[4 + v]);
#pragma unroll
                            for (int e = 0; e < 8; e++) {
                                r0[v * 8 + e] = __float_as_uint(__uint_as_float(r0[v * 8 + e]) + __bfloat162float(h0[e]));
                                r1[v * 8 + e] = __float_as_uint(__uint_as_float(r1[v * 8 + e]) + __bfloat162float(h1[e]));
                            }
                        }
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
                    const int gcol = ni * BN + c * GEMM_EPI_COLS + (lane & 7) * 8;
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int rr = i * 4 + (lane >> 3);
                        const int grow = row0 + rr;
                        if (grow < row_limit && gcol < P.N) {
                            uint4 v = *reinterpret_cast<const uint4*>(stage + rr * GEMM_EPI_ROW_BYTES + (lane & 7) * 16);
                            *reinterpret_cast<uint4*>(cbase + (size_t)grow * ldc + gcol) = v;
                        }
                    }
                    __syncwarp();
                }
                if (P.mode == GM_RS && !(P.rs_ring && ring_final)) {
                    // publish: this warp's quarter of the tile has landed (ring: at the next rank down, in
                    // the inbox region of the tile's owner; otherwise at the owner, in my slot)
                    __syncwarp();
                    if (lane == 0) {
                        if (P.rs_ring)
                            dev::red_release_sys_add(cp->aux[(rank + W - 1) % W] + P.flag_off +
                                                         ((size_t)owner * tiles_m_per + mb_local) * tiles_n + ni,
                                                     1u);
                        else
                            dev::red_release_sys_add(
                                cp->aux[owner] + P.flag_off + ((size_t)rank * tiles_m_per + mb_local) * tiles_n + ni, 1u);
                    }
                }
            }
        }

        // ---------------------------------------------------------- converge, free TMEM
        tc_fence_before_sync();
        __syncthreads();
        if (warp == 2) {
            tc_fence_after_sync();
            tmem_dealloc(tmem_base, 512);
        }

        // ---------------------------------------------------------- GM_RS: reduce the tiles I own
        if (P.mode == GM_RS) {
            const int M_per = P.M / W;
            const __nv_bfloat16* part = (const __nv_bfloat16*)(cp->heap[rank] + P.part_off);
            const int items = P.rs_ring ? 0 : tiles_m_per * tiles_n; // ring: the last step wrote the result
            __shared__ int item_fail;
            for (int item = g; item < items; item += G) {
                const int mb = item / tiles_n, ni = item % tiles_n;
                if (threadIdx.x == 0)
                    item_fail = 0;
                __syncthreads();
                if ((int)threadIdx.x < W) {
                    const uint32_t* f =
                        cp->aux[rank] + P.flag_off + ((size_t)threadIdx.x * tiles_m_per + mb) * tiles_n + ni;
                    if (*abort_flag || !wait_word<true>(f, seq * 4u, abort_flag, limit)) {
                        gemm_fail(fr, abort_flag, GE_FLAG_TIMEOUT, (uint32_t)item);
                        item_fail = 1;
                    }
                }
                __syncthreads();
                if (item_fail)
                    break;
                constexpr int PPR = BN / 8; // 16-byte packs per tile row
                for (int p = threadIdx.x; p < GEMM_BM * PPR; p += GEMM_THREADS) {
                    const int rl = mb * GEMM_BM + p / PPR;
                    const int col = ni * BN + (p % PPR) * 8;
                    if (rl >= M_per || col >= P.N)
                        continue;
                    float acc[8];
#pragma unroll
                    for (int k = 0; k < 8; k++)
                        acc[k] = 0.f;
                    for (int src = 0; src < W; src++) {
                        uint4 v = dev::ld_cv16(part + ((size_t)src * M_per + rl) * P.N + col);
                        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
                        for (int k = 0; k < 8; k++)
                            acc[k] += __bfloat162float(h[k]);
                    }
                    uint4 o;
                    __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(&o);
#pragma unroll
                    for (int k = 0; k < 8; k++)
                        oh[k] = __float2bfloat16_rn(acc[k]);
                    *reinterpret_cast<uint4*>(fr.C + (size_t)rl * P.N + col) = o;
                }
            }
            // barrier-slot epoch accounting (one peer_barrier per GEMM CTA)
            __syncthreads();
            if (threadIdx.x == 0) {
                __threadfence();
                uint32_t done = atomicAdd(cp->state + dev::STATE_DONE, 1u);
                if (done == (uint32_t)G - 1) {
                    cp->state[dev::STATE_EPOCH] += 1;
                    __threadfence();
                    cp->state[dev::STATE_DONE] = 0;
                }
            }
        }
    }

    // ---------------------------------------------------------------- plan sequence number
    if (fused) {
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            uint32_t done = atomicAdd(fr.plan_state + PLAN_DONE, 1u);
            if (done == gridDim.x - 1) {
                fr.plan_state[PLAN_SEQ] += 1;
                __threadfence();
                fr.plan_state[PLAN_DONE] = 0;
            }
        }
    }
}

} // namespace gpu
} // namespace cclx
