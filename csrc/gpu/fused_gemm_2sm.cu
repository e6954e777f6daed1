// All-gather -> GEMM and GEMM -> reduce-scatter on CTA pairs (tcgen05.mma.cta_group::2).
//
// The collective side is the one of fused_gemm.cuh (copy CTAs that pull the peers' row shards with bulk
// copies and publish a flag per 128-row block; epilogues that store partial tiles into the owning rank's
// memory and count them in; the ring form that adds the neighbour's partial sum on the way), the main loop is
// the one of gemm_2sm.cu: two CTAs of a cluster share a 256 x 256 tile, each stages its own 128 rows of A and
// its own 128-row half of the B tile (32 KB per K step and CTA instead of 48 KB), the even CTA issues the MMAs
// for both, each CTA drains its own 128 accumulator rows.  Every unit of the collective protocol is a 128-row
// block, which is exactly what one CTA of a pair owns, so flags, slots and counters keep their layout.
//
// Loads are per CTA and never multicast (tma_load_2d_2sm addresses the leader's barrier, not the peer's shared
// memory); peer GPUs are touched by plain loads / stores and non-multicast bulk copies only.
// Tiles are visited shard by shard (all-gather: the local shard first; reduce-scatter: the local rows last) and
// in column groups of 8 inside a shard, so that the clusters of one wave share A and B tiles in the L2.
#include <algorithm>
#include <cstring>

#include "core/env.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"
#include "gpu/fused_gemm.cuh"
#include "gpu/fused_gemm.hpp"

namespace cclx {
namespace gpu {

constexpr int F2_STAGES = 6;
constexpr int F2_BN = 256;
constexpr int F2_HALF = 128;
constexpr int F2_STAGE_A = F2_HALF * GEMM_BK * 2;
constexpr int F2_STAGE_B = F2_HALF * GEMM_BK * 2;
constexpr int F2_RING = F2_STAGES * (F2_STAGE_A + F2_STAGE_B);
constexpr int F2_EPI = 4 * 32 * GEMM_EPI_ROW_BYTES;
constexpr int F2_DATA = F2_RING + F2_EPI; // the copy CTAs lay their ring of COPY_NBUF pieces over it
constexpr int F2_SMEM = 1024 + F2_DATA + 256;
constexpr int F2_GROUP_N = 8;
static_assert(COPY_NBUF * COPY_PIECE <= F2_DATA, "copy ring must fit the GEMM CTA's shared memory");

namespace {

// tile t of a shard of tiles_m x tiles_n tiles -> (row, column), column groups of F2_GROUP_N
__device__ __forceinline__ void f2_tile(int t, int tiles_m, int tiles_n, int& mi, int& ni) {
    const int per_group = F2_GROUP_N * tiles_m;
    const int grp = t / per_group, in = t % per_group;
    const int width = min(F2_GROUP_N, tiles_n - grp * F2_GROUP_N);
    mi = in / width;
    ni = grp * F2_GROUP_N + in % width;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    fused_gemm2_kernel(const dev::comm_dev* tab, const __grid_constant__ fused_params P) {
    using namespace sm100;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = smem + F2_STAGES * F2_STAGE_A;
    uint8_t* sEpi = smem + F2_RING;
    uint64_t* bars = (uint64_t*)(smem + F2_DATA);
    uint64_t* full = bars; // [STAGES]  used in the leader: bytes of both CTAs
    uint64_t* empty = bars + F2_STAGES; // [STAGES]  per CTA, signalled by the MMA commit
    uint64_t* tfull = bars + 2 * F2_STAGES; // [2] per CTA
    uint64_t* tempty = bars + 2 * F2_STAGES + 2; // [2] used in the leader: 4 warps x 2 CTAs
    uint64_t* cbar = bars + 2 * F2_STAGES + 4; // [COPY_NBUF] copy CTAs only
    uint32_t* tmem_holder = (uint32_t*)(bars + 2 * F2_STAGES + 4 + COPY_NBUF);
    volatile int* abort_flag = (volatile int*)(tmem_holder + 1);

    const int er = P.emu ? (int)blockIdx.y : 0;
    const fused_rank& fr = P.r[er];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = P.world;
    const dev::comm_dev* cp = tab + er;
    const int rank = cp->rank;
    const int G = (int)gridDim.x - P.n_comm; // GEMM CTAs (even), the copy CTAs follow (even)
    const bool is_copy_cta = (int)blockIdx.x >= G;
    const uint32_t cr = cluster_ctarank(); // 0 = leader of the pair
    const bool leader = cr == 0;
    const int n_clusters = G >> 1, cluster = blockIdx.x >> 1;
    const int tiles_m = P.M / 256, tiles_n = (P.N + F2_BN - 1) / F2_BN; // 256-row tiles
    const int tiles_m_per = tiles_m / W; // 256-row tiles per shard
    const int blocks_per = 2 * tiles_m_per; // 128-row blocks per shard: the unit of the collective protocol
    const int per_shard = tiles_m_per * tiles_n;
    const int total_tiles = tiles_m * tiles_n;
    const int KB = (P.K + GEMM_BK - 1) / GEMM_BK;
    const unsigned long long limit = P.timeout_ns;
    const uint32_t seq = dev::ld_volatile_u32(fr.plan_state + PLAN_SEQ) + 1;
    // shard order: all-gather starts with the local shard, reduce-scatter ends with the local rows
    const int rot = P.mode == GM_AG ? rank : (rank + 1) % W;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int i = 0; i < F2_STAGES; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&tfull[i], 1);
            mbar_init(&tempty[i], 8);
        }
        for (int i = 0; i < COPY_NBUF; i++)
            mbar_init(&cbar[i], 1);
        mbar_fence_init();
        tma_prefetch_desc(&fr.tmA);
        tma_prefetch_desc(&fr.tmB);
    }
    if (warp == 2 && !is_copy_cta) {
        tmem_alloc_2sm(tmem_holder, 512);
        tc_fence_before_sync();
    }
    __syncthreads();
    uint32_t tmem_base = 0;
    if (!is_copy_cta) {
        cluster_sync_all(); // the partner's barriers exist before anything is signalled across the pair
        tc_fence_after_sync();
        tmem_base = *tmem_holder;
    }

    // ------------------------------------------------------------------ copy CTAs (GM_AG)
    if (is_copy_cta) {
        dev::block_sync s;
        dev::sync_begin(*cp, s);
        // every peer has written its shard (stream order on its side) once it reaches this barrier
        bool ok = dev::peer_barrier(*cp, s);
        if (ok && threadIdx.x == 0) {
            const int cid = (int)blockIdx.x - G;
            const size_t chunk_bytes = (size_t)GEMM_BM * P.K * 2;
            const int n_remote = (W - 1) * blocks_per;
            uint32_t ld_cnt = 0, st_cnt = 0;
            uint8_t* ring = smem;
            for (int ci = cid; ci < n_remote && !*abort_flag; ci += P.n_comm) {
                const int src = (rank + 1 + ci / blocks_per) % W;
                const int mb = src * blocks_per + ci % blocks_per;
                const size_t off = P.x_off + (size_t)mb * chunk_bytes;
                const char* gsrc = cp->heap[src] + off;
                char* gdst = cp->heap[rank] + off;
                const size_t bytes = chunk_bytes;
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
                dev::st_release_gpu(cp->aux[rank] + P.flag_off + mb, seq);
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
        __syncthreads();
        if (threadIdx.x == 0) { // epoch accounting for the barrier slots used by the copy CTAs
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
        // -------------------------------------------------------------- GEMM CTA pairs
        const int g = blockIdx.x;
        dev::block_sync s;
        if (P.mode == GM_RS) {
            // the owners' partial slots are free again once every rank entered this call
            dev::sync_begin(*cp, s);
            if (!dev::peer_barrier(*cp, s))
                gemm_fail(fr, abort_flag, GE_BARRIER, 0);
        }
        // tile t of this cluster -> 256-row tile index and column tile
        auto locate = [&](int t, int& mi, int& ni) {
            const int sh = (t / per_shard + rot) % W;
            int ml;
            f2_tile(t % per_shard, tiles_m_per, tiles_n, ml, ni);
            mi = sh * tiles_m_per + ml;
        };

        if (warp == 0) {
            if (lane == 0) {
                uint32_t it = 0;
                for (int t = cluster; t < total_tiles && !*abort_flag; t += n_clusters) {
                    int mi, ni;
                    locate(t, mi, ni);
                    const int mb = mi * 2 + (int)cr; // my 128-row block of the tile
                    if (P.mode == GM_AG && mb / blocks_per != rank) {
                        if (!wait_word<false>(cp->aux[rank] + P.flag_off + mb, seq, abort_flag, limit)) {
                            gemm_fail(fr, abort_flag, GE_FLAG_TIMEOUT, (uint32_t)mb);
                            break;
                        }
                        fence_proxy_async();
                    }
                    for (int kb = 0; kb < KB; kb++, it++) {
                        const uint32_t st = it % F2_STAGES, ph = (it / F2_STAGES) & 1;
                        if (!mbar_wait(&empty[st], ph ^ 1, abort_flag, limit)) {
                            gemm_fail(fr, abort_flag, GE_MBAR_TIMEOUT, 2);
                            break;
                        }
                        if (leader)
                            mbar_expect_tx(&full[st], 2 * (F2_STAGE_A + F2_STAGE_B));
                        tma_load_2d_2sm(sA + st * F2_STAGE_A, &fr.tmA, kb * GEMM_BK, mb * F2_HALF, &full[st]);
                        tma_load_2d_2sm(sB + st * F2_STAGE_B, &fr.tmB, kb * GEMM_BK, ni * F2_BN + (int)cr * F2_HALF,
                                        &full[st]);
                    }
                }
                if (leader) { // copies of both CTAs still in flight must land before the pair may exit
                    const uint32_t first = it > (uint32_t)F2_STAGES ? it - F2_STAGES : 0;
                    for (uint32_t i = first; i < it; i++)
                        mbar_wait(&full[i % F2_STAGES], (i / F2_STAGES) & 1, abort_flag, limit);
                }
            }
            __syncwarp();
        }
        else if (warp == 1) {
            if (lane == 0 && leader) {
                constexpr uint32_t idesc = make_idesc_bf16(256, F2_BN);
                uint32_t it = 0, tc = 0;
                for (int t = cluster; t < total_tiles && !*abort_flag; t += n_clusters, tc++) {
                    const uint32_t acc = tc & 1, aph = (tc >> 1) & 1;
                    if (!mbar_wait(&tempty[acc], aph ^ 1, abort_flag, limit)) {
                        gemm_fail(fr, abort_flag, GE_MBAR_TIMEOUT, 3);
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + acc * F2_BN;
                    bool bad = false;
                    for (int kb = 0; kb < KB; kb++, it++) {
                        const uint32_t st = it % F2_STAGES, ph = (it / F2_STAGES) & 1;
                        if (!mbar_wait(&full[st], ph, abort_flag, limit)) {
                            gemm_fail(fr, abort_flag, GE_MBAR_TIMEOUT, 4);
                            bad = true;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t a_addr = smem_u32(sA + st * F2_STAGE_A);
                        const uint32_t b_addr = smem_u32(sB + st * F2_STAGE_B);
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
            const int M_per = P.M / W;
            uint32_t tc = 0;
            for (int t = cluster; t < total_tiles && !*abort_flag; t += n_clusters, tc++) {
                int mi, ni;
                locate(t, mi, ni);
                const int mb = mi * 2 + (int)cr;
                const uint32_t acc = tc & 1, aph = (tc >> 1) & 1;
                if (!mbar_wait(&tfull[acc], aph, abort_flag, limit)) {
                    if (lane == 0)
                        gemm_fail(fr, abort_flag, GE_MBAR_TIMEOUT, 5);
                    break;
                }
                tc_fence_after_sync();
                // destination of my 128 rows of this tile
                __nv_bfloat16* cbase = fr.C;
                const size_t ldc = (size_t)P.N;
                int row0 = mb * F2_HALF + q * 32; // first row handled by this warp
                int row_limit = P.M;
                int owner = 0, mb_local = 0;
                const __nv_bfloat16* incoming = nullptr; // ring: partial sum of the previous rank for this block
                bool ring_final = false;
                bool lost = false;
                if (P.mode == GM_RS) {
                    owner = mb / blocks_per;
                    mb_local = mb % blocks_per;
                    row0 = mb_local * F2_HALF + q * 32;
                    row_limit = M_per;
                    if (P.rs_ring) {
                        const int step = (owner - rank - 1 + W) % W; // 0 .. W-1, my own rows come last
                        const size_t slot = (size_t)owner * M_per * P.N; // inbox region of this owner's rows
                        if (step > 0) {
                            const uint32_t* f =
                                cp->aux[rank] + P.flag_off + ((size_t)owner * blocks_per + mb_local) * tiles_n + ni;
                            bool got = true;
                            if (lane == 0)
                                got = wait_word<true>(f, seq * 4u, abort_flag, limit);
                            got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
                            if (!got) {
                                if (lane == 0)
                                    gemm_fail(fr, abort_flag, GE_FLAG_TIMEOUT, (uint32_t)mb);
                                lost = true;
                            }
                            incoming = (const __nv_bfloat16*)(cp->heap[rank] + P.part_off) + slot;
                        }
                        ring_final = step == W - 1;
                        if (!ring_final)
                            cbase = (__nv_bfloat16*)(cp->heap[(rank + W - 1) % W] + P.part_off) + slot;
                    }
                    else
                        cbase = (__nv_bfloat16*)(cp->heap[owner] + P.part_off) + (size_t)rank * M_per * P.N;
                }
#pragma unroll 1
                for (int c = 0; c < F2_BN / GEMM_EPI_COLS; c++) {
                    uint32_t r0[32], r1[32];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * F2_BN + c * GEMM_EPI_COLS;
                    tmem_ld_32x32(taddr, r0);
                    tmem_ld_32x32(taddr + 32, r1);
                    tmem_ld_wait();
                    if (c == F2_BN / GEMM_EPI_COLS - 1) {
                        // all reads of this accumulator are done: hand it back to the leader's MMA warp (also on the
                        // failure path, so that the pair winds down instead of waiting for this warp)
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0)
                            mbar_arrive_cluster(tempty_leader + acc * 8);
                    }
                    if (lost)
                        continue;
                    if (incoming) {
                        // my row of the incoming partial tile: 64 bf16 = eight 16-byte loads
                        const int irow = row0 + lane;
                        const int icol = ni * F2_BN + c * GEMM_EPI_COLS;
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
                    const int gcol = ni * F2_BN + c * GEMM_EPI_COLS + (lane & 7) * 8;
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
                if (lost)
                    break;
                if (P.mode == GM_RS && !(P.rs_ring && ring_final)) {
                    // publish: this warp's quarter of the block has landed (ring: at the next rank down, in the
                    // inbox region of the block's owner; otherwise at the owner, in my slot)
                    __syncwarp();
                    if (lane == 0) {
                        if (P.rs_ring)
                            dev::red_release_sys_add(cp->aux[(rank + W - 1) % W] + P.flag_off +
                                                         ((size_t)owner * blocks_per + mb_local) * tiles_n + ni,
                                                     1u);
                        else
                            dev::red_release_sys_add(
                                cp->aux[owner] + P.flag_off + ((size_t)rank * blocks_per + mb_local) * tiles_n + ni, 1u);
                    }
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

        // ---------------------------------------------------------- GM_RS: reduce the blocks I own
        if (P.mode == GM_RS) {
            const int M_per = P.M / W;
            const __nv_bfloat16* part = (const __nv_bfloat16*)(cp->heap[rank] + P.part_off);
            const int items = P.rs_ring ? 0 : blocks_per * tiles_n; // ring: the last step wrote the result
            __shared__ int item_fail;
            for (int item = g; item < items; item += G) {
                const int mb = item / tiles_n, ni = item % tiles_n;
                if (threadIdx.x == 0)
                    item_fail = 0;
                __syncthreads();
                if ((int)threadIdx.x < W) {
                    const uint32_t* f = cp->aux[rank] + P.flag_off + ((size_t)threadIdx.x * blocks_per + mb) * tiles_n + ni;
                    if (*abort_flag || !wait_word<true>(f, seq * 4u, abort_flag, limit)) {
                        gemm_fail(fr, abort_flag, GE_FLAG_TIMEOUT, (uint32_t)item);
                        item_fail = 1;
                    }
                }
                __syncthreads();
                if (item_fail)
                    break;
                constexpr int PPR = F2_BN / 8; // 16-byte packs per tile row
                for (int p = threadIdx.x; p < F2_HALF * PPR; p += GEMM_THREADS) {
                    const int rl = mb * F2_HALF + p / PPR;
                    const int col = ni * F2_BN + (p % PPR) * 8;
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
            __syncthreads();
            if (threadIdx.x == 0) { // barrier-slot epoch accounting (one peer_barrier per GEMM CTA)
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

} // namespace

bool fused_gemm2_usable(int world, int M, int N, int K) {
    return env_data::get().gemm_2sm && M % (world * 256) == 0 && N % F2_BN == 0 && K % 8 == 0;
}

// CTAs of this kernel that can be resident at once (2 x the number of co-resident clusters, which may be below
// SMs / 2 where a GPC has an odd number of usable SMs).  The grid must not exceed it: GEMM pairs wait for flags
// that the copy CTAs at the end of the grid publish, so a copy CTA queued behind them would never run.
int fused_gemm2_max_ctas() {
    int dev_now = 0;
    CUDA_CHECK(cudaGetDevice(&dev_now));
    static int cached[64] = {};
    if (dev_now < 64 && cached[dev_now])
        return cached[dev_now];
    CUDA_CHECK(cudaFuncSetAttribute(fused_gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F2_SMEM));
    int sms = 0;
    CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev_now));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(sms & ~1);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = F2_SMEM;
    int clusters = 0;
    CUDA_CHECK(cudaOccupancyMaxActiveClusters(&clusters, fused_gemm2_kernel, &cfg));
    const int n = std::max(2, 2 * clusters);
    if (dev_now < 64)
        cached[dev_now] = n;
    return n;
}

// `ctas` CTAs per rank (even), of which the last `P.n_comm` (even) are copy CTAs; `ranks` > 1 = emulation
// (cooperative launch, blockIdx.y = rank)
void launch_fused_gemm2(const dev::comm_dev* tab, const fused_params& P, int ctas, int ranks, bool coop, cudaStream_t st) {
    int dev_now = 0;
    CUDA_CHECK(cudaGetDevice(&dev_now));
    static bool attr_done[64] = {}; // the attribute is per device
    if (dev_now >= 64 || !attr_done[dev_now]) {
        CUDA_CHECK(cudaFuncSetAttribute(fused_gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F2_SMEM));
        if (dev_now < 64)
            attr_done[dev_now] = true;
    }
    CCL_THROW_IF_NOT(ctas % 2 == 0 && P.n_comm % 2 == 0 && ctas - P.n_comm >= 2, "CTA pairs need even CTA counts");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas, ranks);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = F2_SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = coop ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CUDA_CHECK(cudaLaunchKernelEx(&cfg, fused_gemm2_kernel, tab, P));
}

} // namespace gpu
} // namespace cclx
