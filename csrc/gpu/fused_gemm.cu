#include "gpu/fused_gemm.cuh"

#include <algorithm>
#include <cstring>
#include <map>
#include <vector>

#include "core/env.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"
#include "gpu/device_comm.hpp"
#include "gpu/fused_gemm.hpp"

namespace cclx {
namespace gpu {

namespace {

// [rows, cols] row-major bf16 matrix, box = 64 columns x box_rows rows, 128-byte swizzle
CUtensorMap make_map(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    const driver_api& d = driver();
    CCL_THROW_IF_NOT(d.loaded && d.TensorMapEncodeTiled, "CUDA driver not available: ", d.error);
    CCL_THROW_IF_NOT(((uintptr_t)base & 15) == 0, "GEMM operand must be 16-byte aligned");
    CCL_THROW_IF_NOT(cols % 8 == 0, "GEMM inner dimension must be a multiple of 8 (16-byte row pitch)");
    CUtensorMap m;
    cuuint64_t gdim[2] = { cols, rows };
    cuuint64_t gstride[1] = { cols * 2 };
    cuuint32_t box[2] = { (cuuint32_t)GEMM_BK, box_rows };
    cuuint32_t estr[2] = { 1, 1 };
    CU_CHECK(d.TensorMapEncodeTiled(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride,
                                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return m;
}

} // namespace

CUtensorMap make_bf16_kmajor_map(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    return make_map(base, rows, cols, box_rows);
}

namespace {

int pick_bn(int N) {
    return (N % 256 == 0 || N % 128 != 0) ? 256 : 128;
}

template <int BN>
void set_smem_attr() {
    int dev_now = 0;
    CUDA_CHECK(cudaGetDevice(&dev_now));
    static bool done[64] = {}; // the attribute is per device
    if (dev_now >= 64 || !done[dev_now]) {
        CUDA_CHECK(cudaFuncSetAttribute(fused_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        gemm_smem<BN>::TOTAL));
        if (dev_now < 64)
            done[dev_now] = true;
    }
}

void launch(const dev::comm_dev* tab, const fused_params& P, int bn, int ctas, int ranks, bool coop, cudaStream_t st) {
    dim3 grid(ctas, ranks);
    void* argv[] = { (void*)&tab, (void*)&P };
    if (bn == 256) {
        set_smem_attr<256>();
        if (coop)
            CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)fused_gemm_kernel<256>, grid, dim3(GEMM_THREADS), argv,
                                                   gemm_smem<256>::TOTAL, st));
        else
            fused_gemm_kernel<256><<<grid, GEMM_THREADS, gemm_smem<256>::TOTAL, st>>>(tab, P);
    }
    else {
        set_smem_attr<128>();
        if (coop)
            CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)fused_gemm_kernel<128>, grid, dim3(GEMM_THREADS), argv,
                                                   gemm_smem<128>::TOTAL, st));
        else
            fused_gemm_kernel<128><<<grid, GEMM_THREADS, gemm_smem<128>::TOTAL, st>>>(tab, P);
    }
    CUDA_CHECK(cudaGetLastError());
}

int sm_count() {
    int dev = 0, n = 0;
    CUDA_CHECK(cudaGetDevice(&dev));
    CUDA_CHECK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    return n;
}

} // namespace

void gemm_bf16_plain(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int ctas,
                     uint32_t* err, cudaStream_t st) {
    CCL_THROW_IF_NOT(M > 0 && N > 0 && K > 0 && N % 8 == 0 && K % 8 == 0, "unsupported GEMM shape ", M, "x", N, "x", K);
    // CTA pairs (two-SM MMA) when the problem has at least one 256-row tile per pair; a negative `ctas` forces
    // the single-CTA kernel, CCL_CUDA_GEMM_2SM=0 turns the pairs off
    if (ctas >= 0 && env_data::get().gemm_2sm && M >= 256 && N >= 128) {
        gemm_bf16_2sm(A, B, C, M, N, K, epilogue, ctas / 2, err, st);
        return;
    }
    if (ctas < 0)
        ctas = -ctas - 1; // -(n + 1) asks for the single-CTA kernel on n CTAs (0 = all SMs)
    const int bn = pick_bn(N);
    fused_params P;
    std::memset(&P, 0, sizeof(P));
    P.r[0].tmA = make_map(A, M, K, GEMM_BM);
    P.r[0].tmB = make_map(B, N, K, bn);
    P.r[0].C = (__nv_bfloat16*)C;
    P.r[0].err = err;
    P.r[0].plan_state = nullptr;
    P.M = M;
    P.N = N;
    P.K = K;
    P.mode = GM_PLAIN;
    P.epilogue = epilogue;
    P.world = 1;
    P.timeout_ns = (unsigned long long)env_data::get().wait_timeout_ms * 1000000ull;
    const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + bn - 1) / bn);
    int g = ctas > 0 ? ctas : sm_count();
    g = std::min(g, tiles);
    launch(nullptr, P, bn, g, 1, false, st);
}

// CTA-pair form of the fused kernels (fused_gemm_2sm.cu)
bool fused_gemm2_usable(int world, int M, int N, int K);
int fused_gemm2_max_ctas();
void launch_fused_gemm2(const dev::comm_dev* tab, const fused_params& P, int ctas, int ranks, bool coop, cudaStream_t st);

struct fused_plan {
    device_comm* dc = nullptr;
    bool two_sm = false; // CTA pairs (cta_group::2): rows per rank a multiple of 256, N a multiple of 256
    int mode = 0, M = 0, N = 0, K = 0, epilogue = 0, n_comm = 0, ctas = 0, bn = 256;
    int entries = 1;
    size_t x_off = 0, part_off = 0;
    uint32_t flag_off = 0;
    uint32_t* state_dev = nullptr; // entries * (PLAN_WORDS + 4 err words)
    // cached maps, rebuilt when the operand pointers change
    std::vector<const void*> lastA, lastB;
    fused_params P;
    // all-gather by the copy engines (n_comm == 0): a side stream carries the peer copies and the
    // flag kernels while every SM runs GEMM tiles
    bool ce_gather = false;
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
};

namespace {
// flags of one gathered shard: its 128-row blocks may be loaded (sequence number of the running call)
__global__ void publish_shard_kernel(uint32_t* flags, int n, const uint32_t* plan_state) {
    const uint32_t seq = dev::ld_volatile_u32(plan_state + PLAN_SEQ) + 1;
    __threadfence();
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        dev::st_release_gpu(flags + i, seq);
}
} // namespace

// auxiliary flag words are handed out linearly per communicator
static uint32_t take_flag_words(device_comm& dc, uint32_t n) {
    static std::map<device_comm*, uint32_t> next;
    uint32_t& cur = next[&dc];
    if (cur == 0)
        cur = dev::A2A_HDR_WORDS;
    const uint32_t cap = (uint32_t)(dc.heap().regions().aux_flags_bytes / sizeof(uint32_t));
    CCL_THROW_IF_NOT(cur + n <= cap, "out of auxiliary flag words");
    uint32_t off = cur;
    cur += n;
    return off;
}

fused_plan* fused_plan_create(device_comm& dc, int mode, int M, int N, int K, int epilogue, int n_comm, int ctas) {
    CCL_THROW_IF_NOT(mode == GM_AG || mode == GM_RS, "fused plan mode must be 1 (AG+GEMM) or 2 (GEMM+RS)");
    const int W = dc.world();
    CCL_THROW_IF_NOT(M % (W * GEMM_BM) == 0, "rows (", M, ") must be a multiple of world*128");
    CCL_THROW_IF_NOT(N % 8 == 0 && K % 8 == 0, "N and K must be multiples of 8");
    CCL_THROW_IF_NOT(!dc.emulated() || W <= GEMM_EMU_MAX, "emulated fused GEMM supports at most 4 ranks");
    fused_plan* p = new fused_plan();
    p->dc = &dc;
    p->mode = mode;
    p->M = M;
    p->N = N;
    p->K = K;
    p->epilogue = epilogue;
    p->bn = pick_bn(N);
    p->entries = dc.emulated() ? W : 1;
    const int sms = sm_count();
    int per_rank = dc.emulated() ? sms / W : sms;
    if (ctas > 0)
        per_rank = std::min(per_rank, ctas);
    // n_comm < 0 (or CCL_CUDA_AG_GEMM_CE=1 with n_comm == 0): the copy engines gather, no copy CTAs
    p->two_sm = W > 1 && fused_gemm2_usable(W, M, N, K);
    if (p->two_sm) {
        const int cap = fused_gemm2_max_ctas() / (dc.emulated() ? W : 1);
        per_rank = std::min(per_rank, cap) & ~1; // whole pairs, all of them resident at once
        if (per_rank < 4)
            p->two_sm = false;
    }
    p->ce_gather = mode == GM_AG && W > 1 && (n_comm < 0 || (n_comm == 0 && env_data::get().ag_gemm_ce));
    p->n_comm = mode == GM_AG ? (n_comm > 0 ? n_comm : std::max(1, per_rank / 8)) : 0;
    if (W == 1)
        p->n_comm = mode == GM_AG ? 1 : 0;
    if (p->two_sm && p->n_comm > 0)
        p->n_comm = std::max(2, (p->n_comm + 1) & ~1); // copy CTAs come in pairs too (clusters of two)
    if (p->ce_gather) {
        p->n_comm = 0;
        CUDA_CHECK(cudaStreamCreateWithFlags(&p->side, cudaStreamNonBlocking));
        CUDA_CHECK(cudaEventCreateWithFlags(&p->ev_fork, cudaEventDisableTiming));
        CUDA_CHECK(cudaEventCreateWithFlags(&p->ev_join, cudaEventDisableTiming));
    }
    CCL_THROW_IF_NOT(per_rank - p->n_comm >= 1, "not enough CTAs");
    CCL_THROW_IF_NOT(per_rank <= dev::MAX_BLOCKS, "too many CTAs for the barrier slots");
    p->ctas = per_rank;
    const int tiles_m = M / GEMM_BM, tiles_n = (N + p->bn - 1) / p->bn;
    if (mode == GM_AG) {
        p->x_off = dc.heap().alloc((size_t)M * K * 2);
        p->flag_off = take_flag_words(dc, tiles_m);
    }
    else {
        p->part_off = dc.heap().alloc((size_t)M * N * 2); // world slots of [M/world, N]
        p->flag_off = take_flag_words(dc, (uint32_t)(tiles_m * tiles_n));
    }
    const size_t words = (size_t)p->entries * (PLAN_WORDS + 4);
    CUDA_CHECK(cudaMalloc((void**)&p->state_dev, words * sizeof(uint32_t)));
    CUDA_CHECK(cudaMemset(p->state_dev, 0, words * sizeof(uint32_t)));
    std::memset(&p->P, 0, sizeof(p->P));
    p->P.M = M;
    p->P.N = N;
    p->P.K = K;
    p->P.mode = mode;
    p->P.epilogue = epilogue;
    p->P.emu = dc.emulated() ? 1 : 0;
    p->P.world = W;
    p->P.n_comm = p->n_comm;
    // GEMM -> reduce-scatter: ring of partial sums inside the epilogue unless n_comm == -1 or the knob is off
    // The ring needs the neighbour's tile of the previous step to be finished well before this rank reaches
    // the same tile: with fewer than about one and a half waves of tiles per step the epilogues would wait on one another
    // (measured: faster at 4 ranks with 256 tiles per step, slower at 8 ranks with 128), so the owner-side
    // reduction stays the default there.  n_comm == -2 forces the ring.
    const bool ring_pays = 2 * (size_t)(tiles_m / W) * tiles_n >= 3 * (size_t)per_rank;
    p->P.rs_ring = (mode == GM_RS && W > 1 && n_comm != -1 && env_data::get().gemm_rs_ring && (ring_pays || n_comm == -2)) ? 1 : 0;
    p->P.x_off = p->x_off;
    p->P.part_off = p->part_off;
    p->P.flag_off = p->flag_off;
    p->P.timeout_ns = (unsigned long long)env_data::get().wait_timeout_ms * 1000000ull;
    for (int e = 0; e < p->entries; e++) {
        p->P.r[e].plan_state = p->state_dev + (size_t)e * (PLAN_WORDS + 4);
        p->P.r[e].err = p->state_dev + (size_t)e * (PLAN_WORDS + 4) + PLAN_WORDS;
    }
    p->lastA.assign(p->entries, nullptr);
    p->lastB.assign(p->entries, nullptr);
    CUDA_CHECK(cudaDeviceSynchronize());
    return p;
}

void fused_plan_destroy(fused_plan* p) {
    if (!p)
        return;
    cudaDeviceSynchronize();
    if (p->mode == GM_AG)
        p->dc->heap().free(p->x_off);
    else
        p->dc->heap().free(p->part_off);
    cudaFree(p->state_dev);
    if (p->side) {
        cudaStreamDestroy(p->side);
        cudaEventDestroy(p->ev_fork);
        cudaEventDestroy(p->ev_join);
    }
    delete p;
}

void* fused_plan_x_full(fused_plan* p, int r) {
    const int owner = p->dc->emulated() ? r : p->dc->rank();
    return p->dc->heap().base(owner) + p->x_off;
}

void* fused_plan_x_shard(fused_plan* p, int r) {
    const int owner = p->dc->emulated() ? r : p->dc->rank();
    const size_t shard = (size_t)(p->M / p->dc->world()) * p->K * 2;
    return p->dc->heap().base(owner) + p->x_off + (size_t)owner * shard;
}

void fused_plan_run(fused_plan* p, const void* const* A, const void* const* B, void* const* C, cudaStream_t st) {
    device_comm& dc = *p->dc;
    dc.check_status();
    for (int e = 0; e < p->entries; e++) {
        const void* a = p->mode == GM_AG ? fused_plan_x_full(p, e) : A[e];
        if (a != p->lastA[e]) {
            p->P.r[e].tmA = make_map(a, p->M, p->K, GEMM_BM);
            p->lastA[e] = a;
        }
        if (B[e] != p->lastB[e]) {
            p->P.r[e].tmB = make_map(B[e], p->N, p->K, p->two_sm ? 128 : p->bn); // a pair's CTA stages half of the B tile
            p->lastB[e] = B[e];
        }
        p->P.r[e].C = (__nv_bfloat16*)C[e];
    }
    auto go = [&] {
        if (p->two_sm)
            launch_fused_gemm2(dc.table(), p->P, p->ctas, p->entries, dc.emulated(), st);
        else
            launch(dc.table(), p->P, p->bn, p->ctas, p->entries, dc.emulated(), st);
    };
    if (!p->ce_gather) {
        go();
        return;
    }
    // every rank has written its shard once it passed this barrier
    launch_barrier(dc, st);
    CUDA_CHECK(cudaEventRecord(p->ev_fork, st));
    CUDA_CHECK(cudaStreamWaitEvent(p->side, p->ev_fork, 0));
    const int W = dc.world();
    const int tiles_m_per = p->M / GEMM_BM / W;
    const size_t shard = (size_t)(p->M / W) * p->K * 2;
    for (int k = 1; k < W; k++) {
        for (int e = 0; e < p->entries; e++) {
            const int r = dc.emulated() ? e : dc.rank();
            const int src = (r + k) % W;
            const size_t off = p->x_off + (size_t)src * shard;
            CUDA_CHECK(cudaMemcpyAsync(dc.heap().base(r) + off, dc.heap().base(src) + off, shard, cudaMemcpyDeviceToDevice,
                                       p->side));
            uint32_t* flags = dc.host_entry(e).aux[dc.emulated() ? e : dc.rank()] + p->flag_off + (size_t)src * tiles_m_per;
            publish_shard_kernel<<<1, 32, 0, p->side>>>(flags, tiles_m_per, p->P.r[e].plan_state);
            CUDA_CHECK(cudaGetLastError());
        }
    }
    CUDA_CHECK(cudaEventRecord(p->ev_join, p->side));
    // the GEMM starts on the local shard at once and waits per 128-row block for the others
    go();
    CUDA_CHECK(cudaStreamWaitEvent(st, p->ev_join, 0));
    // peers may overwrite their shard (next call) only after everybody has copied it
    launch_barrier(dc, st);
}

uint32_t fused_plan_error(fused_plan* p, int r) {
    uint32_t v[4] = { 0, 0, 0, 0 };
    CUDA_CHECK(cudaMemcpy(v, p->state_dev + (size_t)r * (PLAN_WORDS + 4) + PLAN_WORDS, sizeof(v),
                          cudaMemcpyDeviceToHost));
    return v[0];
}

} // namespace gpu
} // namespace cclx
