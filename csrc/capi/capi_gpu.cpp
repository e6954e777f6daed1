// Flat C API over the device communicator: what the Python package calls
// through ctypes.  Every function returns 0 on success and -1 on error
// (message via cclx_last_error) unless stated.
#include <cstring>
#include <vector>

#include "capi/capi_common.hpp"
#include "core/env.hpp"
#include "core/log.hpp"
#include "gpu/cuda_driver.hpp"
#include "gpu/device_comm.hpp"
#include "gpu/fused_gemm.hpp"

using namespace cclx;
using namespace cclx::gpu;

namespace cclx {
namespace capi {
static thread_local std::string last_error;
void set_last_error(const std::string& msg) {
    last_error = msg;
}
} // namespace capi
} // namespace cclx

CCLX_API const char* cclx_last_error() {
    return capi::last_error.c_str();
}

CCLX_API int cclx_env_reload() {
    return capi::guard([] { env_data::reload(); });
}

CCLX_API int cclx_cuda_device_count() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

// The library carries its own (static) CUDA runtime, whose notion of the
// current device is per thread and independent of the caller's runtime: the
// bindings call this before every launch with the caller's current device.
CCLX_API int cclx_set_device(int dev) {
    return capi::guard([&] { CUDA_CHECK(cudaSetDevice(dev)); });
}

// ---- emulated group (all ranks on the current device) ---------------------------
CCLX_API void* cclx_emu_create(int world, size_t heap_bytes, size_t staging_bytes) {
    device_comm* dc = nullptr;
    int rc = capi::guard([&] {
        dc = new device_comm();
        dc->init_emulated(world, heap_bytes, staging_bytes);
    });
    if (rc != 0) {
        delete dc;
        return nullptr;
    }
    return dc;
}

CCLX_API int cclx_dc_destroy(void* h) {
    return capi::guard([&] { delete (device_comm*)h; });
}

CCLX_API int cclx_dc_world(void* h) {
    return ((device_comm*)h)->world();
}
CCLX_API int cclx_dc_rank(void* h) {
    return ((device_comm*)h)->rank();
}
CCLX_API int cclx_dc_nvls(void* h) {
    return ((device_comm*)h)->nvls() ? 1 : 0;
}
CCLX_API size_t cclx_dc_staging_bytes(void* h) {
    return ((device_comm*)h)->staging_bytes();
}
CCLX_API int cclx_dc_status(void* h, int r) {
    return (int)((device_comm*)h)->status_code(r);
}
CCLX_API int cclx_dc_check(void* h) {
    return capi::guard([&] { ((device_comm*)h)->check_status(); });
}
CCLX_API int cclx_dc_clear_status(void* h) {
    return capi::guard([&] { ((device_comm*)h)->clear_status(); });
}
CCLX_API int cclx_dc_abort(void* h) {
    return capi::guard([&] { ((device_comm*)h)->abort(); });
}
// test hook: the next collectives of emulated rank `rank` (-1: none) carry a falsified argument signature
CCLX_API int cclx_dc_test_sig_skew(void* h, int rank) {
    return capi::guard([&] { ((device_comm*)h)->test_sig_skew = rank + 1; });
}
CCLX_API int cclx_dc_set_timeout_ms(void* h, size_t ms) {
    return capi::guard([&] { ((device_comm*)h)->set_timeout_ms(ms); });
}
// registration of ordinary device allocations for zero-copy peer access (collective; arrays hold one
// entry in real mode and `world` entries in emulation mode); returns the registration id or -1
CCLX_API int cclx_dc_register(void* h, void* const* ptrs, const size_t* bytes) {
    int id = -1;
    capi::guard([&] { id = ((device_comm*)h)->register_user(ptrs, bytes); });
    return id;
}
CCLX_API int cclx_dc_deregister(void* h, int id) {
    return capi::guard([&] { ((device_comm*)h)->deregister_user(id); });
}

CCLX_API unsigned long long cclx_dc_algo_hits(void* h, int coll, int algo) {
    return ((device_comm*)h)->algo_hits[coll * ga_last + algo];
}
CCLX_API int cclx_gpu_algo_from_name(const char* s) {
    return gpu_algo_from_name(s);
}

// symmetric heap: returns the heap offset (same on every rank) or (size_t)-1
CCLX_API size_t cclx_dc_symm_alloc(void* h, size_t bytes) {
    size_t off = (size_t)-1;
    capi::guard([&] { off = ((device_comm*)h)->heap().alloc(bytes); });
    return off;
}
CCLX_API int cclx_dc_symm_free(void* h, size_t off) {
    return capi::guard([&] { ((device_comm*)h)->heap().free(off); });
}
CCLX_API void* cclx_dc_heap_base(void* h, int r) {
    return ((device_comm*)h)->heap().base(r);
}
CCLX_API void* cclx_dc_mc_base(void* h) {
    return ((device_comm*)h)->heap().mc_base();
}
CCLX_API size_t cclx_dc_aux_offset(void* h) {
    return ((device_comm*)h)->heap().regions().aux_flags_off;
}

// ---- collectives ------------------------------------------------------------------
// send/recv: arrays of `n` pointers, n = 1 in real mode and world in emulation mode
static std::vector<dev::rank_args> make_ra(device_comm* dc, const void* const* send, void* const* recv) {
    const int n = dc->emulated() ? dc->world() : 1;
    std::vector<dev::rank_args> ra(n);
    std::memset(ra.data(), 0, n * sizeof(dev::rank_args));
    for (int e = 0; e < n; e++) {
        ra[e].send = send ? send[e] : nullptr;
        ra[e].recv = recv ? recv[e] : nullptr;
    }
    return ra;
}

static launch_opts make_opts(int algo, int blocks, float scale, int do_scale) {
    launch_opts o;
    o.algo = algo;
    o.blocks = blocks;
    o.scale = scale;
    o.do_scale = do_scale != 0;
    return o;
}

CCLX_API int cclx_dc_allreduce(void* h, const void* const* send, void* const* recv, size_t count, int dt_in,
                               int dt_out, int op, int algo, int blocks, float scale, int do_scale, void* stream) {
    return capi::guard([&] {
        device_comm* dc = (device_comm*)h;
        auto ra = make_ra(dc, send, recv);
        launch_allreduce(*dc, ra.data(), count, dt_in, dt_out, op, make_opts(algo, blocks, scale, do_scale),
                         (cudaStream_t)stream);
    });
}

CCLX_API int cclx_dc_reduce_scatter(void* h, const void* const* send, void* const* recv, size_t recv_count,
                                    int dt_in, int dt_out, int op, int algo, int blocks, float scale, int do_scale,
                                    void* stream) {
    return capi::guard([&] {
        device_comm* dc = (device_comm*)h;
        auto ra = make_ra(dc, send, recv);
        launch_reduce_scatter(*dc, ra.data(), recv_count, dt_in, dt_out, op,
                              make_opts(algo, blocks, scale, do_scale), (cudaStream_t)stream);
    });
}

CCLX_API int cclx_dc_reduce(void* h, const void* const* send, void* const* recv, size_t count, int dt_in, int dt_out,
                            int op, int root, int blocks, float scale, int do_scale, void* stream) {
    return capi::guard([&] {
        device_comm* dc = (device_comm*)h;
        auto ra = make_ra(dc, send, recv);
        launch_reduce(*dc, ra.data(), count, dt_in, dt_out, op, root, make_opts(ga_auto, blocks, scale, do_scale),
                      (cudaStream_t)stream);
    });
}

// byte_counts / byte_displs: world entries, identical on every rank
CCLX_API int cclx_dc_allgatherv(void* h, const void* const* send, void* const* recv, const size_t* byte_counts,
                                const size_t* byte_displs, int algo, int blocks, void* stream) {
    return capi::guard([&] {
        device_comm* dc = (device_comm*)h;
        auto ra = make_ra(dc, send, recv);
        for (auto& r : ra)
            for (int p = 0; p < dc->world(); p++) {
                r.scount[p] = byte_counts[p];
                r.sdispl[p] = byte_displs[p];
            }
        launch_allgatherv(*dc, ra.data(), make_opts(algo, blocks, 1.f, 0), (cudaStream_t)stream);
    });
}

// tables: n x 4 x world size_t (send counts, send displs, recv counts, recv displs) in bytes
CCLX_API int cclx_dc_alltoallv(void* h, const void* const* send, void* const* recv, const size_t* tables, int blocks,
                               void* stream) {
    return capi::guard([&] {
        device_comm* dc = (device_comm*)h;
        auto ra = make_ra(dc, send, recv);
        const int W = dc->world();
        for (size_t e = 0; e < ra.size(); e++) {
            const size_t* t = tables + e * 4 * W;
            for (int p = 0; p < W; p++) {
                ra[e].scount[p] = t[p];
                ra[e].sdispl[p] = t[W + p];
                ra[e].rcount[p] = t[2 * W + p];
                ra[e].rdispl[p] = t[3 * W + p];
            }
        }
        launch_alltoallv(*dc, ra.data(), make_opts(ga_auto, blocks, 1.f, 0), (cudaStream_t)stream);
    });
}

// alltoall with one block size for every pair of ranks (bytes per peer)
CCLX_API int cclx_dc_alltoall(void* h, const void* const* send, void* const* recv, size_t bytes_per_peer, int algo,
                              int blocks, void* stream) {
    return capi::guard([&] {
        device_comm* dc = (device_comm*)h;
        auto ra = make_ra(dc, send, recv);
        const int W = dc->world();
        for (size_t e = 0; e < ra.size(); e++)
            for (int p = 0; p < W; p++) {
                ra[e].scount[p] = ra[e].rcount[p] = bytes_per_peer;
                ra[e].sdispl[p] = ra[e].rdispl[p] = (size_t)p * bytes_per_peer;
            }
        launch_opts o = make_opts(algo, blocks, 1.f, 0);
        o.uniform = true;
        launch_alltoallv(*dc, ra.data(), o, (cudaStream_t)stream);
    });
}

CCLX_API int cclx_dc_broadcast(void* h, const void* const* send, void* const* recv, size_t bytes, int root, int blocks,
                               void* stream) {
    return capi::guard([&] {
        device_comm* dc = (device_comm*)h;
        auto ra = make_ra(dc, send, recv);
        launch_broadcast(*dc, ra.data(), bytes, root, make_opts(ga_auto, blocks, 1.f, 0), (cudaStream_t)stream);
    });
}

CCLX_API int cclx_dc_barrier(void* h, void* stream) {
    return capi::guard([&] { launch_barrier(*(device_comm*)h, (cudaStream_t)stream); });
}

// real mode: n_ops operations of this rank (arrays of n_ops).  emulation mode: one
// operation per emulated rank (arrays of world entries, peer -1 = idle).
CCLX_API int cclx_dc_sendrecv(void* h, const void* const* send, void* const* recv, const size_t* bytes,
                              const int* peers, const int* is_send, int n_ops, void* stream) {
    return capi::guard([&] {
        device_comm* dc = (device_comm*)h;
        if (dc->emulated()) {
            std::vector<dev::p2p_ops> ops(dc->world());
            for (int e = 0; e < dc->world(); e++) {
                ops[e].n = 1;
                ops[e].op[0] = dev::p2p_op{ send ? send[e] : nullptr, recv ? recv[e] : nullptr, bytes[e], peers[e],
                                            is_send[e] };
            }
            launch_sendrecv(*dc, ops.data(), (cudaStream_t)stream);
        }
        else {
            dev::p2p_ops ops{};
            CCL_THROW_IF_NOT(n_ops <= dev::P2P_MAX_OPS, "at most ", dev::P2P_MAX_OPS, " operations per launch");
            ops.n = n_ops;
            for (int i = 0; i < n_ops; i++)
                ops.op[i] = dev::p2p_op{ send ? send[i] : nullptr, recv ? recv[i] : nullptr, bytes[i], peers[i],
                                         is_send[i] };
            launch_sendrecv(*dc, &ops, (cudaStream_t)stream);
        }
    });
}

CCLX_API int cclx_dc_wait_unset_flag(void* h, void* stream) {
    return capi::guard([&] { launch_wait_unset_flag(*(device_comm*)h, (cudaStream_t)stream); });
}

CCLX_API int cclx_reduce_local(const void* in, void* inout, size_t count, int dt, int op, void* stream) {
    return capi::guard([&] { launch_reduce_local(in, inout, count, dt, op, (cudaStream_t)stream); });
}

CCLX_API int cclx_transpose_blocks(const void* in, void* out, int rows, int cols, size_t block_bytes, void* stream) {
    return capi::guard([&] { launch_transpose_blocks(in, out, rows, cols, block_bytes, (cudaStream_t)stream); });
}

// fused small-message allreduce: n tensors per entry (tensor-major pointer arrays), one pack kernel, one
// zero-copy allreduce on the fused symmetric buffer, one unpack kernel
CCLX_API int cclx_dc_allreduce_fused(void* h, const void* const* send, void* const* recv, const size_t* counts, int n,
                                     int dt, int op, float scale, int do_scale, void* stream) {
    return capi::guard([&] {
        launch_allreduce_fused(*(device_comm*)h, send, recv, counts, n, dt, op, make_opts(ga_auto, 0, scale, do_scale),
                               (cudaStream_t)stream);
    });
}
CCLX_API unsigned long long cclx_dc_fused_batches(void* h) {
    return ((device_comm*)h)->fuse().batches;
}

// ---- tcgen05 GEMM, plain and fused with a collective ------------------------------
CCLX_API int cclx_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int ctas,
                            void* err_words, void* stream) {
    return capi::guard(
        [&] { gemm_bf16_plain(A, B, C, M, N, K, epilogue, ctas, (uint32_t*)err_words, (cudaStream_t)stream); });
}

CCLX_API int cclx_gemm_bf16_2sm(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int clusters,
                                void* err_words, void* stream) {
    return capi::guard(
        [&] { gemm_bf16_2sm(A, B, C, M, N, K, epilogue, clusters, (uint32_t*)err_words, (cudaStream_t)stream); });
}

// The same product over the first min(M, *rows_dev) rows of A: the count is read on the device, so a kernel in
// front (the MoE dispatch) can decide it without the host in between.  M bounds the buffers.
CCLX_API int cclx_gemm_bf16_rows(const void* A, const void* B, void* C, int M, int N, int K, int epilogue,
                                 const void* rows_dev, void* err_words, void* stream) {
    return capi::guard([&] {
        gemm_bf16_2sm(A, B, C, M, N, K, epilogue, 0, (uint32_t*)err_words, (cudaStream_t)stream, (const int*)rows_dev);
    });
}

CCLX_API void* cclx_fused_plan_create(void* dc, int mode, int M, int N, int K, int epilogue, int n_comm, int ctas) {
    fused_plan* p = nullptr;
    capi::guard([&] { p = fused_plan_create(*(device_comm*)dc, mode, M, N, K, epilogue, n_comm, ctas); });
    return p;
}
CCLX_API int cclx_fused_plan_destroy(void* p) {
    return capi::guard([&] { fused_plan_destroy((fused_plan*)p); });
}
CCLX_API void* cclx_fused_plan_x_shard(void* p, int r) {
    return fused_plan_x_shard((fused_plan*)p, r);
}
CCLX_API void* cclx_fused_plan_x_full(void* p, int r) {
    return fused_plan_x_full((fused_plan*)p, r);
}
CCLX_API int cclx_fused_plan_run(void* p, const void* const* A, const void* const* B, void* const* C, void* stream) {
    return capi::guard([&] { fused_plan_run((fused_plan*)p, A, B, C, (cudaStream_t)stream); });
}
CCLX_API int cclx_fused_plan_error(void* p, int r) {
    int v = -1;
    capi::guard([&] { v = (int)fused_plan_error((fused_plan*)p, r); });
    return v;
}
