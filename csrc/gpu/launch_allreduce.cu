// Allreduce on GPU buffers: selection by size / registration and launch.
// Counterpart of allreduce_sycl_single_node (reference
// src/coll/algorithms/allreduce/sycl/allreduce_sycl.cpp:27-168): world==1 is a
// copy, small messages take the one-shot kernel, larger ordinary buffers the
// chunk-pipelined kernel (two-shot below its threshold), buffers from the
// symmetric heap or from a registered allocation skip staging (NVLS when both
// lie in the heap).
#include "gpu/launch_common.cuh"

namespace cclx {
namespace gpu {

namespace {

template <class T, class Tout>
__global__ void __launch_bounds__(1024) scale_cast_kernel(const T* in, Tout* out, size_t count, float scale,
                                                          int do_scale) {
    typedef typename dev::acc_of<T>::type A;
    constexpr int N = dev::pack_traits<T>::N;
    const size_t npacks = (count + N - 1) / N;
    const bool vin = (((uintptr_t)in) & 15) == 0;
    const bool vout = dev::out_vec_ok<Tout, N>(out);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < npacks;
         i += (size_t)gridDim.x * blockDim.x) {
        A acc[N];
        dev::unpack16<T, A>(dev::load_pack<T>(in, i, count, vin), acc);
        dev::store_pack<Tout, A, N>(out, i, count, vout, acc, scale, do_scale != 0);
    }
}

// debug scan of a result buffer (the reference's sycl_check_nan,
// src/coll/algorithms/utils/sycl_coll_base.hpp:516-549)
template <class T>
__global__ void __launch_bounds__(256) check_finite_kernel(const T* p, size_t count, volatile uint32_t* status) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        const float v = (float)p[i];
        if (!isfinite(v) && status[0] == dev::ST_OK) {
            status[1] = blockIdx.x;
            status[3] = (uint32_t)i;
            __threadfence_system();
            status[0] = dev::ST_NOT_FINITE;
        }
    }
}

} // namespace

void launch_check_finite(device_comm& dc, const void* buf, size_t count, int dt, cudaStream_t st) {
    if (count == 0 || dc.emulated())
        return;
    volatile uint32_t* status = dc.host_entry(0).status;
    const int blocks = (int)std::min<size_t>((count + 255) / 256, (size_t)dc.sm_count() * 4);
    if (dt == dt_float32)
        check_finite_kernel<float><<<blocks, 256, 0, st>>>((const float*)buf, count, status);
    else if (dt == dt_bfloat16)
        check_finite_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)buf, count, status);
    else if (dt == dt_float16)
        check_finite_kernel<__half><<<blocks, 256, 0, st>>>((const __half*)buf, count, status);
    else if (dt == dt_float64)
        check_finite_kernel<double><<<blocks, 256, 0, st>>>((const double*)buf, count, status);
    else
        return;
    CUDA_CHECK(cudaGetLastError());
}

int selected_allreduce_algo(const device_comm& dc, size_t bytes, bool symmetric, int dt, int op) {
    const env_data& env = env_data::get();
    if (dc.world() == 1)
        return ga_copy;
    const bool fits_oneshot = (size_t)dc.world() * ((bytes + 15) & ~(size_t)15) <= dc.staging_bytes();
    // one-shot sends (n-1) copies of the message: its break-even size shrinks with the rank
    // count (the configured threshold is the 8-rank value)
    // between two ranks one-shot moves exactly what two-shot moves and saves a barrier: measured faster up to
    // 8 MiB (2 MiB: 17.3 us against 21.4 us)
    const size_t oneshot_max = dc.world() == 2 ? env.ar_oneshot_threshold * 32
                                               : env.ar_oneshot_threshold * 8 / (size_t)std::max(dc.world(), 2);
    if (bytes <= oneshot_max && fits_oneshot)
        return (dc.nvls() && bytes >= 4096 && dc.world() >= env.nvls_min_ranks) ? ga_nvls_oneshot : ga_oneshot;
    // in-switch reduction moves (1 + 1/n) S per direction, peer loads 2 (n-1)/n S: NVLS wins from 3 ranks on
    if (symmetric)
        return (dc.nvls() && nvls_type_ok(dt, op) && dc.world() >= env.nvls_min_ranks) ? ga_nvls : ga_symm;
    // ordinary buffers: the chunk pipeline hides the staging copies under the NVLink traffic
    return bytes >= env.ar_pipelined_min ? ga_pipelined : ga_twoshot;
}

void launch_allreduce(device_comm& dc, const dev::rank_args* ra, size_t count, int dt_in, int dt_out, int op,
                      const launch_opts& o, cudaStream_t st) {
    if (count == 0)
        return;
    const int W = dc.world();
    const size_t esz = predefined_dtype_size(dt_in);
    const size_t bytes = count * esz;
    const int entries = dc.emulated() ? W : 1;

    // zero-copy needs both buffers of every rank in the symmetric heap or in a registered allocation,
    // at equal offsets; the in-switch reduction needs both in the heap (the multicast window covers only it)
    // Ordinary buffers have two ways: share them (CUDA IPC) and reduce by peer loads, or copy them chunk by chunk
    // through the heap's staging area, where the switch can reduce.  The in-switch reduction moves (1 + 1/W) S
    // over a GPU's links instead of 2 (W - 1)/W S, which pays for the copies from five ranks on (8 B200s, bf16,
    // ordinary tensors: 1 GiB in 2.55 ms staged against 3.17 ms by peer loads, 16 MiB in 64 us against 86 us; on 4
    // ranks the two are equal within 1 %).  All terms are the same on every rank.
    const env_data& env0 = env_data::get();
    const bool staged_nvls = dc.nvls() && nvls_type_ok(dt_in, op) &&
                             W >= std::max(env0.nvls_min_ranks, env0.nvls_staged_min_ranks);
    zc_view vin, vout;
    if (dt_in == dt_out && W > 1)
        zero_copy_views(dc, ra, true, bytes, true, bytes, vin, vout, !staged_nvls);
    const bool symmetric = vin.ok && vout.ok;
    const bool in_heap = symmetric && !vin.registered && !vout.registered;
    const size_t in_off = vin.off, out_off = vout.off;
    (void)entries;

    int algo = o.algo;
    if (algo == ga_auto)
        algo = selected_allreduce_algo(dc, bytes, symmetric, dt_in, op);
    if ((algo == ga_symm || algo == ga_nvls) && !symmetric)
        CCL_THROW("allreduce algorithm ", gpu_algo_name(algo),
                  " needs buffers from the symmetric heap or from a registered allocation");
    if (algo == ga_nvls && !in_heap)
        algo = ga_symm;
    if ((algo == ga_nvls || algo == ga_nvls_oneshot) && !dc.nvls())
        algo = algo == ga_nvls ? ga_symm : ga_oneshot;
    if (algo == ga_nvls && !nvls_type_ok(dt_in, op))
        algo = ga_symm;
    if (W == 1)
        algo = ga_copy;
    dc.algo_hits[coll_allreduce * ga_last + algo]++;

    dev::coll_args a{};
    a.scale = o.scale;
    a.do_scale = o.do_scale ? 1 : 0;
    a.flags = 0;
    const int threads = dc.threads();

    if (algo == ga_copy) {
        dispatch_reduce_types(dt_in, dt_out, op, [&](auto tin, auto tout, auto) {
            typedef decltype(tin) T;
            typedef decltype(tout) Tout;
            for (int e = 0; e < entries; e++) {
                if (ra[e].send == ra[e].recv && !o.do_scale && dt_in == dt_out)
                    continue;
                const size_t npacks = (bytes + 15) / 16;
                int blocks = (int)std::min<size_t>((npacks + threads - 1) / threads, (size_t)dc.sm_count() * 4);
                scale_cast_kernel<T, Tout><<<std::max(blocks, 1), threads, 0, st>>>(
                    (const T*)ra[e].send, (Tout*)ra[e].recv, count, o.scale, a.do_scale);
                CUDA_CHECK(cudaGetLastError());
            }
        });
        return;
    }

    if (algo == ga_symm || algo == ga_nvls) {
        a.count = count;
        a.in_off = in_off;
        a.out_off = out_off;
        a.flags = dev::CF_SYMM_IN | dev::CF_SYMM_OUT | (algo == ga_nvls ? dev::CF_NVLS : 0);
        if (vin.registered)
            fill_registered(dc, a, vin, false);
        if (vout.registered)
            fill_registered(dc, a, vout, true);
        prepare_args(dc, a, ra, st);
        // Grid width.  In-switch reduction: the traffic of a GPU's links is carried by a handful of blocks (measured
        // on 4 and 8 B200s: 4 to 8 blocks of 1024 threads with eight loads in flight per thread are as fast as or
        // faster than any wider grid from 1 MB to 1 GiB), so the automatic choice stays narrow and leaves the SMs
        // to whatever else runs.  Peer loads need their requests spread over many SMs: 8 KiB of the per-rank
        // slice per block, up to the whole GPU.
        int blocks;
        bool narrow;
        if (algo == ga_nvls && o.blocks == 0) {
            blocks = pick_blocks(dc, bytes / 16 / W + 1, 128, 8);
            blocks = std::min(blocks, (int)((bytes / 16 / W) / 128 + 1));
            narrow = true;
        }
        else {
            blocks = pick_blocks(dc, bytes / 16 / W + 1, 512, o.blocks);
            // a grid that the caller kept narrow (it runs beside a compute kernel) makes up for the missing
            // blocks with full-size blocks and twice the loads in flight per thread
            narrow = o.blocks > 0 && blocks * 4 <= dc.sm_count();
        }
        const int th = narrow ? 1024 : threads;
        CCLX_DISPATCH_DTYPE(dt_in, T, {
            if (algo == ga_nvls) {
                if constexpr (std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value ||
                              std::is_same<T, __half>::value) {
                    if (narrow)
                        launch_kernel(dc, dev::allreduce_symm_kernel<T, dev::op_sum, true, 8>, blocks, th, st,
                                      dc.table(), a);
                    else
                        launch_kernel(dc, dev::allreduce_symm_kernel<T, dev::op_sum, true, 4>, blocks, th, st,
                                      dc.table(), a);
                }
            }
            else {
                CCLX_DISPATCH_OP(op, OP,
                                 launch_kernel(dc, dev::allreduce_symm_kernel<T, OP, false>, blocks, th, st,
                                               dc.table(), a));
            }
        });
        return;
    }

    if (algo == ga_oneshot || algo == ga_nvls_oneshot) {
        const size_t slot = (bytes + 15) & ~(size_t)15;
        if ((size_t)W * slot > dc.staging_bytes())
            algo = ga_twoshot;
        else {
            a.count = count;
            a.flags = algo == ga_nvls_oneshot ? dev::CF_NVLS : 0;
            prepare_args(dc, a, ra, st);
            const int blocks = pick_blocks(dc, slot / 16, 512, o.blocks); // one pack per thread: latency, not throughput, counts here
            dispatch_reduce_types(dt_in, dt_out, op, [&](auto tin, auto tout, auto opv) {
                launch_kernel(dc, dev::allreduce_oneshot_kernel<decltype(tin), decltype(tout), decltype(opv)>, blocks,
                              threads, st, dc.table(), a);
            });
            return;
        }
    }

    const size_t osz = predefined_dtype_size(dt_out);
    const size_t N = 16 / esz;
    const size_t out_pack = std::max<size_t>(N * osz, 16); // reduced packs are staged in whole 16-byte units

    if (algo == ga_pipelined) {
        const env_data& env = env_data::get();
        const size_t npacks = (bytes + 15) / 16;
        int blocks = o.blocks > 0 ? o.blocks : env.ar_pipelined_blocks;
        blocks = std::max(1, std::min(blocks, dc.max_blocks()));
        // a few hundred packs per block and rank at least, so that small messages do not pay for idle blocks
        while (blocks > 1 && npacks < (size_t)blocks * W * 256)
            blocks /= 2;
        const size_t unit = (size_t)blocks * W; // a chunk divides evenly among blocks, then ranks
        size_t cp = dc.staging_bytes() / (2 * 16 + 2 * out_pack) / unit * unit;
        CCL_THROW_IF_NOT(cp >= unit, "staging buffer too small for the pipelined allreduce");
        cp = std::min(cp, (npacks + unit - 1) / unit * unit);
        a.count = count;
        a.stride = cp;
        const bool nvls = dc.nvls() && nvls_type_ok(dt_in, op) && W >= env.nvls_min_ranks;
        prepare_args(dc, a, ra, st);
        dispatch_reduce_types(dt_in, dt_out, op, [&](auto tin, auto tout, auto opv) {
            typedef decltype(tin) T;
            typedef decltype(tout) Tout;
            typedef decltype(opv) OP;
            if constexpr (std::is_same<OP, dev::op_sum>::value &&
                          (std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value ||
                           std::is_same<T, __half>::value)) {
                if (nvls) {
                    launch_kernel(dc, dev::allreduce_pipelined_kernel<T, Tout, OP, true>, blocks, threads, st,
                                  dc.table(), a);
                    return;
                }
            }
            launch_kernel(dc, dev::allreduce_pipelined_kernel<T, Tout, OP, false>, blocks, threads, st, dc.table(),
                          a);
        });
        return;
    }

    // two-shot, chunked so that IN slots + OUT region fit one staging generation
    CCL_THROW_IF_NOT(algo == ga_twoshot, "unknown allreduce algorithm ", algo);
    size_t max_packs = (dc.staging_bytes() - 16 * (size_t)W) / (16 + out_pack);
    max_packs = max_packs / W * W; // whole slices
    CCL_THROW_IF_NOT(max_packs >= (size_t)W, "staging buffer too small for a two-shot allreduce");
    const size_t chunk_elems = max_packs * N;
    std::vector<dev::rank_args> cur(ra, ra + entries);
    for (size_t done = 0; done < count; done += chunk_elems) {
        const size_t n = std::min(chunk_elems, count - done);
        for (int e = 0; e < entries; e++) {
            cur[e].send = (const char*)ra[e].send + done * esz;
            cur[e].recv = (char*)ra[e].recv + done * osz;
        }
        a.count = n;
        prepare_args(dc, a, cur.data(), st);
        const int blocks = pick_blocks(dc, (n * esz + 15) / 16 / W + 1, 1024, o.blocks);
        dispatch_reduce_types(dt_in, dt_out, op, [&](auto tin, auto tout, auto opv) {
            launch_kernel(dc, dev::allreduce_twoshot_kernel<decltype(tin), decltype(tout), decltype(opv)>, blocks,
                          threads, st, dc.table(), a);
        });
    }
}

} // namespace gpu
} // namespace cclx
