// Launchers of the remaining GPU collectives (reduce_scatter, reduce,
// allgatherv, alltoallv, broadcast, barrier, point-to-point) and the local
// helper kernels.  Size thresholds follow the reference's structure
// (small / large variants, src/common/env/env.cpp:171-184) with values tuned
// for NVLink 5.
#include "gpu/launch_common.cuh"

namespace cclx {
namespace gpu {

namespace {
size_t r16(size_t b) {
    return (b + 15) & ~(size_t)15;
}
} // namespace

void launch_reduce_scatter(device_comm& dc, const dev::rank_args* ra, size_t rc, int dt_in, int dt_out, int op,
                           const launch_opts& o, cudaStream_t st) {
    if (rc == 0)
        return;
    const int W = dc.world();
    if (W == 1) { // a single rank keeps its only block: the copy / cast / scale path of allreduce
        launch_allreduce(dc, ra, rc, dt_in, dt_out, op, o, st);
        return;
    }
    const int entries = dc.emulated() ? W : 1;
    const size_t esz = predefined_dtype_size(dt_in), osz = predefined_dtype_size(dt_out);
    const int threads = dc.threads();
    dev::coll_args a{};
    a.scale = o.scale;
    a.do_scale = o.do_scale ? 1 : 0;

    // send buffers in the symmetric heap or in a registered allocation: pull (or NVLS) without staging
    // From five ranks on the in-switch reduction beats peer loads up to blocks of 64 MiB, and an ordinary send buffer
    // is better staged (chunk pipeline with the switch reducing) than shared up to 128 MiB in total (8 B200s,
    // bf16, 32 MiB: 70 us staged, 73 us symmetric NVLS, 97 us shared + peer loads, NCCL 85 us; from 128 MiB on
    // shared + peer loads is ahead: 247 against 259 us).
    const env_data& env0 = env_data::get();
    const bool many = dc.nvls() && nvls_type_ok(dt_in, op) && W >= std::max(env0.nvls_min_ranks, env0.nvls_staged_min_ranks);
    const size_t nvls_max_block = many ? env0.rs_nvls_max_block * 16 : env0.rs_nvls_max_block;
    zc_view vin, vnone;
    if (dt_in == dt_out)
        zero_copy_views(dc, ra, true, rc * esz * W, false, 0, vin, vnone, !(many && rc * esz * W < (128u << 20)));
    const bool symmetric = vin.ok;
    const size_t in_off = vin.off;
    (void)entries;
    int algo = o.algo;
    if (algo == ga_auto)
        algo = (symmetric && W > 1 && rc * esz > env_data::get().rs_small_threshold)
                   // the in-switch reduction wins while latency counts; large blocks are reduced faster from peer
                   // loads (measured on 4 B200s, 1 GiB: 1.28 ms by peer loads, 1.58 ms by multimem.ld_reduce, NCCL 1.38 ms)
                   ? ((dc.nvls() && nvls_type_ok(dt_in, op) && !vin.registered && W >= env_data::get().nvls_min_ranks &&
                       rc * esz <= nvls_max_block)
                          ? ga_nvls
                          : ga_symm)
                   : ga_push;
    if ((algo == ga_symm || algo == ga_nvls) && !symmetric)
        CCL_THROW("reduce_scatter algorithm ", gpu_algo_name(algo),
                  " needs a send buffer from the symmetric heap or from a registered allocation");
    if (algo == ga_nvls && (!dc.nvls() || !nvls_type_ok(dt_in, op) || vin.registered))
        algo = ga_symm;
    if (algo == ga_push && o.algo == ga_auto && W > 1 && rc * esz * W >= env_data::get().rs_pipelined_min)
        algo = ga_pipelined;
    dc.algo_hits[coll_reduce_scatter * ga_last + algo]++;

    if (algo == ga_symm || algo == ga_nvls) {
        a.count = rc;
        a.in_off = in_off;
        if (vin.registered)
            fill_registered(dc, a, vin, false);
        prepare_args(dc, a, ra, st);
        const int blocks = pick_blocks(dc, rc * esz / 16 + 1, 1024, o.blocks);
        CCLX_DISPATCH_DTYPE(dt_in, T, {
            if (algo == ga_nvls) {
                if constexpr (std::is_same<T, float>::value || std::is_same<T, __nv_bfloat16>::value ||
                              std::is_same<T, __half>::value)
                    launch_kernel(dc, dev::reduce_scatter_symm_kernel<T, dev::op_sum, true>, blocks, threads, st,
                                  dc.table(), a);
            }
            else {
                CCLX_DISPATCH_OP(op, OP,
                                 launch_kernel(dc, dev::reduce_scatter_symm_kernel<T, OP, false>, blocks, threads,
                                               st, dc.table(), a));
            }
        });
        return;
    }

    // large ordinary buffers: chunk pipeline (staging copy of chunk j under the reduction of chunk j-1)
    const env_data& env = env_data::get();
    if (algo == ga_pipelined && W > 1) {
        const size_t rpacks = r16(rc * esz) / 16;
        int blocks = o.blocks > 0 ? o.blocks : env.ar_pipelined_blocks;
        blocks = std::max(1, std::min(blocks, dc.max_blocks()));
        while (blocks > 1 && rpacks < (size_t)blocks * 256)
            blocks /= 2;
        size_t cs = dc.staging_bytes() / (2 * 16 * (size_t)W) / blocks * blocks;
        CCL_THROW_IF_NOT(cs >= (size_t)blocks, "staging buffer too small for the pipelined reduce_scatter");
        cs = std::min(cs, (rpacks + blocks - 1) / blocks * blocks);
        a.count = rc;
        a.stride = rc;
        a.in_off = cs;
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
                    launch_kernel(dc, dev::reduce_scatter_pipelined_kernel<T, Tout, OP, true>, blocks, threads, st,
                                  dc.table(), a);
                    return;
                }
            }
            launch_kernel(dc, dev::reduce_scatter_pipelined_kernel<T, Tout, OP, false>, blocks, threads, st,
                          dc.table(), a);
        });
        return;
    }

    // staged push, chunked over the per-rank block so that world slots fit
    const size_t N = 16 / esz;
    size_t max_packs = dc.staging_bytes() / 16 / W;
    CCL_THROW_IF_NOT(max_packs >= 1, "staging buffer too small for reduce_scatter");
    const size_t chunk = max_packs * N;
    std::vector<dev::rank_args> cur(ra, ra + entries);
    if (rc <= chunk) {
        a.count = rc;
        a.stride = rc;
        prepare_args(dc, a, ra, st);
        const int blocks = pick_blocks(dc, r16(rc * esz) / 16, 512, o.blocks);
        dispatch_reduce_types(dt_in, dt_out, op, [&](auto tin, auto tout, auto opv) {
            launch_kernel(dc, dev::reduce_scatter_kernel<decltype(tin), decltype(tout), decltype(opv)>, blocks,
                          threads, st, dc.table(), a);
        });
        return;
    }
    // large: chunks of every rank block, addressed through the block stride
    for (size_t done = 0; done < rc; done += chunk) {
        const size_t n = std::min(chunk, rc - done);
        for (int e = 0; e < entries; e++) {
            cur[e].send = (const char*)ra[e].send + done * esz;
            cur[e].recv = (char*)ra[e].recv + done * osz;
        }
        a.count = n;
        a.stride = rc;
        prepare_args(dc, a, cur.data(), st);
        const int blocks = pick_blocks(dc, r16(n * esz) / 16, 1024, o.blocks);
        dispatch_reduce_types(dt_in, dt_out, op, [&](auto tin, auto tout, auto opv) {
            launch_kernel(dc, dev::reduce_scatter_kernel<decltype(tin), decltype(tout), decltype(opv)>, blocks,
                          threads, st, dc.table(), a);
        });
    }
}

void launch_reduce(device_comm& dc, const dev::rank_args* ra, size_t count, int dt_in, int dt_out, int op, int root,
                   const launch_opts& o, cudaStream_t st) {
    if (count == 0)
        return;
    const int W = dc.world();
    const int entries = dc.emulated() ? W : 1;
    const size_t esz = predefined_dtype_size(dt_in), osz = predefined_dtype_size(dt_out);
    const size_t N = 16 / esz;
    size_t max_packs = dc.staging_bytes() / 16 / W;
    const size_t chunk = max_packs * N;
    dev::coll_args a{};
    a.scale = o.scale;
    a.do_scale = o.do_scale ? 1 : 0;
    a.root = root;
    dc.algo_hits[coll_reduce * ga_last + ga_push]++;
    std::vector<dev::rank_args> cur(ra, ra + entries);
    for (size_t done = 0; done < count; done += chunk) {
        const size_t n = std::min(chunk, count - done);
        for (int e = 0; e < entries; e++) {
            cur[e].send = (const char*)ra[e].send + done * esz;
            cur[e].recv = ra[e].recv ? (char*)ra[e].recv + done * osz : nullptr;
        }
        a.count = n;
        prepare_args(dc, a, cur.data(), st);
        const int blocks = pick_blocks(dc, r16(n * esz) / 16, 1024, o.blocks);
        dispatch_reduce_types(dt_in, dt_out, op, [&](auto tin, auto tout, auto opv) {
            launch_kernel(dc, dev::reduce_kernel<decltype(tin), decltype(tout), decltype(opv)>, blocks,
                          dc.threads(), st, dc.table(), a);
        });
    }
}

void launch_barrier(device_comm& dc, cudaStream_t st);

void launch_allgatherv(device_comm& dc, const dev::rank_args* ra, const launch_opts& o, cudaStream_t st) {
    const int W = dc.world();
    const int entries = dc.emulated() ? W : 1;
    size_t total = 0, maxb = 0, rounded = 0;
    for (int p = 0; p < W; p++) {
        total += ra[0].scount[p];
        maxb = std::max(maxb, ra[0].scount[p]);
        rounded += r16(ra[0].scount[p]);
    }
    if (total == 0)
        return;
    const int threads = dc.threads();
    dev::coll_args a{};

    // equal 16-byte-multiple blocks into a symmetric or registered recv buffer: direct stores
    zc_view vout, vnone;
    if (W > 1)
        zero_copy_views(dc, ra, false, 0, true, total, vnone, vout);
    bool symm = vout.ok;
    const size_t out_off = vout.off;
    for (int p = 0; p < W && symm; p++)
        if (ra[0].scount[p] != maxb || (maxb & 15) || ra[0].sdispl[p] != (size_t)p * maxb)
            symm = false;

    int algo = o.algo;
    if (algo == ga_auto) {
        if (W == 1)
            algo = ga_copy;
        else if (symm && maxb > env_data::get().ag_small_threshold && env_data::get().cuda_copy_engine)
            algo = ga_ce; // CCL_CUDA_COPY_ENGINE=1: large blocks move by the copy engines, the SMs stay free
        else if (symm && (maxb > env_data::get().ag_small_threshold || vout.registered))
            // one multimem.st reaches every peer, which wins while latency counts; large blocks move faster as
            // plain peer stores (measured on 4 B200s: 1 GiB gathered in 1.27 ms by peer stores, 1.55 ms by multimem.st)
            algo = (dc.nvls() && !vout.registered && W >= env_data::get().nvls_min_ranks &&
                    maxb <= env_data::get().ag_nvls_max_block)
                       ? ga_nvls
                       : ga_symm;
        else if (maxb <= env_data::get().ag_small_threshold && rounded <= dc.staging_bytes())
            algo = ga_push;
        else
            algo = ga_pull;
    }
    if (algo == ga_ce) {
        // Copy engines instead of SMs (the reference's copy-engine allgather, src/coll/algorithms/allgatherv/
        // sycl/allgatherv_large_sycl_impl.hpp:77-200): barrier, every rank pulls the peers' blocks out of
        // their recv buffers with asynchronous copies, barrier.  Between the two tiny barrier kernels no
        // SM is busy, so a concurrent GEMM keeps the whole GPU.
        CCL_THROW_IF_NOT(symm, "allgather algorithm ce needs equal 16-byte-multiple blocks and a recv buffer from the "
                               "symmetric heap or a registered allocation");
        dc.algo_hits[coll_allgatherv * ga_last + ga_ce]++;
        for (int e = 0; e < entries; e++) {
            const int r = dc.emulated() ? e : dc.rank();
            char* mine = (char*)ra[e].recv + (size_t)r * maxb;
            if (ra[e].send && ra[e].send != mine)
                CUDA_CHECK(cudaMemcpyAsync(mine, ra[e].send, maxb, cudaMemcpyDeviceToDevice, st));
        }
        launch_barrier(dc, st); // every block sits in its owner's recv buffer
        for (int e = 0; e < entries; e++) {
            const int r = dc.emulated() ? e : dc.rank();
            for (int k = 1; k < W; k++) {
                const int p = (r + k) % W;
                const char* peer = vout.registered ? view_ptr(dc, vout, p) : dc.heap().base(p) + out_off;
                CUDA_CHECK(cudaMemcpyAsync((char*)ra[e].recv + (size_t)p * maxb, peer + (size_t)p * maxb, maxb,
                                           cudaMemcpyDeviceToDevice, st));
            }
        }
        launch_barrier(dc, st); // nobody overwrites its block while a peer still reads it
        return;
    }
    if ((algo == ga_symm || algo == ga_nvls) && !symm)
        CCL_THROW("allgather algorithm ", gpu_algo_name(algo),
                  " needs equal 16-byte-multiple blocks and a recv buffer from the symmetric heap");
    if (algo == ga_nvls && (!dc.nvls() || vout.registered))
        algo = ga_symm;
    dc.algo_hits[coll_allgatherv * ga_last + algo]++;

    if (algo == ga_copy) {
        for (int e = 0; e < entries; e++) {
            const int r = dc.emulated() ? e : dc.rank();
            char* dst = (char*)ra[e].recv + ra[e].sdispl[r];
            if (ra[e].send && ra[e].send != dst)
                CUDA_CHECK(cudaMemcpyAsync(dst, ra[e].send, ra[e].scount[r], cudaMemcpyDeviceToDevice, st));
        }
        return;
    }
    if (algo == ga_symm || algo == ga_nvls) {
        a.count = maxb;
        a.out_off = out_off;
        if (vout.registered)
            fill_registered(dc, a, vout, true);
        prepare_args(dc, a, ra, st);
        const int blocks = pick_blocks(dc, maxb / 16, 2048, o.blocks);
        if (algo == ga_nvls)
            launch_kernel(dc, dev::allgather_symm_kernel<true>, blocks, threads, st, dc.table(), a);
        else
            launch_kernel(dc, dev::allgather_symm_kernel<false>, blocks, threads, st, dc.table(), a);
        return;
    }
    if (algo == ga_push && rounded > dc.staging_bytes())
        algo = ga_pull;
    if (algo == ga_push) {
        bool uniform = (maxb & 15) == 0;
        for (int p = 0; p < W && uniform; p++)
            uniform = ra[0].scount[p] == maxb && ra[0].sdispl[p] == (size_t)p * maxb;
        for (int e = 0; e < entries && uniform; e++)
            uniform = (((uintptr_t)ra[e].recv) & 15) == 0;
        a.flags = (dc.nvls() && W >= env_data::get().nvls_min_ranks ? dev::CF_NVLS : 0) |
                  (uniform ? dev::CF_UNIFORM : 0);
        prepare_args(dc, a, ra, st);
        const int blocks = pick_blocks(dc, r16(maxb) / 16, 1024, o.blocks);
        launch_kernel(dc, dev::allgatherv_kernel<true>, blocks, threads, st, dc.table(), a);
        return;
    }
    // pull, in rounds of at most one staging generation per block
    const size_t cap = dc.staging_bytes() & ~(size_t)15;
    std::vector<dev::rank_args> cur(ra, ra + entries);
    for (size_t done = 0; done < maxb; done += cap) {
        for (int e = 0; e < entries; e++) {
            const int r = dc.emulated() ? e : dc.rank();
            const char* src = ra[e].send ? (const char*)ra[e].send : (const char*)ra[e].recv + ra[e].sdispl[r];
            cur[e].send = src + done;
            for (int p = 0; p < W; p++) {
                size_t b = ra[e].scount[p] > done ? ra[e].scount[p] - done : 0;
                cur[e].scount[p] = std::min(b, cap);
                cur[e].sdispl[p] = ra[e].sdispl[p] + done;
            }
        }
        prepare_args(dc, a, cur.data(), st);
        const int blocks = pick_blocks(dc, std::min(cap, maxb - done) / 16 + 1, 2048, o.blocks);
        launch_kernel(dc, dev::allgatherv_kernel<false>, blocks, threads, st, dc.table(), a);
    }
}

void launch_alltoallv(device_comm& dc, const dev::rank_args* ra, const launch_opts& o, cudaStream_t st) {
    const int W = dc.world();
    const int entries = dc.emulated() ? W : 1;
    // local estimate only sizes the grid; the number of rounds is agreed inside the kernel
    size_t lmax = 0;
    for (int e = 0; e < entries; e++)
        for (int p = 0; p < W; p++)
            lmax = std::max(lmax, std::max(ra[e].scount[p], ra[e].rcount[p]));
    const size_t slot = (dc.staging_bytes() / W) & ~(size_t)15;
    CCL_THROW_IF_NOT(slot >= 16, "staging buffer too small for alltoallv");
    dev::coll_args a{};
    // equal blocks (alltoall): the block size is the same on every rank, so it may size the grid
    const size_t b = ra[0].scount[0];
    bool uniform = o.uniform && W > 1 && b > 0 && (b & 15) == 0;
    bool symm = uniform && o.algo != ga_push;
    for (int e = 0; e < entries && uniform; e++) {
        for (int p = 0; p < W; p++)
            uniform = uniform && ra[e].scount[p] == b && ra[e].rcount[p] == b && ra[e].sdispl[p] == (size_t)p * b &&
                      ra[e].rdispl[p] == (size_t)p * b;
        const bool aligned = ((((uintptr_t)ra[e].send) | ((uintptr_t)ra[e].recv)) & 15) == 0;
        if (!aligned || ra[e].send == ra[e].recv)
            symm = false;
        uniform = uniform && aligned;
    }
    // the direct path must be chosen by every rank or by none: it depends only on the block size and
    // on recv being a symmetric or registered allocation, which is a collective property
    zc_view vout, vnone;
    if (symm && uniform)
        zero_copy_views(dc, ra, false, 0, true, b * W, vnone, vout);
    symm = symm && vout.ok;
    const size_t out_off = vout.off;
    symm = symm && uniform;
    if (symm) {
        dc.algo_hits[coll_alltoallv * ga_last + ga_symm]++;
        a.count = b;
        a.out_off = out_off;
        if (vout.registered)
            fill_registered(dc, a, vout, true);
        prepare_args(dc, a, ra, st);
        const int blocks = pick_blocks(dc, b / 16, 512, o.blocks);
        launch_kernel(dc, dev::alltoall_symm_kernel, blocks, dc.threads(), st, dc.table(), a);
        return;
    }
    dc.algo_hits[coll_alltoallv * ga_last + ga_push]++;
    a.flags = uniform ? dev::CF_UNIFORM : 0;
    prepare_args(dc, a, ra, st);
    // every rank must use the same grid: derive it from what all ranks know (the common block size
    // of an alltoall, else a fixed size), never from local counts
    (void)lmax;
    int blocks;
    if (o.blocks > 0)
        blocks = pick_blocks(dc, 1, 1, o.blocks);
    else if (o.uniform)
        blocks = pick_blocks(dc, std::min(b, slot) / 16 + 1, 512, 0);
    else
        blocks = std::min(dc.max_blocks(), 32);
    launch_kernel(dc, dev::alltoallv_kernel, blocks, dc.threads(), st, dc.table(), a);
}

void launch_broadcast(device_comm& dc, const dev::rank_args* ra, size_t bytes, int root, const launch_opts& o,
                      cudaStream_t st) {
    if (bytes == 0)
        return;
    const int W = dc.world();
    const int entries = dc.emulated() ? W : 1;
    if (W == 1) {
        if (ra[0].send != ra[0].recv)
            CUDA_CHECK(cudaMemcpyAsync(ra[0].recv, ra[0].send, bytes, cudaMemcpyDeviceToDevice, st));
        return;
    }
    dc.algo_hits[coll_broadcast * ga_last + (dc.nvls() ? ga_nvls : ga_push)]++;
    const size_t cap = dc.staging_bytes() & ~(size_t)15;
    dev::coll_args a{};
    a.root = root;
    a.flags = dc.nvls() ? dev::CF_NVLS : 0;
    std::vector<dev::rank_args> cur(ra, ra + entries);
    for (size_t done = 0; done < bytes; done += cap) {
        const size_t n = std::min(cap, bytes - done);
        for (int e = 0; e < entries; e++) {
            cur[e].send = ra[e].send ? (const char*)ra[e].send + done : nullptr;
            cur[e].recv = (char*)ra[e].recv + done;
        }
        a.count = n;
        prepare_args(dc, a, cur.data(), st);
        const int blocks = pick_blocks(dc, n / 16 + 1, 2048, o.blocks);
        launch_kernel(dc, dev::broadcast_kernel, blocks, dc.threads(), st, dc.table(), a);
    }
}

void launch_barrier(device_comm& dc, cudaStream_t st) {
    if (dc.world() == 1)
        return;
    dev::coll_args a{};
    dev::rank_args dummy[dev::MAX_RANKS] = {};
    prepare_args(dc, a, dummy, st);
    dc.algo_hits[coll_barrier * ga_last + ga_push]++;
    launch_kernel(dc, dev::barrier_kernel, 1, 64, st, dc.table(), a);
}

void launch_sendrecv(device_comm& dc, const dev::p2p_ops* ops, cudaStream_t st) {
    const int entries = dc.emulated() ? dc.world() : 1;
    size_t maxb = 0;
    int max_n = 0;
    for (int e = 0; e < entries; e++) {
        CCL_THROW_IF_NOT(ops[e].n >= 0 && ops[e].n <= dev::P2P_MAX_OPS, "too many point-to-point operations in one launch");
        max_n = std::max(max_n, ops[e].n);
        for (int i = 0; i < ops[e].n; i++) {
            const dev::p2p_op& o = ops[e].op[i];
            if (o.peer < 0)
                continue;
            CCL_THROW_IF_NOT(o.peer < dc.world(), "invalid peer ", o.peer);
            maxb = std::max(maxb, o.bytes);
            dc.algo_hits[(o.is_send ? coll_send : coll_recv) * ga_last + ga_push]++;
            for (int k = 0; k < i; k++)
                CCL_THROW_IF_NOT(ops[e].op[k].peer != o.peer || ops[e].op[k].is_send != o.is_send,
                                 "two operations of one launch address the same peer in the same direction");
        }
    }
    if (max_n == 0)
        return;
    dc.check_status();
    const dev::p2p_ops* tab = nullptr;
    if (dc.emulated()) {
        CUDA_CHECK(cudaStreamSynchronize(st));
        CUDA_CHECK(cudaMemcpy(dc.emu_ops_dev(), ops, entries * sizeof(dev::p2p_ops), cudaMemcpyHostToDevice));
        tab = dc.emu_ops_dev();
    }
    const int emu = dc.emulated() ? 1 : 0;
    // Blocks wait for the peer's blocks, so all blocks of a launch must be resident at once: the lanes of an
    // operation are shared out among as many blocks as fit (each side decides for itself; the lane a chunk
    // travels through depends on the byte count alone).
    const int threads = 1024; // one control warp and 31 warps that copy
    const int fit = resident_blocks(dc, dev::sendrecv_kernel, threads) / (entries * max_n);
    CCL_THROW_IF_NOT(fit >= 1, "point-to-point launch of ", entries * max_n, " operations does not fit the GPU");
    const dev::p2p_layout L = dc.p2p();
    const size_t chunks = std::max<size_t>(1, (maxb + dev::P2P_CHUNK_BYTES - 1) / dev::P2P_CHUNK_BYTES);
    int blocks = (int)std::min<size_t>(std::min(fit, L.lanes), chunks);
    if (env_data::get().p2p_max_blocks > 0)
        blocks = std::min(blocks, env_data::get().p2p_max_blocks);
    dim3 grid(blocks, entries, max_n);
    const dev::comm_dev* t = dc.table();
    dev::p2p_ops r0 = ops[0];
    if (dc.emulated()) {
        void* argv[] = { (void*)&t, (void*)&L, (void*)&r0, (void*)&tab, (void*)&emu };
        CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)dev::sendrecv_kernel, grid, dim3(threads), argv, 0, st));
    }
    else {
        dev::sendrecv_kernel<<<grid, threads, 0, st>>>(t, L, r0, tab, emu);
        CUDA_CHECK(cudaGetLastError());
    }
}

void launch_wait_unset_flag(device_comm& dc, cudaStream_t st) {
    dev::coll_args a{};
    dev::rank_args dummy[dev::MAX_RANKS] = {};
    prepare_args(dc, a, dummy, st);
    if (dc.emulated()) {
        void* argv[] = { (void*)nullptr, (void*)&a };
        const dev::comm_dev* t = dc.table();
        argv[0] = (void*)&t;
        CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)dev::wait_unset_flag_kernel, dim3(1, dc.world()),
                                               dim3(64), argv, 0, st));
    }
    else {
        dev::wait_unset_flag_kernel<<<1, 64, 0, st>>>(dc.table(), a);
        CUDA_CHECK(cudaGetLastError());
    }
}

void launch_reduce_local(const void* in, void* inout, size_t count, int dt, int op, cudaStream_t st) {
    if (count == 0)
        return;
    const int threads = 512;
    const int blocks = (int)std::min<size_t>((count + threads - 1) / threads, 148 * 4);
    CCLX_DISPATCH_DTYPE(dt, T, CCLX_DISPATCH_OP(op, OP, {
                            dev::reduce_local_kernel<T, OP><<<blocks, threads, 0, st>>>((const T*)in, (T*)inout, count);
                        }));
    CUDA_CHECK(cudaGetLastError());
}

// Block transpose: `in` holds rows x cols blocks of block_bytes each, row-major; `out` gets the same
// blocks column-major (block (r, c) moves to position c * rows + r).  A reduce_scatter across nodes
// needs it: send buffers are ordered by global rank (node-major), the node-level stage wants the
// blocks grouped by local rank (reference src/coll/algorithms/reduce_scatter/sycl/reduce_scatter_sycl.cpp:176-204).
template <class V>
__global__ void transpose_blocks_kernel(const V* __restrict__ in, V* __restrict__ out, int rows, int cols,
                                        size_t per_block) {
    const size_t total = (size_t)rows * (size_t)cols * per_block;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t blk = i / per_block, e = i - blk * per_block; // output block and offset inside it
        const size_t c = blk / (size_t)rows, r = blk - c * (size_t)rows;
        out[i] = in[(r * (size_t)cols + c) * per_block + e];
    }
}

void launch_transpose_blocks(const void* in, void* out, int rows, int cols, size_t block_bytes, cudaStream_t st) {
    if (rows <= 0 || cols <= 0 || block_bytes == 0)
        return;
    CCL_THROW_IF_NOT(in != out, "block transpose works out of place only");
    const bool wide = block_bytes % 16 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0;
    const size_t per_block = wide ? block_bytes / 16 : block_bytes;
    const size_t total = (size_t)rows * (size_t)cols * per_block;
    const int threads = 256;
    const int blocks = (int)std::min<size_t>((total + threads - 1) / threads, 148 * 8);
    if (wide)
        transpose_blocks_kernel<uint4><<<blocks, threads, 0, st>>>((const uint4*)in, (uint4*)out, rows, cols, per_block);
    else
        transpose_blocks_kernel<unsigned char>
            <<<blocks, threads, 0, st>>>((const unsigned char*)in, (unsigned char*)out, rows, cols, per_block);
    CUDA_CHECK(cudaGetLastError());
}

void launch_pack(const void* const* ptrs_dev, const size_t* offs_dev, const size_t* lens_dev, int n, void* fused,
                 bool unpack, size_t max_tensor_bytes, cudaStream_t st) {
    if (n <= 0)
        return;
    dev::pack_table t{ ptrs_dev, offs_dev, lens_dev, n };
    const int bx = (int)std::max<size_t>(1, std::min<size_t>(max_tensor_bytes / (64 << 10) + 1, 32));
    dim3 grid(bx, std::min(n, 1024));
    if (unpack)
        dev::pack_kernel<true><<<grid, 512, 0, st>>>(t, (char*)fused);
    else
        dev::pack_kernel<false><<<grid, 512, 0, st>>>(t, (char*)fused);
    CUDA_CHECK(cudaGetLastError());
}

void launch_allreduce_fused(device_comm& dc, const void* const* send, void* const* recv, const size_t* counts, int n,
                            int dt, int op, const launch_opts& o, cudaStream_t st) {
    if (n <= 0)
        return;
    const int W = dc.world();
    const int entries = dc.emulated() ? W : 1;
    const size_t esz = predefined_dtype_size(dt);
    typedef device_comm::fuse_state FS;
    FS& f = dc.fuse();
    const env_data& env = env_data::get();
    if (f.buf_off == (size_t)-1) {
        // first use (the same call on every rank: symmetric allocations are collective by program order)
        f.buf_bytes = std::max<size_t>(env.fusion_bytes_threshold * env.fusion_count_threshold, (size_t)4 << 20);
        char* p = (char*)dc.symm_alloc(f.buf_bytes, 0);
        f.buf_off = dc.symm_offset(p, dc.emulated() ? 0 : -1);
        const size_t per_entry = (size_t)FS::MAX_TENSORS * (sizeof(void*) + 2 * sizeof(size_t));
        CUDA_CHECK(cudaHostAlloc((void**)&f.tab_host, (size_t)FS::SLOTS * entries * per_entry, cudaHostAllocMapped));
        CUDA_CHECK(cudaHostGetDevicePointer((void**)&f.tab_dev, f.tab_host, 0));
        for (auto& e : f.used)
            CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    // per entry: MAX_TENSORS pointers (send then recv of a group), MAX_TENSORS offsets, MAX_TENSORS byte lengths
    const size_t per_entry = (size_t)FS::MAX_TENSORS * (sizeof(void*) + 2 * sizeof(size_t));

    auto single = [&](int k) {
        std::vector<dev::rank_args> ra(entries);
        for (int e = 0; e < entries; e++) {
            ra[e] = dev::rank_args{};
            ra[e].send = send[(size_t)k * entries + e];
            ra[e].recv = recv[(size_t)k * entries + e];
        }
        launch_allreduce(dc, ra.data(), counts[k], dt, dt, op, o, st);
    };

    int k = 0;
    while (k < n) {
        // next group: consecutive tensors whose 16-byte-rounded sizes fit the fused buffer
        if (r16(counts[k] * esz) > f.buf_bytes / 2) {
            single(k++);
            continue;
        }
        int first = k;
        size_t used = 0, biggest = 0;
        std::vector<size_t> offs;
        while (k < n && k - first < FS::MAX_TENSORS / 2 && r16(counts[k] * esz) <= f.buf_bytes / 2 &&
               used + r16(counts[k] * esz) <= f.buf_bytes) {
            offs.push_back(used);
            used += r16(counts[k] * esz);
            biggest = std::max(biggest, counts[k] * esz);
            k++;
        }
        const int m = k - first;
        if (m == 1) {
            single(first);
            continue;
        }
        // a table slot may be rewritten only when the kernels that read it have run
        const int slot = f.next;
        f.next = (f.next + 1) % FS::SLOTS;
        CUDA_CHECK(cudaEventSynchronize(f.used[slot]));
        std::vector<dev::rank_args> ra(entries);
        // Rounded slots leave up to 15 bytes of padding behind a tensor; the allreduce runs over `used` bytes, so the
        // padding is reduced too (whatever it holds) and never unpacked.
        for (int pass = 0; pass < 2; pass++) { // 0: send pointers for the pack, 1: recv pointers for the unpack
            if (pass == 1) {
                for (int e = 0; e < entries; e++) {
                    ra[e] = dev::rank_args{};
                    ra[e].send = ra[e].recv = dc.heap().base(dc.emulated() ? e : dc.rank()) + f.buf_off;
                }
                launch_allreduce(dc, ra.data(), used / esz, dt, dt, op, o, st);
            }
            for (int e = 0; e < entries; e++) {
                char* th = f.tab_host + ((size_t)(slot * entries + e)) * per_entry;
                char* td = f.tab_dev + ((size_t)(slot * entries + e)) * per_entry;
                // pack and unpack read different halves of the pointer table: [0, m) send, [m, 2m) recv
                const void** ptrs = (const void**)th;
                size_t* of = (size_t*)(th + (size_t)FS::MAX_TENSORS * sizeof(void*));
                size_t* ln = of + FS::MAX_TENSORS;
                if (pass == 0) {
                    for (int j = 0; j < m; j++) {
                        ptrs[j] = send[(size_t)(first + j) * entries + e];
                        ptrs[m + j] = recv[(size_t)(first + j) * entries + e];
                        of[j] = offs[j];
                        ln[j] = counts[first + j] * esz;
                    }
                }
                char* fused = dc.heap().base(dc.emulated() ? e : dc.rank()) + f.buf_off;
                const void* const* pd = (const void* const*)td + (pass == 0 ? 0 : m);
                const size_t* od = (const size_t*)(td + (size_t)FS::MAX_TENSORS * sizeof(void*));
                launch_pack(pd, od, od + FS::MAX_TENSORS, m, fused, pass == 1, biggest, st);
            }
        }
        CUDA_CHECK(cudaEventRecord(f.used[slot], st));
        f.batches++;
        f.tensors += m;
    }
}

} // namespace gpu
} // namespace cclx
