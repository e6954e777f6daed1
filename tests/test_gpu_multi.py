"""Real multi-GPU path: one process per GPU, symmetric heaps exchanged over
Unix sockets, device kernels driven through the Communicator API.  Skipped on
boxes with a single GPU (the emulated tests cover the kernels there)."""
import os

import pytest
import torch

from mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


needs2 = pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
ENV = {"CCL_CUDA_SYMM_HEAP_SIZE": "512M", "CCL_CUDA_TMP_BUF_SIZE": "16M", "CCL_CUDA_WAIT_TIMEOUT_MS": "5000"}


def _world():
    return min(_ngpu(), 8)


def _collectives(comm):
    r, W = comm.rank, comm.size
    torch.cuda.set_device(r)
    dev = torch.device("cuda", r)
    g = comm.device_group
    out = {"nvls": g.nvls}
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        for n in (1, 17, 4096, 262144, 3 * (1 << 20) + 5):
            gen = [torch.Generator().manual_seed(100 + p) for p in range(W)]
            xs = [(torch.rand(n, generator=gen[p]) * 2 - 1).to(dtype) for p in range(W)]
            ref = torch.stack([x.double() for x in xs]).sum(0)
            x = xs[r].to(dev)
            y = torch.empty_like(x)
            comm.allreduce(x, y).wait()
            assert torch.allclose(y.double().cpu(), ref, rtol=tol, atol=tol * W), (dtype, n)
            comm.allreduce(x).wait()  # in place
            assert torch.allclose(x.double().cpu(), ref, rtol=tol, atol=tol * W), (dtype, n, "inplace")
    # symmetric (registered) buffers: zero-copy two-shot, NVLS when the switch offers it
    for n in (1000, 5 << 20):  # the large one is beyond the one-shot range of every world size (8 MiB between two ranks)
        s = g.symm_empty((n,), dtype=torch.float32)
        s.copy_(torch.full((n,), float(r + 1), device=dev))
        comm.allreduce(s).wait()
        assert torch.all(s == W * (W + 1) / 2)
        sb = g.symm_empty((n,), dtype=torch.bfloat16)
        sb.copy_(torch.full((n,), float(r + 1), device=dev).to(torch.bfloat16))
        comm.allreduce(sb, scale=1.0 / W).wait()
        assert torch.allclose(sb.float(), torch.full((n,), (W + 1) / 2, device=dev), rtol=1e-2, atol=1e-2)
        g.symm_free(s)
        g.symm_free(sb)
    out["ar_symm_hits"] = g.algo_hits("allreduce", "symm") + g.algo_hits("allreduce", "nvls")
    # an ordinary torch allocation registered through CUDA IPC: peers read and write it directly
    n = 3 << 20
    plain = torch.full((n + 128,), float(r + 1), device=dev)
    rid = g.register(plain)
    view = plain[64:64 + n]
    before = g.algo_hits("allreduce", "symm")
    comm.allreduce(view).wait()
    torch.cuda.synchronize()
    assert g.algo_hits("allreduce", "symm") == before + 1
    assert torch.all(view == W * (W + 1) / 2) and torch.all(plain[:64] == r + 1) and torch.all(plain[64 + n:] == r + 1)
    gathered = torch.zeros(W * 4096, device=dev)
    rid2 = g.register(gathered)
    g.allgatherv(torch.full((4096,), float(r), device=dev), gathered, algo="symm")
    torch.cuda.synchronize()
    assert torch.equal(gathered, torch.arange(W, device=dev, dtype=torch.float32).repeat_interleave(4096))
    g.deregister(rid)
    g.deregister(rid2)
    # reduce_scatter / allgather / alltoall / broadcast / reduce
    n = 5000
    x = (torch.arange(n * W, dtype=torch.float32) + r).to(dev)
    y = torch.empty(n, device=dev)
    comm.reduce_scatter(x, y).wait()
    assert torch.allclose(y.cpu(), (torch.arange(n * W, dtype=torch.float32)[r * n:(r + 1) * n] * W + sum(range(W))))
    z = torch.empty(n * W, device=dev)
    comm.allgather(y, z).wait()
    assert torch.allclose(z.cpu(), torch.arange(n * W, dtype=torch.float32) * W + sum(range(W)))
    counts = [100 + 11 * p for p in range(W)]
    zz = torch.zeros(sum(counts), device=dev)
    comm.allgatherv(torch.full((counts[r],), float(r), device=dev), zz, counts).wait()
    assert torch.equal(zz.cpu(), torch.cat([torch.full((c,), float(p)) for p, c in enumerate(counts)]))
    a = (torch.arange(W * 300, dtype=torch.float32) + 10000 * r).to(dev)
    b = torch.empty_like(a)
    comm.alltoall(a, b).wait()
    refb = torch.cat([torch.arange(300, dtype=torch.float32) + 300 * r + 10000 * p for p in range(W)])
    assert torch.equal(b.cpu(), refb)
    for root in (0, W - 1):
        t = torch.full((70001,), float(r), device=dev)
        comm.broadcast(t, root=root).wait()
        assert torch.all(t == root)
        o = torch.zeros(999, device=dev)
        comm.reduce(torch.full((999,), float(r + 1), device=dev), o, root=root).wait()
        if r == root:
            assert torch.all(o == W * (W + 1) / 2)
    # send / recv, alone and batched in a group (both directions at once)
    from oneccl_b200.comm import group_end, group_start

    nxt, prv = (r + 1) % W, (r - 1) % W
    m = torch.full((200000,), float(r), device=dev)
    got = torch.zeros_like(m)
    if W == 2:
        if r == 0:
            comm.send(m, 1).wait()
            comm.recv(got, 1).wait()
        else:
            comm.recv(got, 0).wait()
            comm.send(m, 0).wait()
        assert torch.all(got == prv)
    got.zero_()
    group_start()
    e1 = comm.send(m, nxt)
    e2 = comm.recv(got, prv)
    group_end()
    e1.wait()
    e2.wait()
    assert torch.all(got == prv)
    comm.barrier().wait()
    torch.cuda.synchronize()
    g.check()
    return out


@needs2
def test_device_collectives_real():
    res = run_ranks(_collectives, _world(), env=ENV, timeout=300)
    assert all(r["ar_symm_hits"] >= 2 for r in res)


@needs2
def test_device_collectives_real_nvls_off():
    env = dict(ENV, CCL_CUDA_NVLS="0")
    res = run_ranks(_collectives, 2, env=env, timeout=300)
    assert not any(r["nvls"] for r in res)


def _fused(comm):
    from oneccl_b200.ops.gemm import FusedPlan

    r, W = comm.rank, comm.size
    torch.cuda.set_device(r)
    dev = torch.device("cuda", r)
    g = comm.device_group
    M, N, K = W * 256, 512, 256
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(M, K, generator=gen).to(torch.bfloat16)
    ws = [(torch.randn(N, K, generator=gen) * 0.1).to(torch.bfloat16) for _ in range(W)]
    per = M // W
    plan = FusedPlan(g, "ag_gemm", M, N, K, epilogue="silu", n_comm=4)
    for it in range(3):
        plan.x_shard(r).copy_((x[r * per:(r + 1) * per] * (it + 1)).to(dev))
        out = plan.run(None, ws[r].to(dev))
        torch.cuda.synchronize()
        assert plan.error() == 0
        ref = torch.nn.functional.silu((x * (it + 1)).float() @ ws[r].float().t())
        err = (out.float().cpu() - ref).abs().max().item()
        assert err < 2e-2 * ref.abs().max().item() + 1e-3, err
    plan.close()
    # GEMM -> reduce-scatter
    K2 = 192
    hs = [torch.randn(M, K2, generator=gen).to(torch.bfloat16) for _ in range(W)]
    w2 = [(torch.randn(N, K2, generator=gen) * 0.1).to(torch.bfloat16) for _ in range(W)]
    full = sum((h.float() @ w.float().t()).to(torch.bfloat16).float() for h, w in zip(hs, w2))
    plan2 = FusedPlan(g, "gemm_rs", M, N, K2)
    for it in range(3):
        out = plan2.run(hs[r].to(dev), w2[r].to(dev))
        torch.cuda.synchronize()
        assert plan2.error() == 0
        ref = full[r * per:(r + 1) * per]
        err = (out.float().cpu() - ref).abs().max().item()
        assert err < 2e-2 * ref.abs().max().item() + 1e-3, err
    plan2.close()
    g.check()
    return True


def _auto_shared(comm):
    """Ordinary torch tensors, at a different offset of their allocation on every rank and re-allocated between
    iterations (the reference's dynamic-pointer mode, tests/functional/test_impl.hpp:326-372): from 256 KiB on
    the ranks exchange allocation handles by themselves and the zero-copy kernels run."""
    r, W = comm.rank, comm.size
    torch.cuda.set_device(r)
    dev = torch.device("cuda", r)
    g = comm.device_group
    n = 3 << 20  # 12 MiB of float32: beyond the one-shot range of every world size
    keep = []
    for it in range(4):
        pad = 16 * (r + it)
        raw = torch.empty(n + 4096, device=dev)
        x = raw[pad:pad + n]
        x.fill_(float(r + 1))
        # from five ranks on, where the switch can reduce, allreduce stages ordinary buffers for it instead
        algo = "pipelined" if (g.nvls and W >= 5) else "symm"
        before = g.algo_hits("allreduce", algo)
        comm.allreduce(x).wait()
        torch.cuda.synchronize()
        assert g.algo_hits("allreduce", algo) == before + 1, "ordinary buffers did not take the expected kernel"
        assert torch.all(x == W * (W + 1) / 2)
        # reduce_scatter: zero-copy on the send side; allgather / alltoall: on the recv side
        per = 1 << 17
        send = torch.arange(per * W, device=dev, dtype=torch.float32) + r
        out = torch.empty(per + 64, device=dev)[32 + 4 * r:32 + 4 * r + per]
        comm.reduce_scatter(send, out).wait()
        ref = torch.arange(per * W, dtype=torch.float32)[r * per:(r + 1) * per] * W + sum(range(W))
        assert torch.equal(out.cpu(), ref)
        gathered = torch.empty(per * W + 256, device=dev)[4 * r:4 * r + per * W]
        comm.allgather(out, gathered).wait()
        assert torch.equal(gathered.cpu(), torch.arange(per * W, dtype=torch.float32) * W + sum(range(W)))
        a = (torch.arange(per * W, dtype=torch.float32) + 1e6 * r).to(dev)
        b = torch.empty(per * W + 128, device=dev)[8 * r:8 * r + per * W]
        comm.alltoall(a, b).wait()
        refb = torch.cat([torch.arange(per, dtype=torch.float32) + per * r + 1e6 * p for p in range(W)])
        assert torch.equal(b.cpu(), refb)
        if it % 2 == 0:
            keep.append(raw)  # some allocations stay, some are freed and their addresses reused
        del raw, x, send, out, gathered, a, b
    torch.cuda.synchronize()
    g.check()
    return True


@needs2
def test_ordinary_buffers_are_shared_automatically():
    assert all(run_ranks(_auto_shared, _world(), env=ENV, timeout=300))


def _mismatch(comm):
    """Two ranks pass different offsets of a symmetric buffer to a small (locally decided) zero-copy allreduce:
    the kernels notice at their first barrier and report ST_ARG_MISMATCH instead of reducing the wrong bytes."""
    from oneccl_b200 import CclError

    r = comm.rank
    torch.cuda.set_device(r)
    g = comm.device_group
    s = g.symm_empty((4096,), dtype=torch.float32)
    s.fill_(float(r + 1))
    torch.cuda.synchronize()
    g.barrier()
    view = s[16 * r:16 * r + 1000]
    g.allreduce(view, view, algo="symm")
    torch.cuda.synchronize()
    code = g.status()
    raised = False
    try:
        g.check()
    except CclError:
        raised = True
    untouched = bool(torch.all(s == float(r + 1)))
    g.clear_status()
    g.barrier()
    g.allreduce(s, s, algo="symm")
    torch.cuda.synchronize()
    g.check()
    return code, raised, untouched, float(s[0])


@needs2
def test_unequal_symmetric_offsets_are_reported():
    res = run_ranks(_mismatch, 2, env=ENV, timeout=120)
    for code, raised, untouched, total in res:
        assert code == 7 and raised and untouched and total == 3.0, res


@needs2
def test_fused_gemm_real():
    assert all(run_ranks(_fused, _world(), env=ENV, timeout=300))


def _ddp(comm):
    from oneccl_b200.models.gpt2 import GPT2, GPT2Config
    from oneccl_b200.parallel.ddp import DataParallel, train_step

    r, W = comm.rank, comm.size
    torch.cuda.set_device(r)
    torch.manual_seed(0)  # same initial weights everywhere; rank 0's are broadcast anyway
    cfg = GPT2Config.named("gpt2-tiny")
    model = GPT2(cfg).cuda().to(torch.bfloat16)
    ddp = DataParallel(model, comm.device_group, bucket_mb=0.05)
    opt = ddp.make_optimizer(lr=1e-3)
    gen = torch.Generator().manual_seed(77)
    idx = torch.randint(0, cfg.vocab, (W * 2, cfg.seq_len), generator=gen)
    tgt = torch.randint(0, cfg.vocab, (W * 2, cfg.seq_len), generator=gen)
    losses = []
    for _ in range(4):
        loss = train_step(ddp, opt, idx[2 * r:2 * r + 2].cuda(), tgt[2 * r:2 * r + 2].cuda())
        losses.append(float(loss))
    torch.cuda.synchronize()
    # every replica holds identical weights after synchronous data-parallel steps
    digest = ddp.flat_param.float().double().sum().item()
    return losses, digest, len(ddp.buckets)


@needs2
def test_data_parallel_replicas_stay_identical():
    res = run_ranks(_ddp, 2, env=ENV, timeout=300)
    assert res[0][1] == res[1][1]
    assert res[0][2] > 1  # several buckets were reduced
    assert res[0][0][-1] < res[0][0][0]


def _leaver(comm):
    """Failure detection without a GPU fault: rank 1 leaves between steps (nothing in
    flight); rank 0 learns it on the host through the heartbeat keys and, if it launches
    anyway, its device wait runs out and reports a status instead of hanging."""
    import time

    r = comm.rank
    torch.cuda.set_device(r)
    g = comm.device_group
    x = torch.ones(1000, device="cuda")
    comm.heartbeat()
    comm.allreduce(x).wait()
    torch.cuda.synchronize()
    if r == 1:
        return "left"
    time.sleep(1.5)
    alive = comm.peer_alive(1, max_age_ms=500)
    g.set_timeout_ms(700)
    status = None
    try:
        comm.allreduce(x).wait()
    except Exception as e:  # noqa: BLE001
        status = str(e)
    code = g.status()
    # the context is still usable
    y = torch.ones(10, device="cuda") * 3
    torch.cuda.synchronize()
    return alive, code, status is not None, float(y.sum())


@needs2
def test_rank_leaving_is_detected_on_host_and_device_wait_is_bounded():
    import multiprocessing as mp
    import tempfile
    import time

    env = dict(ENV, CCL_CUDA_NVLS="0")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    addr = os.path.join(tempfile.mkdtemp(prefix="cclx_"), "addr")

    procs = [ctx.Process(target=_child_noclose, args=(rk, 2, addr, q, env)) for rk in range(2)]
    for p in procs:
        p.start()
    got = {}
    t0 = time.time()
    while len(got) < 2 and time.time() - t0 < 120:
        try:
            rk, st, out = q.get(timeout=1)
            got[rk] = (st, out)
        except Exception:
            pass
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.terminate()
    assert got[1] == ("ok", "left")
    st, out = got[0]
    assert st == "ok", out
    alive, code, raised, ysum = out
    assert alive is False
    assert code == 1 and raised  # ST_BARRIER_TIMEOUT reported through the status word
    assert ysum == 30.0


def _child_noclose(rank, world, addr_file, q, env):
    """Like mp_util._child but without the closing barrier: one rank leaves early on purpose."""
    import time
    import traceback

    try:
        os.environ.update(env)
        from oneccl_b200.comm import KVS, Communicator

        if rank == 0:
            kvs = KVS.create_main()
            with open(addr_file + ".tmp", "w") as f:
                f.write(kvs.address)
            os.replace(addr_file + ".tmp", addr_file)
        else:
            t0 = time.time()
            while not os.path.exists(addr_file):
                if time.time() - t0 > 60:
                    raise RuntimeError("no kvs address")
                time.sleep(0.01)
            kvs = KVS.connect(open(addr_file).read())
        comm = Communicator(world, rank, kvs)
        out = _leaver(comm)
        q.put((rank, "ok", out))
        q.close()
        q.join_thread()  # the result must reach the parent before the hard exit below
        # leave without the collective teardown (the peer is gone or about to go)
        os._exit(0)
    except Exception:
        q.put((rank, "error", traceback.format_exc()))
        q.close()
        q.join_thread()


def _tp_and_moe(comm):
    from oneccl_b200.parallel.ep import ExpertParallelMoE, reference_moe
    from oneccl_b200.parallel.tp import TensorParallelMLP

    r, W = comm.rank, comm.size
    torch.cuda.set_device(r)
    g = comm.device_group
    # tensor-parallel MLP: fused kernels against separate collectives + cuBLAS
    tokens, d_model, d_ff = W * 128, 256, W * 128
    mlp = TensorParallelMLP(g, tokens, d_model, d_ff, n_comm=2)
    gen = torch.Generator(device="cuda").manual_seed(100 + r)
    x_local = torch.randn(tokens // W, d_model, generator=gen, device="cuda").to(torch.bfloat16)
    for _ in range(2):
        mlp.x_shard.copy_(x_local)
        y = mlp.forward().float().clone()
        y_ref = mlp.forward_unfused(x_local).float()
        torch.cuda.synchronize()
        assert (y - y_ref).abs().max().item() < 3e-2 * y_ref.abs().max().item() + 1e-3
    mlp.close()
    # expert-parallel MoE against the dense restatement (all experts gathered on every rank)
    T, H, F = 96, 64, 128
    moe = ExpertParallelMoE(g, H, F, topk=2)
    x = torch.randn(T, H, generator=gen, device="cuda").to(torch.bfloat16)
    logits = torch.randn(T, W, generator=gen, device="cuda")
    out = moe(x, logits).float()
    w1s = [torch.empty_like(moe.w1) for _ in range(W)]
    w2s = [torch.empty_like(moe.w2) for _ in range(W)]
    w1all = torch.empty((W,) + tuple(moe.w1.shape), dtype=torch.bfloat16, device="cuda")
    w2all = torch.empty((W,) + tuple(moe.w2.shape), dtype=torch.bfloat16, device="cuda")
    g.allgatherv(moe.w1, w1all)
    g.allgatherv(moe.w2, w2all)
    torch.cuda.synchronize()
    ref = reference_moe(x, logits, list(w1all), list(w2all), topk=2)
    assert (out - ref).abs().max().item() < 3e-2 * ref.abs().max().item() + 1e-3
    out2 = moe.forward_alltoall(x, logits).float()
    assert (out2 - ref).abs().max().item() < 3e-2 * ref.abs().max().item() + 1e-3
    assert sum(moe.stats["sent_rows"]) == T * 2
    out3 = moe(x, logits).float()  # buffers and count table are reused
    assert torch.equal(out3, out)
    g.check()
    return True


@needs2
def test_tensor_parallel_mlp_and_moe():
    assert all(run_ranks(_tp_and_moe, _world(), env=ENV, timeout=300))


def _pipeline_cuda(comm):
    """GPipe over device send / recv: stream-ordered transfers, activations of 6 MiB (several chunks per
    lane), more micro-batches than a pair's ring holds; gradients against the whole model on one GPU."""
    import copy

    from oneccl_b200.parallel.pp import PipelineStage, run_gpipe
    from oneccl_b200.parallel.sp import ring_attention

    r, W = comm.rank, comm.size
    torch.cuda.set_device(r)
    torch.manual_seed(0)
    D, rows, n_micro = 768, 2048, 7
    layers = [torch.nn.Sequential(torch.nn.Linear(D, D), torch.nn.Tanh()) for _ in range(W)]
    full = torch.nn.Sequential(*layers).cuda()
    ref = copy.deepcopy(full)
    mine = full[r]
    gen = torch.Generator(device="cuda").manual_seed(5)
    micro = [torch.randn(rows, D, generator=gen, device="cuda") for _ in range(n_micro)]
    stage = PipelineStage(comm)
    losses = run_gpipe(stage, mine, micro, act_like=torch.empty(rows, D, device="cuda"),
                       loss_fn=lambda y, m: (y ** 2).mean())
    torch.cuda.synchronize()
    ref_losses = []
    for m in range(n_micro):
        loss = (ref(micro[m]) ** 2).mean()
        loss.backward()
        ref_losses.append(float(loss))
    for a, b in zip(mine.parameters(), ref[r].parameters()):
        assert (a.grad - b.grad).abs().max().item() < 1e-4 * max(1.0, b.grad.abs().max().item())
    if stage.is_last:
        assert all(abs(a - b) < 1e-4 for a, b in zip(losses, ref_losses))
    # ring attention on CUDA tensors: the next K / V block travels on a side stream during the math
    s, H, Dh = 64, 4, 32
    g2 = torch.Generator(device="cuda").manual_seed(9)
    q, k, v = (torch.randn(W * s, H, Dh, generator=g2, device="cuda") for _ in range(3))
    out = ring_attention(comm, q[r * s:(r + 1) * s], k[r * s:(r + 1) * s], v[r * s:(r + 1) * s])
    att = torch.softmax(torch.einsum("qhd,khd->hqk", q[r * s:(r + 1) * s], k) * Dh ** -0.5, dim=-1)
    want = torch.einsum("hqk,khd->qhd", att, v)
    torch.cuda.synchronize()
    assert (out - want).abs().max().item() < 1e-4
    comm.device_group.check()
    return True


@needs2
def test_gpipe_and_ring_attention_on_device_buffers():
    assert all(run_ranks(_pipeline_cuda, min(_world(), 4), env=ENV, timeout=300))


def _nan_check(comm):
    r = comm.rank
    torch.cuda.set_device(r)
    dev = torch.device("cuda", r)
    g = comm.device_group
    x = torch.ones(5000, device=dev)
    comm.allreduce(x).wait()
    torch.cuda.synchronize()
    g.check()  # finite result: nothing recorded
    x[1234] = float("inf") if r == 0 else 1.0
    try:  # the scan's record surfaces at the first status check: the event wait or an explicit check
        comm.allreduce(x).wait()
        torch.cuda.synchronize()
        g.check()
        found = False
    except Exception as e:  # noqa: BLE001
        found = "NaN or Inf" in str(e) and "1234" in str(e)
    g.clear_status()
    comm.allreduce(torch.ones(8, device=dev)).wait()  # the communicator stays usable
    torch.cuda.synchronize()
    g.check()
    return found


@needs2
def test_debug_scan_reports_non_finite_results():
    assert all(run_ranks(_nan_check, 2, env=dict(ENV, CCL_CUDA_CHECK_NAN="1"), timeout=200))


def _fake_nodes(rank, world, addr_file, q, chunks=0):
    """Two ranks that pretend to sit on different hosts and share GPU 0: the node communicators have one
    rank each (their kernels wait on nobody), the slice crosses the 'nodes' on the host path."""
    try:
        os.environ["CCL_TOPO_FAKE_HOST"] = f"node{rank}"
        os.environ["CCL_CUDA_NVLS"] = "0"
        os.environ["CCL_CUDA_SYMM_HEAP_SIZE"] = "64M"
        os.environ["CCL_CUDA_TMP_BUF_SIZE"] = "8M"
        os.environ["CCL_ALLREDUCE_PIPE_CHUNK_COUNT"] = str(chunks)
        import time

        from oneccl_b200.comm import KVS, Communicator

        if rank == 0:
            kvs = KVS.create_main()
            with open(addr_file + ".tmp", "w") as f:
                f.write(kvs.address)
            os.replace(addr_file + ".tmp", addr_file)
        else:
            t0 = time.time()
            while not os.path.exists(addr_file):
                assert time.time() - t0 < 60
                time.sleep(0.01)
            kvs = KVS.connect(open(addr_file).read())
        comm = Communicator(world, rank, kvs)
        torch.cuda.set_device(0)
        x = torch.full((4096,), float(rank + 1), device="cuda")
        y = torch.zeros_like(x)
        comm.allreduce(x, y).wait()
        torch.cuda.synchronize()
        ok = bool(torch.all(y == world * (world + 1) / 2)) and comm.local_size == 1
        z = torch.arange(1000, device="cuda", dtype=torch.float32) + rank
        comm.allreduce(z).wait()  # in place
        torch.cuda.synchronize()
        ok = ok and bool(torch.all(z == 2 * torch.arange(1000, device="cuda") + 1))
        # a message of several parts (when chunks > 1), values that differ per element, out of place and in place
        n = 3 * 7 * 1024
        big = torch.arange(n, device="cuda", dtype=torch.float32) * (rank + 1)
        out = torch.zeros_like(big)
        comm.allreduce(big, out).wait()
        comm.allreduce(big).wait()
        torch.cuda.synchronize()
        want = torch.arange(n, device="cuda", dtype=torch.float32) * 3
        ok = ok and bool(torch.equal(out, want)) and bool(torch.equal(big, want))
        # broadcast and reduce take the node stage on the device and cross the 'nodes' once, on the host path
        from oneccl_b200.comm import stats

        b = torch.full((5000,), float(rank + 7), device="cuda")
        comm.broadcast(b, root=1).wait()
        src = torch.arange(300, device="cuda", dtype=torch.float32) + 10 * rank
        dst = torch.zeros(300, device="cuda")
        comm.broadcast(src, root=0, recv=dst).wait()
        o = torch.zeros(777, device="cuda")
        comm.reduce(torch.full((777,), float(rank + 1), device="cuda"), o, root=1).wait()
        torch.cuda.synchronize()
        ok = ok and bool(torch.all(b == 8.0)) and bool(torch.all(dst == torch.arange(300, device="cuda")))
        ok = ok and (rank != 1 or bool(torch.all(o == 3.0)))
        ok = ok and stats("device_calls", "bcast") >= 1 and stats("device_calls", "broadcast") >= 1
        ok = ok and stats("device_calls", "reduce") >= 1
        comm.barrier().wait()
        comm.close()
        q.put((rank, "ok", ok))
    except Exception:
        import traceback

        q.put((rank, "error", traceback.format_exc()))


@pytest.mark.skipif(_ngpu() < 1, reason="needs a GPU")
@pytest.mark.parametrize("chunks", [0, 3, 5], ids=["one-part", "three-parts", "five-asked-four-fit"])
def test_collectives_across_fake_nodes_take_the_hierarchical_path(chunks):
    import multiprocessing as mp
    import tempfile

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    addr = os.path.join(tempfile.mkdtemp(prefix="cclx_fn_"), "addr")
    procs = [ctx.Process(target=_fake_nodes, args=(r, 2, addr, q, chunks)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(2):
        rank, status, out = q.get(timeout=180)
        assert status == "ok", out
        res[rank] = out
    for p in procs:
        p.join(timeout=30)
    assert res == {0: True, 1: True}
