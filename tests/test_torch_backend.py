"""torch.distributed 'ccl' backend on CPU tensors with real processes; the CUDA
variant runs when at least two GPUs are visible."""
import multiprocessing as mp
import os
import socket
import traceback

import pytest
import torch


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, device, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["CCL_CUDA_SYMM_HEAP_SIZE"] = "256M"
        os.environ["CCL_CUDA_TMP_BUF_SIZE"] = "16M"
        import torch.distributed as dist

        import oneccl_b200.torch_backend  # noqa: F401  registers "ccl"

        if device == "cuda":
            torch.cuda.set_device(rank)
        dist.init_process_group("ccl", rank=rank, world_size=world)
        dev = torch.device(device, rank) if device == "cuda" else torch.device("cpu")
        W = world
        x = torch.arange(1000, dtype=torch.float32, device=dev) + rank
        dist.all_reduce(x)
        assert torch.allclose(x.cpu(), torch.arange(1000, dtype=torch.float32) * W + sum(range(W)))
        y = torch.full((7,), float(rank), device=dev)
        dist.all_reduce(y, op=dist.ReduceOp.MAX)
        assert torch.all(y == W - 1)
        z = torch.full((5,), float(rank + 1), device=dev)
        dist.all_reduce(z, op=dist.ReduceOp.AVG)
        assert torch.allclose(z.cpu(), torch.full((5,), (W + 1) / 2))
        b = torch.full((33,), float(rank), device=dev)
        dist.broadcast(b, src=W - 1)
        assert torch.all(b == W - 1)
        outs = [torch.zeros(4, device=dev) for _ in range(W)]
        dist.all_gather(outs, torch.full((4,), float(rank), device=dev))
        for p in range(W):
            assert torch.all(outs[p] == p)
        flat = torch.zeros(4 * W, device=dev)
        dist.all_gather_into_tensor(flat, torch.full((4,), float(rank), device=dev))
        assert torch.equal(flat.cpu(), torch.repeat_interleave(torch.arange(W, dtype=torch.float32), 4))
        rs = torch.zeros(3, device=dev)
        dist.reduce_scatter_tensor(rs, torch.arange(3 * W, dtype=torch.float32, device=dev))
        assert torch.allclose(rs.cpu(), torch.arange(3 * W, dtype=torch.float32)[3 * rank:3 * rank + 3] * W)
        a2a = torch.zeros(2 * W, device=dev)
        dist.all_to_all_single(a2a, torch.arange(2 * W, dtype=torch.float32, device=dev) + 100 * rank)
        ref = torch.cat([torch.arange(2, dtype=torch.float32) + 2 * rank + 100 * p for p in range(W)])
        assert torch.equal(a2a.cpu(), ref)
        red = torch.full((9,), float(rank + 1), device=dev)
        dist.reduce(red, dst=0)
        if rank == 0:
            assert torch.all(red == W * (W + 1) / 2)
        if rank == 0:
            dist.send(torch.full((6,), 42.0, device=dev), dst=1)
        elif rank == 1:
            got = torch.zeros(6, device=dev)
            dist.recv(got, src=0)
            assert torch.all(got == 42)
        dist.barrier()
        # DistributedDataParallel over the backend
        torch.manual_seed(0)
        model = torch.nn.Linear(16, 4).to(dev)
        ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[rank] if device == "cuda" else None)
        inp = torch.randn(8, 16, generator=torch.Generator().manual_seed(rank)).to(dev)
        ddp(inp).sum().backward()
        g = model.weight.grad.detach().cpu().clone()
        gathered = [torch.zeros_like(g) for _ in range(W)]
        dist.all_gather(gathered, g.to(dev) if device == "cuda" else g)
        for t in gathered:
            assert torch.allclose(t.cpu(), g, rtol=1e-5, atol=1e-6)
        dist.barrier()
        if device == "cuda":
            torch.cuda.synchronize()
        dist.destroy_process_group()
        q.put((rank, "ok", ""))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def _run(world, device):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, device, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = []
    try:
        for _ in range(world):
            res.append(q.get(timeout=240))
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.terminate()
    for rank, status, msg in res:
        assert status == "ok", f"rank {rank}: {msg}"


def test_process_group_cpu_world2():
    _run(2, "cpu")


def test_process_group_cpu_world3():
    _run(3, "cpu")


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_process_group_cuda():
    _run(2, "cuda")


def _worker_more(rank, world, port, q):
    """Remaining operations on CPU tensors: gather / scatter, list forms of all_to_all and
    reduce_scatter, coalesced and object collectives, sub-groups, uneven all_to_all splits."""
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import torch.distributed as dist

        import oneccl_b200.torch_backend  # noqa: F401

        dist.init_process_group("ccl", rank=rank, world_size=world)
        W = world
        # gather / scatter
        got = [torch.zeros(3) for _ in range(W)] if rank == 1 else None
        dist.gather(torch.full((3,), float(rank)), got, dst=1)
        if rank == 1:
            assert all(torch.all(got[p] == p) for p in range(W))
        out = torch.zeros(2)
        dist.scatter(out, [torch.full((2,), float(10 + p)) for p in range(W)] if rank == 0 else None, src=0)
        assert torch.all(out == 10 + rank)
        # list forms
        outs = [torch.zeros(2) for _ in range(W)]
        dist.all_to_all(outs, [torch.full((2,), float(rank * 10 + p)) for p in range(W)])
        assert all(torch.all(outs[p] == p * 10 + rank) for p in range(W))
        rs = torch.zeros(4)
        dist.reduce_scatter(rs, [torch.full((4,), float(p + 1)) for p in range(W)])
        assert torch.all(rs == (rank + 1) * W)
        # uneven all_to_all_single: rank r sends r + 1 elements to everybody
        send = torch.full(((rank + 1) * W,), float(rank))
        recv = torch.zeros(sum(p + 1 for p in range(W)))
        dist.all_to_all_single(recv, send, output_split_sizes=[p + 1 for p in range(W)],
                               input_split_sizes=[rank + 1] * W)
        assert torch.equal(recv, torch.cat([torch.full((p + 1,), float(p)) for p in range(W)]))
        # object collectives ride on byte tensors
        objs = [None] * W
        dist.all_gather_object(objs, {"rank": rank, "name": "r%d" % rank})
        assert [o["rank"] for o in objs] == list(range(W))
        box = [{"lr": 3e-4} if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        assert box[0] == {"lr": 3e-4}
        # sub-group of the even ranks plus a reduce to its first member
        evens = list(range(0, W, 2))
        sub = dist.new_group(evens)
        if rank in evens:
            t = torch.full((5,), float(rank + 1))
            dist.all_reduce(t, group=sub)
            assert torch.all(t == sum(e + 1 for e in evens))
            r = torch.full((2,), 1.0)
            dist.reduce(r, dst=evens[0], group=sub)
            if rank == evens[0]:
                assert torch.all(r == len(evens))
        # asynchronous work objects
        w1 = dist.all_reduce(torch.ones(10), async_op=True)
        w2 = dist.broadcast(torch.ones(3), src=0, async_op=True)
        w1.wait()
        w2.wait()
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok", ""))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def test_ccl_backend_cpu_remaining_operations():
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_more, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    for rank, status, msg in res:
        assert status == "ok", f"rank {rank}:\n{msg}"


def _worker_p2p_and_dtypes(rank, world, port, q):
    """Point-to-point batches, the coalescing manager, every tensor dtype the backend maps, reductions,
    non-contiguous inputs, and the tensor forms that sharded data parallelism uses."""
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import torch.distributed as dist

        import oneccl_b200.torch_backend  # noqa: F401

        dist.init_process_group("ccl", rank=rank, world_size=world)
        W = world
        nxt, prv = (rank + 1) % W, (rank - 1) % W
        # isend / irecv
        got = torch.zeros(6)
        rr = dist.irecv(got, src=prv)
        rs = dist.isend(torch.full((6,), float(rank)), dst=nxt)
        rr.wait()
        rs.wait()
        assert torch.all(got == prv)
        # a batch in both directions at once
        a, b = torch.zeros(4), torch.zeros(4)
        ops = [dist.P2POp(dist.isend, torch.full((4,), float(rank + 1)), nxt),
               dist.P2POp(dist.isend, torch.full((4,), float(-rank - 1)), prv),
               dist.P2POp(dist.irecv, a, prv), dist.P2POp(dist.irecv, b, nxt)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        assert torch.all(a == prv + 1) and torch.all(b == -(nxt + 1))
        # dtypes x reductions
        for dt in (torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int32,
                   torch.int64):
            t = (torch.arange(33) % 3 + rank + 1).to(dt)
            dist.all_reduce(t)
            ref = sum((torch.arange(33) % 3 + p + 1) for p in range(W)).to(dt)
            assert torch.equal(t, ref), dt
            for op, fn in ((dist.ReduceOp.MAX, max), (dist.ReduceOp.MIN, min)):
                t = torch.full((5,), rank + 1).to(dt)
                dist.all_reduce(t, op=op)
                assert torch.all(t == fn(range(1, W + 1))), (dt, op)
        t = torch.full((3,), 2.0)
        dist.all_reduce(t, op=dist.ReduceOp.PRODUCT)
        assert torch.all(t == 2.0 ** W)
        t = torch.full((4,), float(rank))
        dist.all_reduce(t, op=dist.ReduceOp.AVG)
        assert torch.allclose(t, torch.full((4,), (W - 1) / 2))
        # bool travels as uint8
        flag = torch.tensor([rank == 0, True])
        dist.all_reduce(flag, op=dist.ReduceOp.MAX)
        assert flag.tolist() == [True, True]
        # non-contiguous input
        m = (torch.arange(12, dtype=torch.float32).reshape(3, 4) + rank).t()
        assert not m.is_contiguous()
        dist.all_reduce(m)
        assert torch.equal(m, (torch.arange(12, dtype=torch.float32).reshape(3, 4) * W + sum(range(W))).t())
        # sharded-parameter pattern: gather the shards, reduce-scatter the gradients
        shard = torch.full((8,), float(rank))
        full = torch.zeros(8 * W)
        dist.all_gather_into_tensor(full, shard)
        assert torch.equal(full, torch.arange(W, dtype=torch.float32).repeat_interleave(8))
        grad = torch.arange(8 * W, dtype=torch.float32) + rank
        out = torch.zeros(8)
        dist.reduce_scatter_tensor(out, grad, op=dist.ReduceOp.AVG)
        assert torch.allclose(out, torch.arange(8 * rank, 8 * rank + 8, dtype=torch.float32) + (W - 1) / 2)
        # coalescing manager
        xs = [torch.full((k + 1,), float(rank + k)) for k in range(4)]
        with dist._coalescing_manager():
            for x in xs:
                dist.all_reduce(x)
        for k, x in enumerate(xs):
            assert torch.all(x == sum(p + k for p in range(W))), k
        lst = [[torch.zeros(2) for _ in range(W)] for _ in range(2)]
        dist.all_gather_coalesced(lst, [torch.full((2,), float(rank)), torch.full((2,), float(rank * 2))])
        for p in range(W):
            assert torch.all(lst[0][p] == p) and torch.all(lst[1][p] == 2 * p)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok", ""))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def test_ccl_backend_cpu_p2p_batches_dtypes_and_sharded_patterns():
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_p2p_and_dtypes, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=30)
    for rank, status, msg in res:
        assert status == "ok", f"rank {rank}: {msg}"
