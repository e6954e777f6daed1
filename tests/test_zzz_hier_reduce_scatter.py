"""reduce_scatter on device buffers across nodes: the block regrouping kernel against a plain PyTorch
permutation, and the whole path with two ranks that report different host names and share GPU 0 (their
node communicators have one rank each, so no kernel waits on another process)."""
import multiprocessing as mp
import os
import tempfile
import time
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols,block,dtype", [(3, 4, 1000, torch.float32), (2, 8, 7, torch.bfloat16),
                                                   (5, 2, 4096, torch.int64), (1, 6, 33, torch.uint8),
                                                   (4, 4, 65536, torch.bfloat16)])
def test_block_transpose_matches_a_permute(rows, cols, block, dtype):
    from oneccl_b200.ops.device_group import transpose_blocks

    n = rows * cols * block
    x = (torch.arange(n, device="cuda") % 251).to(dtype)
    out = transpose_blocks(x, rows, cols)
    torch.cuda.synchronize()
    ref = x.view(rows, cols, block).permute(1, 0, 2).contiguous().view(-1)
    assert torch.equal(out, ref)
    # an offset that breaks the 16-byte alignment takes the byte-wise kernel
    if block % 2 == 1 or dtype == torch.uint8:
        y = torch.empty(n + 1, device="cuda", dtype=dtype)[1:]
        y.copy_(x)
        out2 = transpose_blocks(y.contiguous(), rows, cols)
        torch.cuda.synchronize()
        assert torch.equal(out2, ref)


def _rs_fake_nodes(rank, world, addr_file, q, mode="reduce_scatter"):
    try:
        os.environ["CCL_TOPO_FAKE_HOST"] = f"node{rank}"
        os.environ["CCL_CUDA_NVLS"] = "0"
        os.environ["CCL_CUDA_SYMM_HEAP_SIZE"] = "64M"
        os.environ["CCL_CUDA_TMP_BUF_SIZE"] = "8M"
        if mode == "allgather":
            os.environ["CCL_ALLGATHER"] = "topo"
        from oneccl_b200.comm import KVS, Communicator, stats

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
        ok = comm.local_size == 1
        for count, dtype in ((1000, torch.float32), (4099, torch.bfloat16), (70000, torch.float32)):
            if mode != "reduce_scatter":
                break
            base = (torch.arange(count * world, device="cuda") % 7).to(dtype)
            send = base + rank
            recv = torch.zeros(count, device="cuda", dtype=dtype)
            comm.reduce_scatter(send, recv).wait()
            torch.cuda.synchronize()
            ref = base[rank * count:(rank + 1) * count].float() * world + sum(range(world))
            ok = ok and bool(torch.equal(recv.float(), ref))
            ok = ok and bool(torch.equal(send, base + rank))  # the send buffer is left alone
        # allgather on request (CCL_ALLGATHER=topo): my block crosses the nodes on the host path, the node gathers
        for count, dtype in ((1000, torch.float32), (4099, torch.bfloat16)):
            if mode != "allgather":
                break
            mine = torch.full((count,), float(rank + 1), device="cuda", dtype=dtype)
            out = torch.zeros(count * world, device="cuda", dtype=dtype)
            comm.allgather(mine, out).wait()
            torch.cuda.synchronize()
            ref = torch.arange(1, world + 1, device="cuda").repeat_interleave(count).to(dtype)
            ok = ok and bool(torch.equal(out, ref))
        calls = stats("device_calls", mode)
        comm.barrier().wait()
        comm.close()
        q.put((rank, "ok", ok and calls >= 2))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def _run_fake_nodes(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    addr = os.path.join(tempfile.mkdtemp(prefix="cclx_hrs_"), "addr")
    procs = [ctx.Process(target=_rs_fake_nodes, args=(r, 2, addr, q, mode)) for r in range(2)]
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


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_reduce_scatter_across_fake_nodes_takes_the_hierarchical_path():
    _run_fake_nodes("reduce_scatter")


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
def test_allgather_across_fake_nodes_on_request():
    """CCL_ALLGATHER=topo: own block across the nodes on the host path, node-level gather on the device."""
    _run_fake_nodes("allgather")
