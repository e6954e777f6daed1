"""CPU path over the TCP transport with real processes (no mpirun), mirroring the
reference's functional suite: closed-form oracle, every algorithm per collective
through the CCL_<COLL> override, sizes incl. odd counts, in-place and out-of-place."""
import numpy as np
import pytest

from mp_util import run_ranks


def _cfg1(comm):
    """fp32 sum allreduce with counts {1, 17, 4096, 1048576}, uniform[-1,1) seed 0 per rank;
    allgatherv with per-rank counts {1000, 1500}; barrier."""
    W, r = comm.size, comm.rank
    errs = []
    for count in (1, 17, 4096, 1048576):
        data = [np.random.default_rng(0 + p).uniform(-1, 1, count).astype(np.float32) for p in range(W)]
        out = np.empty(count, np.float32)
        comm.allreduce(data[r], out).wait()
        ref = np.sum(np.stack(data).astype(np.float64), axis=0)
        errs.append(float(np.max(np.abs(out - ref))))
    counts = [1000, 1500][:W] + [700] * max(0, W - 2)
    send = np.full(counts[r], r + 1, np.float32)
    recv = np.zeros(sum(counts), np.float32)
    comm.allgatherv(send, recv, counts).wait()
    ref = np.concatenate([np.full(c, p + 1, np.float32) for p, c in enumerate(counts)])
    assert np.array_equal(recv, ref)
    comm.barrier().wait()
    return errs


@pytest.mark.parametrize("env", [{}, {"CCL_ATL_SHM": "0"}, {"CCL_ATL_SHM_RING_BYTES": "65536"}],
                         ids=["shm", "sockets", "small-rings"])
def test_baseline_config1_world2(env):
    """fp32 sum allreduce at 1 / 17 / 4096 / 1M elements, allgatherv with unequal counts, barrier:
    over the shared-memory rings, over sockets only, and with rings smaller than the messages."""
    for errs in run_ranks(_cfg1, 2, env=env):
        assert max(errs) < 1e-5


def _allreduce_matrix(comm, algo):
    W, r = comm.size, comm.rank
    for dtype in (np.float32, np.int32, np.float64, np.int8):
        for count in (1, 17, 32771):
            base = np.arange(count) % 7
            send = (base + r).astype(dtype)
            # in place
            buf = send.copy()
            comm.allreduce(buf).wait()
            ref = (base * W + sum(range(W))).astype(dtype)
            assert np.array_equal(buf, ref), (algo, dtype, count)
            # out of place, other reductions
            out = np.empty_like(send)
            comm.allreduce(send, out, op="max").wait()
            assert np.array_equal(out, (base + W - 1).astype(dtype))
            assert np.array_equal(send, (base + r).astype(dtype))
    return True


@pytest.mark.parametrize("algo", ["ring", "recursive_doubling", "rabenseifner", "nreduce", "double_tree", "2d", "direct"])
@pytest.mark.parametrize("world", [2, 3, 5])
def test_allreduce_every_algorithm(algo, world):
    assert all(run_ranks(_allreduce_matrix, world, algo, env={"CCL_ALLREDUCE": algo}))


def _others(comm):
    W, r = comm.size, comm.rank
    # allgather
    send = np.full(33, r, np.int32)
    recv = np.zeros(33 * W, np.int32)
    comm.allgather(send, recv).wait()
    assert np.array_equal(recv, np.repeat(np.arange(W, dtype=np.int32), 33))
    # allgatherv with per-rank destination buffers
    counts = [5 + p for p in range(W)]
    bufs = [np.zeros(c, np.float32) for c in counts]
    comm.allgatherv(np.full(counts[r], r, np.float32), None, counts, recv_bufs=bufs).wait()
    for p in range(W):
        assert np.array_equal(bufs[p], np.full(counts[p], p, np.float32))
    # alltoall
    send = (np.arange(W * 10) + 1000 * r).astype(np.int64)
    recv = np.zeros(W * 10, np.int64)
    comm.alltoall(send, recv).wait()
    ref = np.concatenate([(np.arange(10) + 10 * r + 1000 * p) for p in range(W)]).astype(np.int64)
    assert np.array_equal(recv, ref)
    # alltoallv: rank r sends (q+1) elements of value r*100+q to q
    sc = [q + 1 for q in range(W)]
    rc = [r + 1] * W
    send = np.concatenate([np.full(q + 1, r * 100 + q, np.int32) for q in range(W)])
    recv = np.zeros(sum(rc), np.int32)
    comm.alltoallv(send, sc, recv, rc).wait()
    assert np.array_equal(recv, np.concatenate([np.full(r + 1, p * 100 + r, np.int32) for p in range(W)]))
    # broadcast in place and out of place
    for root in range(W):
        buf = np.full(1001, r, np.float32)
        comm.broadcast(buf, root=root).wait()
        assert np.all(buf == root)
        out = np.zeros(77, np.float64)
        comm.broadcast(np.full(77, 5.0 + r), root=root, recv=out).wait()
        assert np.all(out == 5.0 + root)
    # reduce
    for root in (0, W - 1):
        out = np.zeros(513, np.float64)
        comm.reduce(np.full(513, float(r + 1)), out, root=root).wait()
        if r == root:
            assert np.all(out == W * (W + 1) / 2)
    # reduce_scatter incl. the in-place position recv = send + rank*recv_count
    rcnt = 129
    send = np.tile(np.arange(rcnt, dtype=np.float32), W) + r
    out = np.zeros(rcnt, np.float32)
    comm.reduce_scatter(send, out).wait()
    assert np.allclose(out, np.arange(rcnt) * W + sum(range(W)))
    buf = np.tile(np.arange(rcnt, dtype=np.float32), W) + r
    comm.reduce_scatter(buf, buf[r * rcnt:(r + 1) * rcnt]).wait()
    assert np.allclose(buf[r * rcnt:(r + 1) * rcnt], np.arange(rcnt) * W + sum(range(W)))
    # send / recv ring
    nxt, prv = (r + 1) % W, (r - 1) % W
    got = np.zeros(100, np.int32)
    e1 = comm.recv(got, prv)
    e2 = comm.send(np.full(100, r, np.int32), nxt)
    e1.wait()
    e2.wait()
    assert np.all(got == prv)
    return True


@pytest.mark.parametrize("world", [2, 4])
def test_other_collectives_default_algorithms(world):
    assert all(run_ranks(_others, world))


@pytest.mark.parametrize("env", [
    {"CCL_ALLGATHERV": "ring", "CCL_ALLGATHER": "ring", "CCL_ALLTOALL": "scatter", "CCL_ALLTOALLV": "scatter",
     "CCL_BCAST": "ring", "CCL_BROADCAST": "naive", "CCL_REDUCE": "rabenseifner", "CCL_REDUCE_SCATTER": "ring",
     "CCL_BARRIER": "ring"},
    {"CCL_ALLGATHERV": "multi_bcast", "CCL_ALLGATHER": "flat", "CCL_BCAST": "naive", "CCL_BROADCAST": "ring",
     "CCL_REDUCE": "ring", "CCL_REDUCE_SCATTER": "direct", "CCL_WORKER_COUNT": "2"},
    {"CCL_REDUCE": "double_tree", "CCL_BCAST": "double_tree", "CCL_WORKER_OFFLOAD": "0"},
    {"CCL_ATL_SHM": "0", "CCL_WORKER_COUNT": "2"},
    {"CCL_MAX_FLOW_CREDITS": "1", "CCL_ALLTOALL": "naive", "CCL_ALLTOALLV": "naive"},  # one entry in flight at a time
])
def test_other_collectives_algorithm_overrides(env):
    assert all(run_ranks(_others, 3, env=env))


def _split_ops(comm):
    """Sizes long enough for every partition rule: ring allgather(v) cut per worker, alltoall cut per worker,
    allreduce / broadcast / reduce and send / recv cut by the large-message size."""
    W, r = comm.size, comm.rank
    n = 5003
    send = (np.arange(n) + 7 * r).astype(np.float32)
    recv = np.zeros(n * W, np.float32)
    comm.allgather(send, recv).wait()
    assert np.array_equal(recv, np.concatenate([(np.arange(n) + 7 * p).astype(np.float32) for p in range(W)]))
    counts = [3001 + 500 * p for p in range(W)]
    recv = np.zeros(sum(counts), np.float64)
    comm.allgatherv(np.arange(counts[r], dtype=np.float64) + r, recv, counts).wait()
    assert np.array_equal(recv, np.concatenate([np.arange(c, dtype=np.float64) + p for p, c in enumerate(counts)]))
    inplace = np.zeros(n * W, np.float32)
    inplace[r * n:(r + 1) * n] = send
    comm.allgather(inplace[r * n:(r + 1) * n], inplace).wait()
    assert np.array_equal(inplace, np.concatenate([(np.arange(n) + 7 * p).astype(np.float32) for p in range(W)]))
    a = (np.arange(W * n) + 100000 * r).astype(np.int64)
    b = np.zeros(W * n, np.int64)
    comm.alltoall(a, b).wait()
    assert np.array_equal(b, np.concatenate([(np.arange(n) + n * r + 100000 * p) for p in range(W)]).astype(np.int64))
    x = (np.arange(32771) % 13 + r).astype(np.float32)
    comm.allreduce(x).wait()
    assert np.array_equal(x, ((np.arange(32771) % 13) * W + sum(range(W))).astype(np.float32))
    buf = np.full(20001, float(r), np.float64)
    comm.broadcast(buf, root=W - 1).wait()
    assert np.all(buf == W - 1)
    out = np.zeros(9999, np.float32)
    comm.reduce(np.full(9999, float(r + 1), np.float32), out, root=0).wait()
    if r == 0:
        assert np.all(out == W * (W + 1) / 2)
    nxt, prv = (r + 1) % W, (r - 1) % W
    got = np.zeros(30000, np.int32)
    e1 = comm.recv(got, prv)
    e2 = comm.send(np.arange(30000, dtype=np.int32) + r, nxt)
    e1.wait()
    e2.wait()
    assert np.array_equal(got, np.arange(30000, dtype=np.int32) + prv)
    return True


@pytest.mark.parametrize("env", [
    {"CCL_WORKER_COUNT": "2", "CCL_ALLGATHER": "ring", "CCL_ALLGATHERV": "ring", "CCL_ALLTOALL": "naive"},
    {"CCL_WORKER_COUNT": "3", "CCL_ALLGATHER": "ring", "CCL_ALLGATHERV": "ring", "CCL_ALLTOALL": "scatter",
     "CCL_ATL_LARGE_MSG_SIZE": "4096"},
    {"CCL_ATL_LARGE_MSG_SIZE": "10000"},
], ids=["two-workers", "three-workers-small-large-msg", "one-worker-small-large-msg"])
def test_partition_rules_of_every_collective(env):
    assert all(run_ranks(_split_ops, 3, env=env))


def test_double_tree_is_a_pair_of_complementary_binary_trees():
    """Both trees span all ranks with at most two children per node, the parent / child relations agree, and
    a rank that forwards data in one tree (has children) is a leaf in the other, except where an odd size
    leaves no choice; an explicit root swaps places with the tree's own root."""
    import ctypes as C

    from oneccl_b200 import _lib

    lib = _lib.load()

    def tree(n, which, root=-1):
        nodes = []
        for r in range(n):
            out = (C.c_int * 4)()
            assert lib.cclx_bin_tree(n, r, which, root, out) == 0
            nodes.append(tuple(out))
        return nodes

    for n in list(range(2, 34)) + [64, 100]:
        inner = []
        for which in (0, 1):
            t = tree(n, which)
            roots = [r for r in range(n) if t[r][0] < 0]
            assert roots == [t[0][3]], (n, which, roots)
            seen = {roots[0]}
            stack = [roots[0]]
            depth = {roots[0]: 0}
            while stack:  # every rank reachable exactly once, children point back at their parent
                u = stack.pop()
                for ch in t[u][1:3]:
                    if ch >= 0:
                        assert ch not in seen and t[ch][0] == u, (n, which, u, ch)
                        seen.add(ch)
                        depth[ch] = depth[u] + 1
                        stack.append(ch)
            assert len(seen) == n
            assert max(depth.values()) <= n.bit_length()  # logarithmic height
            inner.append({r for r in range(n) if t[r][1] >= 0 or t[r][2] >= 0})
        both = inner[0] & inner[1]
        assert len(both) <= 1, (n, both)  # complementary: forwarding in one tree means leaf in the other
    t = tree(10, 0, root=7)
    assert t[7][0] == -1 and t[7][3] == 7


def _double_tree_ops(comm):
    W, r = comm.size, comm.rank
    for count in (1, 2, 17, 4099):
        base = np.arange(count, dtype=np.float64) % 11
        for root in sorted({0, W - 1, W // 2}):
            buf = (base + 100 * root).astype(np.float32) if r == root else np.zeros(count, np.float32)
            comm.broadcast(buf, root=root).wait()
            assert np.array_equal(buf, (base + 100 * root).astype(np.float32)), ("bcast", count, root)
            out = np.zeros(count, np.float32)
            comm.reduce((base + r).astype(np.float32), out, root=root).wait()
            if r == root:
                assert np.array_equal(out, (base * W + sum(range(W))).astype(np.float32)), ("reduce", count, root)
        x = (base + r).astype(np.float32)
        comm.allreduce(x).wait()
        assert np.array_equal(x, (base * W + sum(range(W))).astype(np.float32)), ("allreduce", count)
    return True


@pytest.mark.parametrize("world", [2, 3, 4, 7])
@pytest.mark.parametrize("parts", ["1", "3"])
def test_double_tree_broadcast_reduce_allreduce(world, parts):
    env = {"CCL_BCAST": "double_tree", "CCL_BROADCAST": "double_tree", "CCL_REDUCE": "double_tree",
           "CCL_ALLREDUCE": "double_tree", "CCL_DTREE_PARTITION_COUNT": parts}
    assert all(run_ranks(_double_tree_ops, world, env=env))


def _bcast_1000(comm):
    b = np.arange(1000, dtype=np.float32)
    comm.broadcast(b, root=0).wait()
    return True


def test_double_tree_schedule_uses_both_trees(capfd):
    """The schedule dump of a double-tree broadcast names the two tree sub-schedules: the name is not an
    alias of the single binomial tree."""
    run_ranks(_bcast_1000, 4, env={"CCL_BCAST": "double_tree", "CCL_BROADCAST": "double_tree", "CCL_SCHED_DUMP": "1",
                                   "CCL_LOG_LEVEL": "info"})
    text = "".join(capfd.readouterr())
    assert "DTREE_BCAST_A" in text and "DTREE_BCAST_B" in text, text[-2000:]


def _lowp_and_custom(comm):
    import ctypes as C

    import torch

    from oneccl_b200.comm import REDUCTION_FN

    W, r = comm.size, comm.rank
    x = (torch.arange(1000, dtype=torch.float32) / 64 + r).to(torch.bfloat16)
    out = torch.empty_like(x)
    comm.allreduce(x, out).wait()
    ref = sum((torch.arange(1000, dtype=torch.float32) / 64 + p).to(torch.bfloat16).float() for p in range(W))
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    h = (torch.arange(500, dtype=torch.float32) / 16 + r).to(torch.float16)
    comm.allreduce(h).wait()
    refh = sum((torch.arange(500, dtype=torch.float32) / 16 + p).to(torch.float16).float() for p in range(W))
    assert torch.allclose(h.float(), refh, rtol=5e-3, atol=5e-3)

    # custom reduction: elementwise "absolute maximum" on int32
    @REDUCTION_FN
    def absmax(inp, n, inout, out_n, dtype, ctx):
        a = np.ctypeslib.as_array(C.cast(inp, C.POINTER(C.c_int32)), (n,))
        b = np.ctypeslib.as_array(C.cast(inout, C.POINTER(C.c_int32)), (n,))
        np.copyto(b, np.where(np.abs(a) > np.abs(b), a, b))

    v = np.array([r - 1, -(r + 1), 3 * (-1) ** r], np.int32)
    res = np.empty_like(v)
    comm.allreduce(v, res, op="custom", reduction_fn=absmax).wait()
    assert list(res[:2]) == [W - 2 if W > 2 else (-1 if W == 1 else (1 if abs(1) > abs(-1) else -1)), -W] or res[1] == -W
    return True


def test_low_precision_and_custom_reduction():
    assert all(run_ranks(_lowp_and_custom, 3))


def _chunked(comm, fake_nodes):
    """allreduce / reduce_scatter / alltoallv with sizes that do and do not divide into the chunk counts."""
    import os

    W, r = comm.size, comm.rank
    if fake_nodes:
        os.environ["CCL_TOPO_FAKE_HOST"] = f"node{r // (W // fake_nodes)}"
    for count in (7, 4099, 70001):
        base = (np.arange(count) % 11).astype(np.float64)
        buf = base + r
        comm.allreduce(buf).wait()
        assert np.array_equal(buf, base * W + sum(range(W))), count
        send = (base + 2 * r).astype(np.float32)
        out = np.zeros(count, np.float32)
        comm.allreduce(send, out, op="max").wait()
        assert np.array_equal(out, (base + 2 * (W - 1)).astype(np.float32))
        assert np.array_equal(send, (base + 2 * r).astype(np.float32))
    rcnt = 3001
    send = np.tile(np.arange(rcnt, dtype=np.float64), W) + r
    out = np.zeros(rcnt, np.float64)
    comm.reduce_scatter(send, out).wait()
    assert np.array_equal(out, np.arange(rcnt) * W + sum(range(W)))
    # alltoallv with unequal blocks, some of them shorter than one chunk
    sc = [(q + 1) * 997 if (q + r) % 2 else 3 for q in range(W)]
    rc = [(r + 1) * 997 if (p + r) % 2 else 3 for p in range(W)]
    send = np.concatenate([np.full(sc[q], r * 100 + q, np.int32) for q in range(W)])
    recv = np.zeros(sum(rc), np.int32)
    comm.alltoallv(send, sc, recv, rc).wait()
    assert np.array_equal(recv, np.concatenate([np.full(rc[p], p * 100 + r, np.int32) for p in range(W)]))
    for root in range(W):
        b = np.full(50001, float(r))
        comm.broadcast(b, root=root).wait()
        assert np.all(b == root)
    return True


@pytest.mark.parametrize("env,world,nodes", [
    ({"CCL_ALLREDUCE": "ring", "CCL_REDUCE_SCATTER": "ring", "CCL_RS_CHUNK_COUNT": "4", "CCL_RS_MIN_CHUNK_SIZE": "64"}, 3, 0),
    ({"CCL_ALLREDUCE": "ring", "CCL_RS_CHUNK_COUNT": "16", "CCL_RS_MIN_CHUNK_SIZE": "1", "CCL_ATL_SHM": "0"}, 4, 0),
    ({"CCL_ALLREDUCE": "nreduce", "CCL_ALLREDUCE_NREDUCE_SEGMENT_SIZE": "4096"}, 3, 0),
    ({"CCL_ALLREDUCE": "nreduce", "CCL_ALLREDUCE_NREDUCE_SEGMENT_SIZE": "16K", "CCL_ALLREDUCE_NREDUCE_BUFFERING": "1"}, 4, 0),
    ({"CCL_ALLREDUCE": "double_tree", "CCL_DTREE_PARTITION_COUNT": "3"}, 5, 0),
    ({"CCL_ALLREDUCE": "2d"}, 4, 2),
    ({"CCL_ALLREDUCE": "2d", "CCL_ALLREDUCE_2D_CHUNK_COUNT": "3", "CCL_ALLREDUCE_2D_MIN_CHUNK_SIZE": "256"}, 4, 2),
    ({"CCL_ALLREDUCE": "2d", "CCL_ALLREDUCE_2D_CHUNK_COUNT": "5", "CCL_ALLREDUCE_2D_MIN_CHUNK_SIZE": "1",
      "CCL_ALLREDUCE_2D_SWITCH_DIMS": "1", "CCL_RS_CHUNK_COUNT": "2", "CCL_RS_MIN_CHUNK_SIZE": "128"}, 6, 3),
    ({"CCL_ALLTOALLV": "naive", "CCL_CHUNK_COUNT": "4", "CCL_MIN_CHUNK_SIZE": "16"}, 3, 0),
    ({"CCL_ALLTOALLV": "scatter", "CCL_CHUNK_COUNT": "3", "CCL_MIN_CHUNK_SIZE": "1024", "CCL_ALLTOALL_SCATTER_MAX_OPS": "1"}, 4, 0),
    ({"CCL_WORKER_COUNT": "2", "CCL_BCAST_PART_COUNT": "3", "CCL_MIN_CHUNK_SIZE": "1024"}, 3, 0),
    ({"CCL_WORKER_COUNT": "2", "CCL_MAX_SHORT_SIZE": "64K", "CCL_MIN_CHUNK_SIZE": "1024"}, 2, 0),
    ({"CCL_BUFFER_CACHE": "0", "CCL_ALLREDUCE": "rabenseifner"}, 3, 0),
], ids=["rs-chunks", "rs-chunks-16-sockets", "nreduce-segments", "nreduce-buffering", "dtree-parts", "2d-two-nodes",
        "2d-chunks", "2d-chunks-switched", "alltoallv-naive-chunks", "alltoallv-scatter-chunks", "bcast-parts",
        "max-short-size", "no-buffer-cache"])
def test_chunking_and_partition_knobs(env, world, nodes):
    """Every knob that cuts a message into chunks, segments or parts gives the same results as the uncut
    algorithm: CCL_RS_CHUNK_COUNT, CCL_ALLREDUCE_NREDUCE_SEGMENT_SIZE / _BUFFERING, CCL_DTREE_PARTITION_COUNT,
    CCL_ALLREDUCE_2D_CHUNK_COUNT / _SWITCH_DIMS over two and three simulated nodes, CCL_CHUNK_COUNT,
    CCL_BCAST_PART_COUNT, CCL_MAX_SHORT_SIZE, CCL_BUFFER_CACHE."""
    assert all(run_ranks(_chunked, world, nodes, env=env))


def _ring_rma(comm):
    W, r = comm.size, comm.rank
    for count in (5, 4099, 300001):
        base = (np.arange(count) % 13).astype(np.float64)
        for _ in range(3):  # repeated runs reuse scratch memory and flags
            buf = base + r
            comm.allreduce(buf).wait()
            assert np.array_equal(buf, base * W + sum(range(W))), count
        send = (base + r).astype(np.int32)
        out = np.zeros(count, np.int32)
        comm.allreduce(send, out, op="max").wait()
        assert np.array_equal(out, (base + W - 1).astype(np.int32))
    # a cached schedule is started again with the same buffers
    buf = np.zeros(1000, np.float32)
    for it in range(4):
        buf[:] = r + it
        comm.allreduce(buf, match_id="rma_cached", to_cache=True).wait()
        assert np.all(buf == sum(range(W)) + W * it)
    return comm.transport_stats()


@pytest.mark.parametrize("env,direct", [
    ({}, True),
    ({"CCL_ATL_CMA": "0"}, False),
    ({"CCL_ATL_CMA": "0", "CCL_ATL_SHM": "0", "CCL_WORKER_COUNT": "2"}, False),
], ids=["cross-memory", "messages-over-rings", "messages-over-sockets"])
@pytest.mark.parametrize("world", [2, 5])
def test_allreduce_ring_by_one_sided_writes(env, direct, world):
    """CCL_ALLREDUCE=ring_rma with CCL_ATL_RMA=1: blocks and flags are written into the neighbour's registered
    memory, by process_vm_writev between processes of one host or as messages that the owner applies."""
    env = dict(env, CCL_ALLREDUCE="ring_rma", CCL_ATL_RMA="1")
    for st in run_ranks(_ring_rma, world, env=env):
        if direct:
            assert st["rma_direct_writes"] > 0 and st["rma_message_writes"] == 0, st
        else:
            assert st["rma_message_writes"] > 0 and st["rma_direct_writes"] == 0, st


def test_ring_rma_without_the_transport_switch_falls_back():
    for st in run_ranks(_ring_rma_off, 2, env={"CCL_ALLREDUCE": "ring_rma"}):
        assert st["rma_direct_writes"] == 0 and st["rma_message_writes"] == 0


def _ring_rma_off(comm):
    buf = np.full(100000, comm.rank + 1.0)
    comm.allreduce(buf).wait()
    assert np.all(buf == 3.0)
    return comm.transport_stats()


def _rendezvous(comm):
    import time

    W, r = comm.size, comm.rank
    n = 600000  # 4.8 MB: above the ring capacity, where one-way point-to-point sends take the rendezvous too
    nxt, prv = (r + 1) % W, (r - 1) % W
    # the send is issued first everywhere: descriptors arrive before any receive is posted
    out = np.arange(n, dtype=np.float64) + r
    es = comm.send(out, nxt)
    time.sleep(0.2)
    got = np.zeros(n)
    comm.recv(got, prv).wait()
    es.wait()
    assert np.array_equal(got, np.arange(n, dtype=np.float64) + prv)
    # receive posted first
    got[:] = 0
    er = comm.recv(got, nxt)
    time.sleep(0.05)
    comm.send(out, prv).wait()
    er.wait()
    assert np.array_equal(got, np.arange(n, dtype=np.float64) + nxt)
    # collectives with long and short messages mixed
    buf = np.full(1 << 20, float(r + 1), np.float32)
    comm.allreduce(buf).wait()
    assert np.all(buf == W * (W + 1) / 2)
    small = np.full(10, float(r), np.float32)
    comm.allreduce(small).wait()
    assert np.all(small == sum(range(W)))
    return comm.transport_stats()


@pytest.mark.parametrize("env,expect", [({}, True), ({"CCL_ATL_SHM": "0"}, True), ({"CCL_ATL_CMA": "0"}, False),
                                        ({"CCL_ATL_CMA_THRESHOLD": "16M"}, False)],
                         ids=["rings", "sockets", "cma-off", "threshold-above"])
def test_long_messages_between_processes_of_one_host_go_by_rendezvous(env, expect):
    """A long message travels as a descriptor; the receiver reads the sender's buffer with one
    cross-memory copy and acknowledges.  Descriptors that arrive before their receive wait in the
    unexpected queue without any data."""
    for st in run_ranks(_rendezvous, 3, env=env):
        assert (st["rndv_sends"] > 0) == expect, st
