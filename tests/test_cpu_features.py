"""Scheduler features through real ranks: schedule cache + relaunch, fusion, priorities,
dependencies, sub-communicators, strict order, worker modes, hang detector."""
import numpy as np
import pytest

from mp_util import run_ranks


def _cache(comm):
    from oneccl_b200.comm import stats

    W, r = comm.size, comm.rank
    x = np.full(5000, r + 1.0, np.float32)
    y = np.zeros_like(x)
    evs = []
    before = stats("cache_hits")
    # the same operation launched repeatedly without waiting: relaunches queue behind the running one
    for _ in range(6):
        evs.append(comm.allreduce(x, y, to_cache=True, match_id="w0"))
    for e in evs:
        e.wait()
    assert np.all(y == W * (W + 1) / 2)
    assert comm.cache_size() == 1
    hits = stats("cache_hits") - before
    # a different buffer under the same name is a different schedule
    z = np.zeros_like(x)
    comm.allreduce(x, z, to_cache=True, match_id="w0").wait()
    assert comm.cache_size() == 2 and np.all(z == W * (W + 1) / 2)
    return hits


def test_schedule_cache_and_relaunch():
    assert all(h == 5 for h in run_ranks(_cache, 2))


def _cache_bound(comm):
    W, r = comm.size, comm.rank
    # one name, a new buffer every step: every call misses (keys hold the addresses) and the cache must not grow
    keep = []
    for step in range(40):
        x = np.full(300, float(r + step), np.float32)
        keep.append(x)  # keeps the addresses distinct
        comm.allreduce(x, to_cache=True, match_id="grad").wait()
        assert np.all(x == sum(p + step for p in range(W)))
        assert comm.cache_size() <= 8
    # un-waited events of evicted schedules stay valid
    evs = []
    for step in range(20):
        x = np.full(100, 1.0, np.float32)
        keep.append(x)
        evs.append((comm.allreduce(x, to_cache=True, match_id="g2"), x))
    for e, x in evs:
        e.wait()
        assert np.all(x == W)
    # schedules that were running could not be evicted; the next insertion trims the cache again
    last = np.ones(10, np.float32)
    comm.allreduce(last, to_cache=True, match_id="g3").wait()
    return comm.cache_size()


def test_schedule_cache_is_bounded():
    assert all(n <= 8 for n in run_ranks(_cache_bound, 3, env={"CCL_SCHED_CACHE_MAX_ENTRIES": "8"}))


def _fusion(comm):
    from oneccl_b200.comm import stats

    W, r = comm.size, comm.rank
    bufs = [np.full(10 + k, float(r + k), np.float32) for k in range(40)]
    outs = [np.zeros_like(b) for b in bufs]
    evs = [comm.allreduce(b, o) for b, o in zip(bufs, outs)]
    big = np.full(100000, 1.0, np.float32)  # above the fusion threshold: cuts the batch, runs alone
    bo = np.zeros_like(big)
    eb = comm.allreduce(big, bo)
    more = [comm.allreduce(b, o) for b, o in zip(bufs[:5], outs[:5])]
    for e in evs + [eb] + more:
        e.wait()
    for k, o in enumerate(outs):
        assert np.all(o == sum(p + k for p in range(W))), k
    assert np.all(bo == W)
    return stats("fused_ops"), stats("fused_batches")


def test_fusion_packs_small_allreduces():
    res = run_ranks(_fusion, 3, env={"CCL_FUSION": "1"})
    for ops, batches in res:
        assert ops == 45 and batches == 2


def test_fusion_count_threshold_cuts_batches():
    res = run_ranks(_fusion, 2, env={"CCL_FUSION": "1", "CCL_FUSION_COUNT_THRESHOLD": "16"})
    for ops, batches in res:
        assert ops == 45 and batches >= 4


def _subcomms_and_deps(comm):
    W, r = comm.size, comm.rank
    # split by parity: allreduce inside each half
    half = comm.split(r % 2)
    x = np.full(100, float(r), np.float64)
    half.allreduce(x).wait()
    expect = sum(p for p in range(W) if p % 2 == r % 2)
    assert np.all(x == expect) and half.size == len([p for p in range(W) if p % 2 == r % 2])
    # node / r2r communicators on one host: node == world, r2r == self
    node, r2r = comm.node_comm(), comm.r2r_comm()
    assert node.size == W and r2r.size == 1
    assert comm.local_rank == r and comm.local_size == W
    # dependency chain: the second operation starts only after the first event completed
    a = np.full(3000, 1.0, np.float32)
    b = np.zeros_like(a)
    e1 = comm.allreduce(a, b)
    c = np.zeros_like(a)
    e2 = comm.allreduce(b, c, deps=[e1])
    e2.wait()
    assert np.all(c == W * W)
    # priorities and ids are per communicator
    assert half.id != comm.id
    half.close()
    return True


@pytest.mark.parametrize("env", [{}, {"CCL_PRIORITY": "lifo"}, {"CCL_PRIORITY": "direct", "CCL_STRICT_ORDER": "1"},
                                 {"CCL_WORKER_COUNT": "2", "CCL_WORKER_AFFINITY": "0,1"},
                                 {"CCL_WORKER_OFFLOAD": "0", "CCL_SCHED_PROFILE": "1"}])
def test_subcommunicators_dependencies_and_modes(env):
    assert all(run_ranks(_subcomms_and_deps, 4, env=env))


def _hang(comm):
    """A peer that never joins: the entry hang detector turns the stall into an error."""
    import time

    from oneccl_b200 import CclError

    r = comm.rank
    x = np.ones(10, np.float32)
    if r == 0:
        try:
            comm.allreduce(x).wait()
        except CclError as e:
            return "timeout" if "no progress" in str(e) else str(e)
        return "completed"
    time.sleep(2.5)  # rank 1 skips the collective
    return "skipped"


def test_entry_hang_detector_reports_missing_peer():
    import multiprocessing as mp
    import os
    import tempfile

    # ranks do not run the closing barrier here (rank 0's communicator is broken on purpose)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    addr = os.path.join(tempfile.mkdtemp(prefix="cclx_"), "addr")
    procs = [ctx.Process(target=_hang_child, args=(r, addr, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.terminate()
    assert got[0] == "timeout" and got[1] == "skipped"


def _hang_child(rank, addr_file, q):
    import os
    import time

    os.environ["CCL_ENTRY_MAX_UPDATE_TIME_SEC"] = "1"
    from oneccl_b200.comm import KVS, Communicator

    if rank == 0:
        kvs = KVS.create_main()
        with open(addr_file + ".tmp", "w") as f:
            f.write(kvs.address)
        os.replace(addr_file + ".tmp", addr_file)
    else:
        while not os.path.exists(addr_file):
            time.sleep(0.01)
        kvs = KVS.connect(open(addr_file).read())
    comm = Communicator(2, rank, kvs)
    q.put((rank, _hang(comm)))
    q.close()
    q.join_thread()
    os._exit(0)


def _unordered(comm):
    from oneccl_b200.comm import stats

    W, r = comm.size, comm.rank
    names = [f"grad.{i}" for i in range(7)]
    n = 3000
    xs = {m: np.full(n + i, (r + 1.0) * (i + 1), np.float32) for i, m in enumerate(names)}
    ys = {m: np.zeros_like(xs[m]) for m in names}
    # every rank issues the operations in its own order, and waits in yet another one
    order = np.random.RandomState(100 + r).permutation(len(names))
    evs = {}
    for i in order:
        m = names[i]
        evs[m] = comm.allreduce(xs[m], ys[m], match_id=m, to_cache=bool(i % 2))
    for i in np.random.RandomState(200 + r).permutation(len(names)):
        evs[names[i]].wait()
    for i, m in enumerate(names):
        assert np.all(ys[m] == (i + 1) * W * (W + 1) / 2), m
    # a second pass reuses the names without coordination; allgatherv shares the mechanism
    for i in reversed(order):
        m = names[i]
        ys[m][:] = 0
        evs[m] = comm.allreduce(xs[m], ys[m], match_id=m, to_cache=bool(i % 2))
    g = np.zeros(4 * W, np.int32)
    ge = comm.allgatherv(np.full(4, r, np.int32), g, [4] * W, match_id="gather")
    for m in names:
        evs[m].wait()
        assert np.all(ys[m] == (names.index(m) + 1) * W * (W + 1) / 2), m
    ge.wait()
    assert np.all(g == np.repeat(np.arange(W), 4))
    return stats("postponed")


@pytest.mark.parametrize("env", [{}, {"CCL_WORKER_OFFLOAD": "0"}, {"CCL_WORKER_COUNT": "2"}])
def test_unordered_collectives_match_by_name(env):
    env = dict(env, CCL_UNORDERED_COLL="1")
    postponed = run_ranks(_unordered, 3, env=env)
    assert postponed[0] == 0  # the coordinator never parks an operation
