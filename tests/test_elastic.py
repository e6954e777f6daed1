"""Elastic membership: pods agree on a member list, a pod that dies without saying so is
noticed through its heartbeat, the survivors re-form a smaller communicator, a newcomer is
taken in.  Failures are injected on the host only (a process that exits)."""
import multiprocessing as mp
import os
import tempfile
import time

import numpy as np


def _pod(name, addr_file, q, script):
    try:
        from oneccl_b200.comm import KVS, ElasticGroup

        if name == "pod0":
            kvs = KVS.create_main()
            tmp = addr_file + ".tmp"
            with open(tmp, "w") as f:
                f.write(kvs.address)
            os.replace(tmp, addr_file)
        else:
            t0 = time.time()
            while not os.path.exists(addr_file):
                assert time.time() - t0 < 60
                time.sleep(0.01)
            kvs = KVS.connect(open(addr_file).read())
        eg = ElasticGroup(kvs, pod_id=name, heartbeat_ms=50, dead_after_ms=600, min_size=script["min_size"])
        log = []
        comm = None
        for phase in script["phases"]:
            want = phase["size"]
            deadline = time.time() + 60
            while True:
                rank, size, gen = eg.form(timeout_ms=30000)
                if size == want:
                    break
                assert time.time() < deadline, f"{name}: stuck at size {size}, want {want}"
                time.sleep(0.1)
            comm = eg.communicator()
            x = np.full(1000, float(rank + 1), np.float32)
            y = np.zeros_like(x)
            comm.allreduce(x, y).wait()
            assert np.all(y == size * (size + 1) / 2), (name, y[0], size)
            log.append((size, rank, gen, list(eg.members)))
            comm.barrier().wait()
            if phase.get("die") == name:
                q.put((name, "ok", log))
                q.close()
                q.join_thread()
                os._exit(0)  # no leave(), no close(): the others must notice by themselves
            comm.close()
            if phase.get("leave") == name:
                eg.leave()
                q.put((name, "ok", log))
                return
            # wait for the membership change that ends this phase
            if phase is not script["phases"][-1]:
                t0 = time.time()
                while not eg.changed():
                    assert time.time() - t0 < 30, f"{name}: no membership change seen"
                    time.sleep(0.05)
        eg.leave()
        q.put((name, "ok", log))
        if name == "pod0":
            time.sleep(1.0)  # the store lives here: let the others finish their last requests
    except Exception:
        import traceback

        q.put((name, "error", traceback.format_exc()))


def test_pods_die_and_join():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    addr = os.path.join(tempfile.mkdtemp(prefix="cclx_el_"), "addr")
    # three pods; pod2 dies silently after phase 1; the two survivors regroup; pod3 joins for phase 3
    first = {"min_size": 2, "phases": [{"size": 3, "die": "pod2"}, {"size": 2}, {"size": 3}]}
    procs = {n: ctx.Process(target=_pod, args=(n, addr, q, first)) for n in ("pod0", "pod1", "pod2")}
    for p in procs.values():
        p.start()
    results = {}
    newcomer = None
    deadline = time.time() + 150
    while len(results) < 4 and time.time() < deadline:
        try:
            name, status, log = q.get(timeout=1.0)
        except Exception:
            continue
        assert status == "ok", f"{name}:\n{log}"
        results[name] = log
        if name == "pod2" and newcomer is None:
            time.sleep(2.0)  # let the survivors run their two-pod phase first
            late = {"min_size": 2, "phases": [{"size": 3}]}
            newcomer = ctx.Process(target=_pod, args=("pod3", addr, q, late))
            newcomer.start()
    for p in list(procs.values()) + ([newcomer] if newcomer else []):
        p.join(timeout=20)
        if p.is_alive():
            p.kill()
    assert set(results) == {"pod0", "pod1", "pod2", "pod3"}, results.keys()
    sizes = [entry[0] for entry in results["pod0"]]
    assert sizes == [3, 2, 3]
    gens = [entry[2] for entry in results["pod0"]]
    assert gens == sorted(gens) and len(set(gens)) == 3
    # ranks follow the join order; the newcomer takes the last rank
    assert results["pod0"][-1][3] == ["pod0", "pod1", "pod3"] and results["pod3"][0][1] == 2
    assert results["pod1"][1][:2] == (2, 1)


def _pod_window(name, addr_file, q, go_file):
    """pod0 / pod1 agree on a list of two; inside pod1's agreement window (list published, others' not yet
    read) a third pod registers.  Whatever each of the two saw at that moment, both must end up with the same
    member lists generation by generation, and finally with all three."""
    try:
        from oneccl_b200.comm import KVS, ElasticGroup

        if name == "pod0":
            kvs = KVS.create_main()
            tmp = addr_file + ".tmp"
            with open(tmp, "w") as f:
                f.write(kvs.address)
            os.replace(tmp, addr_file)
        else:
            t0 = time.time()
            while not os.path.exists(addr_file):
                assert time.time() - t0 < 60
                time.sleep(0.01)
            kvs = KVS.connect(open(addr_file).read())
        if name == "pod2":  # the newcomer waits until pod1 is inside its window
            t0 = time.time()
            while not os.path.exists(go_file):
                assert time.time() - t0 < 60
                time.sleep(0.005)
        eg = ElasticGroup(kvs, pod_id=name, heartbeat_ms=50, dead_after_ms=600, min_size=2)
        fired = []

        def window(gen):
            if name == "pod1" and not fired:
                fired.append(gen)
                open(go_file, "w").close()
                time.sleep(0.4)  # long enough for pod2 to register and beat

        eg.set_window_hook(window)
        history = []
        deadline = time.time() + 60
        while True:
            rank, size, gen = eg.form(timeout_ms=30000)
            history.append((gen, list(eg.members)))
            comm = eg.communicator()  # every adopted view must be usable: all its members adopted it too
            x = np.full(16, float(rank + 1), np.float32)
            y = np.zeros_like(x)
            comm.allreduce(x, y).wait()
            assert np.all(y == size * (size + 1) / 2), (name, gen, y[0], size)
            comm.close()
            if size == 3:
                break
            assert time.time() < deadline, f"{name}: never reached three members: {history}"
            t0 = time.time()
            while not eg.changed():
                assert time.time() - t0 < 30, f"{name}: no membership change seen"
                time.sleep(0.02)
        kvs.barrier("window_done", 3, 30000)
        eg.leave()
        q.put((name, "ok", history))
        if name == "pod0":
            time.sleep(1.0)
    except Exception:
        import traceback

        q.put((name, "error", traceback.format_exc()))


def test_pod_registers_inside_the_agreement_window():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    d = tempfile.mkdtemp(prefix="cclx_el_")
    addr, go = os.path.join(d, "addr"), os.path.join(d, "go")
    procs = [ctx.Process(target=_pod_window, args=(n, addr, q, go)) for n in ("pod0", "pod1", "pod2")]
    for p in procs:
        p.start()
    results = {}
    deadline = time.time() + 120
    while len(results) < 3 and time.time() < deadline:
        try:
            name, status, hist = q.get(timeout=1.0)
        except Exception:
            continue
        assert status == "ok", f"{name}:\n{hist}"
        results[name] = dict(hist)
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.kill()
    assert set(results) == {"pod0", "pod1", "pod2"}, results.keys()
    # a generation that two pods adopted has the same member list on both, and every member of it adopted it
    for a in results:
        for gen, members in results[a].items():
            for m in members:
                assert results[m].get(gen) == members, (a, gen, members, results[m])
    assert all(sorted(max(r.items())[1]) == ["pod0", "pod1", "pod2"] for r in results.values())
