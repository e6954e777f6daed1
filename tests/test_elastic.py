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
