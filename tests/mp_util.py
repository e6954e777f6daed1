"""Spawns `world` local processes that rendezvous through the library's own KVS
(no mpirun): the parent creates nothing, rank 0 of the children creates the main
KVS and publishes its address through a file."""
from __future__ import annotations

import multiprocessing as mp
import os
import tempfile
import time
import traceback


def _child(fn, rank, world, addr_file, q, env, args):
    try:
        os.environ.update(env)
        os.environ["CCL_LOCAL_RANK"] = str(rank)
        os.environ["CCL_LOCAL_SIZE"] = str(world)
        for name in env.get("CCLX_TEST_UNSET", "").split(","):  # a test of what happens without them
            os.environ.pop(name, None)
        from oneccl_b200.comm import KVS, Communicator

        if rank == 0:
            kvs = KVS.create_main()
            tmp = addr_file + ".tmp"
            with open(tmp, "w") as f:
                f.write(kvs.address)
            os.replace(tmp, addr_file)
        else:
            t0 = time.time()
            while not os.path.exists(addr_file):
                if time.time() - t0 > 60:
                    raise RuntimeError("kvs address never appeared")
                time.sleep(0.01)
            kvs = KVS.connect(open(addr_file).read())
        comm = Communicator(world, rank, kvs)
        out = fn(comm, *args)
        comm.barrier().wait()
        comm.close()
        q.put((rank, "ok", out))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))


def run_ranks(fn, world, *args, env=None, timeout=120):
    """Runs fn(comm, *args) on `world` ranks; returns the list of return values by rank."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    d = tempfile.mkdtemp(prefix="cclx_")
    addr_file = os.path.join(d, "kvs_addr")
    procs = [ctx.Process(target=_child, args=(fn, r, world, addr_file, q, env or {}, args)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    deadline = time.time() + timeout
    try:
        while len(results) < world:
            left = deadline - time.time()
            if left <= 0:
                raise TimeoutError(f"ranks did not finish: got {sorted(results)}")
            try:
                rank, status, out = q.get(timeout=min(left, 1.0))
            except Exception:
                if any(p.exitcode not in (None, 0) for p in procs):
                    dead = [i for i, p in enumerate(procs) if p.exitcode not in (None, 0)]
                    raise RuntimeError(f"rank(s) {dead} died")
                continue
            if status != "ok":
                raise RuntimeError(f"rank {rank} failed:\n{out}")
            results[rank] = out
    finally:
        for p in procs:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()  # exactly the children started above
    return [results[r] for r in range(world)]
