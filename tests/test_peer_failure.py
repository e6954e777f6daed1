"""A rank that dies between two collectives: the others get an exception that names the lost peer instead of
waiting forever.  The failure is made on the host (the process exits); no timeout knob is set, the transport
itself notices the closed connection or, behind shared-memory rings, the missing process."""
import multiprocessing as mp
import os
import tempfile
import time
import traceback

import numpy as np
import pytest


def _rank(rank, world, addr_file, q, env, big):
    try:
        os.environ.update(env)
        os.environ["CCL_LOCAL_RANK"] = str(rank)
        os.environ["CCL_LOCAL_SIZE"] = str(world)
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
        n = 400000 if big else 100
        x = np.full(n, rank + 1.0, np.float32)
        comm.allreduce(x).wait()
        assert np.all(x == world * (world + 1) / 2)
        if rank == world - 1:
            q.put((rank, "left", 0.0))
            q.close()
            q.join_thread()
            os._exit(0)  # gone without a word: no barrier, no close
        time.sleep(0.3)
        t0 = time.time()
        try:
            comm.allreduce(x).wait()
            q.put((rank, "no error", time.time() - t0))
        except Exception as ex:  # noqa: BLE001
            secs = time.time() - t0
            # the failed launch's other partial schedules may still sit in a second worker's queue: dropping
            # the event and launching again must not pull the schedule from under them
            for _ in range(3):
                try:
                    ev = comm.allreduce(x)  # launched and dropped without waiting
                    del ev
                except Exception:  # noqa: BLE001
                    pass
                time.sleep(0.1)
            q.put((rank, "error: " + str(ex), secs))
        q.close()
        q.join_thread()
        os._exit(0)  # the communicator cannot say goodbye to a dead peer
    except Exception:
        q.put((rank, "crash: " + traceback.format_exc(), 0.0))


@pytest.mark.parametrize("env,big", [({}, False), ({}, True), ({"CCL_ATL_SHM": "0"}, False),
                                     ({"CCL_ATL_SHM": "0", "CCL_ALLREDUCE": "ring"}, True),
                                     ({"CCL_ATL_CMA": "0", "CCL_ALLREDUCE": "ring"}, True),
                                     ({"CCL_WORKER_COUNT": "2", "CCL_ALLREDUCE": "ring"}, True)],
                         ids=["rings-small", "rings-rendezvous", "sockets-small", "sockets-rendezvous", "rings-long",
                              "two-workers"])
def test_survivors_get_an_error_when_a_rank_dies(env, big):
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    addr = os.path.join(tempfile.mkdtemp(prefix="cclx_pf_"), "addr")
    procs = [ctx.Process(target=_rank, args=(r, world, addr, q, env, big)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        rank, what, secs = q.get(timeout=60)
        res[rank] = (what, secs)
    for p in procs:
        p.join(timeout=20)
    assert res[world - 1][0] == "left"
    for r in range(world - 1):
        what, secs = res[r]
        assert what.startswith("error:") and "left the job" in what, res
        assert secs < 10, res
