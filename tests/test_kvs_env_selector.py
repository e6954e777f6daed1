"""Unit tests of the bootstrap store, the environment parser and the algorithm selector
(all in-process or with plain child processes; no transport involved)."""
import ctypes as C
import os
import subprocess
import sys
import threading
import time

import pytest

from oneccl_b200 import CclError, _lib
from oneccl_b200.comm import KVS, select_cpu_algo


def test_kvs_set_get_add_count_barrier():
    main = KVS.create_main()
    peers = [KVS.connect(main.address) for _ in range(3)]
    assert "_" in main.address
    peers[0].set("a/x", b"hello")
    assert peers[1].get("a/x") == b"hello"
    assert peers[2].try_get("a/missing") is None
    big = os.urandom(300000)  # far beyond the reference's 130-byte value records
    peers[0].set("a/big", big)
    assert peers[2].get("a/big") == big
    assert [peers[i % 3].add("ctr", 2) for i in range(5)][-1] == 10
    assert main.count("a/") == 2
    peers[0].delete("a/x")
    assert main.count("a/") == 1

    # blocking get is released by a later set
    got = {}

    def getter():
        got["v"] = peers[1].get("late", timeout_ms=5000)

    t = threading.Thread(target=getter)
    t.start()
    time.sleep(0.1)
    peers[2].set("late", b"now")
    t.join()
    assert got["v"] == b"now"

    # counted barrier: every participant returns only when all arrived
    order = []

    def arrive(k, delay):
        time.sleep(delay)
        peers[k].barrier("b0", 3)
        order.append(time.time())

    ts = [threading.Thread(target=arrive, args=(k, 0.1 * k)) for k in range(3)]
    t0 = time.time()
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert min(order) - t0 >= 0.19
    with pytest.raises(CclError):
        peers[0].get("never", timeout_ms=100)
    with pytest.raises(CclError):
        peers[0].barrier("lonely", 2, timeout_ms=100)
    for p in peers:
        p.close()
    main.close()


def test_kvs_fixed_address_and_connect_timeout():
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    main = KVS.create_main(f"127.0.0.1_{port}")
    assert main.address == f"127.0.0.1_{port}"
    main.close()
    os.environ["CCL_KVS_CONNECTION_TIMEOUT"] = "1"
    try:
        _lib.load().cclx_env_reload()
        with pytest.raises(CclError):
            KVS.connect(f"127.0.0.1_{port}")  # nobody listens any more
    finally:
        del os.environ["CCL_KVS_CONNECTION_TIMEOUT"]
        _lib.load().cclx_env_reload()


def test_env_size_parser():
    lib = _lib.load()
    out = C.c_size_t()
    for text, val in (("4096", 4096), ("16K", 16384), ("2m", 2 << 20), ("1G", 1 << 30), ("1.5K", 1536), ("64KB", 65536)):
        assert lib.cclx_env_size(text.encode(), C.byref(out)) == 0 and out.value == val
    for bad in ("", "abc", "12Q", "-5"):
        assert lib.cclx_env_size(bad.encode(), C.byref(out)) == -1


def test_selector_defaults_follow_size_tables():
    assert select_cpu_algo("allreduce", 1024) == "recursive_doubling"
    assert select_cpu_algo("allreduce", 100000) == "nreduce"
    assert select_cpu_algo("allreduce", 8 << 20) == "ring"
    assert select_cpu_algo("allgatherv", 1000) == "naive"
    assert select_cpu_algo("allgatherv", 1 << 20) == "ring"
    assert select_cpu_algo("alltoall", 4 << 20) == "scatter"
    assert select_cpu_algo("barrier", 0) == "dissemination"


def test_algorithm_grammar_parse_errors():
    lib = _lib.load()
    from oneccl_b200.dtypes import COLL

    ok = ["ring", "ring:0-8192;direct:8193-max", "rabenseifner:0-1M;ring:1048577-max", "2d"]
    bad = ["", "rign", "ring:5", "ring:9-3", "ring:a-b", "ring;bogus:0-max"]
    for spec in ok:
        assert lib.cclx_parse_algo_spec(COLL["allreduce"], spec.encode()) == 0, spec
    for spec in bad:
        assert lib.cclx_parse_algo_spec(COLL["allreduce"], spec.encode()) == -1, spec
    assert lib.cclx_parse_algo_spec(COLL["barrier"], b"ring") == 0
    assert lib.cclx_parse_algo_spec(COLL["barrier"], b"rabenseifner") == -1


def test_selector_env_override_in_child_process():
    code = (
        "from oneccl_b200.comm import select_cpu_algo as s;"
        "print(s('allreduce', 100), s('allreduce', 10000), s('allreduce', 1<<22), s('reduce', 10))"
    )
    env = dict(os.environ, CCL_ALLREDUCE="ring:0-8192;rabenseifner:8193-max", CCL_REDUCE="double_tree",
               PYTHONPATH=str(_lib.LIBDIR.parent.parent))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["ring", "rabenseifner", "rabenseifner", "double_tree"]


def test_scaleout_table_applies_to_the_inter_node_stage_only():
    code = (
        "from oneccl_b200.comm import select_cpu_algo as s;"
        "print(s('allreduce', 1 << 20), s('allreduce', 1 << 20, scaleout=True), s('allreduce', 100, scaleout=True),"
        " s('allgatherv', 1 << 20, scaleout=True))"
    )
    env = dict(os.environ, CCL_ALLREDUCE="ring", CCL_ALLREDUCE_SCALEOUT="rabenseifner:65536-max",
               PYTHONPATH=str(_lib.LIBDIR.parent.parent))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env)
    assert out.returncode == 0, out.stderr
    # ordinary operation: CCL_ALLREDUCE; scale-out stage: its own table where it has a range, else CCL_ALLREDUCE
    assert out.stdout.split() == ["ring", "rabenseifner", "ring", "ring"]


def test_datatype_table_and_cpu_reductions():
    import numpy as np

    lib = _lib.load()
    idx = lib.cclx_datatype_create(24)
    assert idx >= 12 and lib.cclx_datatype_size(idx) == 24
    assert lib.cclx_datatype_size(11) == 2 and lib.cclx_datatype_size(10) == 8
    assert lib.cclx_datatype_free(idx) == 0
    assert lib.cclx_datatype_size(idx) == -1
    assert lib.cclx_datatype_free(3) == -1  # predefined
    # bf16 / fp16 reductions go through fp32 and round to nearest even
    import torch

    a = torch.randn(1003).to(torch.bfloat16)
    b = torch.randn(1003).to(torch.bfloat16)
    ref = (a.float() + b.float()).to(torch.bfloat16)
    bb = b.clone()
    assert lib.cclx_comp_reduce(a.data_ptr(), 1003, bb.data_ptr(), 11, 0) == 0
    assert torch.equal(bb, ref)
    h = torch.randn(517).to(torch.float16)
    g = torch.randn(517).to(torch.float16)
    refh = torch.maximum(h, g)
    gg = g.clone()
    assert lib.cclx_comp_reduce(h.data_ptr(), 517, gg.data_ptr(), 8, 3) == 0
    assert torch.equal(gg, refh)
    x = np.arange(100, dtype=np.int64)
    y = np.full(100, 3, np.int64)
    assert lib.cclx_comp_reduce(x.ctypes.data, 100, y.ctypes.data, 6, 1) == 0
    assert np.array_equal(y, x * 3)
    assert lib.cclx_comp_impl(0).decode() in ("avx512f", "scalar")


def test_init_from_env_under_torchrun_uses_the_agent_store(tmp_path):
    """Three ranks under torchrun: the KVS address travels through the agent's store (no second fixed port),
    two communicators in one job."""
    script = tmp_path / "job.py"
    script.write_text(
        "import numpy as np\n"
        "from oneccl_b200.comm import init_from_env\n"
        "c = init_from_env(); c2 = init_from_env()\n"
        "x = np.full(10, c.rank + 1.0, np.float32); c.allreduce(x).wait()\n"
        "assert np.all(x == c.size * (c.size + 1) / 2)\n"
        "y = np.ones(3, np.float32); c2.allreduce(y).wait(); assert np.all(y == c2.size)\n"
        "c.barrier().wait(); print('rank-ok', c.rank, flush=True); c2.close(); c.close()\n")
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, PYTHONPATH=str(_lib.LIBDIR.parent.parent))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "3",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                         capture_output=True, text=True, env=env, timeout=240)
    assert out.returncode == 0, out.stderr[-3000:]
    assert out.stdout.count("rank-ok") == 3


def _run_py(code, **env):
    full = dict(os.environ, PYTHONPATH=str(_lib.LIBDIR.parent.parent), **env)
    return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=full)


def test_algo_fallback_switch():
    """A requested algorithm that exists only for device buffers falls back to the size table, unless
    CCL_ALGO_FALLBACK=0 makes that an error."""
    code = "from oneccl_b200.comm import select_cpu_algo as s; print(s('allreduce', 1 << 20))"
    out = _run_py(code, CCL_ALLREDUCE="topo")
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["ring"]  # the size table's choice at 1 MiB
    out = _run_py(code, CCL_ALLREDUCE="topo", CCL_ALGO_FALLBACK="0")
    assert out.returncode != 0
    assert "CCL_ALGO_FALLBACK" in out.stderr


def test_names_without_effect_are_reported():
    """Settings carried over from the reference that change nothing here are named in a warning, the
    Level Zero / SYCL families included; names that do something stay silent."""
    code = "from oneccl_b200.comm import select_cpu_algo as s; s('allreduce', 8)"
    out = _run_py(code, CCL_FUSION_CYCLE_MS="1", CCL_ZE_ENABLE="1", CCL_SYCL_ALLREDUCE_TMP_BUF="1",
                  CCL_ATL_SYNC_COLL="1", CCL_WORKER_COUNT="2")
    assert out.returncode == 0, out.stderr
    for name in ("CCL_FUSION_CYCLE_MS", "CCL_ZE_ENABLE", "CCL_SYCL_ALLREDUCE_TMP_BUF", "CCL_ATL_SYNC_COLL"):
        assert name + " is set but has no effect" in out.stderr, out.stderr
    assert "CCL_WORKER_COUNT is set" not in out.stderr


def test_kvs_mode_and_ip_exchange_values():
    code = "from oneccl_b200.comm import KVS; k = KVS.create_main(); print(k.address)"
    assert _run_py(code, CCL_KVS_MODE="pmi").returncode == 0
    out = _run_py(code, CCL_KVS_MODE="mpi")
    assert out.returncode != 0 and "no MPI" in out.stderr
    # env exchange: the address must be given outside the program
    out = _run_py(code, CCL_KVS_IP_EXCHANGE="env")
    assert out.returncode != 0 and "CCL_KVS_IP_PORT" in out.stderr
    out = _run_py(code, CCL_KVS_IP_EXCHANGE="env", CCL_KVS_IP_PORT="127.0.0.1_29871")
    assert out.returncode == 0, out.stderr
    assert "29871" in out.stdout
