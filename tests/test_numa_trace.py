"""NUMA / placement helpers against a fake sysfs tree, and the tracing level knob."""
import ctypes as C
import os
import subprocess
import sys

from oneccl_b200 import _lib


def _query(root, what, arg=0, text=None, cap=256):
    lib = _lib.load()
    out = (C.c_int * cap)()
    n = lib.cclx_numa_query(root.encode(), what, arg, text.encode() if text is not None else None, out, cap)
    assert n >= 0
    return list(out[:n])


def _fake_sysfs(tmp_path):
    for node, cpus in ((0, "0-3,8-11"), (1, "4-7,12-15")):
        d = tmp_path / "devices/system/node" / f"node{node}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(cpus + "\n")
    pci = tmp_path / "bus/pci/devices/0000:1b:00.0"
    pci.mkdir(parents=True)
    (pci / "numa_node").write_text("1\n")
    return str(tmp_path)


def test_cpulist_parser():
    assert _query("", 4, text="0-2,5,7-8") == [0, 1, 2, 5, 7, 8]
    assert _query("", 4, text="") == []
    assert _query("", 4, text="3") == [3]


def test_fake_sysfs_nodes_and_pci(tmp_path):
    root = _fake_sysfs(tmp_path)
    assert _query(root, 0) == [2]
    assert _query(root, 1, arg=1) == [4, 5, 6, 7, 12, 13, 14, 15]
    assert _query(root, 2, arg=9) == [0]
    assert _query(root, 2, arg=13) == [1]
    assert _query(root, 2, arg=99) == [-1]
    assert _query(root, 3, text="0000:1b:00.0") == [1]
    assert _query(root, 3, text="00000000:1B:00.0") == [1]  # NVML spelling: 8-digit domain, upper case
    assert _query(root, 3, text="0000:ff:00.0") == [-1]


def test_this_machine_has_at_least_one_node():
    assert _query("", 0)[0] >= 1
    allowed = _query("", 5, cap=4096)
    assert len(allowed) >= 1 and all(_query("", 2, arg=c)[0] >= 0 for c in allowed[:4])
    assert _lib.load().cclx_numa_selftest(0, 1 << 20) == 0


def test_auto_worker_placement():
    lib = _lib.load()
    cpus = (C.c_int * 32)(*range(32))
    out = (C.c_int * 8)()
    # 4 ranks x 2 workers on 32 cores: disjoint cores taken from the end
    got = []
    for lr in range(4):
        n = lib.cclx_numa_auto_worker_cpus(cpus, 32, lr, 4, 2, out)
        assert n == 2
        got += list(out[:n])
    assert sorted(got) == list(range(24, 32)) and got[:2] == [31, 30]
    # too few cores to spare any: no pinning
    assert lib.cclx_numa_auto_worker_cpus(cpus, 8, 0, 4, 2, out) == 0
    # unknown local rank: no pinning
    assert lib.cclx_numa_auto_worker_cpus(cpus, 32, -1, -1, 1, out) == 0


def test_tracing_levels_do_not_disturb_results():
    code = (
        "import numpy as np\n"
        "from oneccl_b200.comm import KVS, Communicator\n"
        "k = KVS.create_main(); c = Communicator(1, 0, k)\n"
        "x = np.arange(5, dtype=np.float32); y = np.zeros_like(x)\n"
        "c.allreduce(x, y).wait(); assert (x == y).all(); c.close(); print('ok')\n"
    )
    for level in ("0", "1", "2"):
        env = dict(os.environ, CCL_ITT_LEVEL=level, CCL_WORKER_AFFINITY="auto")
        r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120,
                           cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        assert r.returncode == 0 and "ok" in r.stdout, r.stderr
