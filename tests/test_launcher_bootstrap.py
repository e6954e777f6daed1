"""Communicators whose rank, size and key-value store come from the launcher alone: a PMI-1 process manager
(played here by a small server that speaks the wire protocol on socket pairs handed down in PMI_FD, and in a
second run on a TCP port named in PMI_PORT) and torchrun-style variables, from Python and from C++."""
import os
import socket
import subprocess
import sys
import threading
from pathlib import Path

import pytest

from test_cpp_examples import ROOT, _build, _free_port_pair  # noqa: F401

CHILD = """
import numpy as np
from oneccl_b200.comm import Communicator
comm = Communicator.from_launcher()
x = np.full(1000, comm.rank + 1.0, np.float32)
comm.allreduce(x).wait()
assert np.all(x == comm.size * (comm.size + 1) / 2), x[:4]
comm.barrier().wait()
print("rank", comm.rank, "of", comm.size, "ok", flush=True)
comm.close()
"""


class FakeProcessManager:
    """The manager's side of PMI-1 for `size` clients: one thread per connection, a shared key-value
    space, a barrier that releases everybody when the last client arrives."""

    def __init__(self, size):
        self.size = size
        self.kvs = {}
        self.lock = threading.Lock()
        self.arrived = 0
        self.generation = 0
        self.cond = threading.Condition(self.lock)
        self.commands = []

    def serve(self, conn, rank, tcp=False):
        f = conn.makefile("rwb", buffering=0)

        def send(line):
            f.write((line + "\n").encode())

        for raw in f:
            line = raw.decode().strip()
            fields = dict(kv.split("=", 1) for kv in line.split(" ") if "=" in kv)
            cmd = fields.get("cmd")
            with self.lock:
                self.commands.append(cmd)
            if cmd == "initack":
                send("cmd=initack")
                send(f"cmd=set size={self.size}")
                send(f"cmd=set rank={rank}")
                send("cmd=set debug=0")
            elif cmd == "init":
                send("cmd=response_to_init pmi_version=1 pmi_subversion=1 rc=0")
            elif cmd == "get_maxes":
                send("cmd=maxes kvsname_max=256 keylen_max=64 vallen_max=1024")
            elif cmd == "get_my_kvsname":
                send("cmd=my_kvsname kvsname=kvs_test_0")
            elif cmd == "put":
                with self.lock:
                    self.kvs[fields["key"]] = fields["value"]
                send("cmd=put_result rc=0 msg=success")
            elif cmd == "get":
                with self.lock:
                    v = self.kvs.get(fields["key"])
                send(f"cmd=get_result rc=0 msg=success value={v}" if v is not None else "cmd=get_result rc=-1 msg=missing")
            elif cmd == "barrier_in":
                with self.cond:
                    gen = self.generation
                    self.arrived += 1
                    if self.arrived == self.size:
                        self.arrived = 0
                        self.generation += 1
                        self.cond.notify_all()
                    else:
                        while gen == self.generation:
                            self.cond.wait(timeout=60)
                send("cmd=barrier_out")
            elif cmd == "finalize":
                send("cmd=finalize_ack")
                break
        conn.close()


def _env(extra):
    env = dict(os.environ, PYTHONPATH=str(ROOT), **extra)
    for k in ("RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "PMI_FD", "PMI_PORT", "PMI_RANK", "PMI_SIZE", "PMI_ID"):
        if k not in extra:
            env.pop(k, None)
    return env


def test_pmi1_process_manager_on_inherited_sockets():
    size = 3
    pm = FakeProcessManager(size)
    procs, threads = [], []
    for r in range(size):
        ours, theirs = socket.socketpair()
        t = threading.Thread(target=pm.serve, args=(ours, r), daemon=True)
        t.start()
        threads.append(t)
        env = _env({"PMI_FD": str(theirs.fileno()), "PMI_RANK": str(r), "PMI_SIZE": str(size)})
        procs.append(subprocess.Popen([sys.executable, "-c", CHILD], env=env, pass_fds=(theirs.fileno(),),
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
        theirs.close()
    for r, p in enumerate(procs):
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0 and f"rank {r} of {size} ok" in out, err[-2000:]
    for t in threads:
        t.join(timeout=10)
    assert "ccl_kvs_address" in pm.kvs
    assert pm.commands.count("barrier_in") == 2 * size and pm.commands.count("finalize") == size


def test_pmi1_process_manager_on_a_port():
    size = 2
    pm = FakeProcessManager(size)
    srv = socket.socket()
    srv.bind(("127.0.0.1", 0))
    srv.listen(8)
    port = srv.getsockname()[1]

    def accept_all():
        for _ in range(size):
            conn, _ = srv.accept()
            first = conn.recv(4096).decode()  # cmd=initack pmiid=<rank>
            rank = int(first.strip().split("pmiid=")[1])
            conn.sendall(f"cmd=initack\ncmd=set size={size}\ncmd=set rank={rank}\ncmd=set debug=0\n".encode())
            threading.Thread(target=pm.serve, args=(conn, rank), daemon=True).start()

    threading.Thread(target=accept_all, daemon=True).start()
    procs = [subprocess.Popen([sys.executable, "-c", CHILD], env=_env({"PMI_PORT": f"127.0.0.1:{port}", "PMI_ID": str(r)}),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(size)]
    for r, p in enumerate(procs):
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0 and f"rank {r} of {size} ok" in out, err[-2000:]
    srv.close()


def test_torchrun_style_variables_and_single_process():
    port = _free_port_pair()
    procs = [subprocess.Popen([sys.executable, "-c", CHILD],
                              env=_env({"RANK": str(r), "WORLD_SIZE": "3", "MASTER_ADDR": "localhost", "MASTER_PORT": str(port)}),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(3)]
    for r, p in enumerate(procs):
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0 and f"rank {r} of 3 ok" in out, err[-2000:]
    alone = subprocess.run([sys.executable, "-c", CHILD], env=_env({}), capture_output=True, text=True, timeout=120)
    assert alone.returncode == 0 and "rank 0 of 1 ok" in alone.stdout, alone.stderr[-2000:]


def test_cpp_preview_create_communicator(tmp_path):
    src = tmp_path / "launcher_comm.cpp"
    src.write_text('''
#include <iostream>
#include <vector>
#include "oneapi/ccl.hpp"
int main() {
    ccl::init();
    auto comm = ccl::preview::create_communicator();
    std::vector<int> x(100, comm.rank() + 1), y(100, 0);
    ccl::allreduce(x.data(), y.data(), x.size(), ccl::reduction::sum, comm).wait();
    const int n = comm.size();
    auto halves = ccl::preview::split_communicators(
        { { comm, ccl::preview::create_comm_split_attr(ccl::attr_val<ccl::comm_split_attr_id::color>(comm.rank() % 2)) } });
    const bool ok = y[99] == n * (n + 1) / 2 && halves.size() == 1 && halves[0].size() == (n + 1 - comm.rank() % 2) / 2;
    ccl::barrier(comm).wait();
    std::cout << (ok ? "PASSED" : "FAILED") << std::endl;
    return ok ? 0 : 1;
}
''')
    exe = tmp_path / "launcher_comm"
    _build(src, exe)
    port = _free_port_pair()
    procs = [subprocess.Popen([str(exe)], env=_env({"RANK": str(r), "WORLD_SIZE": "4", "MASTER_ADDR": "127.0.0.1",
                                                    "MASTER_PORT": str(port)}),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(4)]
    for p in procs:
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0 and "PASSED" in out, out + err[-2000:]
