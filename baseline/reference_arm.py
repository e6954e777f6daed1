"""Loader of the unmodified reference library for ``bench.py --impl reference``.

``baseline/_ref`` holds an installation of the reference built from its own CMake project
(CPU path, libfabric transport); ``ref_shim.cpp`` is a C binding over its public C++ API.
This module sets the environment the reference reads (transport, libfabric location, local
rank), loads the binding with ctypes and exposes an in-place host allreduce.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
PREFIX = HERE / "_ref"


def available() -> str:
    """Empty string when the reference installation is usable, else the reason."""
    if not (PREFIX / "lib" / "libccl.so").exists():
        return "baseline/_ref/lib/libccl.so is missing (the reference was not built on this machine)"
    if not (PREFIX / "opt" / "mpi" / "libfabric" / "lib" / "libfabric.so").exists():
        return "the reference's libfabric is missing from baseline/_ref"
    return ""


def _build_shim() -> Path:
    so = PREFIX / "ref_shim.so"
    src = HERE / "ref_shim.cpp"
    if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", str(src), f"-I{PREFIX / 'include'}",
                               f"-L{PREFIX / 'lib'}", "-lccl", "-Wl,-rpath,$ORIGIN/lib", "-o", str(so)])
    return so


class ReferenceComm:
    """One rank of a reference communicator.  ``store`` is any object with ``set(key, bytes)`` /
    ``get(key) -> bytes`` shared by the ranks (a ``torch.distributed.TCPStore``); it carries the
    256-byte address of the reference's own key-value store from rank 0 to the others."""

    def __init__(self, rank: int, size: int, local_rank: int, local_size: int, store=None):
        fab = PREFIX / "opt" / "mpi" / "libfabric" / "lib"
        os.environ.setdefault("CCL_ATL_TRANSPORT", "ofi")
        os.environ.setdefault("CCL_OFI_LIBRARY_PATH", str(fab / "libfabric.so"))
        os.environ.setdefault("FI_PROVIDER_PATH", str(fab / "prov"))
        os.environ.setdefault("CCL_PROCESS_LAUNCHER", "none")
        os.environ.setdefault("CCL_LOCAL_RANK", str(local_rank))
        os.environ.setdefault("CCL_LOCAL_SIZE", str(local_size))
        os.environ.setdefault("CCL_KVS_IFACE", "lo")
        self.lib = C.CDLL(str(_build_shim()))
        self.lib.refshim_last_error.restype = C.c_char_p
        self.lib.refshim_allreduce.argtypes = [C.c_void_p, C.c_size_t, C.c_int]
        n = self.lib.refshim_addr_size()
        addr = (C.c_ubyte * n)()
        if rank == 0:
            self._check(self.lib.refshim_main_kvs(addr))
            if store is not None:
                store.set("reference_kvs_address", bytes(addr))
        else:
            raw = store.get("reference_kvs_address")
            C.memmove(addr, raw, n)
        self._check(self.lib.refshim_init(size, rank, addr))
        self.rank, self.size = rank, size

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError("reference oneCCL: " + self.lib.refshim_last_error().decode())

    def allreduce_(self, host_tensor):
        """In-place sum of a contiguous CPU tensor (float32 or bfloat16) over all ranks."""
        import torch

        code = {torch.float32: 0, torch.bfloat16: 1}[host_tensor.dtype]
        self._check(self.lib.refshim_allreduce(host_tensor.data_ptr(), host_tensor.numel(), code))
        return host_tensor

    def barrier(self):
        self._check(self.lib.refshim_barrier())

    def close(self):
        self.lib.refshim_finalize()
