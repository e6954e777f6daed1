"""``torch.distributed`` backend named ``ccl``.

    import oneccl_b200.torch_backend          # registers the backend
    torch.distributed.init_process_group("ccl", ...)

The backend is the native extension ``_ccl_torch.so`` (a ``c10d::Backend``
subclass, see ``ProcessGroupCCL.cpp``) built in-tree by ``oneccl_b200._build``.
CPU tensors use the library's scheduler path, CUDA tensors its device kernels.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import torch
import torch.distributed as dist

from .. import _lib

_EXT = None


def load_extension():
    global _EXT
    if _EXT is not None:
        return _EXT
    _lib.load()  # libccl_b200.so first: the extension links against it
    path = Path(__file__).resolve().parent.parent / "lib" / "_ccl_torch.so"
    if not path.exists():
        from .. import _build

        _build.build_torch_backend()
    spec = importlib.util.spec_from_file_location("_ccl_torch", str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["_ccl_torch"] = mod
    _EXT = mod
    return mod


def _create(store, rank, size, timeout):
    return load_extension().create_backend(store, rank, size, timeout)


def register():
    if "ccl" not in getattr(dist.Backend, "backend_list", []):
        dist.Backend.register_backend("ccl", _create, devices=["cpu", "cuda"])


register()
