"""KVS, communicators and collectives on host (numpy / CPU torch) and device
(CUDA torch) buffers - the Python face of the ``ccl::`` API.

    kvs = KVS.create_main()              # rank 0; ship kvs.address out of band
    kvs = KVS.connect(address)           # other ranks
    comm = Communicator(size, rank, kvs)
    comm.allreduce(x).wait()             # CPU tensor -> scheduler path
    comm.allreduce(x_cuda).wait()        # CUDA tensor -> device kernels on the current stream

``init_from_env()`` builds the world communicator under torchrun
(RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT): rank 0 starts
the KVS server on MASTER_PORT + 1 + CCL_KVS_PORT_OFFSET and everybody connects.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from .dtypes import COLL, GPU_ALGO, reduce_op_code

_NP_CODES = {
    np.dtype("int8"): 0, np.dtype("uint8"): 1, np.dtype("int16"): 2, np.dtype("uint16"): 3,
    np.dtype("int32"): 4, np.dtype("uint32"): 5, np.dtype("int64"): 6, np.dtype("uint64"): 7,
    np.dtype("float16"): 8, np.dtype("float32"): 9, np.dtype("float64"): 10,
}


class _CollDesc(C.Structure):
    _fields_ = [
        ("ctype", C.c_int), ("send_buf", C.c_void_p), ("recv_buf", C.c_void_p), ("count", C.c_size_t),
        ("dtype", C.c_int), ("reduction", C.c_int), ("root", C.c_int), ("peer", C.c_int),
        ("send_counts", C.POINTER(C.c_size_t)), ("recv_counts", C.POINTER(C.c_size_t)),
        ("recv_bufs", C.POINTER(C.c_void_p)), ("stream", C.c_void_p), ("device", C.c_int),
        ("priority", C.c_int), ("synchronous", C.c_int), ("to_cache", C.c_int), ("match_id", C.c_char_p),
        ("reduction_fn", C.c_void_p), ("do_scale", C.c_int), ("scale", C.c_float), ("out_dtype", C.c_int),
        ("gpu_algo", C.c_char_p), ("deps", C.POINTER(C.c_void_p)), ("n_deps", C.c_int),
    ]


# signature of a custom reduction: (in, in_count, inout, out_count*, dtype, ctx*)
REDUCTION_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_size_t, C.c_void_p, C.POINTER(C.c_size_t), C.c_int, C.c_void_p)


def _buf_info(x):
    """(pointer, element count, ccl dtype code, is_device, keepalive)"""
    if x is None:
        return 0, 0, 9, False, None
    if isinstance(x, np.ndarray):
        assert x.flags["C_CONTIGUOUS"], "buffers must be contiguous"
        return x.ctypes.data, x.size, _NP_CODES[x.dtype], False, x
    import torch

    from .dtypes import torch_to_ccl

    if isinstance(x, torch.Tensor):
        assert x.is_contiguous(), "buffers must be contiguous"
        return x.data_ptr(), x.numel(), torch_to_ccl(x.dtype), x.is_cuda, x
    raise TypeError(f"unsupported buffer {type(x)}")


class Event:
    def __init__(self, handle, keep=()):
        self._lib = _lib.load()
        self._h = C.c_void_p(handle)
        self._keep = keep

    def wait(self):
        _lib.check(self._lib.cclx_event_wait(self._h))
        return self

    def test(self) -> bool:
        r = self._lib.cclx_event_test(self._h)
        if r < 0:
            _lib.check(-1)
        return r == 1

    @property
    def native(self):
        return self._lib.cclx_event_native(self._h)

    def __del__(self):
        try:
            if self._h:
                self._lib.cclx_event_destroy(self._h)
        except Exception:
            pass


class KVS:
    def __init__(self, handle, is_main):
        self._lib = _lib.load()
        self._h = C.c_void_p(handle)
        self.is_main = is_main

    @classmethod
    def create_main(cls, ip_port: str = "") -> "KVS":
        lib = _lib.load()
        h = lib.cclx_kvs_create_main(ip_port.encode() if ip_port else None)
        if not h:
            raise _lib.CclError(lib.cclx_last_error().decode())
        return cls(h, True)

    @classmethod
    def connect(cls, address: str) -> "KVS":
        lib = _lib.load()
        h = lib.cclx_kvs_create_peer(address.encode())
        if not h:
            raise _lib.CclError(lib.cclx_last_error().decode())
        return cls(h, False)

    @property
    def address(self) -> str:
        buf = C.create_string_buffer(256)
        _lib.check(self._lib.cclx_kvs_address(self._h, buf, 256))
        return buf.value.decode()

    def set(self, key: str, value: bytes):
        _lib.check(self._lib.cclx_kvs_set(self._h, key.encode(), value, len(value)))

    def get(self, key: str, timeout_ms: int = 30000) -> Optional[bytes]:
        cap = 1 << 16
        while True:
            buf = C.create_string_buffer(cap)
            n = self._lib.cclx_kvs_get(self._h, key.encode(), buf, cap, timeout_ms)
            if n < 0:
                if timeout_ms < 0:
                    return None
                raise _lib.CclError(self._lib.cclx_last_error().decode())
            if n <= cap:
                return buf.raw[:n]
            cap = n

    def try_get(self, key: str) -> Optional[bytes]:
        return self.get(key, timeout_ms=-1)

    def add(self, key: str, delta: int = 1) -> int:
        return int(self._lib.cclx_kvs_add(self._h, key.encode(), delta))

    def count(self, prefix: str) -> int:
        return int(self._lib.cclx_kvs_count(self._h, prefix.encode()))

    def delete(self, key: str):
        _lib.check(self._lib.cclx_kvs_del(self._h, key.encode()))

    def barrier(self, name: str, participants: int, timeout_ms: int = 30000):
        _lib.check(self._lib.cclx_kvs_barrier(self._h, name.encode(), participants, timeout_ms))

    def close(self):
        if self._h:
            self._lib.cclx_kvs_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Communicator:
    def __init__(self, size: int = 0, rank: int = 0, kvs: Optional[KVS] = None, _handle=None, _parent=None):
        self._lib = _lib.load()
        self._kvs = kvs
        self._parent = _parent
        if _handle is None:
            h = self._lib.cclx_comm_create(size, rank, kvs._h)
            if not h:
                raise _lib.CclError(self._lib.cclx_last_error().decode())
            _handle = h
        self._h = C.c_void_p(_handle)
        self.rank = self._lib.cclx_comm_rank(self._h)
        self.size = self._lib.cclx_comm_size(self._h)
        self._device_group = None
        self._group_keep = []

    # ---- structure ----------------------------------------------------------------------
    def split(self, color: int, key: Optional[int] = None) -> "Communicator":
        h = self._lib.cclx_comm_split(self._h, color, self.rank if key is None else key)
        if not h:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        return Communicator(_handle=h, _parent=self)

    def node_comm(self) -> "Communicator":
        h = self._lib.cclx_comm_node(self._h)
        if not h:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        return Communicator(_handle=h, _parent=self)

    def r2r_comm(self) -> "Communicator":
        h = self._lib.cclx_comm_r2r(self._h)
        if not h:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        return Communicator(_handle=h, _parent=self)

    @classmethod
    def from_launcher(cls) -> "Communicator":
        """World communicator whose rank, size and key-value store come from the process launcher: a PMI-1
        process manager (Hydra's ``mpiexec``: ``PMI_FD`` / ``PMI_PORT``) or torchrun-style variables; the
        C++ form is ``ccl::preview::create_communicator()``."""
        lib = _lib.load()
        h = lib.cclx_comm_create_from_launcher()
        if not h:
            raise _lib.CclError(lib.cclx_last_error().decode())
        return cls(_handle=h)

    @property
    def id(self) -> int:
        return int(self._lib.cclx_comm_id(self._h))

    @property
    def transport_name(self) -> str:
        """"tcp" (the library's socket / shared-memory mesh) or "ofi:<provider>" (libfabric)."""
        return self._lib.cclx_comm_transport_name(self._h).decode()

    def transport_stats(self) -> dict:
        """Counters of the host transport under this communicator: messages and bytes, messages that
        arrived before their receive was posted, one-sided writes by cross-memory copy and by message."""
        names = ("msgs_sent", "bytes_sent", "bytes_received", "unexpected_msgs", "rma_direct_writes",
                 "rma_message_writes", "rndv_sends")
        return {n: int(self._lib.cclx_comm_transport_stat(self._h, k)) for k, n in enumerate(names)}

    @property
    def local_rank(self) -> int:
        return self._lib.cclx_comm_local_rank(self._h)

    @property
    def local_size(self) -> int:
        return self._lib.cclx_comm_local_size(self._h)

    @property
    def device_group(self):
        """The node's device communicator (symmetric heap, kernels).  First use is collective."""
        if self._device_group is None:
            import torch

            from .ops.device_group import DeviceGroup

            self._lib.cclx_set_device(torch.cuda.current_device())
            h = self._lib.cclx_comm_device(self._h)
            if not h:
                raise _lib.CclError(self._lib.cclx_last_error().decode())
            self._device_group = DeviceGroup(h, False, owns=False)
        return self._device_group

    def abort(self):
        _lib.check(self._lib.cclx_comm_abort(self._h))

    def heartbeat(self):
        _lib.check(self._lib.cclx_comm_heartbeat(self._h))

    def peer_alive(self, peer: int, max_age_ms: int = 2000) -> bool:
        return self._lib.cclx_comm_peer_alive(self._h, peer, max_age_ms) == 1

    def close(self):
        if self._h:
            if self._device_group is not None:
                import torch

                torch.cuda.synchronize()
                self._device_group._h = None
                self._device_group = None
                self._lib.cclx_comm_release_device(self._h)
            self._lib.cclx_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- generic launcher ---------------------------------------------------------------
    def _run(self, ctype, send=None, recv=None, count=None, op="sum", root=0, peer=-1, send_counts=None,
             recv_counts=None, recv_bufs=None, priority=0, synchronous=False, to_cache=False, match_id=None,
             reduction_fn=None, scale=None, out_dtype=None, gpu_algo=None, deps=(), stream=None, dtype=None) -> Event:
        sp, sn, sdt, sdev, k1 = _buf_info(send)
        rp, rn, rdt, rdev, k2 = _buf_info(recv)
        keep = [k1, k2]
        d = _CollDesc()
        d.ctype = COLL[ctype]
        d.send_buf, d.recv_buf = sp, rp
        d.dtype = dtype if dtype is not None else (sdt if send is not None else rdt)
        d.count = count if count is not None else (sn if send is not None else rn)
        d.reduction = 4 if reduction_fn is not None and op == "custom" else reduce_op_code(op) if op != "custom" else 4
        d.root, d.peer = root, peer
        if send_counts is not None:
            sc = _lib.size_array(send_counts)
            d.send_counts = sc
            keep.append(sc)
        if recv_counts is not None:
            rc = _lib.size_array(recv_counts)
            d.recv_counts = rc
            keep.append(rc)
        device = sdev or rdev
        if recv_bufs is not None:
            infos = [_buf_info(b) for b in recv_bufs]
            arr = _lib.ptr_array([i[0] for i in infos])
            d.recv_bufs = arr
            keep += [arr] + [i[4] for i in infos]
            device = device or any(i[3] for i in infos)
            if recv is None:
                d.dtype = infos[0][2] if send is None else sdt
        d.device = 1 if device else 0
        if device:
            from .ops.device_group import _stream_ptr

            d.stream = _stream_ptr(stream)
            if out_dtype is None and send is not None and recv is not None and sdt != rdt:
                out_dtype = rdt
        d.priority = priority
        d.synchronous = 1 if synchronous else 0
        d.to_cache = 1 if to_cache else 0
        d.match_id = match_id.encode() if match_id else None
        if reduction_fn is not None:
            d.reduction_fn = C.cast(reduction_fn, C.c_void_p)
            keep.append(reduction_fn)
        d.do_scale = 0 if scale is None else 1
        d.scale = 1.0 if scale is None else float(scale)
        d.out_dtype = -1 if out_dtype is None else int(out_dtype)
        d.gpu_algo = gpu_algo.encode() if gpu_algo else None
        if deps:
            arr = _lib.ptr_array([e._h.value for e in deps])
            d.deps = arr
            d.n_deps = len(deps)
            keep += [arr, list(deps)]
        h = self._lib.cclx_coll(self._h, C.byref(d))
        if not h:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        return Event(h, keep)

    # ---- the twelve operations ------------------------------------------------------------
    def allreduce(self, send, recv=None, op="sum", **kw) -> Event:
        return self._run("allreduce", send, send if recv is None else recv, op=op, **kw)

    def allgather(self, send, recv, **kw) -> Event:
        return self._run("allgather", send, recv, count=_buf_info(send)[1], **kw)

    def allgatherv(self, send, recv, recv_counts: Sequence[int], recv_bufs=None, **kw) -> Event:
        count = recv_counts[self.rank]
        return self._run("allgatherv", send, recv, count=count, recv_counts=recv_counts, recv_bufs=recv_bufs, **kw)

    def alltoall(self, send, recv, **kw) -> Event:
        return self._run("alltoall", send, recv, count=_buf_info(send)[1] // self.size, **kw)

    def alltoallv(self, send, send_counts, recv, recv_counts, **kw) -> Event:
        return self._run("alltoallv", send, recv, count=0, send_counts=send_counts, recv_counts=recv_counts, **kw)

    def barrier(self, stream=None) -> Event:
        d = _CollDesc()
        d.ctype = COLL["barrier"]
        d.out_dtype = -1
        h = self._lib.cclx_coll(self._h, C.byref(d))
        if not h:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        return Event(h)

    def broadcast(self, buf, root=0, recv=None, **kw) -> Event:
        if recv is None:
            return self._run("bcast", buf, buf, root=root, **kw)
        return self._run("broadcast", buf, recv, root=root, count=_buf_info(recv)[1], **kw)

    def reduce(self, send, recv, root=0, op="sum", **kw) -> Event:
        return self._run("reduce", send, recv, count=_buf_info(send)[1], op=op, root=root, **kw)

    def reduce_scatter(self, send, recv, op="sum", **kw) -> Event:
        return self._run("reduce_scatter", send, recv, count=_buf_info(recv)[1], op=op, **kw)

    def send(self, buf, peer: int, **kw) -> Event:
        return self._run("send", buf, None, peer=peer, **kw)

    def recv(self, buf, peer: int, **kw) -> Event:
        return self._run("recv", None, buf, peer=peer, **kw)

    def cache_size(self) -> int:
        return int(self._lib.cclx_comm_cache_size(self._h))


def group_start():
    _lib.check(_lib.load().cclx_group_start())


def group_end():
    _lib.check(_lib.load().cclx_group_end())


def stats(which: str, coll: str = "allreduce") -> int:
    idx = {"calls": 0, "device_calls": 1, "fused_ops": 2, "fused_batches": 3, "cache_hits": 4, "postponed": 5}[which]
    return int(_lib.load().cclx_stats(idx, COLL[coll]))


def select_cpu_algo(coll: str, nbytes: int, comm_size: int = 2, scaleout: bool = False) -> str:
    """Name of the host algorithm the selector picks; ``scaleout`` asks for the inter-node stage of a
    hierarchical device collective (``CCL_<COLL>_SCALEOUT`` is consulted first)."""
    buf = C.create_string_buffer(64)
    _lib.check(_lib.load().cclx_select_cpu_algo(COLL[coll], nbytes, comm_size, 1 if scaleout else 0, buf, 64))
    return buf.value.decode()


def topo_describe() -> str:
    buf = C.create_string_buffer(16384)
    _lib.check(_lib.load().cclx_topo_describe(buf, 16384))
    return buf.value.decode()


_init_calls = 0


def init_from_env(port_offset: Optional[int] = None) -> Communicator:
    """World communicator under torchrun-style environment variables.

    Under a torchrun agent (``TORCHELASTIC_USE_AGENT_STORE=True``) rank 0 starts the KVS on a free port
    and publishes its address through the agent's store at MASTER_ADDR:MASTER_PORT, so no second
    well-known port is needed.  Otherwise the KVS listens on MASTER_PORT + 1 (+ ``CCL_KVS_PORT_OFFSET``)."""
    global _init_calls
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    if addr in ("localhost",):
        addr = "127.0.0.1"
    port = int(os.environ.get("MASTER_PORT", "29500"))
    call = _init_calls
    _init_calls += 1
    if port_offset is None and os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "").lower() == "true" \
            and os.environ.get("CCL_KVS_USE_AGENT_STORE", "1") == "1":
        try:
            from datetime import timedelta

            from torch.distributed import TCPStore

            store = TCPStore(addr, port, world, False, timeout=timedelta(seconds=60))
            key = f"ccl_b200/kvs/{os.environ.get('TORCHELASTIC_RESTART_COUNT', '0')}/{call}"
            if rank == 0:
                kvs = KVS.create_main(f"{addr}_0" if addr[0].isdigit() else "")
                store.set(key, kvs.address)
            else:
                kvs = KVS.connect(store.get(key).decode())
            return Communicator(world, rank, kvs)
        except Exception as e:  # noqa: BLE001  fall back to the fixed port
            if rank == 0:
                print(f"oneccl_b200: agent store not usable ({e}); using MASTER_PORT + 1", flush=True)
    if port_offset is None:  # a further communicator of the same job takes the next port
        port_offset = 1 + int(os.environ.get("CCL_KVS_PORT_OFFSET", "0")) + call
    ip_port = f"{addr}_{port + port_offset}"
    kvs = KVS.create_main(ip_port) if rank == 0 else KVS.connect(ip_port)
    return Communicator(world, rank, kvs)


class ElasticGroup:
    """Membership that survives pods leaving and joining (the reference's resizable process
    manager, ``CCL_PM_TYPE=resizable``): every pod heart-beats into the KVS, the live pods agree
    on a member list ("generation") and re-form their communicator over it.

        eg = ElasticGroup(kvs, pod_id="worker-3", min_size=2)
        rank, size, gen = eg.form()            # blocks until the live pods agree
        comm = eg.communicator()
        ...
        if eg.changed():                        # somebody died, left or joined
            comm.close(); eg.form(); comm = eg.communicator()

    ``resize_fn(n)`` may veto a size: return "wait", "run" or "finalize"."""

    _ACTIONS = {"wait": 0, "run": 1, "finalize": 2}

    def __init__(self, kvs: "KVS", pod_id: Optional[str] = None, heartbeat_ms: int = 100, dead_after_ms: int = 1000,
                 min_size: int = 1, resize_fn=None):
        import os
        import socket

        self._lib = _lib.load()
        self._kvs = kvs
        pod_id = pod_id or f"{socket.gethostname()}-{os.getpid()}"
        h = self._lib.cclx_elastic_create(kvs._h, pod_id.encode(), heartbeat_ms, dead_after_ms, min_size)
        if not h:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        self._h = C.c_void_p(h)
        self.pod_id = pod_id
        self.rank = self.size = -1
        self.generation = 0
        self.members: List[str] = []
        self._cb = None
        if resize_fn is not None:
            proto = C.CFUNCTYPE(C.c_int, C.c_size_t)
            self._cb = proto(lambda n: self._ACTIONS[resize_fn(int(n))])
            _lib.check(self._lib.cclx_elastic_set_resize_fn(self._h, C.cast(self._cb, C.c_void_p)))

    def set_window_hook(self, fn):
        """``fn(generation)`` runs inside ``form`` right after this pod published its member list for a
        generation and before it reads the others' lists (tests use it to change the membership there)."""
        if fn is None:
            self._win = None
            _lib.check(self._lib.cclx_elastic_set_window_hook(self._h, None))
            return
        proto = C.CFUNCTYPE(None, C.c_ulonglong)
        self._win = proto(lambda g: fn(int(g)))
        _lib.check(self._lib.cclx_elastic_set_window_hook(self._h, C.cast(self._win, C.c_void_p)))

    def form(self, timeout_ms: int = 60000):
        out = (C.c_longlong * 3)()
        buf = C.create_string_buffer(1 << 16)
        _lib.check(self._lib.cclx_elastic_form(self._h, timeout_ms, out, buf, len(buf)))
        self.rank, self.size, self.generation = int(out[0]), int(out[1]), int(out[2])
        self.members = buf.value.decode().split(",") if buf.value else []
        return self.rank, self.size, self.generation

    def changed(self) -> bool:
        r = self._lib.cclx_elastic_changed(self._h)
        if r < 0:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        return bool(r)

    def communicator(self) -> "Communicator":
        h = self._lib.cclx_elastic_comm_create(self._h)
        if not h:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        return Communicator(_handle=h, kvs=self._kvs)

    def leave(self):
        if self._h:
            _lib.check(self._lib.cclx_elastic_leave(self._h))

    def close(self):
        if self._h:
            self._lib.cclx_elastic_destroy(self._h)
            self._h = None
