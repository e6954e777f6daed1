"""Python face of the native device communicator.

``DeviceGroup`` wraps one ``cclx::gpu::device_comm``.  It exists in two
flavours that share every kernel:

* *real*: one process per GPU, created by :class:`oneccl_b200.comm.Communicator`
  after the symmetric heaps were exchanged; every method takes this rank's
  tensor(s);
* *emulated* (``DeviceGroup.emulated(world)``): all ranks live on the current
  GPU and each call takes a list with one tensor per rank.  The launch is
  cooperative, so blocks of different emulated ranks can wait on one another.
  This is how the multi-rank kernels are tested on a single device.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Optional, Sequence

import torch

from .. import _lib
from ..dtypes import GPU_ALGO, COLL, reduce_op_code, torch_to_ccl


def _stream_ptr(stream=None) -> int:
    """Raw handle of the launch stream; also points the library's own CUDA runtime
    (per-thread current device) at the caller's device."""
    s = stream if stream is not None else torch.cuda.current_stream()
    idx = s.device.index if s.device.index is not None else torch.cuda.current_device()
    if getattr(_tls, "device", None) != idx:  # the library's runtime keeps the device per thread too
        _lib.load().cclx_set_device(idx)
        _tls.device = idx
    return s.cuda_stream


_tls = threading.local()


class _SymmStorage:
    """Exposes a slice of the symmetric heap through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (ptr, False),
            "version": 3,
            "strides": None,
        }
        self._owner = owner


class DeviceGroup:
    def __init__(self, handle: int, emulated: bool, owns: bool = True):
        self._lib = _lib.load()
        self._h = C.c_void_p(handle)
        self.emulated_mode = emulated
        self._owns = owns
        self.world = self._lib.cclx_dc_world(self._h)
        self.rank = self._lib.cclx_dc_rank(self._h)
        self._symm = {}  # data_ptr -> offset

    # ---- construction -----------------------------------------------------------
    @classmethod
    def emulated(cls, world: int, heap_bytes: int = 256 << 20, staging_bytes: int = 16 << 20) -> "DeviceGroup":
        lib = _lib.load()
        if not torch.cuda.is_available():
            raise _lib.CclError("an emulated device group needs a CUDA device")
        torch.cuda.init()
        torch.zeros(1, device="cuda")  # make the primary context current
        lib.cclx_set_device(torch.cuda.current_device())
        h = lib.cclx_emu_create(world, heap_bytes, staging_bytes)
        if not h:
            raise _lib.CclError(lib.cclx_last_error().decode())
        return cls(h, True)

    def close(self):
        if self._h and self._owns:
            torch.cuda.synchronize()
            self._lib.cclx_dc_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    @property
    def nvls(self) -> bool:
        return bool(self._lib.cclx_dc_nvls(self._h))

    @property
    def n_entries(self) -> int:
        return self.world if self.emulated_mode else 1

    # ---- status -------------------------------------------------------------------
    def status(self, r: int = 0) -> int:
        return self._lib.cclx_dc_status(self._h, r)

    def check(self):
        _lib.check(self._lib.cclx_dc_check(self._h))

    def clear_status(self):
        _lib.check(self._lib.cclx_dc_clear_status(self._h))

    def abort(self):
        _lib.check(self._lib.cclx_dc_abort(self._h))

    def set_timeout_ms(self, ms: int):
        _lib.check(self._lib.cclx_dc_set_timeout_ms(self._h, ms))

    def test_sig_skew(self, rank: int):
        """Test hook: falsify the argument signature that emulated rank `rank` presents in the next
        collectives (-1 switches it off), to exercise the cross-rank argument check on one GPU."""
        _lib.check(self._lib.cclx_dc_test_sig_skew(self._h, rank))

    def algo_hits(self, coll: str, algo: str) -> int:
        return int(self._lib.cclx_dc_algo_hits(self._h, COLL[coll], GPU_ALGO[algo]))

    # ---- symmetric tensors --------------------------------------------------------
    def symm_empty(self, shape, dtype=torch.float32):
        """Allocate from the symmetric heap.  Real mode: collective call, returns
        this rank's tensor.  Emulated mode: returns one tensor per rank."""
        shape = tuple(shape) if not isinstance(shape, int) else (shape,)
        n = 1
        for s in shape:
            n *= s
        nbytes = max(n * torch.empty((), dtype=dtype).element_size(), 16)
        off = self._lib.cclx_dc_symm_alloc(self._h, nbytes)
        if off == C.c_size_t(-1).value:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        outs = []
        ranks = range(self.world) if self.emulated_mode else [self.rank]
        for r in ranks:
            base = self._lib.cclx_dc_heap_base(self._h, r)
            st = _SymmStorage(base + off, nbytes, self)
            t = torch.as_tensor(st, device="cuda").view(torch.uint8)[: n * torch.empty((), dtype=dtype).element_size()]
            t = t.view(dtype).view(shape)
            self._symm[t.data_ptr()] = off
            outs.append(t)
        return outs if self.emulated_mode else outs[0]

    def symm_free(self, t):
        ts = t if isinstance(t, (list, tuple)) else [t]
        off = self._symm.pop(ts[0].data_ptr())
        for x in ts[1:]:
            self._symm.pop(x.data_ptr(), None)
        _lib.check(self._lib.cclx_dc_symm_free(self._h, off))

    # ---- registration of ordinary tensors ---------------------------------------------
    def register(self, t) -> int:
        """Makes an ordinary CUDA tensor (not from the symmetric heap) directly readable and writable by
        the peers' kernels: collective; every rank passes its own tensor (emulation: one per rank).  The
        whole allocation is exported once through a CUDA IPC handle; afterwards collectives whose buffers
        lie inside the registered tensors (same offset on every rank) run without staging copies."""
        ts = list(t) if self.emulated_mode else [t]
        rid = self._lib.cclx_dc_register(self._h, self._ptrs(ts),
                                         _lib.size_array([x.numel() * x.element_size() for x in ts]))
        if rid < 0:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        self._registered = getattr(self, "_registered", {})
        self._registered[rid] = ts  # keeps the tensors alive while peers may touch them
        return rid

    def deregister(self, rid: int):
        _lib.check(self._lib.cclx_dc_deregister(self._h, rid))
        getattr(self, "_registered", {}).pop(rid, None)

    # ---- helpers ------------------------------------------------------------------
    def _lists(self, send, recv):
        if self.emulated_mode:
            if self.world == 1:  # a single emulated rank may pass bare tensors
                send = [send] if isinstance(send, torch.Tensor) else send
                recv = [recv] if isinstance(recv, torch.Tensor) else recv
            assert send is None or len(send) == self.world
            assert recv is None or len(recv) == self.world
            return send, recv
        s = None if send is None else [send]
        r = None if recv is None else [recv]
        return s, r

    @staticmethod
    def _ptrs(ts):
        if ts is None:
            return None
        return _lib.ptr_array([0 if t is None else t.data_ptr() for t in ts])

    def _finish(self, rc):
        _lib.check(rc)

    # ---- collectives --------------------------------------------------------------
    def allreduce(self, send, recv=None, op="sum", algo="auto", blocks=0, scale: Optional[float] = None, stream=None):
        recv = send if recv is None else recv
        s, r = self._lists(send, recv)
        for a, b in zip(s, r):
            assert a.is_contiguous() and b.is_contiguous() and a.numel() == b.numel()
        rc = self._lib.cclx_dc_allreduce(
            self._h, self._ptrs(s), self._ptrs(r), s[0].numel(), torch_to_ccl(s[0].dtype), torch_to_ccl(r[0].dtype),
            reduce_op_code(op), GPU_ALGO[algo], blocks, 1.0 if scale is None else float(scale),
            0 if scale is None else 1, _stream_ptr(stream))
        self._finish(rc)
        return recv

    def allreduce_fused(self, tensors, op="sum", scale: Optional[float] = None, stream=None):
        """In-place allreduce of a list of (small) tensors as ONE collective: one kernel packs them into a
        buffer of the symmetric heap, one zero-copy allreduce reduces it, one kernel unpacks.  Real mode:
        ``tensors`` is this rank's list.  Emulated mode: a list (per tensor) of lists (per rank)."""
        n = len(tensors)
        if self.emulated_mode:
            flat = [t for per_rank in tensors for t in per_rank]  # tensor-major
            first = tensors[0][0]
            counts = [per_rank[0].numel() for per_rank in tensors]
        else:
            flat = list(tensors)
            first = tensors[0]
            counts = [t.numel() for t in tensors]
        for t in flat:
            assert t.is_contiguous() and t.dtype == first.dtype
        ptrs = self._ptrs(flat)
        rc = self._lib.cclx_dc_allreduce_fused(self._h, ptrs, ptrs, _lib.size_array(counts), n, torch_to_ccl(first.dtype),
                                               reduce_op_code(op), 1.0 if scale is None else float(scale),
                                               0 if scale is None else 1, _stream_ptr(stream))
        self._finish(rc)
        return tensors

    @property
    def fused_batches(self) -> int:
        return int(self._lib.cclx_dc_fused_batches(self._h))

    def reduce_scatter(self, send, recv, op="sum", algo="auto", blocks=0, scale: Optional[float] = None, stream=None):
        s, r = self._lists(send, recv)
        for a, b in zip(s, r):
            assert a.is_contiguous() and b.is_contiguous() and a.numel() == b.numel() * self.world
        rc = self._lib.cclx_dc_reduce_scatter(
            self._h, self._ptrs(s), self._ptrs(r), r[0].numel(), torch_to_ccl(s[0].dtype), torch_to_ccl(r[0].dtype),
            reduce_op_code(op), GPU_ALGO[algo], blocks, 1.0 if scale is None else float(scale),
            0 if scale is None else 1, _stream_ptr(stream))
        self._finish(rc)
        return recv

    def reduce(self, send, recv, root=0, op="sum", blocks=0, scale: Optional[float] = None, stream=None):
        s, r = self._lists(send, recv)
        rc = self._lib.cclx_dc_reduce(
            self._h, self._ptrs(s), self._ptrs(r), s[0].numel(), torch_to_ccl(s[0].dtype),
            torch_to_ccl(next(t for t in r if t is not None).dtype), reduce_op_code(op), root, blocks,
            1.0 if scale is None else float(scale), 0 if scale is None else 1, _stream_ptr(stream))
        self._finish(rc)
        return recv

    def allgatherv(self, send, recv, counts: Optional[Sequence[int]] = None, algo="auto", blocks=0, stream=None):
        """``counts`` are elements per rank (default: equal blocks); ``send`` may be None for in-place."""
        s, r = self._lists(send, recv)
        esz = r[0].element_size()
        if counts is None:
            per = r[0].numel() // self.world
            counts = [per] * self.world
        bc = [c * esz for c in counts]
        bd = [0] * self.world
        for p in range(1, self.world):
            bd[p] = bd[p - 1] + bc[p - 1]
        sp = self._ptrs(s) if s is not None else _lib.ptr_array([0] * self.n_entries)
        rc = self._lib.cclx_dc_allgatherv(self._h, sp, self._ptrs(r), _lib.size_array(bc), _lib.size_array(bd),
                                          GPU_ALGO[algo], blocks, _stream_ptr(stream))
        self._finish(rc)
        return recv

    def alltoall(self, send, recv, algo="auto", blocks=0, stream=None):
        """Equal blocks: block q of `send` goes to rank q.  With `recv` from the symmetric heap the
        blocks are stored straight into the peers' buffers (algo="push" forces the staged kernel)."""
        s, r = self._lists(send, recv)
        per = s[0].numel() // self.world * s[0].element_size()
        rc = self._lib.cclx_dc_alltoall(self._h, self._ptrs(s), self._ptrs(r), per, GPU_ALGO[algo], blocks,
                                        _stream_ptr(stream))
        self._finish(rc)
        return recv

    def alltoallv(self, send, recv, send_counts=None, recv_counts=None, blocks=0, stream=None):
        """Counts are in elements; emulated mode takes one row of counts per rank."""
        if send_counts is None:
            return self.alltoall(send, recv, blocks=blocks, stream=stream)
        s, r = self._lists(send, recv)
        W = self.world
        esz = s[0].element_size()
        n = self.n_entries
        if not self.emulated_mode:
            send_counts, recv_counts = [list(send_counts)], [list(recv_counts)]
        table = []
        for e in range(n):
            sc = [c * esz for c in send_counts[e]]
            rcnt = [c * esz for c in recv_counts[e]]
            sd, rd = [0] * W, [0] * W
            for p in range(1, W):
                sd[p] = sd[p - 1] + sc[p - 1]
                rd[p] = rd[p - 1] + rcnt[p - 1]
            table += sc + sd + rcnt + rd
        rc = self._lib.cclx_dc_alltoallv(self._h, self._ptrs(s), self._ptrs(r), _lib.size_array(table), blocks,
                                         _stream_ptr(stream))
        self._finish(rc)
        return recv

    def broadcast(self, send, recv=None, root=0, blocks=0, stream=None):
        recv = send if recv is None else recv
        s, r = self._lists(send, recv)
        nbytes = r[0].numel() * r[0].element_size()
        rc = self._lib.cclx_dc_broadcast(self._h, self._ptrs(s), self._ptrs(r), nbytes, root, blocks,
                                         _stream_ptr(stream))
        self._finish(rc)
        return recv

    def barrier(self, stream=None):
        self._finish(self._lib.cclx_dc_barrier(self._h, _stream_ptr(stream)))

    def sendrecv(self, send, recv, peers, is_send, nbytes=None, stream=None):
        """Point-to-point.  Real mode: lists of operations of this rank posted in one launch
        (``send[i]`` / ``recv[i]`` tensor or None, ``peers[i]``, ``is_send[i]``); scalars are
        accepted for a single operation.  Emulated mode: one operation per rank (peer -1 = idle)."""
        if not self.emulated_mode and not isinstance(peers, (list, tuple)):
            send, recv, peers, is_send = [send], [recv], [peers], [is_send]
        n = len(peers)
        sizes = []
        for k in range(n):
            t = send[k] if is_send[k] else recv[k]
            if nbytes is not None:
                sizes.append(nbytes if not isinstance(nbytes, (list, tuple)) else nbytes[k])
            else:
                sizes.append(0 if (t is None or peers[k] < 0) else t.numel() * t.element_size())
        rc = self._lib.cclx_dc_sendrecv(self._h, self._ptrs(send), self._ptrs(recv), _lib.size_array(sizes),
                                        _lib.int_array(peers), _lib.int_array([1 if x else 0 for x in is_send]), n,
                                        _stream_ptr(stream))
        self._finish(rc)

    def wait_unset_flag(self, stream=None):
        self._finish(self._lib.cclx_dc_wait_unset_flag(self._h, _stream_ptr(stream)))


def reduce_local(inp: torch.Tensor, inout: torch.Tensor, op="sum", stream=None):
    lib = _lib.load()
    _lib.check(lib.cclx_reduce_local(inp.data_ptr(), inout.data_ptr(), inout.numel(), torch_to_ccl(inout.dtype),
                                     reduce_op_code(op), _stream_ptr(stream)))
    return inout


def transpose_blocks(inp: torch.Tensor, rows: int, cols: int, out: Optional[torch.Tensor] = None, stream=None):
    """``inp`` seen as ``rows x cols`` equal blocks (row-major) comes out with the blocks in column-major
    order: the regrouping from rank order (node-major) to local-rank order that a reduce_scatter across
    nodes starts with."""
    assert inp.is_cuda and inp.is_contiguous() and inp.numel() % (rows * cols) == 0
    if out is None:
        out = torch.empty_like(inp)
    block_bytes = inp.numel() // (rows * cols) * inp.element_size()
    lib = _lib.load()
    _lib.check(lib.cclx_transpose_blocks(inp.data_ptr(), out.data_ptr(), rows, cols, block_bytes, _stream_ptr(stream)))
    return out
