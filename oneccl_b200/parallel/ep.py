"""Expert parallelism: top-k routing, dispatch all-to-all, expert FFN on the
tcgen05 GEMM, combine all-to-all with the weighted sum fused into the
un-permute kernel.

One expert per rank (``world`` experts).  Default path: ``fused_dispatch`` stores
every routed row straight into the owning expert's symmetric receive buffer and
``fused_combine`` pulls the expert outputs back with peer loads while forming the
weighted sum (no staging, no gather or un-permute pass).  ``forward_alltoall`` is
the same layer on the library's ``alltoallv`` kernel (variable per-destination
counts; rounds are agreed on the device) with separate gather / combine kernels;
all kernels are in ``csrc/gpu/moe_kernels.cu``.
"""
from __future__ import annotations

import torch

from .. import _lib
from ..ops.device_group import DeviceGroup, _stream_ptr
from ..ops.gemm import gemm_bf16

launches = 0


def gather_rows(x: torch.Tensor, src_row: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    global launches
    n, hidden = src_row.numel(), x.shape[1]
    if out is None:
        out = torch.empty((n, hidden), dtype=x.dtype, device=x.device)
    _lib.check(_lib.load().cclx_moe_gather_rows(x.data_ptr(), src_row.data_ptr(), out.data_ptr(), n, hidden,
                                                _stream_ptr()))
    launches += 1
    return out


def combine_rows(y: torch.Tensor, pos: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    global launches
    n_tok, topk = pos.shape
    hidden = y.shape[1]
    if out is None:
        out = torch.empty((n_tok, hidden), dtype=y.dtype, device=y.device)
    _lib.check(_lib.load().cclx_moe_combine(y.data_ptr(), pos.data_ptr(), w.data_ptr(), out.data_ptr(), n_tok, topk,
                                            hidden, _stream_ptr()))
    launches += 1
    return out


def _per_entry(group: DeviceGroup, t):
    """Real mode takes one tensor, emulation a list with one tensor per rank."""
    return list(t) if group.emulated_mode else [t]


def fused_dispatch(group: DeviceGroup, x, order, send_counts, meta, recv_buf, cnt_table, topk: int, blocks: int = 0):
    """Stores row ``order[i] // topk`` of ``x`` into the receive buffer of the expert that owns item i
    (items sorted by expert), straight over NVLink.  ``recv_buf`` ([cap, hidden] bf16) and ``cnt_table``
    (int32, >= 256 * world**2) are symmetric allocations; ``meta`` (int32 [2 * world + 2]) receives the row
    offsets, the number of rows this rank's expert got (``meta[2 * world]``) and an overflow flag."""
    global launches
    xs, orders, counts, metas = (_per_entry(group, v) for v in (x, order, send_counts, meta))
    rb, ct = _per_entry(group, recv_buf)[0], _per_entry(group, cnt_table)[0]
    _lib.check(_lib.load().cclx_moe_dispatch(
        group.handle, group._ptrs(xs), group._ptrs(orders), group._ptrs(counts), group._ptrs(metas),
        orders[0].numel(), topk, xs[0].shape[1], rb.data_ptr(), rb.shape[0], ct.data_ptr(), blocks, _stream_ptr()))
    launches += 1


def fused_combine(group: DeviceGroup, expert, pos, weight, out, meta, expert_out, topk: int, blocks: int = 0):
    """out[t] = sum_s weight[t, s] * (row of item (t, s) in the output buffer of its expert), read with
    peer loads.  ``expert_out`` is the symmetric [cap, hidden] bf16 buffer every expert wrote its rows to,
    in the order ``fused_dispatch`` delivered them."""
    global launches
    es, ps, ws, outs, metas = (_per_entry(group, v) for v in (expert, pos, weight, out, meta))
    eo = _per_entry(group, expert_out)[0]
    _lib.check(_lib.load().cclx_moe_combine_peer(
        group.handle, group._ptrs(es), group._ptrs(ps), group._ptrs(ws), group._ptrs(outs), group._ptrs(metas),
        es[0].numel(), topk, outs[0].shape[1], eo.data_ptr(), blocks, _stream_ptr()))
    launches += 1


def route_device(logits: torch.Tensor, topk: int):
    """Top-k routing in two kernels: expert ids [T, k] (int64), softmax weights over the chosen logits [T, k]
    (fp32), items per expert [E] (int64), a permutation ``order`` of the T * k (token, slot) items that groups
    them by expert, and its inverse ``pos``.  What ``torch.topk`` + ``softmax`` + ``bincount`` + ``argsort`` +
    a scatter compute, without the sort (the order inside an expert's group is arbitrary)."""
    global launches
    assert logits.is_cuda and logits.dim() == 2
    lg = logits.float().contiguous()
    T, E = lg.shape
    dev = lg.device
    idx = torch.empty((T, topk), dtype=torch.int64, device=dev)
    wts = torch.empty((T, topk), dtype=torch.float32, device=dev)
    counts = torch.empty((E,), dtype=torch.int64, device=dev)
    order = torch.empty((T * topk,), dtype=torch.int64, device=dev)
    pos = torch.empty((T * topk,), dtype=torch.int64, device=dev)
    scratch = torch.empty((E,), dtype=torch.int32, device=dev)
    _lib.check(_lib.load().cclx_moe_route(lg.data_ptr(), T, E, topk, idx.data_ptr(), wts.data_ptr(), counts.data_ptr(),
                                          order.data_ptr(), pos.data_ptr(), scratch.data_ptr(), _stream_ptr()))
    launches += 2
    return idx, wts, counts, order, pos


class ExpertParallelMoE:
    """x [T, H] bf16 on every rank -> y [T, H]: every token visits its top-k experts."""

    def __init__(self, group: DeviceGroup, hidden: int, ffn: int, topk: int = 2, seed: int = 0,
                 use_native_gemm: bool = True, fused: bool = True, max_tokens: int = 0):
        self.group = group
        self.world = group.world
        self.rank = group.rank
        self.hidden, self.ffn, self.topk = hidden, ffn, topk
        self.use_native_gemm = use_native_gemm
        g = torch.Generator(device="cuda").manual_seed(seed + 17 * group.rank)
        # this rank's expert: W1 [ffn, hidden], W2 [hidden, ffn] (nn.Linear layout = K-major operands)
        self.w1 = (torch.randn(ffn, hidden, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        self.w2 = (torch.randn(hidden, ffn, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
        self.stats = {}
        # fused path: rows travel straight into / out of symmetric buffers sized for the worst case
        # (every token of every rank choosing this expert); set up lazily for the first batch size
        self.fused = fused
        self._cap = 0
        self._max_tokens = max_tokens
        self._xrecv = self._yout = self._cnt = self._meta = self._hmid = self._last = None

    def _buffers(self, tokens: int):
        cap = max(tokens, self._max_tokens) * self.topk * self.world
        if cap > self._cap:  # collective: every rank sees the same token count
            for t in (self._xrecv, self._yout):
                if t is not None:
                    self.group.symm_free(t)
            self._xrecv = self.group.symm_empty((cap, self.hidden), dtype=torch.bfloat16)
            self._yout = self.group.symm_empty((cap, self.hidden), dtype=torch.bfloat16)
            self._hmid = torch.empty((cap, self.ffn), dtype=torch.bfloat16, device="cuda")  # FFN intermediate
            if self._cnt is None:
                self._cnt = self.group.symm_empty((256 * self.world * self.world,), dtype=torch.int32)
                self._meta = torch.zeros(2 * self.world + 2, dtype=torch.int32, device="cuda")
            self._cap = cap

    def forward_fused(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        global launches
        T, H = x.shape
        W, k = self.world, self.topk
        self._buffers(T)
        mark = self._mark
        mark("start")
        idx, wts, send_counts, order, pos = route_device(logits, k)
        flat_e = idx.view(-1)
        mark("routed")
        fused_dispatch(self.group, x, order, send_counts, self._meta, self._xrecv, self._cnt, k)
        # the number of rows that arrived stays on the device: the expert GEMMs read it there and skip the tiles
        # behind it, so the host issues dispatch, FFN and combine without waiting for anything
        n_dev = self._meta[2 * W:2 * W + 1]
        mark("dispatched")
        if self.use_native_gemm:
            gemm_bf16(self._xrecv, self.w1, out=self._hmid, epilogue="silu", rows=n_dev)
            gemm_bf16(self._hmid, self.w2, out=self._yout, rows=n_dev)
            launches += 2
        else:  # library GEMMs take their shape from the host: this form pays the read
            n_recv = int(n_dev.item())
            if n_recv > 0:
                torch.matmul(torch.nn.functional.silu(self._xrecv[:n_recv] @ self.w1.t()), self.w2.t(),
                             out=self._yout[:n_recv])
        mark("ffn")
        out = torch.empty_like(x)
        fused_combine(self.group, flat_e, pos, wts.view(-1), out, self._meta, self._yout, k)
        mark("combined")
        self._last = self._meta[2 * W:2 * W + 2].clone()  # rows received, overflow flag: read on request
        return out

    def _mark(self, name: str):
        """With ``self.phase_events`` set to a dict, records a CUDA event per phase boundary of the fused
        forward (start, routed, dispatched, ffn, combined) so that a benchmark can time the phases."""
        ev = getattr(self, "phase_events", None)
        if ev is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            ev.setdefault(name, []).append(e)

    def recv_rows(self) -> int:
        """Rows this rank's expert received in the last fused forward (a host read of two device words);
        raises if the receive buffer had been too small for them."""
        n_recv, over = self._last.tolist()
        if over:
            raise RuntimeError("expert receive buffer overflow")
        self.stats = {"recv_rows": n_recv}
        return n_recv

    def route(self, logits: torch.Tensor):
        """Returns expert ids [T, k] and normalised weights [T, k] (fp32)."""
        val, idx = torch.topk(logits.float(), self.topk, dim=-1)
        return idx, torch.softmax(val, dim=-1)

    def expert(self, rows: torch.Tensor) -> torch.Tensor:
        global launches
        if rows.shape[0] == 0:
            return rows.new_empty((0, self.hidden))
        if self.use_native_gemm:
            h = gemm_bf16(rows, self.w1, epilogue="silu")
            launches += 2
            return gemm_bf16(h, self.w2)
        return torch.nn.functional.silu(rows @ self.w1.t()) @ self.w2.t()

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        if self.fused:
            return self.forward_fused(x, logits)
        return self.forward_alltoall(x, logits)

    def forward_alltoall(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        T, H = x.shape
        W, k = self.world, self.topk
        idx, wts = self.route(logits)
        flat_e = idx.reshape(-1)  # [T*k] expert of every (token, slot)
        order = torch.argsort(flat_e, stable=True)  # dispatch order: grouped by destination
        send_counts = torch.bincount(flat_e, minlength=W)
        # counts travel first (tiny all-to-all), then the host learns the row counts once
        recv_counts = torch.empty_like(send_counts)
        self.group.alltoallv(send_counts, recv_counts)
        sc = send_counts.tolist()
        rc = recv_counts.tolist()
        xs = gather_rows(x, order // k)  # [T*k, H] rows in dispatch order
        n_recv = sum(rc)
        recv = torch.empty((max(n_recv, 1), H), dtype=x.dtype, device=x.device)
        self.group.alltoallv(xs, recv, send_counts=[c * H for c in sc], recv_counts=[c * H for c in rc])
        y = self.expert(recv[:n_recv])
        back = torch.empty_like(xs)
        ysend = y if n_recv > 0 else recv
        self.group.alltoallv(ysend, back, send_counts=[c * H for c in rc], recv_counts=[c * H for c in sc])
        # position of (token, slot) inside `back`
        pos = torch.empty_like(order)
        pos[order] = torch.arange(order.numel(), device=order.device)
        out = combine_rows(back, pos.view(T, k), wts.contiguous())
        self.stats = {"sent_rows": sc, "recv_rows": rc}
        return out

    __call__ = forward


def reference_moe(x, logits, w1s, w2s, topk=2):
    """Dense fp32 restatement used by the tests: every expert on one device."""
    val, idx = torch.topk(logits.float(), topk, dim=-1)
    wts = torch.softmax(val, dim=-1)
    out = torch.zeros_like(x, dtype=torch.float32)
    for e in range(len(w1s)):
        for slot in range(topk):
            m = idx[:, slot] == e
            if m.any():
                h = torch.nn.functional.silu(x[m].float() @ w1s[e].float().t()).to(torch.bfloat16).float()
                y = (h @ w2s[e].float().t()).to(torch.bfloat16).float()
                out[m] += wts[m, slot:slot + 1] * y
    return out
