"""Expert parallelism: top-k routing, dispatch all-to-all, expert FFN on the
tcgen05 GEMM, combine all-to-all with the weighted sum fused into the
un-permute kernel.

One expert per rank (``world`` experts).  The exchange is the library's
``alltoallv`` kernel (variable per-destination counts; rounds are agreed on
the device), the gather / combine passes are ``csrc/gpu/moe_kernels.cu``.
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


class ExpertParallelMoE:
    """x [T, H] bf16 on every rank -> y [T, H]: every token visits its top-k experts."""

    def __init__(self, group: DeviceGroup, hidden: int, ffn: int, topk: int = 2, seed: int = 0,
                 use_native_gemm: bool = True):
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
