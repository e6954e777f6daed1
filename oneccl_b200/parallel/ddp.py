"""Data-parallel training on top of the device communicator.

``DataParallel`` re-homes a module's parameters into one flat bf16/fp32 buffer
and its gradients into one flat buffer taken from the symmetric heap, cut into
buckets (default 25 MB, the reference's fusion idea applied to gradients:
src/fusion/fusion.cpp:145-376 packs small allreduces into one buffer).  Because
``p.grad`` are views of the bucket, no pack / unpack copy exists: autograd
accumulates straight into peer-visible memory.  When the last gradient of a
bucket has been accumulated, the bucket's allreduce is launched on a side
stream (zero-copy two-shot / NVLS kernel, in place, optionally fused with the
1/world scale), so communication overlaps the rest of backward.  The optimizer
(:class:`oneccl_b200.ops.train.FlatAdamW`) then reads the reduced bf16 bucket
directly and keeps fp32 master weights.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from ..ops.device_group import DeviceGroup
from ..ops.train import FlatAdamW


class _Bucket:
    __slots__ = ("start", "end", "params", "pending", "event")

    def __init__(self, start):
        self.start = start
        self.end = start
        self.params = []
        self.pending = 0
        self.event = None


class DataParallel:
    def __init__(self, module: nn.Module, group: DeviceGroup, bucket_mb: float = 25.0, scale_in_allreduce: bool = True,
                 broadcast_from: Optional[int] = 0, algo: str = "auto", comm_blocks: int = 0):
        assert not group.emulated_mode or group.world == 1, "DataParallel drives one rank per process"
        self.module = module
        self.group = group
        self.world = group.world
        self.algo = algo
        self.comm_blocks = comm_blocks
        self.scale_in_allreduce = scale_in_allreduce and self.world > 1
        self.launches = 0

        # ---- flat layout: decay params in reverse registration order, then the rest
        decay = [p for p in module.parameters() if p.requires_grad and p.dim() >= 2]
        other = [p for p in module.parameters() if p.requires_grad and p.dim() < 2]
        seen, order = set(), []
        for p in list(reversed(decay)) + list(reversed(other)):
            if id(p) not in seen:
                seen.add(id(p))
                order.append(p)
        dtype = order[0].dtype
        assert all(p.dtype == dtype for p in order), "mixed parameter dtypes are not supported"
        self.dtype = dtype
        offs, cur = [], 0
        n_decay = 0
        for p in order:
            cur = (cur + 7) // 8 * 8  # 16-byte aligned starts
            offs.append(cur)
            cur += p.numel()
            if p.dim() >= 2:
                n_decay = cur
        total = (cur + 7) // 8 * 8
        self.n_decay = n_decay
        self.total = total
        dev = order[0].device
        self.flat_param = torch.zeros(total, dtype=dtype, device=dev)
        g = group.symm_empty((total,), dtype=dtype)
        self.flat_grad = g[0] if isinstance(g, list) else g
        self.flat_grad.zero_()
        for p, o in zip(order, offs):
            self.flat_param[o:o + p.numel()].copy_(p.data.reshape(-1))
            p.data = self.flat_param[o:o + p.numel()].view_as(p.data)
            p.grad = self.flat_grad[o:o + p.numel()].view_as(p.data)
            # layers that can accumulate straight into the flat buffer (oneccl_b200.ops.nn.linear) use this
            # instead of handing autograd a gradient to add; the callback does the bucket accounting
            p._grad_sink = (p.grad, self._on_grad)

        # ---- buckets over the flat gradient
        cap = max(1, int(bucket_mb * (1 << 20) / self.flat_grad.element_size()))
        self.buckets: List[_Bucket] = []
        b = _Bucket(0)
        for p, o in zip(order, offs):
            if b.params and (o + p.numel() - b.start) > cap:
                b.end = o
                self.buckets.append(b)
                b = _Bucket(o)
            b.params.append(p)
        b.end = total
        self.buckets.append(b)
        self._bucket_of = {}
        for bi, b in enumerate(self.buckets):
            for p in b.params:
                self._bucket_of[id(p)] = bi
        self.comm_stream = torch.cuda.Stream()
        self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in order]
        self._armed = False
        self._seen = set()
        if broadcast_from is not None and self.world > 1:
            group.broadcast(self.flat_param, root=broadcast_from)
            torch.cuda.synchronize()

    # ---- per step -------------------------------------------------------------------
    def zero_grad(self):
        self.flat_grad.zero_()
        for b in self.buckets:
            b.pending = len(b.params)
        self._seen = set()
        self._armed = True

    def _launch_bucket(self, b: _Bucket):
        ev = torch.cuda.Event()
        ev.record()
        self.comm_stream.wait_event(ev)
        seg = self.flat_grad[b.start:b.end]
        with torch.cuda.stream(self.comm_stream):
            self.group.allreduce(seg, seg, algo=self.algo, blocks=self.comm_blocks,
                                 scale=(1.0 / self.world) if self.scale_in_allreduce else None,
                                 stream=self.comm_stream)
        if self.world > 1:
            self.launches += 1

    def _on_grad(self, p):
        if not self._armed or id(p) in self._seen:
            return  # a parameter counts once per step, whether its layer or autograd reports it
        self._seen.add(id(p))
        b = self.buckets[self._bucket_of[id(p)]]
        b.pending -= 1
        if b.pending == 0:
            self._launch_bucket(b)

    def finish(self):
        """Make the compute stream wait for the outstanding bucket allreduces."""
        for b in self.buckets:
            if b.pending > 0:  # parameters that received no gradient this step
                b.pending = 0
                self._launch_bucket(b)
        torch.cuda.current_stream().wait_stream(self.comm_stream)
        self._armed = False

    @property
    def grad_scale(self) -> float:
        return 1.0 if (self.scale_in_allreduce or self.world == 1) else 1.0 / self.world

    def make_optimizer(self, **kw) -> FlatAdamW:
        return FlatAdamW(self.flat_param, self.n_decay, **kw)

    def __call__(self, *a, **kw):
        return self.module(*a, **kw)


def train_step(ddp: DataParallel, opt: FlatAdamW, idx: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """One full data-parallel step: forward, backward with overlapped bucket
    allreduce, gradient clipping + AdamW.  Returns the (device) loss."""
    ddp.zero_grad()
    loss = ddp(idx, targets)
    loss.backward()
    ddp.finish()
    opt.step(ddp.flat_grad, grad_scale=ddp.grad_scale)
    return loss
