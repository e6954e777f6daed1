"""Data-parallel training on top of the device communicator.

``DataParallel`` re-homes a module's parameters into one flat bf16/fp32 buffer
and its gradients into one flat buffer taken from the symmetric heap, cut into
buckets (default 25 MB, the reference's fusion idea applied to gradients:
src/fusion/fusion.cpp:145-376 packs small allreduces into one buffer).  Because
``p.grad`` are views of the flat buffer, no pack / unpack copy exists: autograd
accumulates straight into peer-visible memory.

Overlap with backward (the role of the reference's priority queue,
src/sched/queue/queue.cpp:100-152, played by CUDA stream priorities):

* the flat layout follows the order in which gradients become ready, and a bucket is a
  plain range of it, so a parameter larger than the bucket size (a tied embedding) is cut
  into several buckets instead of forming one oversized one;
* a bucket is reduced as soon as the last parameter overlapping it has its gradient, on a
  high-priority side stream, in place, with the 1/world scale fused (zero-copy NVLS or peer
  load kernel);
* while backward still runs, the allreduce uses a *narrow* grid (``comm_blocks`` thread
  blocks), which leaves the other SMs to the backward GEMMs instead of time-slicing the
  whole GPU with them; buckets that are launched when nothing is left to overlap with
  (the last ones, or whatever ``finish`` still finds) use ``tail_blocks``.

``GraphedTrainStep`` captures the whole step (forward, backward with the bucket
allreduces on their side stream, clipping, AdamW) into one CUDA graph, so that a step costs
one launch on the host; the collective kernels keep their epoch and staging state in device
memory, which is what makes the replay valid.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from ..ops.device_group import DeviceGroup
from ..ops.train import FlatAdamW

# Thread blocks of a bucket allreduce.  Measured with oneccl_b200.benchmarks.ddp_overlap_bench on B200s:
# the in-switch (NVLS) reduction of a 25 MB bucket among 8 GPUs is as fast from 4 to 8 blocks of 1024 threads
# (8 loads of 16 bytes in flight per thread) as from any wider grid, 80 us, and 100 MB are faster narrow
# (0.24 ms) than GPU-wide (0.29 ms), so every bucket uses the narrow grid and the SMs stay with backward.
# The peer-load form that two GPUs use needs its loads spread over more SMs: 32 blocks while backward
# runs, the full width for the last buckets of a step.
NVLS_BLOCKS = 8
PEER_OVERLAP_BLOCKS = 32


class _Bucket:
    __slots__ = ("start", "end", "n_params", "pending", "t_ready", "t_start", "t_end")

    def __init__(self, start, end):
        self.start = start
        self.end = end
        self.n_params = 0
        self.pending = 0
        self.t_ready = self.t_start = self.t_end = None


class DataParallel:
    def __init__(self, module: nn.Module, group: DeviceGroup, bucket_mb: float = 25.0, scale_in_allreduce: bool = True,
                 broadcast_from: Optional[int] = 0, algo: str = "auto", comm_blocks: int = -1,
                 high_priority: bool = True, record_timeline: bool = False, reducer: Optional[str] = None):
        assert not group.emulated_mode or group.world == 1, "DataParallel drives one rank per process"
        self.module = module
        self.group = group
        self.world = group.world
        self.algo = algo
        # -1: the measured default; 0: the kernel's own (full-width) choice
        nvls = group.nvls and group.world >= 3
        self.comm_blocks = (NVLS_BLOCKS if nvls else PEER_OVERLAP_BLOCKS) if comm_blocks < 0 else comm_blocks
        self.tail_blocks = self.comm_blocks if nvls else 0
        self.scale_in_allreduce = scale_in_allreduce and self.world > 1
        self.record_timeline = record_timeline
        # None: this library's allreduce kernels.  "nccl": torch.distributed's default (NCCL) group reduces the
        # buckets instead, everything else unchanged (a comparison arm for the benchmark).
        self.reducer = reducer
        self.launches = 0

        # ---- flat layout in gradient-ready order: matrices in reverse registration order, then the rest
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

        # ---- buckets: ranges of the flat gradient, cut every `cap` elements inside the matrices and
        # inside the rest (a parameter may span several buckets; starts stay 16-byte aligned)
        cap = max(8, int(bucket_mb * (1 << 20) / self.flat_grad.element_size()) // 8 * 8)
        n_decay_al = (n_decay + 7) // 8 * 8
        self.buckets: List[_Bucket] = []
        for lo, hi in ((0, n_decay_al), (n_decay_al, total)):
            s = lo
            while s < hi:
                e = min(s + cap, hi)
                if hi - e < cap // 4:  # no sliver at the end of a region
                    e = hi
                self.buckets.append(_Bucket(s, e))
                s = e
        self._buckets_of = {}
        for p, o in zip(order, offs):
            mine = [bi for bi, b in enumerate(self.buckets) if b.start < o + p.numel() and o < b.end]
            self._buckets_of[id(p)] = mine
            for bi in mine:
                self.buckets[bi].n_params += 1
        lo_pri, hi_pri = torch.cuda.Stream.priority_range()
        self.comm_stream = torch.cuda.Stream(priority=hi_pri if high_priority else lo_pri)
        self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in order]
        self._armed = False
        self._seen = set()
        self._unlaunched = 0
        self.t_step = self.t_backward_end = None
        if broadcast_from is not None and self.world > 1:
            group.broadcast(self.flat_param, root=broadcast_from)
            torch.cuda.synchronize()

    # ---- per step -------------------------------------------------------------------
    def zero_grad(self):
        if self.record_timeline:
            self.t_step = torch.cuda.Event(enable_timing=True)
            self.t_step.record()
        self.flat_grad.zero_()
        for b in self.buckets:
            b.pending = b.n_params
        self._unlaunched = len(self.buckets)
        self._seen = set()
        self._armed = True

    def _launch(self, bs: List[_Bucket], overlapped: bool):
        """One allreduce over the adjacent buckets `bs` (buckets that become ready together travel together)."""
        timing = self.record_timeline
        ev = torch.cuda.Event(enable_timing=timing)
        ev.record()
        self.comm_stream.wait_event(ev)
        seg = self.flat_grad[bs[0].start:bs[-1].end]
        with torch.cuda.stream(self.comm_stream):
            t0 = t1 = None
            if timing:
                t0 = torch.cuda.Event(enable_timing=True)
                t0.record()
            if self.reducer == "nccl":
                if self.world > 1:
                    import torch.distributed as dist

                    dist.all_reduce(seg, op=dist.ReduceOp.AVG if self.scale_in_allreduce else dist.ReduceOp.SUM)
            else:
                self.group.allreduce(seg, seg, algo=self.algo, blocks=self.comm_blocks if overlapped else self.tail_blocks,
                                     scale=(1.0 / self.world) if self.scale_in_allreduce else None,
                                     stream=self.comm_stream)
            if timing:
                t1 = torch.cuda.Event(enable_timing=True)
                t1.record()
            for b in bs:
                b.t_ready, b.t_start, b.t_end = ev, t0, t1
        self._unlaunched -= len(bs)
        if self.world > 1 and self.reducer is None:
            self.launches += 1

    def _launch_ready(self, ready: List[_Bucket]):
        if not ready:
            return
        # nothing else waits for gradients: backward is over, there is no compute left to share the GPU with
        overlapped = self._unlaunched > len(ready)
        run = [ready[0]]
        for b in ready[1:]:
            if b.start == run[-1].end:
                run.append(b)
            else:
                self._launch(run, overlapped)
                run = [b]
        self._launch(run, overlapped)

    def _on_grad(self, p):
        if not self._armed or id(p) in self._seen:
            return  # a parameter counts once per step, whether its layer or autograd reports it
        self._seen.add(id(p))
        ready = []
        for bi in self._buckets_of[id(p)]:
            b = self.buckets[bi]
            b.pending -= 1
            if b.pending == 0:
                ready.append(b)
        self._launch_ready(ready)

    def finish(self):
        """Make the compute stream wait for the outstanding bucket allreduces."""
        if self.record_timeline:
            self.t_backward_end = torch.cuda.Event(enable_timing=True)
            self.t_backward_end.record()
        late = [b for b in self.buckets if b.pending > 0]  # parameters that received no gradient this step
        for b in late:
            b.pending = 0
        self._launch_ready(late)
        torch.cuda.current_stream().wait_stream(self.comm_stream)
        self._armed = False

    def timeline(self):
        """Per-bucket times of the last step in ms after its start (``record_timeline=True``): when the
        bucket's last gradient was ready, when its allreduce started and ended on the side stream, plus
        the end of backward.  Call after a device synchronisation."""
        assert self.record_timeline and self.t_step is not None
        rows = []
        for i, b in enumerate(self.buckets):
            rows.append({"bucket": i, "mbytes": (b.end - b.start) * self.flat_grad.element_size() / 2**20,
                         "ready": self.t_step.elapsed_time(b.t_ready), "start": self.t_step.elapsed_time(b.t_start),
                         "end": self.t_step.elapsed_time(b.t_end)})
        return {"backward_end": self.t_step.elapsed_time(self.t_backward_end), "buckets": rows}

    def close(self):
        """Detach from the module: remove the gradient hooks and give the flat gradient back to the
        symmetric heap (collective in multi-process mode, like the allocation)."""
        for hk in self._hooks:
            hk.remove()
        self._hooks = []
        for p in self.module.parameters():
            if hasattr(p, "_grad_sink"):
                del p._grad_sink
            p.grad = None
        if self.flat_grad is not None:
            torch.cuda.synchronize()
            self.group.symm_free(self.flat_grad)
            self.flat_grad = None

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


class GraphedTrainStep:
    """``train_step`` captured once into a CUDA graph and replayed.

    The optimizer must keep its step number on the device (``make_optimizer(device_step=True)``).
    Capture needs the lazily created state of the libraries involved (cuBLAS workspaces, autograd
    buffers, the column-sum counters) to exist already, so two eager steps run first on a side
    stream; parameters and optimizer state are put back afterwards, so constructing this object does
    not train.  ``__call__`` copies the batch into the graph's static input tensors (the copies are
    ordinary stream work, pinned host tensors are fine), replays the graph and returns the static
    loss tensor, which the next call overwrites.
    """

    def __init__(self, ddp: DataParallel, opt: FlatAdamW, idx: torch.Tensor, targets: torch.Tensor, warmup: int = 2):
        assert opt._step_dev is not None, "GraphedTrainStep needs an optimizer with device_step=True"
        assert not ddp.record_timeline, "event timing cannot be captured; record the timeline on an eager step"
        self.ddp, self.opt = ddp, opt
        dev = ddp.flat_param.device
        self.idx = torch.empty(idx.shape, dtype=idx.dtype, device=dev)
        self.targets = torch.empty(targets.shape, dtype=targets.dtype, device=dev)
        self.idx.copy_(idx)
        self.targets.copy_(targets)
        keep = [t.clone() for t in (ddp.flat_param, opt.master, opt.m, opt.v, opt._step_dev)]
        step_count = opt.step_count
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                train_step(ddp, opt, self.idx, self.targets)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        launches0 = ddp.launches
        from ..ops import train as train_ops

        count0 = train_ops.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = train_step(ddp, opt, self.idx, self.targets)
        # kernels of this library that one replay launches (collective kernels, layer and training kernels)
        self.launches_per_step = (ddp.launches - launches0) + (train_ops.launch_count - count0)
        for t, k in zip((ddp.flat_param, opt.master, opt.m, opt.v, opt._step_dev), keep):
            t.copy_(k)
        opt.step_count = step_count
        torch.cuda.synchronize()

    def __call__(self, idx: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self.idx.copy_(idx, non_blocking=True)
        self.targets.copy_(targets, non_blocking=True)
        self.graph.replay()
        self.opt.step_count += 1
        return self.loss
