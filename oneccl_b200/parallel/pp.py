"""Pipeline parallelism over the library's point-to-point operations.

The reference offers ``send`` / ``recv`` and ``group_start`` / ``group_end`` batching
(src/coll/coll.cpp:1381-1473, src/coll/group/group.cpp:25-59) and leaves the schedule to
the application.  ``PipelineStage`` wraps one rank's neighbours; ``run_gpipe`` is the
fill / drain schedule (all forwards, then all backwards) over micro-batches, enough to
train a model cut into ``world`` stages.  Works on host tensors (CPU transport) and on
CUDA tensors (eager device kernels; a send and the matching recv of one step are posted
inside one group so that neighbouring stages cannot deadlock on ordering)."""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch

from ..comm import Communicator, group_end, group_start


class PipelineStage:
    """One rank's place in the pipeline.  Host tensors: every transfer is waited for.  CUDA tensors: transfers
    are ordered by streams and nothing waits on the host; sends go to a side stream (ordered after the producer
    of the tensor), so the activation of micro-batch m travels while m + 1 is computed, and receives run on the
    caller's stream in front of the kernels that use them.  A send completes without its receive as long as
    the pair's ring at the receiver has room (four 8 MiB activations, say), which is what lets the first stage
    run ahead during the fill phase."""

    def __init__(self, comm: Communicator, stage: Optional[int] = None, n_stages: Optional[int] = None):
        self.comm = comm
        self.stage = comm.rank if stage is None else stage
        self.n_stages = comm.size if n_stages is None else n_stages
        self.prev = self.stage - 1 if self.stage > 0 else None
        self.next = self.stage + 1 if self.stage < self.n_stages - 1 else None
        self._send_stream = None

    @property
    def is_first(self) -> bool:
        return self.prev is None

    @property
    def is_last(self) -> bool:
        return self.next is None

    # transports; a subclass may replace these two (the benchmark does, to time another library's p2p)
    def _send(self, t: torch.Tensor, peer: int):
        if not t.is_cuda:
            self.comm.send(t, peer).wait()
            return
        if self._send_stream is None:
            self._send_stream = torch.cuda.Stream()
        side = self._send_stream
        side.wait_stream(torch.cuda.current_stream())
        self.comm.send(t, peer, stream=side)
        t.record_stream(side)

    def _recv(self, buf: torch.Tensor, peer: int):
        ev = self.comm.recv(buf, peer)
        if not buf.is_cuda:
            ev.wait()

    def send_forward(self, t: torch.Tensor):
        if self.next is not None:
            self._send(t.contiguous(), self.next)

    def recv_forward(self, like: torch.Tensor) -> Optional[torch.Tensor]:
        if self.prev is None:
            return None
        buf = torch.empty_like(like)
        self._recv(buf, self.prev)
        return buf

    def send_backward(self, g: torch.Tensor):
        if self.prev is not None:
            self._send(g.contiguous(), self.prev)

    def recv_backward(self, like: torch.Tensor) -> Optional[torch.Tensor]:
        if self.next is None:
            return None
        buf = torch.empty_like(like)
        self._recv(buf, self.next)
        return buf

    def drain(self):
        """Orders the caller's stream after the sends posted so far (end of a step)."""
        if self._send_stream is not None:
            torch.cuda.current_stream().wait_stream(self._send_stream)

    def exchange(self, send_next=None, recv_prev_like=None, send_prev=None, recv_next_like=None):
        """Posts up to four transfers as one group (steady state of a 1F1B schedule: activation out,
        activation in, gradient out, gradient in) and waits for all of them.  Returns (from_prev, from_next)."""
        evs, from_prev, from_next = [], None, None
        keep = []
        group_start()
        if send_next is not None and self.next is not None:
            keep.append(send_next.contiguous())
            evs.append(self.comm.send(keep[-1], self.next))
        if recv_prev_like is not None and self.prev is not None:
            from_prev = torch.empty_like(recv_prev_like)
            evs.append(self.comm.recv(from_prev, self.prev))
        if send_prev is not None and self.prev is not None:
            keep.append(send_prev.contiguous())
            evs.append(self.comm.send(keep[-1], self.prev))
        if recv_next_like is not None and self.next is not None:
            from_next = torch.empty_like(recv_next_like)
            evs.append(self.comm.recv(from_next, self.next))
        group_end()
        for e in evs:
            e.wait()
        return from_prev, from_next


def run_gpipe(stage: PipelineStage, module: torch.nn.Module, micro_inputs: Sequence[torch.Tensor],
              act_like: torch.Tensor, loss_fn: Optional[Callable[[torch.Tensor, int], torch.Tensor]] = None) -> List[float]:
    """Fill / drain schedule.  ``micro_inputs`` are this job's micro-batches (used by the first stage
    only), ``act_like`` has the shape / dtype of the activation that crosses a stage boundary,
    ``loss_fn(output, micro_index)`` is evaluated on the last stage.  Gradients accumulate in
    ``module``'s parameters; returns the micro-batch losses (last stage) or an empty list.  The losses are
    read back once, after the last backward."""
    n = len(micro_inputs)
    saved_in, saved_out, losses = [], [], []
    for m in range(n):
        if stage.is_first:
            x = micro_inputs[m]
        else:
            x = stage.recv_forward(act_like).requires_grad_(True)
        y = module(x)
        saved_in.append(x)
        if stage.is_last:
            loss = loss_fn(y, m) if loss_fn is not None else y.float().mean()
            saved_out.append(loss)
            losses.append(loss.detach())
        else:
            saved_out.append(y)
            stage.send_forward(y.detach())
    for m in range(n):
        if stage.is_last:
            saved_out[m].backward()
        else:
            g = stage.recv_backward(saved_out[m])
            saved_out[m].backward(g)
        if not stage.is_first:
            stage.send_backward(saved_in[m].grad)
        saved_out[m] = None
    stage.drain()
    return [float(l) for l in losses]
