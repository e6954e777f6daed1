"""Sequence- and context-parallel helpers on top of the collectives.

The reference has no sequence parallelism of its own (a user builds it from allgather /
reduce_scatter or alltoall); these are the two usual constructions:

* ``ulysses_*``: all-to-all that turns a sequence shard with all heads into the full sequence
  with a shard of the heads (and back), so that attention runs locally per head group;
* ``ring_pass``: one rotation step of a ring (send to the next rank, receive from the previous
  one in a single group), the building block of ring / blockwise attention over K and V.

Megatron-style sequence parallelism (all-gather before, reduce-scatter after a tensor-parallel
region) is what ``TensorParallelMLP`` already fuses into its GEMMs."""
from __future__ import annotations

import torch

from ..comm import Communicator, group_end, group_start


def ulysses_seq_to_heads(comm: Communicator, x: torch.Tensor) -> torch.Tensor:
    """[S / W, H, D] (my sequence shard, all heads) -> [S, H / W, D] (whole sequence, my heads)."""
    W = comm.size
    s, H, D = x.shape
    assert H % W == 0
    send = x.view(s, W, H // W, D).permute(1, 0, 2, 3).contiguous()  # block q = heads of rank q
    recv = torch.empty_like(send)
    comm.alltoall(send, recv).wait()
    return recv.view(W * s, H // W, D)  # block p = sequence shard of rank p


def ulysses_heads_to_seq(comm: Communicator, x: torch.Tensor) -> torch.Tensor:
    """Inverse of ``ulysses_seq_to_heads``: [S, H / W, D] -> [S / W, H, D]."""
    W = comm.size
    S, h, D = x.shape
    assert S % W == 0
    send = x.contiguous().view(W, S // W, h, D)  # block q = sequence shard of rank q
    recv = torch.empty_like(send)
    comm.alltoall(send, recv).wait()
    return recv.permute(1, 0, 2, 3).reshape(S // W, W * h, D)  # block p = heads of rank p


class _RingTransfer:
    """A rotation step in flight: ``wait()`` returns what rank - 1 sent."""

    def __init__(self, out, events, stream, keep):
        self.out, self.events, self.stream, self.keep = out, events, stream, keep

    def wait(self) -> torch.Tensor:
        for e in self.events:
            e.wait()
        if self.stream is not None:  # device transfer on a side stream: order the caller's stream after it
            torch.cuda.current_stream().wait_stream(self.stream)
        return self.out


_side_streams = {}


def ring_pass_start(comm: Communicator, t: torch.Tensor) -> _RingTransfer:
    """Starts sending ``t`` to rank + 1 and receiving from rank - 1 and returns at once, so that the caller
    can compute on ``t`` while the next block travels.  Host tensors progress on the worker threads; CUDA
    tensors move on a side stream (the group makes send and recv one launch)."""
    W, r = comm.size, comm.rank
    if W == 1:
        return _RingTransfer(t.clone(), [], None, None)
    out = torch.empty_like(t)
    src = t.contiguous()
    stream = None
    kw = {}
    if t.is_cuda:
        key = (t.device.index, id(comm))
        if key not in _side_streams:
            _side_streams[key] = torch.cuda.Stream(priority=torch.cuda.Stream.priority_range()[1])
        stream = _side_streams[key]
        stream.wait_stream(torch.cuda.current_stream())  # `t` is complete before it is sent
        kw = {"stream": stream}
    group_start()
    es = comm.send(src, (r + 1) % W, **kw)
    er = comm.recv(out, (r - 1) % W, **kw)
    group_end()
    if t.is_cuda:
        src.record_stream(stream)
        out.record_stream(stream)
        return _RingTransfer(out, [], stream, src)  # stream order is enough; no host wait
    return _RingTransfer(out, [es, er], None, src)


def ring_pass(comm: Communicator, t: torch.Tensor) -> torch.Tensor:
    """Sends ``t`` to rank + 1 and returns what rank - 1 sent (one step of a ring rotation)."""
    return ring_pass_start(comm, t).wait()


def ring_attention(comm: Communicator, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Non-causal attention over a sequence sharded across the ranks: K / V blocks travel around the
    ring while every rank keeps a running (max, sum, output) for its queries.  The next block is on its way
    while the current one is being multiplied.  q, k, v: [s, H, D]."""
    W = comm.size
    scale = q.shape[-1] ** -0.5
    qh = q.float().permute(1, 0, 2)  # [H, s, D]
    m = torch.full(qh.shape[:2], float("-inf"), device=q.device)
    l = torch.zeros(qh.shape[:2], device=q.device)
    o = torch.zeros_like(qh)
    kv = torch.stack([k, v]).contiguous()
    for step in range(W):
        nxt = ring_pass_start(comm, kv) if step + 1 < W else None
        kh = kv[0].float().permute(1, 0, 2)
        vh = kv[1].float().permute(1, 0, 2)
        sc = torch.matmul(qh, kh.transpose(1, 2)) * scale  # [H, s, s_blk]
        m_new = torch.maximum(m, sc.max(-1).values)
        p = torch.exp(sc - m_new.unsqueeze(-1))
        alpha = torch.exp(m - m_new)
        l = l * alpha + p.sum(-1)
        o = o * alpha.unsqueeze(-1) + torch.matmul(p, vh)
        m = m_new
        if nxt is not None:
            kv = nxt.wait()
    return (o / l.unsqueeze(-1)).permute(1, 0, 2).to(q.dtype)
