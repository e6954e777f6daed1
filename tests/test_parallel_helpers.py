"""Pipeline, Ulysses and ring-attention helpers over the CPU transport (real ranks, host tensors)."""
import torch

from mp_util import run_ranks


def _pipeline(comm):
    from oneccl_b200.parallel.pp import PipelineStage, run_gpipe

    W, r = comm.size, comm.rank
    torch.manual_seed(0)
    layers = [torch.nn.Linear(16, 16) for _ in range(W)]  # every rank builds all, keeps its own
    full = torch.nn.Sequential(*[torch.nn.Sequential(l, torch.nn.Tanh()) for l in layers])
    mine = full[r]
    micro = [torch.randn(4, 16, generator=torch.Generator().manual_seed(10 + m)) for m in range(3)]
    stage = PipelineStage(comm)
    losses = run_gpipe(stage, mine, micro, act_like=torch.empty(4, 16), loss_fn=lambda y, m: (y ** 2).mean())
    # reference: the whole model on one rank
    import copy

    ref = copy.deepcopy(full)
    for p in ref.parameters():
        p.grad = None
    ref_losses = []
    for m in range(3):
        loss = (ref(micro[m]) ** 2).mean()
        loss.backward()
        ref_losses.append(float(loss))
    # the first call above already accumulated into `full[r]`'s parameters: compare with the copy made before
    return r, losses, ref_losses, [float((a.grad - b.grad).abs().max()) for a, b in
                                   zip(mine.parameters(), ref[r].parameters())]


def test_gpipe_schedule_matches_single_process():
    out = run_ranks(_pipeline, 3)
    for r, losses, ref_losses, diffs in out:
        assert max(diffs) < 1e-5, (r, diffs)
        if r == 2:
            assert all(abs(a - b) < 1e-6 for a, b in zip(losses, ref_losses))


def _ulysses_and_ring(comm):
    from oneccl_b200.parallel.sp import ring_attention, ring_pass, ulysses_heads_to_seq, ulysses_seq_to_heads

    W, r = comm.size, comm.rank
    S, H, D = 8 * W, 2 * W, 4
    g = torch.Generator().manual_seed(3)
    full = torch.randn(S, H, D, generator=g)
    shard = full[r * (S // W):(r + 1) * (S // W)].contiguous()
    heads = ulysses_seq_to_heads(comm, shard)
    ok = torch.equal(heads, full[:, r * (H // W):(r + 1) * (H // W)])
    back = ulysses_heads_to_seq(comm, heads)
    ok = ok and torch.equal(back, shard)
    got = ring_pass(comm, torch.full((5,), float(r)))
    ok = ok and torch.equal(got, torch.full((5,), float((r - 1) % W)))
    q, k, v = (torch.randn(S, H, D, generator=g) for _ in range(3))
    sl = slice(r * (S // W), (r + 1) * (S // W))
    out = ring_attention(comm, q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous())
    ref = torch.nn.functional.scaled_dot_product_attention(q.permute(1, 0, 2), k.permute(1, 0, 2), v.permute(1, 0, 2))
    err = float((out - ref.permute(1, 0, 2)[sl]).abs().max())
    return ok, err


def test_ulysses_all_to_all_and_ring_attention():
    for ok, err in run_ranks(_ulysses_and_ring, 4):
        assert ok and err < 1e-5, err
