"""Fused cross-entropy, gradient norm and flat AdamW against PyTorch fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,vocab,pad", [(64, 1000, 24), (33, 50257, 47), (8, 257, 0), (5, 70000, 0),
                                            (16, 32768, 0), (3, 57347, 5)])
def test_softmax_xent(rows, vocab, pad):
    from oneccl_b200.ops.train import softmax_cross_entropy

    g = torch.Generator(device="cuda").manual_seed(0)
    logits = (torch.randn(rows, vocab + pad, generator=g, device="cuda") * 3).to(torch.bfloat16)
    tgt = torch.randint(0, vocab, (rows,), generator=g, device="cuda")
    ref_in = logits[:, :vocab].float().clone().requires_grad_(True)
    ref_loss = torch.nn.functional.cross_entropy(ref_in, tgt)
    ref_loss.backward()
    x = logits.clone().requires_grad_(True)
    y = x * 1.0  # non-leaf, like the output of the lm head
    loss = softmax_cross_entropy(y, tgt, vocab)
    loss.backward()
    torch.cuda.synchronize()
    torch.testing.assert_close(loss, ref_loss, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(x.grad[:, :vocab].float(), ref_in.grad, rtol=2e-2, atol=1e-5)
    if pad:
        assert torch.count_nonzero(x.grad[:, vocab:]) == 0


def test_flat_adamw_matches_torch():
    from oneccl_b200.ops.train import FlatAdamW

    n, n_decay = 10007, 8000
    g = torch.Generator(device="cuda").manual_seed(1)
    p0 = torch.randn(n, generator=g, device="cuda")
    model = p0.to(torch.bfloat16)
    ref_p = model.float().clone().requires_grad_(True)
    ref_a = ref_p[:n_decay].detach().clone().requires_grad_(True)
    ref_b = ref_p[n_decay:].detach().clone().requires_grad_(True)
    ropt = torch.optim.AdamW([{"params": [ref_a], "weight_decay": 0.1}, {"params": [ref_b], "weight_decay": 0.0}],
                             lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    opt = FlatAdamW(model, n_decay, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_norm=1.0)
    for step in range(3):
        grad = (torch.randn(n, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
        gf = grad.float()
        clip = min(1.0, 1.0 / (gf.norm().item() + 1e-6))
        ref_a.grad = gf[:n_decay] * clip
        ref_b.grad = gf[n_decay:] * clip
        ropt.step()
        opt.step(grad)
    torch.cuda.synchronize()
    ref = torch.cat([ref_a.detach(), ref_b.detach()])
    torch.testing.assert_close(opt.master, ref, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(model.float(), ref, rtol=1e-2, atol=1e-2)


def test_reduce_local_and_pack():
    from oneccl_b200.ops.device_group import reduce_local

    a = torch.arange(1000, device="cuda", dtype=torch.float32)
    b = torch.ones(1000, device="cuda")
    reduce_local(a, b, op="sum")
    torch.cuda.synchronize()
    assert torch.equal(b, a + 1)
    c = torch.full((1000,), 5, device="cuda", dtype=torch.int32)
    d = torch.arange(1000, device="cuda", dtype=torch.int32)
    reduce_local(c, d, op="max")
    torch.cuda.synchronize()
    assert torch.equal(d, torch.clamp(torch.arange(1000, device="cuda", dtype=torch.int32), min=5))


def test_moe_gather_and_combine_kernels():
    from oneccl_b200.parallel.ep import combine_rows, gather_rows

    g = torch.Generator(device="cuda").manual_seed(3)
    T, H, k = 257, 136, 2
    x = torch.randn(T, H, generator=g, device="cuda").to(torch.bfloat16)
    order = torch.randperm(T * k, generator=g, device="cuda")
    xs = gather_rows(x, order // k)
    torch.cuda.synchronize()
    assert torch.equal(xs, x[order // k])
    pos = torch.empty_like(order)
    pos[order] = torch.arange(T * k, device="cuda")
    w = torch.rand(T, k, generator=g, device="cuda")
    out = combine_rows(xs, pos.view(T, k), w)
    ref = (xs[pos].view(T, k, H).float() * w.unsqueeze(-1)).sum(1)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)


def test_graphed_train_step_matches_eager_steps():
    """The whole step (forward, backward with bucket launches on the side stream, clipping, AdamW with the
    step number kept on the device) replayed from one CUDA graph gives the losses and weights of the same
    steps launched eagerly, and building the graph does not train."""
    from oneccl_b200.models.gpt2 import GPT2, GPT2Config
    from oneccl_b200.ops.device_group import DeviceGroup
    from oneccl_b200.parallel.ddp import DataParallel, GraphedTrainStep, train_step

    cfg = GPT2Config(2, 4, 256, 64, 1000)
    gen = torch.Generator().manual_seed(3)
    batches = [(torch.randint(0, cfg.vocab, (4, 64), generator=gen).cuda(),
                torch.randint(0, cfg.vocab, (4, 64), generator=gen).cuda()) for _ in range(4)]
    results = []
    for graphed in (False, True):
        torch.manual_seed(0)
        model = GPT2(cfg, fused_ops=True).cuda().to(torch.bfloat16)
        group = DeviceGroup.emulated(1, heap_bytes=64 << 20, staging_bytes=1 << 20)
        ddp = DataParallel(model, group, bucket_mb=0.25)
        assert len(ddp.buckets) > 3
        opt = ddp.make_optimizer(lr=1e-3, device_step=graphed)
        if graphed:
            before = ddp.flat_param.clone()
            step = GraphedTrainStep(ddp, opt, *batches[0])
            assert torch.equal(before, ddp.flat_param) and opt.step_count == 0
            assert step.launches_per_step > 10
        else:
            def step(i, t):
                return train_step(ddp, opt, i, t)
        losses = [float(step(i, t).detach()) for i, t in batches]
        torch.cuda.synchronize()
        results.append((losses, ddp.flat_param.float().clone()))
        del step
        ddp.close()
        group.close()
    (l0, w0), (l1, w1) = results
    for a, b in zip(l0, l1):
        assert abs(a - b) < 1e-3, (l0, l1)
    torch.testing.assert_close(w0, w1, rtol=0, atol=2e-3)


@pytest.mark.parametrize("T,E,k", [(1, 2, 1), (97, 8, 2), (4096, 8, 2), (1000, 16, 4), (33, 4, 4)])
def test_moe_routing_kernels_match_torch(T, E, k):
    """Expert ids and weights against torch.topk + softmax, counts against bincount, and the permutation: it
    groups the items by expert and `pos` is its inverse."""
    from oneccl_b200.parallel.ep import route_device

    g = torch.Generator(device="cuda").manual_seed(T + E)
    logits = torch.randn(T, E, generator=g, device="cuda")
    idx, wts, counts, order, pos = route_device(logits, k)
    torch.cuda.synchronize()
    val, ref_idx = torch.topk(logits, k, dim=-1)
    assert torch.equal(idx, ref_idx)
    torch.testing.assert_close(wts, torch.softmax(val, dim=-1), rtol=1e-5, atol=1e-6)
    flat = ref_idx.reshape(-1)
    assert torch.equal(counts, torch.bincount(flat, minlength=E))
    assert torch.equal(torch.sort(order).values, torch.arange(T * k, device="cuda"))
    assert torch.equal(order[pos], torch.arange(T * k, device="cuda"))
    grouped = flat[order]
    assert bool((grouped[1:] >= grouped[:-1]).all())
