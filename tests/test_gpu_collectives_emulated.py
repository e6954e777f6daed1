"""Collective kernels against a plain PyTorch fp32 restatement, with all ranks
emulated on one GPU (cooperative launch, blockIdx.y = rank).  Mirrors the
reference's functional matrix (tests/functional/conf.cpp:51-53: sizes 17,
32771, 262144; every datatype / reduction; in-place and out-of-place) with
canary padding around every output buffer."""
import pytest
import torch

pytestmark = pytest.mark.gpu

WORLDS = [2, 4, 8]
SIZES = [1, 17, 4096, 32771, 262144]
CANARY = 64


@pytest.fixture(scope="module", params=WORLDS)
def group(request):
    from oneccl_b200.ops.device_group import DeviceGroup

    g = DeviceGroup.emulated(request.param, heap_bytes=96 << 20, staging_bytes=8 << 20)
    yield g
    g.close()


def _padded(n, dtype, fill=None):
    """Tensor of n elements inside a larger buffer with canary words on both sides."""
    buf = torch.full((n + 2 * CANARY,), 77, dtype=dtype, device="cuda")
    view = buf[CANARY:CANARY + n]
    if fill is not None:
        view.copy_(fill)
    return buf, view


def _canary_ok(buf, n):
    ref = torch.full((CANARY,), 77, dtype=buf.dtype, device="cuda")
    return torch.equal(buf[:CANARY], ref) and torch.equal(buf[CANARY + n:], ref)


def _inputs(world, n, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    outs = []
    for r in range(world):
        if dtype.is_floating_point:
            x = (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)
        else:
            x = torch.randint(-3, 4, (n,), generator=g, device="cuda").to(dtype)
        outs.append(x)
    return outs


def _tol(dtype, world):
    if dtype == torch.bfloat16:
        return dict(rtol=2e-2, atol=2e-2 * world ** 0.5)
    if dtype == torch.float16:
        return dict(rtol=2e-3, atol=2e-3 * world ** 0.5)
    if dtype == torch.float32:
        return dict(rtol=1e-5, atol=1e-5)
    return dict(rtol=0, atol=0)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32])
@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "pipelined"])
def test_allreduce_sum(group, n, dtype, algo):
    W = group.world
    xs = _inputs(W, n, dtype)
    ref = torch.stack([x.double() for x in xs]).sum(0)
    bufs = [_padded(n, dtype) for _ in range(W)]
    group.allreduce(xs, [b[1] for b in bufs], op="sum", algo=algo)
    torch.cuda.synchronize()
    group.check()
    for buf, out in bufs:
        torch.testing.assert_close(out.double(), ref, **_tol(dtype, W))
        assert _canary_ok(buf, n)
    # every rank holds bit-identical results
    for _, out in bufs[1:]:
        assert torch.equal(out, bufs[0][1])


@pytest.mark.parametrize("op", ["prod", "min", "max"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.int64, torch.bfloat16])
def test_allreduce_other_ops(group, op, dtype):
    W, n = group.world, 3001
    xs = _inputs(W, n, dtype, seed=3)
    st = torch.stack([x.double() for x in xs])
    ref = {"prod": st.prod(0), "min": st.min(0).values, "max": st.max(0).values}[op]
    outs = [torch.empty_like(x) for x in xs]
    group.allreduce(xs, outs, op=op, algo="auto")
    torch.cuda.synchronize()
    group.check()
    for o in outs:
        torch.testing.assert_close(o.double(), ref, **_tol(dtype, W))


def test_allreduce_inplace_unaligned_and_repeat(group):
    """In-place, pointer offset by one element (not 16-byte aligned), called several
    times in a row so that both staging generations and the epoch flags are reused."""
    W, n = group.world, 5003
    for it in range(5):
        for algo in ("oneshot", "twoshot", "pipelined"):
            base = [torch.zeros(n + 1, dtype=torch.float32, device="cuda") for _ in range(W)]
            xs = [b[1:] for b in base]
            src = _inputs(W, n, torch.float32, seed=10 + it)
            for x, s in zip(xs, src):
                x.copy_(s)
            ref = torch.stack(src).sum(0)
            group.allreduce(xs, xs, algo=algo)
            torch.cuda.synchronize()
            group.check()
            for x in xs:
                torch.testing.assert_close(x, ref, rtol=1e-5, atol=1e-5)


def test_allreduce_scale_and_cast(group):
    """bf16 in, fp32 out, fused 1/world scale (the data-parallel epilogue)."""
    W, n = group.world, 70001
    xs = _inputs(W, n, torch.bfloat16, seed=5)
    ref = torch.stack([x.float() for x in xs]).sum(0) / W
    for algo in ("oneshot", "twoshot", "pipelined"):
        outs = [torch.empty(n, dtype=torch.float32, device="cuda") for _ in range(W)]
        group.allreduce(xs, outs, algo=algo, scale=1.0 / W)
        torch.cuda.synchronize()
        group.check()
        for o in outs:
            torch.testing.assert_close(o, ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("algo", ["twoshot", "pipelined"])
def test_allreduce_narrowing_cast(group, algo):
    """fp32 in, bf16 out: a reduced pack is 8 bytes, staged in 16-byte units."""
    W, n = group.world, 9001
    xs = _inputs(W, n, torch.float32, seed=6)
    ref = torch.stack(xs).sum(0)
    bufs = [_padded(n, torch.bfloat16) for _ in range(W)]
    group.allreduce(xs, [b[1] for b in bufs], algo=algo)
    torch.cuda.synchronize()
    group.check()
    for buf, o in bufs:
        torch.testing.assert_close(o.float(), ref, rtol=1e-2, atol=1e-2)
        assert _canary_ok(buf, n)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("blocks", [0, 3])
def test_allreduce_pipelined_many_chunks(group, dtype, blocks):
    """Message of several chunks (8 MiB staging holds 2 MiB chunks): the copy-in, reduce and
    copy-out stages of neighbouring chunks overlap; odd length, run twice for the generation flip."""
    W = group.world
    n = (11 << 20) // torch.empty((), dtype=dtype).element_size() + 13
    xs = _inputs(W, n, dtype, seed=8)
    ref = torch.stack([x.double() for x in xs]).sum(0)
    for _ in range(2):
        bufs = [_padded(n, dtype) for _ in range(W)]
        group.allreduce(xs, [b[1] for b in bufs], algo="pipelined", blocks=blocks)
        torch.cuda.synchronize()
        group.check()
        for buf, o in bufs:
            torch.testing.assert_close(o.double(), ref, **_tol(dtype, W))
            assert _canary_ok(buf, n)
        assert group.algo_hits("allreduce", "pipelined") > 0


def test_allreduce_twoshot_chunked(group):
    """Message larger than one staging generation: several launches alternate generations."""
    W = group.world
    n = (20 << 20) // 4  # 20 MiB of fp32 with 8 MiB staging
    xs = _inputs(W, n, torch.float32, seed=7)
    ref = torch.stack(xs).sum(0)
    outs = [torch.empty_like(x) for x in xs]
    group.allreduce(xs, outs, algo="twoshot")
    torch.cuda.synchronize()
    group.check()
    for o in outs:
        torch.testing.assert_close(o, ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [24, 1000, 40003])
def test_allreduce_symmetric_zero_copy(group, dtype, n):
    W = group.world
    bufs = group.symm_empty((n,), dtype=dtype)
    src = _inputs(W, n, dtype, seed=11)
    for b, s in zip(bufs, src):
        b.copy_(s)
    ref = torch.stack([s.double() for s in src]).sum(0)
    group.allreduce(bufs, bufs, algo="symm")
    torch.cuda.synchronize()
    group.check()
    for b in bufs:
        torch.testing.assert_close(b.double(), ref, **_tol(dtype, W))
    assert group.algo_hits("allreduce", "symm") >= 1
    group.symm_free(bufs)


@pytest.mark.parametrize("n", [1, 17, 32771])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reduce_scatter(group, n, dtype):
    W = group.world
    xs = _inputs(W, n * W, dtype, seed=2)
    full = torch.stack([x.double() for x in xs]).sum(0)
    bufs = [_padded(n, dtype) for _ in range(W)]
    group.reduce_scatter(xs, [b[1] for b in bufs])
    torch.cuda.synchronize()
    group.check()
    for r, (buf, out) in enumerate(bufs):
        torch.testing.assert_close(out.double(), full[r * n:(r + 1) * n], **_tol(dtype, W))
        assert _canary_ok(buf, n)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_reduce_scatter_pipelined_many_chunks(group, dtype):
    """Blocks larger than a staging slab (8 MiB staging): several chunks, copy and reduction overlap;
    odd block length, twice for the generation flip, with a fused scale."""
    W = group.world
    esz = torch.empty((), dtype=dtype).element_size()
    n = (3 << 20) // esz // W * 2 + 7
    xs = _inputs(W, n * W, dtype, seed=12)
    full = torch.stack([x.double() for x in xs]).sum(0) / W
    for _ in range(2):
        bufs = [_padded(n, dtype) for _ in range(W)]
        group.reduce_scatter(xs, [b[1] for b in bufs], algo="pipelined", scale=1.0 / W)
        torch.cuda.synchronize()
        group.check()
        for r, (buf, out) in enumerate(bufs):
            torch.testing.assert_close(out.double(), full[r * n:(r + 1) * n], **_tol(dtype, W))
            assert _canary_ok(buf, n)
    assert group.algo_hits("reduce_scatter", "pipelined") >= 2


def test_reduce_scatter_symmetric(group):
    W, n = group.world, 4099
    send = group.symm_empty((n * W,), dtype=torch.float32)
    src = _inputs(W, n * W, torch.float32, seed=4)
    for b, s in zip(send, src):
        b.copy_(s)
    full = torch.stack(src).sum(0)
    outs = [torch.empty(n, dtype=torch.float32, device="cuda") for _ in range(W)]
    group.reduce_scatter(send, outs, algo="symm")
    torch.cuda.synchronize()
    group.check()
    for r, o in enumerate(outs):
        torch.testing.assert_close(o, full[r * n:(r + 1) * n], rtol=1e-5, atol=1e-5)
    group.symm_free(send)


@pytest.mark.parametrize("root", [0, 1])
def test_reduce_and_broadcast(group, root):
    W, n = group.world, 10007
    xs = _inputs(W, n, torch.float32, seed=8)
    ref = torch.stack(xs).sum(0)
    outs = [torch.zeros(n, device="cuda") if r == root else None for r in range(W)]
    group.reduce(xs, outs, root=root)
    torch.cuda.synchronize()
    group.check()
    torch.testing.assert_close(outs[root], ref, rtol=1e-5, atol=1e-5)
    # broadcast the result back out, in place
    bufs = [outs[root].clone() if r == root else torch.zeros(n, device="cuda") for r in range(W)]
    group.broadcast(bufs, bufs, root=root)
    torch.cuda.synchronize()
    group.check()
    for b in bufs:
        assert torch.equal(b, bufs[root])


@pytest.mark.parametrize("algo", ["push", "pull"])
def test_allgatherv_unequal(group, algo):
    W = group.world
    counts = [1000 + 37 * r for r in range(W)]
    counts[0] = 1  # tiny and odd blocks
    src = [torch.arange(c, device="cuda", dtype=torch.float32) + 1000 * r for r, c in enumerate(counts)]
    ref = torch.cat(src)
    total = sum(counts)
    bufs = [_padded(total, torch.float32) for _ in range(W)]
    group.allgatherv(src, [b[1] for b in bufs], counts=counts, algo=algo)
    torch.cuda.synchronize()
    group.check()
    for buf, out in bufs:
        assert torch.equal(out, ref)
        assert _canary_ok(buf, total)


def test_allgather_inplace_and_symmetric(group):
    W, per = group.world, 2048
    outs = [torch.zeros(per * W, device="cuda") for _ in range(W)]
    for r, o in enumerate(outs):
        o[r * per:(r + 1) * per] = torch.arange(per, device="cuda") + r * 10000
    ref = torch.cat([torch.arange(per, device="cuda", dtype=torch.float32) + r * 10000 for r in range(W)])
    group.allgatherv(None, outs)  # in place: send == recv + offset(rank)
    torch.cuda.synchronize()
    group.check()
    for o in outs:
        assert torch.equal(o, ref)
    sym = group.symm_empty((per * W,), dtype=torch.float32)
    src = [ref[r * per:(r + 1) * per].clone() for r in range(W)]
    for algo in ("symm", "ce"):  # stores by SMs / pulls by the copy engines between two barriers
        for s in sym:
            s.zero_()
        group.allgatherv(src, sym, algo=algo)
        torch.cuda.synchronize()
        group.check()
        for s in sym:
            assert torch.equal(s, ref)
        assert group.algo_hits("allgatherv", algo) > 0
    group.symm_free(sym)


def test_alltoallv_variable_counts(group):
    W = group.world
    g = torch.Generator().manual_seed(1)
    cnt = torch.randint(0, 700, (W, W), generator=g).tolist()  # cnt[r][q]: r sends to q
    send = [torch.cat([torch.full((cnt[r][q],), float(r * 100 + q), device="cuda") for q in range(W)])
            for r in range(W)]
    recv_counts = [[cnt[p][r] for p in range(W)] for r in range(W)]
    bufs = [_padded(sum(recv_counts[r]), torch.float32) for r in range(W)]
    group.alltoallv(send, [b[1] for b in bufs], send_counts=cnt, recv_counts=recv_counts)
    torch.cuda.synchronize()
    group.check()
    for r, (buf, out) in enumerate(bufs):
        ref = torch.cat([torch.full((cnt[p][r],), float(p * 100 + r), device="cuda") for p in range(W)])
        assert torch.equal(out, ref)
        assert _canary_ok(buf, ref.numel())


def test_alltoall_multi_round(group):
    """Blocks larger than a staging slot: the kernel agrees on extra rounds on the device."""
    W = group.world
    per = ((8 << 20) // W // 4) * 2 + 123  # two slots and a bit, in fp32 elements
    send = [torch.arange(per * W, device="cuda", dtype=torch.float32) + r * 1e6 for r in range(W)]
    recv = [torch.zeros(per * W, device="cuda") for _ in range(W)]
    group.alltoallv(send, recv)
    torch.cuda.synchronize()
    group.check()
    for r in range(W):
        ref = torch.cat([send[p][r * per:(r + 1) * per] for p in range(W)])
        assert torch.equal(recv[r], ref)


@pytest.mark.parametrize("per", [4, 2052, ((8 << 20) // 8 // 4) * 3 + 8])
@pytest.mark.parametrize("symmetric", [False, True])
def test_alltoall_equal_blocks(group, per, symmetric):
    """Equal 16-byte-multiple blocks: batched staged kernel (one or several rounds) and the
    direct stores into a symmetric recv buffer; run twice to cover buffer reuse."""
    W = group.world
    send = [torch.arange(per * W, device="cuda", dtype=torch.float32) + r * 1e6 for r in range(W)]
    recv = group.symm_empty((per * W,), dtype=torch.float32) if symmetric else \
        [torch.zeros(per * W, device="cuda") for _ in range(W)]
    for it in range(2):
        for x in send:
            x += it
        group.alltoall(send, recv)
        torch.cuda.synchronize()
        group.check()
        for r in range(W):
            ref = torch.cat([send[p][r * per:(r + 1) * per] for p in range(W)])
            assert torch.equal(recv[r], ref)
    assert group.algo_hits("alltoallv", "symm" if symmetric else "push") > 0
    if symmetric:
        group.symm_free(recv)


def test_allgather_push_uniform_and_nvls_flags(group):
    """Equal aligned blocks take the batched copy-out; unequal ones the per-peer copies."""
    W, per = group.world, 4100
    src = [torch.arange(per, device="cuda", dtype=torch.float32) + r * 10000 for r in range(W)]
    bufs = [_padded(per * W, torch.float32) for _ in range(W)]
    group.allgatherv(src, [b[1] for b in bufs], algo="push")
    torch.cuda.synchronize()
    group.check()
    ref = torch.cat(src)
    for buf, o in bufs:
        assert torch.equal(o, ref) and _canary_ok(buf, per * W)


def test_barrier_and_sendrecv(group):
    W = group.world
    group.barrier()
    n = 300000
    src = [torch.arange(n, device="cuda", dtype=torch.float32) + r for r in range(W)]
    dst = [torch.zeros(n, device="cuda") for _ in range(W)]
    # ring: even ranks send to rank+1, odd ranks receive from rank-1 (one launch holds both sides)
    peers, is_send = [], []
    for r in range(W):
        if r % 2 == 0:
            peers.append(r + 1 if r + 1 < W else -1)
            is_send.append(True)
        else:
            peers.append(r - 1)
            is_send.append(False)
    for _ in range(2):  # twice: sequence numbers advance
        group.sendrecv(src, dst, peers, is_send)
    torch.cuda.synchronize()
    group.check()
    for r in range(1, W, 2):
        assert torch.equal(dst[r], src[r - 1])


@pytest.mark.parametrize("nbytes", [0, 1, 65536, 65537, 9 << 20, (40 << 20) + 12])
def test_sendrecv_chunk_pipeline_sizes(group, nbytes):
    """Messages from nothing to several times the pair's ring of stages, odd tails included; a second
    exchange in the opposite direction continues the per-block chunk counters."""
    W = group.world
    gen = torch.Generator(device="cuda").manual_seed(nbytes % 977)
    src = [torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda", generator=gen) for _ in range(W)]
    for flip in (False, True):
        dst = [torch.full((nbytes + 32,), 7, dtype=torch.uint8, device="cuda") for _ in range(W)]
        peers, is_send = [], []
        for r in range(W):
            sender = (r % 2 == 0) != flip
            partner = r + 1 if r % 2 == 0 else r - 1
            peers.append(partner if partner < W else -1)
            is_send.append(sender)
        group.sendrecv(src, [d[:nbytes] for d in dst], peers, is_send)
        torch.cuda.synchronize()
        group.check()
        for r in range(W):
            if peers[r] >= 0 and not is_send[r]:
                assert torch.equal(dst[r][:nbytes], src[peers[r]])
                assert bool((dst[r][nbytes:] == 7).all())


@pytest.mark.parametrize("max_blocks", [0, 3])
def test_sendrecv_pull_mode_and_unequal_block_counts(monkeypatch, max_blocks):
    """The ring at the sender with the receiver loading from it, and fewer blocks than lanes (a block then
    serves several lanes one after the other)."""
    from oneccl_b200 import _lib
    from oneccl_b200.ops.device_group import DeviceGroup

    monkeypatch.setenv("CCL_CUDA_P2P_PULL", "1")
    monkeypatch.setenv("CCL_CUDA_P2P_MAX_BLOCKS", str(max_blocks))
    _lib.load().cclx_env_reload()
    g = DeviceGroup.emulated(2, heap_bytes=48 << 20, staging_bytes=1 << 20)
    try:
        for nbytes in (5, 3 << 20, (20 << 20) + 4):
            src = [torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda") for _ in range(2)]
            dst = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
            g.sendrecv(src, dst, [1, 0], [True, False])
            g.sendrecv(src, dst, [1, 0], [False, True])
            torch.cuda.synchronize()
            g.check()
            assert torch.equal(dst[1], src[0]) and torch.equal(dst[0], src[1])
    finally:
        g.close()
        monkeypatch.delenv("CCL_CUDA_P2P_PULL")
        monkeypatch.delenv("CCL_CUDA_P2P_MAX_BLOCKS")
        _lib.load().cclx_env_reload()


def test_wait_timeout_reports_status():
    """A device-side wait that nothing satisfies runs out after its limit, the
    kernel returns, the status word says so and the context keeps working."""
    from oneccl_b200 import CclError
    from oneccl_b200.ops.device_group import DeviceGroup

    g = DeviceGroup.emulated(2, heap_bytes=48 << 20, staging_bytes=1 << 20)
    g.set_timeout_ms(300)
    g.wait_unset_flag()
    torch.cuda.synchronize()
    assert g.status(0) == 3 and g.status(1) == 3  # ST_FLAG_TIMEOUT
    with pytest.raises(CclError):
        g.check()
    g.clear_status()
    xs = [torch.ones(100, device="cuda") for _ in range(2)]
    g.allreduce(xs, xs)
    torch.cuda.synchronize()
    assert torch.equal(xs[0], torch.full((100,), 2.0, device="cuda"))
    g.close()


@pytest.mark.parametrize("algo", ["symm", "twoshot"])
def test_argument_mismatch_between_ranks_is_reported(algo):
    """Zero-copy kernels apply this rank's offsets and count to the peers' memory, so every rank must pass
    the same ones.  The first barrier of a kernel compares a signature of those arguments across ranks; a
    rank that disagrees (here: one emulated rank's signature is falsified) ends the kernel with
    ST_ARG_MISMATCH before any data is touched, and the communicator works again after the status is cleared."""
    from oneccl_b200 import CclError
    from oneccl_b200.ops.device_group import DeviceGroup

    W = 4
    g = DeviceGroup.emulated(W, heap_bytes=48 << 20, staging_bytes=1 << 20)
    bufs = g.symm_empty((4096,), dtype=torch.float32)
    for r, b in enumerate(bufs):
        b.fill_(float(r + 1))
    g.test_sig_skew(2)
    g.allreduce(bufs, bufs, algo=algo)
    torch.cuda.synchronize()
    assert all(g.status(r) == 7 for r in range(W)), [g.status(r) for r in range(W)]  # ST_ARG_MISMATCH
    for r, b in enumerate(bufs):  # nothing was reduced
        assert torch.equal(b, torch.full_like(b, float(r + 1)))
    with pytest.raises(CclError, match="buffer kind, offset or count"):
        g.check()
    g.clear_status()
    g.test_sig_skew(-1)
    g.allreduce(bufs, bufs, algo=algo)
    torch.cuda.synchronize()
    g.check()
    assert torch.equal(bufs[0], torch.full_like(bufs[0], 10.0))
    g.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("blocks", [1, 2, 5])
def test_allreduce_symmetric_narrow_grid(group, dtype, blocks):
    """The few-block form used beside a compute kernel (1024-thread blocks, eight loads in flight per
    thread in the in-switch variant) against the fp32 sum, on a size that leaves a ragged tail."""
    W = group.world
    n = 300_003
    bufs = group.symm_empty((n,), dtype=dtype)
    src = _inputs(W, n, dtype, seed=5)
    for b, s in zip(bufs, src):
        b.copy_(s)
    ref = torch.stack([s.double() for s in src]).sum(0) / W
    group.allreduce(bufs, bufs, blocks=blocks, scale=1.0 / W)
    torch.cuda.synchronize()
    group.check()
    for b in bufs:
        torch.testing.assert_close(b.double(), ref, **_tol(dtype, W))
    group.symm_free(bufs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_small_allreduces_pack_reduce_unpack(group, dtype):
    """Many small tensors as ONE collective: pack kernel -> one zero-copy allreduce on a buffer of the symmetric
    heap -> unpack kernel, against the fp32 sum; odd sizes, unaligned starts and canaries around every tensor,
    one tensor too large for the fused buffer (reduced on its own), twice in a row (table slots are reused)."""
    W = group.world
    sizes = [1, 17, 255, 4096, 3, 1000, 32771, 8, 2_500_000, 77]
    for rep in range(2):
        bufs, views, refs = [], [], []
        for k, n in enumerate(sizes):
            src = _inputs(W, n, dtype, seed=100 * rep + k)
            per_rank_buf, per_rank_view = [], []
            for r in range(W):
                b, v = _padded(n + 1, dtype)
                v = v[1:]  # starts that are not 16-byte aligned
                v.copy_(src[r])
                per_rank_buf.append(b)
                per_rank_view.append(v)
            bufs.append(per_rank_buf)
            views.append(per_rank_view)
            refs.append(torch.stack([x.double() for x in src]).sum(0) / W)
        before = group.fused_batches
        group.allreduce_fused(views, scale=1.0 / W)
        torch.cuda.synchronize()
        group.check()
        assert group.fused_batches > before
        for k, n in enumerate(sizes):
            for r in range(W):
                torch.testing.assert_close(views[k][r].double(), refs[k], **_tol(dtype, W))
                assert _canary_ok(bufs[k][r], n + 1) and float(bufs[k][r][CANARY]) == 77.0


@pytest.mark.parametrize("topk", [1, 2])
def test_moe_fused_dispatch_and_combine(group, topk):
    """Rows go straight into the owning expert's symmetric buffer and come back by peer loads with
    the weighted sum; checked against a dense restatement, twice (buffer and table reuse)."""
    from oneccl_b200.parallel.ep import fused_combine, fused_dispatch

    W, T, H = group.world, 37, 64
    cap = T * topk * W
    xrecv = group.symm_empty((cap, H), dtype=torch.bfloat16)
    yout = group.symm_empty((cap, H), dtype=torch.bfloat16)
    cnt = group.symm_empty((256 * W * W,), dtype=torch.int32)
    metas = [torch.zeros(2 * W + 2, dtype=torch.int32, device="cuda") for _ in range(W)]
    gen = torch.Generator(device="cuda").manual_seed(5)
    for it in range(2):
        xs = [torch.randn(T, H, generator=gen, device="cuda").to(torch.bfloat16) for _ in range(W)]
        idx = [torch.stack([torch.randperm(W, generator=gen, device="cuda")[:topk] for _ in range(T)]) for _ in range(W)]
        wts = [torch.softmax(torch.randn(T, topk, generator=gen, device="cuda"), -1) for _ in range(W)]
        flat = [i.reshape(-1) for i in idx]
        order = [torch.argsort(f, stable=True) for f in flat]
        counts = [torch.bincount(f, minlength=W) for f in flat]
        for r in xrecv:
            r.zero_()
        fused_dispatch(group, xs, order, counts, metas, xrecv, cnt, topk)
        torch.cuda.synchronize()
        group.check()
        # expert e holds, rank by rank, the rows routed to it in each sender's sorted order
        for e in range(W):
            rows = [xs[r][order[r][flat[r][order[r]] == e] // topk] for r in range(W)]
            ref = torch.cat(rows)
            assert int(metas[e][2 * W]) == ref.shape[0] and int(metas[e][2 * W + 1]) == 0
            assert torch.equal(xrecv[e][:ref.shape[0]], ref)
            yout[e][:ref.shape[0]] = (ref.float() * (e + 1)).to(torch.bfloat16)  # stand-in expert
        pos = []
        for r in range(W):
            p = torch.empty_like(order[r])
            p[order[r]] = torch.arange(order[r].numel(), device="cuda")
            pos.append(p)
        outs = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(W)]
        fused_combine(group, flat, pos, [w.contiguous().view(-1) for w in wts], outs, metas, yout, topk)
        torch.cuda.synchronize()
        group.check()
        for r in range(W):
            ref = torch.zeros(T, H, device="cuda")
            for s in range(topk):
                y = (xs[r].float() * (idx[r][:, s:s + 1] + 1).float()).to(torch.bfloat16).float()
                ref += wts[r][:, s:s + 1] * y
            torch.testing.assert_close(outs[r].float(), ref, rtol=2e-2, atol=2e-2)
    for t in (xrecv, yout, cnt):
        group.symm_free(t)


def test_registered_buffers_zero_copy(group):
    """Ordinary tensors made peer-accessible by registration take the zero-copy kernels: allreduce
    (views at an inner offset, odd length), reduce_scatter, allgather and alltoall."""
    W = group.world
    n = 300_000
    base = [torch.zeros(n + 64, dtype=torch.float32, device="cuda") for _ in range(W)]
    rid = group.register(base)
    xs = [b[32:32 + n - 3] for b in base]  # same offset on every rank, 128-byte aligned, odd length
    src = _inputs(W, n - 3, torch.float32, seed=21)
    for x, s in zip(xs, src):
        x.copy_(s)
    ref = torch.stack(src).sum(0)
    before = group.algo_hits("allreduce", "symm")
    # in place; the automatic choice at this size is zero-copy too, except between two ranks (one-shot up to 8 MiB)
    group.allreduce(xs, xs, algo="auto" if W > 2 else "symm")
    torch.cuda.synchronize()
    group.check()
    assert group.algo_hits("allreduce", "symm") == before + 1
    for x, b in zip(xs, base):
        torch.testing.assert_close(x, ref, rtol=1e-5, atol=1e-5)
        assert torch.count_nonzero(b[:32]) == 0 and torch.count_nonzero(b[32 + n - 3:]) == 0

    # reduce_scatter out of a registered send buffer
    per = 70_000
    sends = [torch.randn(per * W, device="cuda") for _ in range(W)]
    rid2 = group.register(sends)
    outs = [torch.empty(per, device="cuda") for _ in range(W)]
    group.reduce_scatter(sends, outs, algo="symm")
    torch.cuda.synchronize()
    group.check()
    tot = torch.stack(sends).sum(0)
    for r, o in enumerate(outs):
        torch.testing.assert_close(o, tot[r * per:(r + 1) * per], rtol=1e-5, atol=1e-5)

    # allgather and alltoall into registered recv buffers
    recvs = [torch.zeros(per * W, device="cuda") for _ in range(W)]
    rid3 = group.register(recvs)
    parts = [torch.randn(per, device="cuda") for _ in range(W)]
    group.allgatherv(parts, recvs, algo="symm")
    torch.cuda.synchronize()
    group.check()
    for o in recvs:
        assert torch.equal(o, torch.cat(parts))
    a2a_before = group.algo_hits("alltoallv", "symm")
    group.alltoall(sends, recvs)
    torch.cuda.synchronize()
    group.check()
    assert group.algo_hits("alltoallv", "symm") == a2a_before + 1
    for r in range(W):
        assert torch.equal(recvs[r], torch.cat([sends[p][r * per:(r + 1) * per] for p in range(W)]))
    for i in (rid, rid2, rid3):
        group.deregister(i)
    # after deregistration the same buffers go through staging again
    before = group.algo_hits("allreduce", "symm")
    group.allreduce(xs, xs)
    torch.cuda.synchronize()
    group.check()
    assert group.algo_hits("allreduce", "symm") == before
