"""The allocation-free mean cross-entropy entry point, called through its exported
C symbol exactly as a C caller would, against the regular entry point.

Why the entry point exists: a caller that may not obtain device memory when it
needs a loss (all device memory already belongs to the application's own pool,
or the implicit synchronisation of an allocation is not acceptable on its path)
can still get the mean loss and the logit gradients, because the per-row losses
are kept in a fixed array inside the library instead of a caller buffer.

The file name sorts last on purpose: a run that stops at the first failure has
then already executed every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ROWS = 65536


def _lib():
    from oneccl_b200 import _lib

    lib = _lib.load()
    fn = lib.cclx_softmax_xent_mean_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_size_t, C.c_float, C.c_int,
                   C.c_void_p]
    ref = lib.cclx_softmax_xent
    ref.restype = C.c_int
    ref.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_size_t, C.c_float, C.c_int,
                    C.c_void_p]
    lib.cclx_set_device(torch.cuda.current_device())
    return lib, fn, ref


def _case(rows, vocab, pad, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    logits = (torch.randn(rows, vocab + pad, generator=g, device="cuda") * 2.5).to(torch.bfloat16)
    targets = torch.randint(0, vocab, (rows,), generator=g, device="cuda")
    targets[rows // 3] = -1  # an ignored row
    return logits, targets


def test_no_alloc_matches_regular_entry_point_twice():
    lib, fn, ref = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    mean_out = torch.zeros(1, dtype=torch.float32, device="cuda")  # the caller's output, made before the calls
    # two calls in a row on the shared scratch: the second is smaller, so stale entries of the
    # first call sit right behind the rows it uses
    for rows, vocab, pad, seed in ((1500, 1000, 24, 1), (37, 50257, 47, 2)):
        logits, targets = _case(rows, vocab, pad, seed)
        a = logits.clone()
        b = logits.clone()
        loss_rows = torch.empty(rows, dtype=torch.float32, device="cuda")
        scale = 1.0 / rows
        assert ref(a.data_ptr(), targets.data_ptr(), loss_rows.data_ptr(), rows, vocab, a.stride(0), scale, pad,
                   stream) == 0
        rc = fn(b.data_ptr(), targets.data_ptr(), mean_out.data_ptr(), rows, vocab, b.stride(0), scale, pad, stream)
        assert rc == 0, lib.cclx_last_error().decode()
        torch.cuda.synchronize()
        torch.testing.assert_close(mean_out[0], loss_rows.mean(), rtol=1e-5, atol=1e-6)
        assert torch.equal(a, b)  # same kernel, same gradients bit for bit
        # and both agree with PyTorch in fp32
        x = logits[:, :vocab].float().requires_grad_(True)
        valid = targets >= 0
        lp = torch.nn.functional.cross_entropy(x[valid], targets[valid], reduction="sum") / rows
        lp.backward()
        torch.testing.assert_close(mean_out[0], lp.detach(), rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(b[:, :vocab].float(), x.grad, rtol=2e-2, atol=1e-5)


def test_no_alloc_rejects_more_rows_than_its_scratch_holds():
    lib, fn, _ = _lib()
    logits = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda")
    targets = torch.zeros(4, dtype=torch.int64, device="cuda")
    out = torch.full((1,), 7.0, device="cuda")
    rc = fn(logits.data_ptr(), targets.data_ptr(), out.data_ptr(), MAX_ROWS + 1, 64, 64, 1.0, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    msg = lib.cclx_last_error().decode()
    assert "65536" in msg and "rows" in msg
    torch.cuda.synchronize()
    assert float(out[0]) == 7.0  # nothing was launched
