"""Training-step kernels next to the gradient collective: fused softmax
cross-entropy (logits become their own gradient in place), squared gradient
norm and flat fused AdamW with fp32 master weights.  All three are native
kernels from ``csrc/gpu/train_kernels.cu``; ``launch_count`` lets callers
report how many of them ran."""
from __future__ import annotations

import torch

from .. import _lib
from ..dtypes import torch_to_ccl
from .device_group import _stream_ptr

launch_count = 0


def _bump(n=1):
    global launch_count
    launch_count += n


class _SoftmaxXent(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, vocab):
        assert logits.dtype == torch.bfloat16 and logits.dim() == 2 and logits.stride(1) == 1
        rows, cols = logits.shape
        ld = logits.stride(0)
        loss_rows = torch.empty(rows, dtype=torch.float32, device=logits.device)
        lib = _lib.load()
        # the kernel overwrites `logits` with d(mean loss)/d(logits)
        _lib.check(lib.cclx_softmax_xent(logits.data_ptr(), targets.data_ptr(), loss_rows.data_ptr(), rows, vocab, ld,
                                         1.0 / rows, cols - vocab, _stream_ptr()))
        _bump()
        # autograd is not told about the in-place write: the producer of `logits` (a matmul)
        # does not need its output for its own backward
        ctx.save_for_backward(logits)
        return loss_rows.mean()

    @staticmethod
    def backward(ctx, grad_out):
        (grad_logits,) = ctx.saved_tensors
        # the stored gradient assumes d(loss) = 1; scale only when the caller scaled the loss
        if ctx.needs_input_grad[0] and grad_out is not None and _SoftmaxXent.scale_by_upstream:
            grad_logits = grad_logits * grad_out.to(grad_logits.dtype)
        return grad_logits, None, None

    scale_by_upstream = False


def softmax_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, vocab: int | None = None) -> torch.Tensor:
    """Mean cross-entropy over the rows of ``logits`` ([rows, cols] bf16; only the
    first ``vocab`` columns are classes, the rest is alignment padding).  ``logits``
    is consumed: it holds the gradient afterwards.  ``targets`` int64."""
    vocab = logits.shape[1] if vocab is None else vocab
    return _SoftmaxXent.apply(logits, targets.contiguous(), vocab)


_partials = {}


def sq_norm(flat_grad: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[0] += sum(flat_grad**2) (out: 1-element fp32 device tensor).  Two deterministic
    stages (fixed summation order), so every data-parallel rank computes the same bits."""
    lib = _lib.load()
    key = flat_grad.device
    if key not in _partials:
        _partials[key] = torch.empty(1024, dtype=torch.float32, device=flat_grad.device)
    _lib.check(lib.cclx_sq_norm(flat_grad.data_ptr(), flat_grad.numel(), torch_to_ccl(flat_grad.dtype),
                                out.data_ptr(), _partials[key].data_ptr(), _stream_ptr()))
    _bump(2)
    return out


class FlatAdamW:
    """AdamW over one flat parameter buffer.

    ``model_flat`` (bf16) is what the model's parameters are views of; the
    optimizer keeps fp32 master / m / v copies and rewrites ``model_flat`` in
    the same kernel.  Elements ``[0, n_decay)`` receive weight decay.  The
    gradient is read in its own dtype (bf16 buckets are never widened in
    memory).  ``max_norm`` > 0 enables clipping by the global norm, which is
    computed on the device and consumed on the device (no host sync).
    ``device_step=True`` keeps the step number (bias corrections) in a device word that the
    kernel sequence increments itself, which is what a step replayed from a CUDA graph needs.
    """

    def __init__(self, model_flat: torch.Tensor, n_decay: int, lr=3e-4, betas=(0.9, 0.95), eps=1e-8,
                 weight_decay=0.1, max_norm: float = 1.0, device_step: bool = False):
        self.model_flat = model_flat if model_flat.dtype == torch.bfloat16 else None
        self.master = model_flat.detach().to(torch.float32).clone()
        self._fp32_model = model_flat if model_flat.dtype == torch.float32 else None
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.n_decay = int(n_decay)
        self.lr, self.betas, self.eps, self.weight_decay, self.max_norm = lr, betas, eps, weight_decay, max_norm
        self.step_count = 0
        self._norm = torch.zeros(1, dtype=torch.float32, device=model_flat.device)
        self._step_dev = torch.zeros(1, dtype=torch.int32, device=model_flat.device) if device_step else None

    def step(self, flat_grad: torch.Tensor, grad_scale: float = 1.0):
        self.step_count += 1
        lib = _lib.load()
        norm_ptr = 0
        if self.max_norm > 0:
            self._norm.zero_()
            sq_norm(flat_grad, self._norm)
            norm_ptr = self._norm.data_ptr()
        _lib.check(lib.cclx_adamw_flat(
            self.master.data_ptr(), flat_grad.data_ptr(), torch_to_ccl(flat_grad.dtype), self.m.data_ptr(),
            self.v.data_ptr(), 0 if self.model_flat is None else self.model_flat.data_ptr(), self.master.numel(),
            self.n_decay, self.lr, self.betas[0], self.betas[1], self.eps, self.weight_decay, self.step_count,
            grad_scale, self.max_norm, norm_ptr, 0 if self._step_dev is None else self._step_dev.data_ptr(),
            _stream_ptr()))
        _bump(1 if self._step_dev is None else 2)
        if self._fp32_model is not None:
            self._fp32_model.copy_(self.master)

    def grad_norm(self) -> torch.Tensor:
        return self._norm.sqrt()
