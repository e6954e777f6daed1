"""Fused layer pieces for the training path (bf16 activations, fp32 math), each one kernel family of
``csrc/gpu/nn_kernels.cu``:

* ``layer_norm`` / ``add_layer_norm``: LayerNorm whose backward produces the input gradient and the
  weight / bias gradients from one read of the activations; the ``add_`` form also performs the residual
  addition in front of it (and adds the residual branch's gradient inside the backward kernel);
* ``linear``: cuBLAS matmuls with the bias gradient taken by a two-stage column sum;
* ``split_qkv``: views of a packed QKV projection for the attention call, whose backward assembles the
  packed gradient with one strided copy kernel instead of a concatenation.

Shapes the kernels do not cover (LayerNorm width not a multiple of 256 or above 1024, non-bf16, CPU)
fall back to the equivalent PyTorch ops."""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn.functional as F

from .. import _lib
from .device_group import _stream_ptr
from . import train as _train


def _ln_ok(x: torch.Tensor, D: int) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and D % 256 == 0 and 256 <= D <= 1024


class _AddLayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, weight, bias, eps):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        lib = _lib.load()
        if res is not None:
            r2 = res.reshape(-1, D)
            r2 = r2 if r2.is_contiguous() else r2.contiguous()
            total = torch.empty_like(x2)
            _lib.check(lib.cclx_layer_norm_fwd(x2.data_ptr(), r2.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                               y.data_ptr(), total.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, D,
                                               eps, _stream_ptr()))
        else:
            total = x2
            _lib.check(lib.cclx_layer_norm_fwd(x2.data_ptr(), 0, weight.data_ptr(), bias.data_ptr(), y.data_ptr(), 0,
                                               mean.data_ptr(), rstd.data_ptr(), rows, D, eps, _stream_ptr()))
        _train._bump()
        ctx.save_for_backward(total, weight, mean, rstd)
        ctx.has_res = res is not None
        ctx.shape = x.shape
        if res is not None:
            return y.view(x.shape), total.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dsum=None):
        total, weight, mean, rstd = ctx.saved_tensors
        rows, D = total.shape
        lib = _lib.load()
        dy2 = dy.reshape(rows, D)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dres = None
        if ctx.has_res and dsum is not None:
            dres = dsum.reshape(rows, D)
            dres = dres if dres.is_contiguous() else dres.contiguous()
        dx = torch.empty_like(total)
        dgamma = torch.empty_like(weight)
        dbeta = torch.empty_like(weight)
        blocks = lib.cclx_layer_norm_bwd_blocks(rows)
        ws = torch.empty(blocks * 2 * D, dtype=torch.float32, device=total.device)
        _lib.check(lib.cclx_layer_norm_bwd(dy2.data_ptr(), total.data_ptr(), weight.data_ptr(), mean.data_ptr(),
                                           rstd.data_ptr(), 0 if dres is None else dres.data_ptr(), dx.data_ptr(),
                                           dgamma.data_ptr(), dbeta.data_ptr(), ws.data_ptr(), rows, D, _stream_ptr()))
        _train._bump(2)
        dx = dx.view(ctx.shape)
        if ctx.has_res:
            return dx, dx, dgamma, dbeta, None
        return dx, None, dgamma, dbeta, None


def layer_norm(x, weight, bias, eps: float = 1e-5):
    if not _ln_ok(x, x.shape[-1]):
        return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)
    return _AddLayerNorm.apply(x, None, weight, bias, eps)


def add_layer_norm(x, res, weight, bias, eps: float = 1e-5):
    """Returns (LayerNorm(x + res), x + res)."""
    if res is None:
        return layer_norm(x, weight, bias, eps), x
    if not _ln_ok(x, x.shape[-1]):
        s = x + res
        return F.layer_norm(s, (s.shape[-1],), weight, bias, eps), s
    return _AddLayerNorm.apply(x, res, weight, bias, eps)


def colsum(dy2: torch.Tensor) -> torch.Tensor:
    """Sum over the rows of a contiguous [rows, N] bf16 matrix (fp32 accumulation, fixed order)."""
    rows, N = dy2.shape
    out = torch.empty(N, dtype=dy2.dtype, device=dy2.device)
    ws = torch.empty(64 * N, dtype=torch.float32, device=dy2.device)
    key = (dy2.device, torch.cuda.current_stream())
    if key not in _colsum_counters:  # arrival counters per column tile; the kernel leaves them zero
        _colsum_counters[key] = torch.zeros(1024, dtype=torch.int32, device=dy2.device)
    assert N <= 1024 * 256
    _lib.check(_lib.load().cclx_colsum_bf16(dy2.data_ptr(), rows, N, out.data_ptr(), ws.data_ptr(),
                                            _colsum_counters[key].data_ptr(), _stream_ptr()))
    _train._bump()
    return out


_colsum_counters = {}


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, weight, bias)
        ctx.in_shape = x.shape
        return torch.addmm(bias, x2, weight.t()).view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight, bias = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dx = (dy2 @ weight).view(ctx.in_shape) if ctx.needs_input_grad[0] else None
        # A parameter may carry a gradient sink (a view of a flat gradient buffer plus a callback, set by
        # DataParallel): the weight gradient is then accumulated by the GEMM itself (beta = 1) instead of
        # being materialised and added by a separate kernel, and autograd gets no gradient to accumulate.
        wsink = getattr(weight, "_grad_sink", None)
        if wsink is not None:
            wsink[0].addmm_(dy2.t(), x2)
            dw = None
        else:
            dw = dy2.t() @ x2
        bsink = getattr(bias, "_grad_sink", None)
        db = colsum(dy2)
        if bsink is not None:
            bsink[0].add_(db)
            db = None
        if wsink is not None:
            wsink[1](weight)
        if bsink is not None:
            bsink[1](bias)
        return dx, dw, db


def linear(x, weight, bias):
    if bias is None or not (x.is_cuda and x.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0):
        return F.linear(x, weight, bias)
    return _Linear.apply(x, weight, bias)


class _SplitQKV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, n_head):
        B, S, D3 = qkv.shape
        D = D3 // 3
        ctx.dims = (B, S, n_head, D // n_head)
        parts = qkv.view(B, S, 3, n_head, D // n_head).permute(2, 0, 3, 1, 4)  # [3, B, H, S, dh] views
        return parts[0], parts[1], parts[2]

    @staticmethod
    def backward(ctx, dq, dk, dv):
        B, S, H, dh = ctx.dims
        out = torch.empty((B, S, 3, H, dh), dtype=dq.dtype, device=dq.device)
        view = out.permute(2, 0, 3, 1, 4)  # [3, B, H, S, dh]
        srcs = [dq, dk, dv]
        ok = all(g.stride(3) == 1 and g.dtype == torch.bfloat16 for g in srcs) and dh % 8 == 0
        if not ok:
            for i, g in enumerate(srcs):
                view[i].copy_(g)
            return out.view(B, S, 3 * H * dh), None
        strides = []
        for g in srcs:  # gradients are indexed [B, H, S, dh]
            strides += [g.stride(0), g.stride(2), g.stride(1)]
        strides += [view[0].stride(0), view[0].stride(2), view[0].stride(1)]
        arr = (C.c_longlong * 12)(*strides)
        src = _lib.ptr_array([g.data_ptr() for g in srcs])
        dst = _lib.ptr_array([view[i].data_ptr() for i in range(3)])
        _lib.check(_lib.load().cclx_head_copy3(src, dst, arr, B, S, H, dh, _stream_ptr()))
        _train._bump()
        return out.view(B, S, 3 * H * dh), None


def split_qkv(qkv: torch.Tensor, n_head: int):
    """[B, S, 3 * D] -> q, k, v as [B, H, S, D / H] views."""
    if not (qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.is_contiguous()):
        B, S, D3 = qkv.shape
        q, k, v = qkv.view(B, S, 3, n_head, D3 // 3 // n_head).permute(2, 0, 3, 1, 4)
        return q, k, v
    return _SplitQKV.apply(qkv, n_head)
