"""tcgen05 GEMM entry points: plain (single GPU) and fused with a collective.

``gemm_bf16(a, w)`` computes ``a @ w.T`` for bf16 ``a [M,K]`` and ``w [N,K]``
(the layout of ``nn.Linear.weight``) with the hand-written sm_100a kernel.

``FusedPlan`` owns the symmetric buffers of one fused operator:

* mode ``"ag_gemm"``: every rank writes its row shard of X into ``x_shard`` and
  ``run`` returns ``act(allgather(X) @ w.T)``;
* mode ``"gemm_rs"``: ``run(a, w)`` returns this rank's rows of
  ``reduce_scatter(a @ w.T)``.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from .device_group import DeviceGroup, _stream_ptr

EPILOGUE = {None: 0, "none": 0, "silu": 1}
_err_words = {}


def _err_buffer(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    if key not in _err_words:
        _err_words[key] = torch.zeros(4, dtype=torch.int32, device=device)
    return _err_words[key]


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, epilogue=None, ctas: int = 0,
              check: bool = False, kernel: str = "auto", rows: torch.Tensor | None = None) -> torch.Tensor:
    """``kernel``: "auto" (the library decides), "1sm" (one CTA per 128 x 256 tile) or "2sm" (CTA pairs,
    tcgen05 cta_group::2, 256 x 256 tiles; ``ctas`` then counts CTAs, two per pair).  ``rows``: an int32
    device tensor whose first element says how many of ``a``'s rows to multiply (read by the kernel, so the
    host never learns it; the other rows of ``out`` stay as they are)."""
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.is_cuda and w.is_cuda
    assert a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1]
    a = a.contiguous()
    w = w.contiguous()
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    err = _err_buffer(a.device)
    lib = _lib.load()
    if rows is not None:
        assert rows.dtype == torch.int32 and rows.is_cuda
        _lib.check(lib.cclx_gemm_bf16_rows(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, EPILOGUE[epilogue],
                                           rows.data_ptr(), err.data_ptr(), _stream_ptr()))
    elif kernel == "2sm":
        _lib.check(lib.cclx_gemm_bf16_2sm(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, EPILOGUE[epilogue],
                                          ctas // 2, err.data_ptr(), _stream_ptr()))
    else:
        _lib.check(lib.cclx_gemm_bf16(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, EPILOGUE[epilogue],
                                      -(ctas + 1) if kernel == "1sm" else ctas, err.data_ptr(), _stream_ptr()))
    if check:
        code = int(err[0].item())
        if code != 0:
            vals = err.tolist()
            err.zero_()
            raise _lib.CclError(f"tcgen05 GEMM reported error {vals}")
    return out


class FusedPlan:
    MODES = {"ag_gemm": 1, "gemm_rs": 2}

    def __init__(self, group: DeviceGroup, mode: str, M: int, N: int, K: int, epilogue=None, n_comm: int = 0,
                 ctas: int = 0):
        self.group = group
        self.mode = mode
        self.M, self.N, self.K = M, N, K
        self._lib = _lib.load()
        h = self._lib.cclx_fused_plan_create(group.handle, self.MODES[mode], M, N, K, EPILOGUE[epilogue], n_comm, ctas)
        if not h:
            raise _lib.CclError(self._lib.cclx_last_error().decode())
        self._h = C.c_void_p(h)
        self.rows_per_rank = M // group.world

    def close(self):
        if self._h:
            self._lib.cclx_fused_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _view(self, ptr, rows):
        from .device_group import _SymmStorage

        nbytes = rows * self.K * 2
        t = torch.as_tensor(_SymmStorage(ptr, nbytes, self), device="cuda").view(torch.bfloat16)
        return t.view(rows, self.K)

    def x_shard(self, r: int = 0) -> torch.Tensor:
        """ag_gemm: [M/world, K] slot where (emulated) rank r writes its shard of X."""
        assert self.mode == "ag_gemm"
        return self._view(self._lib.cclx_fused_plan_x_shard(self._h, r), self.rows_per_rank)

    def x_full(self, r: int = 0) -> torch.Tensor:
        assert self.mode == "ag_gemm"
        return self._view(self._lib.cclx_fused_plan_x_full(self._h, r), self.M)

    def run(self, a, w, out=None):
        g = self.group
        n = g.n_entries
        ws = w if isinstance(w, (list, tuple)) else [w]
        As = a if isinstance(a, (list, tuple)) else [a] * n
        rows_out = self.M if self.mode == "ag_gemm" else self.rows_per_rank
        if out is None:
            out = [torch.empty((rows_out, self.N), dtype=torch.bfloat16, device="cuda") for _ in range(n)]
            outs = out
        else:
            outs = out if isinstance(out, (list, tuple)) else [out]
        ap = _lib.ptr_array([0 if (x is None or self.mode == "ag_gemm") else x.data_ptr() for x in As])
        _lib.check(self._lib.cclx_fused_plan_run(self._h, ap, _lib.ptr_array([x.data_ptr() for x in ws]),
                                                 _lib.ptr_array([x.data_ptr() for x in outs]), _stream_ptr()))
        return outs if g.emulated_mode else outs[0]

    def error(self, r: int = 0) -> int:
        return self._lib.cclx_fused_plan_error(self._h, r)
