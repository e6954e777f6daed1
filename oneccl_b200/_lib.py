"""ctypes loader of ``libccl_b200.so`` and typed prototypes of its flat C API.

The library is built in-tree by ``oneccl_b200._build`` and must be present on
a GPU machine: ``load()`` raises if it is missing instead of falling back to a
PyTorch implementation, so that a silent eager fallback can not be mistaken
for the native path.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB = None
LIBDIR = Path(__file__).resolve().parent / "lib"
LIBPATH = LIBDIR / "libccl_b200.so"


class CclError(RuntimeError):
    pass


def _proto(lib):
    vp, sz, i, f = C.c_void_p, C.c_size_t, C.c_int, C.c_float
    pp = C.POINTER(C.c_void_p)
    psz = C.POINTER(C.c_size_t)
    pi = C.POINTER(C.c_int)
    P = {
        "cclx_last_error": (C.c_char_p, []),
        "cclx_env_reload": (i, []),
        "cclx_cuda_device_count": (i, []),
        "cclx_set_device": (i, [i]),
        "cclx_emu_create": (vp, [i, sz, sz]),
        "cclx_dc_destroy": (i, [vp]),
        "cclx_dc_world": (i, [vp]),
        "cclx_dc_rank": (i, [vp]),
        "cclx_dc_nvls": (i, [vp]),
        "cclx_dc_staging_bytes": (sz, [vp]),
        "cclx_dc_status": (i, [vp, i]),
        "cclx_dc_check": (i, [vp]),
        "cclx_dc_clear_status": (i, [vp]),
        "cclx_dc_abort": (i, [vp]),
        "cclx_dc_set_timeout_ms": (i, [vp, sz]),
        "cclx_dc_test_sig_skew": (i, [vp, i]),
        "cclx_dc_algo_hits": (C.c_ulonglong, [vp, i, i]),
        "cclx_gpu_algo_from_name": (i, [C.c_char_p]),
        "cclx_dc_symm_alloc": (sz, [vp, sz]),
        "cclx_dc_symm_free": (i, [vp, sz]),
        "cclx_dc_heap_base": (vp, [vp, i]),
        "cclx_dc_mc_base": (vp, [vp]),
        "cclx_dc_allreduce": (i, [vp, pp, pp, sz, i, i, i, i, i, f, i, vp]),
        "cclx_dc_reduce_scatter": (i, [vp, pp, pp, sz, i, i, i, i, i, f, i, vp]),
        "cclx_dc_reduce": (i, [vp, pp, pp, sz, i, i, i, i, i, f, i, vp]),
        "cclx_dc_allgatherv": (i, [vp, pp, pp, psz, psz, i, i, vp]),
        "cclx_dc_alltoallv": (i, [vp, pp, pp, psz, i, vp]),
        "cclx_dc_register": (i, [vp, pp, psz]),
        "cclx_dc_deregister": (i, [vp, i]),
        "cclx_dc_alltoall": (i, [vp, pp, pp, sz, i, i, vp]),
        "cclx_dc_broadcast": (i, [vp, pp, pp, sz, i, i, vp]),
        "cclx_dc_barrier": (i, [vp, vp]),
        "cclx_dc_sendrecv": (i, [vp, pp, pp, psz, pi, pi, i, vp]),
        "cclx_dc_wait_unset_flag": (i, [vp, vp]),
        "cclx_reduce_local": (i, [vp, vp, sz, i, i, vp]),
        "cclx_dc_allreduce_fused": (i, [vp, pp, pp, psz, i, i, i, f, i, vp]),
        "cclx_dc_fused_batches": (C.c_ulonglong, [vp]),
        "cclx_transpose_blocks": (i, [vp, vp, i, i, sz, vp]),
        "cclx_gemm_bf16": (i, [vp, vp, vp, i, i, i, i, i, vp, vp]),
        "cclx_gemm_bf16_2sm": (i, [vp, vp, vp, i, i, i, i, i, vp, vp]),
        "cclx_gemm_bf16_rows": (i, [vp, vp, vp, i, i, i, i, vp, vp, vp]),
        "cclx_fused_plan_create": (vp, [vp, i, i, i, i, i, i, i]),
        "cclx_fused_plan_destroy": (i, [vp]),
        "cclx_fused_plan_x_shard": (vp, [vp, i]),
        "cclx_fused_plan_x_full": (vp, [vp, i]),
        "cclx_fused_plan_run": (i, [vp, pp, pp, pp, vp]),
        "cclx_fused_plan_error": (i, [vp, i]),
    }
    for name, (res, args) in P.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.restype = res
        fn.argtypes = args
    return lib


def _declare_optional(lib, table):
    for name, (res, args) in table.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.restype = res
            fn.argtypes = args


def load():
    """Return the loaded library (building nothing: see ``oneccl_b200._build``)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    override = os.environ.get("CCL_B200_LIBRARY")  # e.g. an instrumented build (see _build.build_native)
    if override:
        _LIB = _proto(C.CDLL(override, mode=C.RTLD_GLOBAL))
        from . import _capi_extra

        _declare_optional(_LIB, _capi_extra.PROTOTYPES)
        return _LIB
    if not LIBPATH.exists():
        if os.environ.get("CCL_B200_AUTOBUILD", "1") == "1":
            from . import _build

            _build.build_native()
        if not LIBPATH.exists():
            raise CclError(f"{LIBPATH} is missing: run `python -m oneccl_b200._build`")
    _LIB = _proto(C.CDLL(str(LIBPATH), mode=C.RTLD_GLOBAL))
    from . import _capi_extra

    _declare_optional(_LIB, _capi_extra.PROTOTYPES)
    return _LIB


def check(rc: int):
    if rc != 0:
        raise CclError(load().cclx_last_error().decode(errors="replace"))


_VOIDP_ARRAYS = {}


def ptr_array(ptrs):
    n = len(ptrs)
    t = _VOIDP_ARRAYS.get(n)
    if t is None:  # ctypes array types are costly to create: one per length
        t = _VOIDP_ARRAYS[n] = C.c_void_p * n
    return t(*ptrs)


def size_array(vals):
    arr = (C.c_size_t * len(vals))()
    for k, v in enumerate(vals):
        arr[k] = int(v)
    return arr


def int_array(vals):
    arr = (C.c_int * len(vals))()
    for k, v in enumerate(vals):
        arr[k] = int(v)
    return arr
