"""Datatype and reduction codes shared with the native library (values of
``cclx::datatype_t`` / ``cclx::reduction_t``, which are the public
``ccl::datatype`` / ``ccl::reduction`` values)."""
from __future__ import annotations

INT8, UINT8, INT16, UINT16, INT32, UINT32, INT64, UINT64, FLOAT16, FLOAT32, FLOAT64, BFLOAT16 = range(12)
SUM, PROD, MIN, MAX, CUSTOM = range(5)

COLL = {
    "allgather": 0, "allgatherv": 1, "allreduce": 2, "alltoall": 3, "alltoallv": 4, "barrier": 5,
    "bcast": 6, "broadcast": 7, "reduce": 8, "reduce_scatter": 9, "recv": 10, "send": 11,
}
GPU_ALGO = {"auto": 0, "oneshot": 1, "twoshot": 2, "symm": 3, "nvls": 4, "nvls_oneshot": 5,
            "push": 6, "pull": 7, "copy": 8, "pipelined": 9, "ce": 10}


_TORCH_TABLE = None


def torch_to_ccl(dtype) -> int:
    global _TORCH_TABLE
    if _TORCH_TABLE is None:  # built once: this sits on the launch path of every collective
        import torch

        table = {
            torch.int8: INT8, torch.uint8: UINT8, torch.int16: INT16, torch.int32: INT32, torch.int64: INT64,
            torch.float16: FLOAT16, torch.float32: FLOAT32, torch.float64: FLOAT64, torch.bfloat16: BFLOAT16,
            torch.bool: UINT8,
        }
        for name, code in (("uint16", UINT16), ("uint32", UINT32), ("uint64", UINT64)):
            if hasattr(torch, name):
                table[getattr(torch, name)] = code
        _TORCH_TABLE = table
    try:
        return _TORCH_TABLE[dtype]
    except KeyError:
        raise TypeError(f"{dtype} has no ccl datatype") from None


_OPS = {"sum": SUM, "prod": PROD, "product": PROD, "min": MIN, "max": MAX, "avg": SUM}


def reduce_op_code(op) -> int:
    if isinstance(op, int):
        return op
    code = _OPS.get(op) if isinstance(op, str) else None
    if code is not None:
        return code
    name = str(op).lower().split(".")[-1]
    if name not in _OPS:
        raise ValueError(f"unsupported reduction {op}")
    return _OPS[name]
