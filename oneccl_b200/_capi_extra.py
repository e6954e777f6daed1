"""Prototypes of the C API groups added on top of the device-communicator core
(optimizer / model kernels, CPU runtime, communicator).  Kept separate so that
each native translation unit has its Python declaration next to the others."""
import ctypes as C

vp, sz, i, f = C.c_void_p, C.c_size_t, C.c_int, C.c_float
fp = C.POINTER(C.c_float)
PROTOTYPES = {
    "cclx_sq_norm": (i, [vp, sz, i, vp, vp]),
    "cclx_adamw_flat": (i, [vp, vp, i, vp, vp, vp, sz, sz, f, f, f, f, f, i, f, f, vp, vp]),
    "cclx_softmax_xent": (i, [vp, vp, vp, sz, i, sz, f, i, vp]),
}
