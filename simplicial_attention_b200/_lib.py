"""ctypes binding of ``libsa2.so`` (C ABI declared in ``include/sa2.h``).

The shared library is the product: if it is missing and cannot be built, or it
does not load, importing this module's ``lib()`` raises.  There is no CPU or
PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

SA2_OK = 0
SA2_F32, SA2_BF16 = 0, 1
KERNEL_AUTO, KERNEL_SIMT, KERNEL_TCGEN05 = 0, 1, 2
KERNELS = {"auto": KERNEL_AUTO, "simt": KERNEL_SIMT, "tcgen05": KERNEL_TCGEN05}
BWD_ROWSUM, BWD_K1, BWD_Q = 1, 2, 4     # sa2_bwd_phase

# symbols declared in include/sa2.h
EXPORTS = ("sa2_fwd", "sa2_bwd", "sa2_bwd_workspace_bytes", "sa2_strerror", "sa2_version",
           "sa2_kernel_launches", "sa2_device_status", "sa2_check_device", "sa2_selftest_wait",
           "sa2_bwd_static_scratch",
           "sa2_headnorm_fwd", "sa2_headnorm_bwd", "sa2_headnorm_partial_bytes")
STATIC_SCRATCH_ROWS = 262144   # SA2_STATIC_SCRATCH_ROWS in include/sa2.h
SELFTEST_WAIT_BIT = 0x10000    # SA2_SELFTEST_WAIT_BIT
SA2_ERR_DEVICE = 5


class Strides(C.Structure):
    _fields_ = [("batch", C.c_int64), ("seq", C.c_int64), ("head", C.c_int64)]


class Shape(C.Structure):
    _fields_ = [
        ("b", C.c_int32), ("n", C.c_int32), ("hq", C.c_int32), ("hk", C.c_int32), ("d", C.c_int32),
        ("w1", C.c_int32), ("w2", C.c_int32), ("off1", C.c_int32), ("off2", C.c_int32),
        ("dtype", C.c_int32), ("kernel", C.c_int32), ("scale", C.c_float),
    ]


class FwdArgs(C.Structure):
    _fields_ = [
        ("shape", Shape),
        ("q", C.c_void_p), ("k1", C.c_void_p), ("k2", C.c_void_p), ("v1", C.c_void_p), ("v2", C.c_void_p),
        ("out", C.c_void_p), ("lse", C.c_void_p),
        ("sq", Strides), ("sk1", Strides), ("sk2", Strides), ("sv1", Strides), ("sv2", Strides), ("sout", Strides),
        ("stream", C.c_void_p),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("shape", Shape),
        ("q", C.c_void_p), ("k1", C.c_void_p), ("k2", C.c_void_p), ("v1", C.c_void_p), ("v2", C.c_void_p),
        ("out", C.c_void_p), ("dout", C.c_void_p), ("lse", C.c_void_p),
        ("dq", C.c_void_p), ("dk1", C.c_void_p), ("dv1", C.c_void_p), ("dk2", C.c_void_p), ("dv2", C.c_void_p),
        ("sq", Strides), ("sk1", Strides), ("sk2", Strides), ("sv1", Strides), ("sv2", Strides),
        ("sout", Strides), ("sdout", Strides), ("sdq", Strides),
        ("sdk1", Strides), ("sdk2", Strides), ("sdv1", Strides), ("sdv2", Strides),
        ("grad_dtype", C.c_int32), ("phases", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("stream", C.c_void_p),
    ]


class HeadnormArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("dy", C.c_void_p), ("weight", C.c_void_p), ("y", C.c_void_p), ("rstd", C.c_void_p),
        ("dweight", C.c_void_p), ("partial", C.c_void_p), ("partial_bytes", C.c_size_t),
        ("rows", C.c_int64), ("x_stride", C.c_int64), ("y_stride", C.c_int64), ("dy_stride", C.c_int64),
        ("channels", C.c_int32), ("d", C.c_int32), ("x_dtype", C.c_int32), ("y_dtype", C.c_int32),
        ("eps", C.c_float), ("stream", C.c_void_p),
    ]


_lock = threading.Lock()
_lib = None


def lib_path() -> str:
    """``SA2_LIBRARY`` names another build of the library (for example a diagnostic build with wait accounting)."""
    return os.environ.get("SA2_LIBRARY") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libsa2.so")


def lib() -> C.CDLL:
    """Load (building first if the sources are newer) and return the library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        from . import build
        if not os.environ.get("SA2_LIBRARY") and (os.environ.get("SA2_REBUILD") or build.is_stale()):
            build.build(force=bool(os.environ.get("SA2_REBUILD")))
        handle = C.CDLL(path)
        handle.sa2_fwd.argtypes = [C.POINTER(FwdArgs)]
        handle.sa2_fwd.restype = C.c_int
        handle.sa2_bwd.argtypes = [C.POINTER(BwdArgs)]
        handle.sa2_bwd.restype = C.c_int
        handle.sa2_bwd_static_scratch.argtypes = [C.POINTER(BwdArgs)]
        handle.sa2_bwd_static_scratch.restype = C.c_int
        handle.sa2_bwd_workspace_bytes.argtypes = [C.POINTER(Shape)]
        handle.sa2_bwd_workspace_bytes.restype = C.c_size_t
        handle.sa2_kernel_launches.argtypes = [C.POINTER(Shape), C.c_int]
        handle.sa2_kernel_launches.restype = C.c_int
        handle.sa2_device_status.argtypes = [C.c_int]
        handle.sa2_device_status.restype = C.c_int
        handle.sa2_selftest_wait.argtypes = [C.c_longlong, C.c_void_p]
        handle.sa2_selftest_wait.restype = C.c_int
        handle.sa2_check_device.argtypes = [C.c_int]
        handle.sa2_check_device.restype = C.c_int
        handle.sa2_strerror.argtypes = [C.c_int]
        handle.sa2_strerror.restype = C.c_char_p
        handle.sa2_headnorm_fwd.argtypes = [C.POINTER(HeadnormArgs)]
        handle.sa2_headnorm_fwd.restype = C.c_int
        handle.sa2_headnorm_bwd.argtypes = [C.POINTER(HeadnormArgs)]
        handle.sa2_headnorm_bwd.restype = C.c_int
        handle.sa2_headnorm_partial_bytes.argtypes = [C.c_int64, C.c_int32]
        handle.sa2_headnorm_partial_bytes.restype = C.c_size_t
        handle.sa2_version.argtypes = []
        handle.sa2_version.restype = C.c_int
        _lib = handle
    return _lib


class Sa2Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().sa2_strerror(status).decode()
        super().__init__(f"{where} failed with status {status}: {msg}")


def check(status: int, where: str) -> None:
    if status != SA2_OK:
        raise Sa2Error(status, where)
