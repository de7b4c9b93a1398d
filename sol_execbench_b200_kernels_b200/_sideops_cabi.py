"""ctypes binding of libsideops.so (C ABI: include/sideops.h).  No fallback: importing this module without
the built library raises."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int64, c_uint64, c_void_p
from . import build as _build

SO_OK, SO_EINVAL_NULL, SO_EINVAL_SHAPE, SO_EINVAL_ALIGN, SO_ECUDA, SO_EDEVICE, SO_ETIMEOUT, SO_EBOUNDS = (
    0, -1, -2, -3, -4, -5, -6, -7)

EXPORTS = ("so_version", "so_error_string", "so_rmsnorm_qk", "so_mamba_conv1d_tail", "so_mamba_in_proj", "so_last_status",
           "so_is_range_checked_build", "so_set_wait_limit_ns", "so_launch_count")


class SideOpsError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libsideops: {message} (code {code})")
        self.code = code


def _load() -> ctypes.CDLL:
    LIB_PATH = _build.SIDE_LIB_PATH  # (a study or debug build can be bound by setting this before the first import)
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python -m sol_execbench_b200_kernels_b200.build` "
            "(needs nvcc); this package has no other implementation to fall back to.")
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.so_version.restype = c_int
    lib.so_error_string.restype = c_char_p
    lib.so_error_string.argtypes = [c_int]
    lib.so_rmsnorm_qk.restype = c_int
    lib.so_rmsnorm_qk.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int64, c_int,
                                  c_void_p]
    lib.so_mamba_conv1d_tail.restype = c_int
    lib.so_mamba_conv1d_tail.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                         c_int64, c_void_p]
    lib.so_mamba_in_proj.restype = c_int
    lib.so_mamba_in_proj.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]
    lib.so_last_status.restype = c_int
    lib.so_last_status.argtypes = [POINTER(c_int), c_int]
    lib.so_is_range_checked_build.restype = c_int
    lib.so_set_wait_limit_ns.restype = c_int
    lib.so_set_wait_limit_ns.argtypes = [c_uint64]
    lib.so_launch_count.restype = c_int64
    return lib


lib = _load()


def error_string(code: int) -> str:
    return lib.so_error_string(code).decode()


def check(code: int) -> None:
    if code == SO_OK:
        return
    if code in (SO_EINVAL_NULL, SO_EINVAL_SHAPE, SO_EINVAL_ALIGN):
        raise ValueError(f"libsideops: {error_string(code)} (code {code})")
    raise SideOpsError(code, error_string(code))
