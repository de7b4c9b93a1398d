"""ctypes binding of libgateup.so (declarations in include/gateup.h).

There is no fallback of any kind: if the library has not been built, importing
this module raises, and every entry point that computes needs a B200.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_int, c_int32, c_int64, c_size_t, c_void_p

from .build import LIB_PATH

GU_OK = 0
GU_EINVAL_NULL = -1
GU_EINVAL_SHAPE = -2
GU_EINVAL_ALIGN = -3
GU_EINVAL_PLAN = -4
GU_EWORKSPACE = -5
GU_ECUDA = -6
GU_EDEVICE = -7
GU_ETIMEOUT = -8
GU_ESTATIC_LIMIT = -9
GU_EBOUNDS = -10

PLAN_AUTO, PLAN_TILE, PLAN_STREAM, PLAN_TILE_DP, PLAN_TILE_SK, PLAN_TILE_PAIR, PLAN_TILE_PAIR_SK = 0, 1, 2, 3, 4, 5, 6
OP_GATEUP, OP_GATEUP_FP8, OP_GEMM = 0, 1, 2
PLAN_NAMES = {PLAN_AUTO: "auto", PLAN_TILE: "tile", PLAN_STREAM: "stream", PLAN_TILE_DP: "tile_dp",
              PLAN_TILE_SK: "tile_sk", PLAN_TILE_PAIR: "tile_pair", PLAN_TILE_PAIR_SK: "tile_pair_sk"}

EXPORTS = (
    "gu_version", "gu_error_string", "gu_select_plan", "gu_select_tile_kernel", "gu_workspace_bytes", "gu_workspace_init",
    "gu_run", "gu_run_concat", "gu_last_status", "gu_launch_count", "gu_run_decode_static", "gu_run_gather", "gu_quantize_activation", "gu_blockwise_gemm", "gu_run_fp8out",
    "gu_blockwise_gemm_scatter", "gu_reduce_gather", "gu_set_wait_limit_ns", "gu_trace_read", "gu_wait_probe", "gu_peer_barrier", "gu_is_range_checked_build",
)


class GuProblem(Structure):
    _fields_ = [
        ("x", c_void_p), ("scale_x", c_void_p),
        ("gate_w", c_void_p), ("scale_gate", c_void_p),
        ("up_w", c_void_p), ("scale_up", c_void_p),
        ("output", c_void_p),
        ("m", c_int64), ("k", c_int64), ("n", c_int64),
        ("ld_output", c_int64),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("plan", c_int32), ("reserved", c_int32),
    ]


class GateUpError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libgateup: {message} (code {code})")
        self.code = code


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python -m sol_execbench_b200_kernels_b200.build` "
            "(needs nvcc); this package has no other implementation to fall back to.")
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.gu_version.restype = c_int
    lib.gu_error_string.restype = c_char_p
    lib.gu_error_string.argtypes = [c_int]
    lib.gu_select_plan.restype = c_int
    lib.gu_select_plan.argtypes = [c_int64, c_int64, c_int64]
    lib.gu_select_tile_kernel.restype = c_int
    lib.gu_select_tile_kernel.argtypes = [c_int, c_int64, c_int64, c_int64, c_int]
    lib.gu_workspace_bytes.restype = c_size_t
    lib.gu_workspace_bytes.argtypes = [c_int64, c_int64, c_int64, c_int]
    lib.gu_workspace_init.restype = c_int
    lib.gu_workspace_init.argtypes = [c_void_p, c_size_t, c_void_p]
    lib.gu_run.restype = c_int
    lib.gu_run.argtypes = [POINTER(GuProblem), c_void_p]
    lib.gu_run_concat.restype = c_int
    lib.gu_run_concat.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                  c_int64, c_void_p, c_size_t, c_int, c_void_p]
    lib.gu_run_decode_static.restype = c_int
    lib.gu_run_decode_static.argtypes = [POINTER(GuProblem), c_void_p]
    lib.gu_run_gather.restype = c_int
    lib.gu_run_gather.argtypes = [POINTER(GuProblem), POINTER(c_void_p), c_int, c_int, c_int64, c_void_p]
    lib.gu_quantize_activation.restype = c_int
    lib.gu_quantize_activation.argtypes = [c_void_p, c_int, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p]
    lib.gu_blockwise_gemm.restype = c_int
    lib.gu_blockwise_gemm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                      c_int64, c_void_p]
    lib.gu_blockwise_gemm_scatter.restype = c_int
    lib.gu_blockwise_gemm_scatter.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, POINTER(c_void_p), c_int, c_int,
                                              c_int64, c_int64, c_int64, c_void_p]
    lib.gu_reduce_gather.restype = c_int
    lib.gu_reduce_gather.argtypes = [c_void_p, POINTER(c_void_p), c_int, c_int, c_int64, c_int64, c_void_p]
    lib.gu_run_fp8out.restype = c_int
    lib.gu_run_fp8out.argtypes = [POINTER(GuProblem), c_void_p, c_void_p, c_void_p]
    lib.gu_last_status.restype = c_int
    lib.gu_last_status.argtypes = [POINTER(c_int), c_int]
    lib.gu_launch_count.restype = c_int64
    lib.gu_set_wait_limit_ns.restype = c_int
    lib.gu_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
    lib.gu_peer_barrier.restype = c_int
    lib.gu_peer_barrier.argtypes = [POINTER(c_void_p), c_int, c_int, ctypes.c_uint64, c_void_p]
    lib.gu_is_range_checked_build.restype = c_int
    lib.gu_wait_probe.restype = c_int
    lib.gu_wait_probe.argtypes = [c_void_p]
    lib.gu_trace_read.restype = c_int
    lib.gu_trace_read.argtypes = [POINTER(ctypes.c_uint64), c_int, c_int]
    return lib


lib = _load()


def error_string(code: int) -> str:
    return lib.gu_error_string(code).decode()


def check(code: int) -> None:
    if code != GU_OK:
        raise GateUpError(code, error_string(code))
