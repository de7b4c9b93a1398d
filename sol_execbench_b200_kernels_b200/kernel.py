"""Drop-in entry point for the FP8 gate/up projection with fused SwiGLU.

``run`` has the signature, tensor layouts, destination-passing style and stream
behaviour of the reference submission's entry point
(kernels/179_fp8_mlp_gate_up_projection/kernel.py:398-407 and
solution.json:14,20): seven positional tensors, the last one written in place,
launched on torch's current CUDA stream.  Where the reference launches two
block-scaled GEMMs and an elementwise SwiGLU kernel (kernel.py:487-503), this
makes one call into libgateup.so, which launches one fused sm_100a kernel.

PyTorch is used for device memory, streams and nothing else.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from . import _cabi
from ._cabi import (PLAN_AUTO, PLAN_STREAM, PLAN_TILE, PLAN_TILE_DP, PLAN_TILE_PAIR, PLAN_TILE_PAIR_SK, PLAN_TILE_SK,
                    GuProblem)

BLOCK = 128
_PLANS = {"auto": PLAN_AUTO, "tile": PLAN_TILE, "stream": PLAN_STREAM, "tile_dp": PLAN_TILE_DP, "tile_sk": PLAN_TILE_SK,
          "tile_pair": PLAN_TILE_PAIR, "tile_pair_sk": PLAN_TILE_PAIR_SK}

# Scratch for the stream-K hand-off, one buffer per (device, stream): it is
# written and consumed inside a single call and carries no result across calls.
_WORKSPACES: Dict[Tuple[int, int], torch.Tensor] = {}


def select_plan(m: int, k: int, n: int) -> str:
    """Name of the kernel the heuristic picks for a shape ('tile' or 'stream').

    Counterpart of the reference's `_select_config` (kernel.py:232-249), which has
    no small-M branch; here decode-sized M on large weights streams them with stream-K.
    """
    code = _cabi.lib.gu_select_plan(m, k, n)
    _cabi.check(min(code, 0))
    return _cabi.PLAN_NAMES[code]


def _raise_for(code: int) -> None:
    """0 returns; a contract violation the library found itself becomes ValueError, like the Python-side checks; any
    other code (workspace, CUDA, device, time-out) GateUpError."""
    if code == _cabi.GU_OK:
        return
    if code in (_cabi.GU_EINVAL_NULL, _cabi.GU_EINVAL_SHAPE, _cabi.GU_EINVAL_ALIGN, _cabi.GU_EINVAL_PLAN):
        raise ValueError(f"libgateup: {_cabi.error_string(code)} (code {code})")
    raise _cabi.GateUpError(code, _cabi.error_string(code))


def _expected_inputs(x, scale_x, gate_w, scale_gate, up_w, scale_up, m_expected=None, n_expected=None):
    """(m, k, n) and the contract's (tensor, shape, dtype) per input name; raises on an unsupported M, K, N."""
    if x.dim() != 2 or gate_w.dim() != 2 or up_w.dim() != 2:
        raise ValueError("x, gate_proj_weight and up_proj_weight must be 2-D")
    m, k = x.shape
    n = gate_w.shape[0]
    if m < 1 or k % BLOCK or n % BLOCK or k < BLOCK or n < BLOCK:
        raise ValueError(f"Unsupported contract shape M={m}, K={k}, N={n}: need M >= 1 and K, N multiples of {BLOCK}")
    if (m_expected is not None and m != m_expected) or (n_expected is not None and n != n_expected):
        raise ValueError(f"Unsupported contract shape M={m}, N={n}: expected M={m_expected}, N={n_expected}")
    kb, nb = k // BLOCK, n // BLOCK
    return (m, k, n), {
        "x": (x, (m, k), torch.float8_e4m3fn),
        "scale_x": (scale_x, (m, kb), torch.float32),
        "gate_proj_weight": (gate_w, (n, k), torch.float8_e4m3fn),
        "scale_gate": (scale_gate, (nb, kb), torch.float32),
        "up_proj_weight": (up_w, (n, k), torch.float8_e4m3fn),
        "scale_up": (scale_up, (nb, kb), torch.float32),
    }


def _check(expected, device) -> None:
    """Same checks as the reference's `_debug_validate` / pybind `run` (kernel.py:345-395,
    variants/cuda_cpp_v4/binding.cpp:26-72): shapes and dtypes first, then device and layout; always on."""
    for name, (t, shape, dtype) in expected.items():
        if tuple(t.shape) != shape or t.dtype != dtype:
            raise ValueError(f"{name}: expected shape={shape}, dtype={dtype}; "
                             f"got shape={tuple(t.shape)}, dtype={t.dtype}")
    for name, (t, shape, dtype) in expected.items():
        if not t.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor (this package has no CPU path)")
        if t.device != device:
            raise ValueError(f"{name} is on {t.device}, x is on {device}")
        if name != "output" and not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")


def _validate_inputs_only(x, scale_x, gate_w, scale_gate, up_w, scale_up, m_expected=None, n_expected=None):
    (m, k, n), expected = _expected_inputs(x, scale_x, gate_w, scale_gate, up_w, scale_up, m_expected, n_expected)
    _check(expected, x.device)
    return m, k, n


def _validate(x, scale_x, gate_w, scale_gate, up_w, scale_up, output) -> Tuple[int, int, int]:
    """Inputs plus the destination: bf16 [M, N] on the same device, row-major with unit column stride."""
    if output.dim() != 2:
        raise ValueError("output must be 2-D")
    (m, k, n), expected = _expected_inputs(x, scale_x, gate_w, scale_gate, up_w, scale_up)
    expected["output"] = (output, (m, n), torch.bfloat16)
    _check(expected, x.device)
    # output may be a column slice of a wider row-major buffer (sharded writes)
    if output.stride(1) != 1 or output.stride(0) < n:
        raise ValueError("output must be row-major with unit column stride")
    return m, k, n


def _workspace(device: torch.device, stream_ptr: int, nbytes: int) -> Optional[torch.Tensor]:
    if nbytes == 0:
        return None
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_ptr)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        # Under stream capture (torch.cuda.graph switches to a stream of its own, which no eager call has used) the
        # scratch comes from the graph's memory pool and its initialisation is recorded with the launch: every replay
        # then starts from zeroed flags and a zero epoch counter, which is a valid state for the kernels.  The tensor
        # kept here holds the pool's block alive for later calls on that stream.
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _cabi.check(_cabi.lib.gu_workspace_init(ws.data_ptr(), nbytes, stream_ptr))
        _WORKSPACES[key] = ws
    return ws


def _launch(x, scale_x, gate_w, scale_gate, up_w, scale_up, output, plan: str, whole_tiles: bool = False) -> None:
    m, k, n = _validate(x, scale_x, gate_w, scale_gate, up_w, scale_up, output)
    plan_id = _PLANS[plan]
    with torch.cuda.device(x.device):
        stream_ptr = torch.cuda.current_stream(x.device).cuda_stream
        nbytes = _cabi.lib.gu_workspace_bytes(m, k, n, plan_id)
        if whole_tiles and (plan_id == PLAN_TILE or (plan_id == PLAN_AUTO and _cabi.lib.gu_select_plan(m, k, n) == PLAN_TILE)):
            nbytes = 0  # the tile plan without scratch never cuts a tile along K
        ws = _workspace(x.device, stream_ptr, nbytes)
        pr = GuProblem(
            x.data_ptr(), scale_x.data_ptr(), gate_w.data_ptr(), scale_gate.data_ptr(),
            up_w.data_ptr(), scale_up.data_ptr(), output.data_ptr(),
            m, k, n, output.stride(0),
            ws.data_ptr() if ws is not None else None, nbytes, plan_id, 0)
        code = _cabi.lib.gu_run(ctypes.byref(pr), stream_ptr)
    _raise_for(code)


@torch.no_grad()
def run(x: torch.Tensor, scale_x: torch.Tensor, gate_proj_weight: torch.Tensor, scale_gate: torch.Tensor,
        up_proj_weight: torch.Tensor, scale_up: torch.Tensor, output: torch.Tensor) -> None:
    """output[M, N] (bf16) = SiLU(x @ gate^T) * (x @ up^T) with block-scaled e4m3 operands.

    Same arguments as the reference `run` (kernel.py:398-407).  Raises ValueError
    for a shape, dtype, device or layout outside the contract.
    """
    _launch(x, scale_x, gate_proj_weight, scale_gate, up_proj_weight, scale_up, output, "auto")


@torch.no_grad()
def run_with_plan(x, scale_x, gate_proj_weight, scale_gate, up_proj_weight, scale_up, output, plan: str,
                  whole_tiles: bool = False) -> None:
    """`run` with the kernel forced: 'auto', 'tile' (kernel and schedule by heuristic), 'tile_pair' / 'tile_pair_sk'
    (CTA-pair kernel, whole tiles / stream-K schedule), 'tile_dp' / 'tile_sk' (lone-CTA kernel, likewise) or 'stream'.

    `whole_tiles=True` keeps the tile plan from cutting any tile along K (it is given no scratch, and then runs its
    data-parallel schedule): the bits of an output row then do not depend on how many other rows the call has, so a
    caller that splits M into chunks gets the result of the unsplit call bit for bit."""
    if plan not in _PLANS:
        raise ValueError(f"unknown plan {plan!r}")
    _launch(x, scale_x, gate_proj_weight, scale_gate, up_proj_weight, scale_up, output, plan, whole_tiles)


@torch.no_grad()
def run_concat(x: torch.Tensor, scale_x: torch.Tensor, w: torch.Tensor, scale_w: torch.Tensor,
               output: torch.Tensor) -> None:
    """Same op with concatenated weights W[2N, K] (gate rows first) and scales [2N/128, K/128].

    Row-major halves are contiguous views, so this slices and forwards to `run`.
    """
    if w.dim() != 2 or w.shape[0] % (2 * BLOCK):
        raise ValueError("w must be [2N, K] with N a multiple of 128")
    n = w.shape[0] // 2
    nb = n // BLOCK
    if scale_w.dim() != 2 or scale_w.shape[0] != 2 * nb:
        raise ValueError(f"scale_w: expected {2 * nb} rows, got {tuple(scale_w.shape)}")
    run(x, scale_x, w[:n], scale_w[:nb], w[n:], scale_w[nb:], output)


@torch.no_grad()
def run_gather(x: torch.Tensor, scale_x: torch.Tensor, gate_shard: torch.Tensor, scale_gate_shard: torch.Tensor,
               up_shard: torch.Tensor, scale_up_shard: torch.Tensor, rank_output_ptrs, rank: int,
               m_n_full: Tuple[int, int], ld_full: int) -> None:
    """This rank's column shard of the op, every output tile stored into all ranks' full [M, N] buffers.

    `rank_output_ptrs[r]` is the device address of rank r's buffer as mapped into this process (see
    `sharded.GatherBuffers`).  Asynchronous; the caller runs a cross-rank barrier before reading any buffer.
    """
    world = len(rank_output_ptrs)
    m, n_full = m_n_full
    n_local = gate_shard.shape[0]
    if n_local * world != n_full:
        raise ValueError(f"shard has {n_local} columns, expected {n_full} / {world}")
    _validate_inputs_only(x, scale_x, gate_shard, scale_gate_shard, up_shard, scale_up_shard, m, n_local)
    k = x.shape[1]
    with torch.cuda.device(x.device):
        stream_ptr = torch.cuda.current_stream(x.device).cuda_stream
        ptrs = (ctypes.c_void_p * world)(*[int(p) for p in rank_output_ptrs])
        pr = GuProblem(
            x.data_ptr(), scale_x.data_ptr(), gate_shard.data_ptr(), scale_gate_shard.data_ptr(),
            up_shard.data_ptr(), scale_up_shard.data_ptr(), int(rank_output_ptrs[rank]),
            m, k, n_local, ld_full, None, 0, PLAN_TILE, 0)
        code = _cabi.lib.gu_run_gather(ctypes.byref(pr), ptrs, world, rank, ld_full, stream_ptr)
    _raise_for(code)


@torch.no_grad()
def run_fp8_output(x: torch.Tensor, scale_x: torch.Tensor, gate_proj_weight: torch.Tensor, scale_gate: torch.Tensor,
                   up_proj_weight: torch.Tensor, scale_up: torch.Tensor, out_q: torch.Tensor,
                   out_scale: torch.Tensor) -> None:
    """`run` with the result re-quantised in the kernel epilogue: e4m3 [M, N] + fp32 scales [M, N/128].

    Feeds `blockwise_gemm` (the down projection) without a bf16 round trip through HBM; the bits equal
    `quantize_activation(run(...))`.
    """
    m, k, n = _validate_inputs_only(x, scale_x, gate_proj_weight, scale_gate, up_proj_weight, scale_up)
    _check({"out_q": (out_q, (m, n), torch.float8_e4m3fn), "out_scale": (out_scale, (m, n // BLOCK), torch.float32)},
           x.device)
    with torch.cuda.device(x.device):
        stream_ptr = torch.cuda.current_stream(x.device).cuda_stream
        pr = GuProblem(
            x.data_ptr(), scale_x.data_ptr(), gate_proj_weight.data_ptr(), scale_gate.data_ptr(),
            up_proj_weight.data_ptr(), scale_up.data_ptr(), None, m, k, n, n, None, 0, PLAN_TILE, 0)
        code = _cabi.lib.gu_run_fp8out(ctypes.byref(pr), out_q.data_ptr(), out_scale.data_ptr(), stream_ptr)
    _raise_for(code)


@torch.no_grad()
def mlp_block(x: torch.Tensor, gate_proj_weight: torch.Tensor, scale_gate: torch.Tensor, up_proj_weight: torch.Tensor,
              scale_up: torch.Tensor, down_proj_weight: torch.Tensor, scale_down: torch.Tensor,
              output: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 / fp32 activations [M, H] -> bf16 [M, H_out]: quantise, gate/up + SwiGLU (e4m3 out), down projection.

    Three launches: `quantize_activation`, `run_fp8_output`, `blockwise_gemm`.  `down_proj_weight` is e4m3
    [H_out, N] with scales [H_out/128, N/128].  The intermediate [M, N] exists only as e4m3 + scales.
    """
    m = x.shape[0]
    n = gate_proj_weight.shape[0]
    h_out = down_proj_weight.shape[0]
    xq, sx = quantize_activation(x)
    mid_q = torch.empty(m, n, dtype=torch.float8_e4m3fn, device=x.device)
    mid_s = torch.empty(m, n // BLOCK, dtype=torch.float32, device=x.device)
    run_fp8_output(xq, sx, gate_proj_weight, scale_gate, up_proj_weight, scale_up, mid_q, mid_s)
    if output is None:
        output = torch.empty(m, h_out, dtype=torch.bfloat16, device=x.device)
    blockwise_gemm(mid_q, mid_s, down_proj_weight, scale_down, output)
    return output


@torch.no_grad()
def blockwise_gemm(a: torch.Tensor, scale_a: torch.Tensor, b: torch.Tensor, scale_b: torch.Tensor,
                   output: torch.Tensor) -> None:
    """output[M, N] (bf16) = block-scaled a[M, K] @ b[N, K]^T with 1x128 scales on a and 128x128 scales on b.

    The single GEMM the reference launches twice per call (kernel.py:487-488), here as one launch of the tile
    kernel in single-projection mode; used for the MLP's down projection.  Destination passing, current stream.
    """
    if a.dim() != 2 or b.dim() != 2 or output.dim() != 2:
        raise ValueError("a, b and output must be 2-D")
    m, k = a.shape
    n = b.shape[0]
    if m < 1 or k % BLOCK or n % BLOCK or k < BLOCK or n < BLOCK:
        raise ValueError(f"Unsupported contract shape M={m}, K={k}, N={n}: need M >= 1 and K, N multiples of {BLOCK}")
    expected = {
        "a": (a, (m, k), torch.float8_e4m3fn), "scale_a": (scale_a, (m, k // BLOCK), torch.float32),
        "b": (b, (n, k), torch.float8_e4m3fn), "scale_b": (scale_b, (n // BLOCK, k // BLOCK), torch.float32),
        "output": (output, (m, n), torch.bfloat16),
    }
    _check(expected, a.device)
    if output.stride(1) != 1 or output.stride(0) < n:
        raise ValueError("output must be row-major with unit column stride")
    with torch.cuda.device(a.device):
        stream_ptr = torch.cuda.current_stream(a.device).cuda_stream
        code = _cabi.lib.gu_blockwise_gemm(a.data_ptr(), scale_a.data_ptr(), b.data_ptr(), scale_b.data_ptr(),
                                           output.data_ptr(), m, k, n, output.stride(0), stream_ptr)
    _raise_for(code)


@torch.no_grad()
def blockwise_gemm_scatter(a: torch.Tensor, scale_a: torch.Tensor, b: torch.Tensor, scale_b: torch.Tensor,
                           rank_slot_ptrs, rank: int) -> None:
    """Row-parallel `blockwise_gemm` whose bf16 partial tiles go straight to the ranks owning their token rows.

    `rank_slot_ptrs[r]` is the device address of rank r's [world, M/world, N] slot buffer as mapped into this
    process (see `sharded.ReduceBuffers`); this rank fills slot `rank` of every buffer.  M must be a multiple
    of 128 * world.  Asynchronous; a cross-rank barrier and `reduce_gather` follow.
    """
    world = len(rank_slot_ptrs)
    m, k = a.shape
    n = b.shape[0]
    if k % BLOCK or n % BLOCK or k < BLOCK or n < BLOCK or m % (BLOCK * world):
        raise ValueError(f"Unsupported contract shape M={m}, K={k}, N={n}: need K, N multiples of {BLOCK} "
                         f"and M a multiple of {BLOCK} * world")
    expected = {
        "a": (a, (m, k), torch.float8_e4m3fn), "scale_a": (scale_a, (m, k // BLOCK), torch.float32),
        "b": (b, (n, k), torch.float8_e4m3fn), "scale_b": (scale_b, (n // BLOCK, k // BLOCK), torch.float32),
    }
    _check(expected, a.device)
    with torch.cuda.device(a.device):
        stream_ptr = torch.cuda.current_stream(a.device).cuda_stream
        ptrs = (ctypes.c_void_p * world)(*[int(p) for p in rank_slot_ptrs])
        code = _cabi.lib.gu_blockwise_gemm_scatter(a.data_ptr(), scale_a.data_ptr(), b.data_ptr(),
                                                   scale_b.data_ptr(), ptrs, world, rank, m, k, n, stream_ptr)
    _raise_for(code)


@torch.no_grad()
def reduce_gather(slots: torch.Tensor, rank_output_ptrs, rank: int, m: int, h: int) -> None:
    """Sum this rank's slots [world, M/world, H] (bf16, fp32 accumulation in rank order) and write the reduced
    rows into every rank's [M, H] result (`rank_output_ptrs[r]`, mapped into this process; a peer entry of None is
    skipped).  Asynchronous."""
    world = len(rank_output_ptrs)
    if slots.dtype != torch.bfloat16 or not slots.is_contiguous() or slots.numel() != m * h or m % world:
        raise ValueError("slots must be a contiguous bf16 [world, M/world, H] tensor")
    with torch.cuda.device(slots.device):
        stream_ptr = torch.cuda.current_stream(slots.device).cuda_stream
        ptrs = (ctypes.c_void_p * world)(*[(int(p) if p else None) for p in rank_output_ptrs])
        code = _cabi.lib.gu_reduce_gather(slots.data_ptr(), ptrs, world, rank, m, h, stream_ptr)
    _raise_for(code)


def peer_barrier(rank_flag_ptrs, rank: int, device, limit_ns: int = 0) -> None:
    """Enqueue the library's bounded cross-rank barrier on the current stream of `device`.  `rank_flag_ptrs[r]` is
    the device address of rank r's 64-word flag array as mapped into this process (see `sharded.PeerBarrier`);
    `limit_ns` = 0 keeps the default time limit of 2 s.  Asynchronous; a rank that never arrives shows up as
    GU_ETIMEOUT in `last_status`, not as a hang."""
    world = len(rank_flag_ptrs)
    dev = torch.device(device)
    with torch.cuda.device(dev):
        stream_ptr = torch.cuda.current_stream(dev).cuda_stream
        ptrs = (ctypes.c_void_p * world)(*[int(p) for p in rank_flag_ptrs])
        code = _cabi.lib.gu_peer_barrier(ptrs, world, rank, int(limit_ns), stream_ptr)
    _raise_for(code)


@torch.no_grad()
def quantize_activation(x: torch.Tensor, q: Optional[torch.Tensor] = None,
                        scale: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 / fp32 activations [M, K] -> (e4m3 [M, K], fp32 scales [M, K/128]), scale = block amax / 448.

    The producer of `run`'s first two arguments (the reference receives them ready-made:
    kernel.py:356-357).  One streaming kernel on the current stream; rows of `x` may be pitched.
    """
    if x.dim() != 2 or x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("x must be a 2-D bf16 or fp32 tensor")
    if not x.is_cuda:
        raise ValueError("x must be a CUDA tensor (this package has no CPU path)")
    m, k = x.shape
    if m < 1 or k < BLOCK or k % BLOCK:
        raise ValueError(f"Unsupported shape M={m}, K={k}: need M >= 1 and K a multiple of {BLOCK}")
    if x.stride(1) != 1 or x.stride(0) < k:
        raise ValueError("x must be row-major with unit column stride")
    if q is None:
        q = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=x.device)
    if scale is None:
        scale = torch.empty(m, k // BLOCK, dtype=torch.float32, device=x.device)
    for name, t, shape, dtype in (("q", q, (m, k), torch.float8_e4m3fn), ("scale", scale, (m, k // BLOCK), torch.float32)):
        if tuple(t.shape) != shape or t.dtype != dtype or t.device != x.device or not t.is_contiguous():
            raise ValueError(f"{name}: expected contiguous shape={shape}, dtype={dtype} on {x.device}")
    with torch.cuda.device(x.device):
        stream_ptr = torch.cuda.current_stream(x.device).cuda_stream
        code = _cabi.lib.gu_quantize_activation(x.data_ptr(), 1 if x.dtype == torch.float32 else 0, x.stride(0),
                                                q.data_ptr(), scale.data_ptr(), m, k, stream_ptr)
    _raise_for(code)
    return q, scale


def last_status(clear: bool = True) -> Tuple[int, int]:
    """(code, detail) of the device-side status word; synchronises the device."""
    detail = ctypes.c_int(0)
    code = _cabi.lib.gu_last_status(ctypes.byref(detail), 1 if clear else 0)
    return code, detail.value


def launch_count() -> int:
    """Kernel launches made by libgateup.so in this process."""
    return int(_cabi.lib.gu_launch_count())
