"""Host-side mirror of the operators that sit beside the FP8 gate/up path in the reference repository.

`rmsnorm_qk` has the signature of the reference's problem-038 entry point
(kernels/038_flux_multi_head_rmsnorm_qk/binding.cpp:26-64: destination passing, current stream, fp32 tensors);
`mamba_conv1d_with_gating` that of problem 029 (kernels/029_mamba_conv1d_with_gating/binding.cpp:31-104:
returns (output_hidden_states, gate)), made of `mamba_in_proj` (the bf16 projection GEMM with bias) and
`mamba_conv1d_tail`.  All call libsideops.so through its C ABI; there is no other implementation behind them.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _sideops_cabi as _so

HEAD_DIM = 128
CONV_TAPS = 4
CONV_CHANNEL_TILE = 64


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _check_f32(t: torch.Tensor, name: str, device) -> None:
    _need(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _need(t.dtype == torch.float32, f"{name} must have float32 dtype")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    _need(t.is_cuda, f"{name} must be a CUDA tensor")
    _need(t.device == device, "all tensors must use the same CUDA device")


@torch.no_grad()
def rmsnorm_qk(query: torch.Tensor, key: torch.Tensor, weight_q: torch.Tensor, weight_k: torch.Tensor, eps: float,
               query_norm: torch.Tensor, key_norm: torch.Tensor) -> None:
    """Per-head RMSNorm of query and key, one launch: out = x * rsqrt(mean(x^2, -1) + eps) * weight[head].

    query, key, query_norm, key_norm: fp32 [..., heads, 128]; weight_q, weight_k: fp32 [heads, 128].
    The reference fixes heads = 48 and four dimensions; any leading dimensions and head count are taken here.
    """
    _need(query.dim() >= 3, "query must be [..., heads, 128]")
    _need(query.shape == key.shape, "query and key shapes must match")
    heads, width = query.shape[-2], query.shape[-1]
    _need(width == HEAD_DIM, f"query and key must have heads of width {HEAD_DIM}")
    _need(tuple(weight_q.shape) == (heads, HEAD_DIM), f"weight_q must have shape [{heads}, {HEAD_DIM}]")
    _need(tuple(weight_k.shape) == (heads, HEAD_DIM), f"weight_k must have shape [{heads}, {HEAD_DIM}]")
    _need(query_norm.shape == query.shape, "query_norm shape must match query")
    _need(key_norm.shape == key.shape, "key_norm shape must match key")
    for t, name in ((query, "query"), (key, "key"), (weight_q, "weight_q"), (weight_k, "weight_k"),
                    (query_norm, "query_norm"), (key_norm, "key_norm")):
        _check_f32(t, name, query.device)
    tokens = query.numel() // (heads * HEAD_DIM)
    if tokens == 0:
        return
    with torch.cuda.device(query.device):
        stream = torch.cuda.current_stream(query.device).cuda_stream
        _so.check(_so.lib.so_rmsnorm_qk(query.data_ptr(), key.data_ptr(), weight_q.data_ptr(), weight_k.data_ptr(),
                                        float(eps), query_norm.data_ptr(), key_norm.data_ptr(), tokens, heads, stream))


def _check_bf16(t: torch.Tensor, name: str, device) -> None:
    _need(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _need(t.dtype == torch.bfloat16, f"{name} must have bfloat16 dtype")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    _need(t.is_cuda, f"{name} must be a CUDA tensor")
    _need(t.device == device, "all tensors must be on the same CUDA device")


@torch.no_grad()
def mamba_conv1d_tail(projected: torch.Tensor, attention_mask: torch.Tensor, conv1d_weight: torch.Tensor,
                      conv1d_bias: torch.Tensor, output_hidden_states: torch.Tensor) -> None:
    """Mask, depthwise causal conv (4 taps) + bias, SiLU, mask, transposed to [B, channels, L]; all bf16.

    projected [B, L, W]: channels [0, C) of the last axis are convolved (the reference: W = 32768, C = 16384);
    attention_mask [B, L] of 0 / 1; conv1d_weight [C, 1, 4]; conv1d_bias [C]; output_hidden_states [B, C, L].
    Rounding boundaries of the reference kernel (kernel.cu:211-251): masked input, convolution, sigmoid and the
    product are each rounded to bf16.
    """
    _need(projected.dim() == 3, "projected must have shape [B, L, W]")
    batch, sequence, width = projected.shape
    channels = conv1d_bias.shape[0] if conv1d_bias.dim() == 1 else -1
    _need(channels >= CONV_CHANNEL_TILE and channels % CONV_CHANNEL_TILE == 0,
          f"conv1d_bias must have shape [C] with C a multiple of {CONV_CHANNEL_TILE}")
    _need(width >= channels and width % 8 == 0, "projected must be at least C wide, a multiple of 8")
    _need(tuple(attention_mask.shape) == (batch, sequence), "attention_mask must have shape [B, L]")
    _need(tuple(conv1d_weight.shape) == (channels, 1, CONV_TAPS), f"conv1d_weight must have shape [{channels}, 1, 4]")
    _need(tuple(output_hidden_states.shape) == (batch, channels, sequence),
          "output_hidden_states must have shape [B, C, L]")
    for t, name in ((projected, "projected"), (attention_mask, "attention_mask"), (conv1d_weight, "conv1d_weight"),
                    (conv1d_bias, "conv1d_bias"), (output_hidden_states, "output_hidden_states")):
        _check_bf16(t, name, projected.device)
    if batch == 0 or sequence == 0:
        return
    with torch.cuda.device(projected.device):
        stream = torch.cuda.current_stream(projected.device).cuda_stream
        _so.check(_so.lib.so_mamba_conv1d_tail(projected.data_ptr(), attention_mask.data_ptr(),
                                               conv1d_weight.data_ptr(), conv1d_bias.data_ptr(),
                                               output_hidden_states.data_ptr(), batch, sequence, channels, width,
                                               stream))


@torch.no_grad()
def mamba_in_proj(hidden_states: torch.Tensor, in_proj_weight: torch.Tensor, in_proj_bias: torch.Tensor,
                  projected: torch.Tensor) -> None:
    """projected[..., N] = bf16(hidden_states[..., K] . in_proj_weight[N, K]^T + in_proj_bias[N]), fp32 accumulation.

    The reference's projection launch (kernels/029_mamba_conv1d_with_gating/kernel.cu:274-312) fixes K = 8192 and
    N = 32768; here K and N are any multiples of 8 and the leading dimensions are flattened into the row count.
    """
    _need(hidden_states.dim() >= 2, "hidden_states must be [..., K]")
    _need(in_proj_weight.dim() == 2, "in_proj_weight must have shape [N, K]")
    n, k = in_proj_weight.shape
    _need(hidden_states.shape[-1] == k, f"hidden_states must have shape [..., {k}]")
    _need(tuple(in_proj_bias.shape) == (n,), f"in_proj_bias must have shape [{n}]")
    _need(tuple(projected.shape) == tuple(hidden_states.shape[:-1]) + (n,),
          "projected must have the leading dimensions of hidden_states and N columns")
    _need(k % 8 == 0 and n % 8 == 0 and k >= 8 and n >= 8, "K and N must be multiples of 8")
    for t, name in ((hidden_states, "hidden_states"), (in_proj_weight, "in_proj_weight"),
                    (in_proj_bias, "in_proj_bias"), (projected, "projected")):
        _check_bf16(t, name, hidden_states.device)
    m = hidden_states.numel() // k
    if m == 0:
        return
    with torch.cuda.device(hidden_states.device):
        stream = torch.cuda.current_stream(hidden_states.device).cuda_stream
        _so.check(_so.lib.so_mamba_in_proj(hidden_states.data_ptr(), in_proj_weight.data_ptr(),
                                           in_proj_bias.data_ptr(), projected.data_ptr(), m, k, n, stream))


def last_status(clear: bool = True) -> Tuple[int, int]:
    """(code, detail) of the library's device status word after a device synchronisation: code 0, or SO_ETIMEOUT
    when a bounded wait inside the projection kernel ran out since the status was last cleared."""
    import ctypes

    detail = ctypes.c_int(0)
    code = _so.lib.so_last_status(ctypes.byref(detail), 1 if clear else 0)
    return code, detail.value


@torch.no_grad()
def mamba_conv1d_with_gating(hidden_states: torch.Tensor, attention_mask: torch.Tensor, in_proj_weight: torch.Tensor,
                             in_proj_bias: torch.Tensor, conv1d_weight: torch.Tensor,
                             conv1d_bias: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Problem 029 as the reference exposes it: (output_hidden_states [B, C, L], gate [B, C, L] view).

    Two launches of this package's kernels: the input projection (a tcgen05 bf16 GEMM with the bias in its epilogue;
    the reference uses a CUTLASS builder GEMM there, kernel.cu:36-160) and the convolution tail.  `gate` is the
    transposed view of the projection's upper half, as in the reference (binding.cpp:88-92).
    """
    _need(hidden_states.dim() == 3, "hidden_states must have shape [B, L, H]")
    projected_width = in_proj_weight.shape[0]
    _need(projected_width % 2 == 0, "in_proj_weight must have an even number of rows")
    channels = projected_width // 2
    projected = torch.empty(hidden_states.shape[0], hidden_states.shape[1], projected_width,
                            dtype=hidden_states.dtype, device=hidden_states.device)
    mamba_in_proj(hidden_states, in_proj_weight, in_proj_bias, projected)
    gate = projected[:, :, channels:].transpose(1, 2)
    out = torch.empty(hidden_states.shape[0], channels, hidden_states.shape[1], dtype=hidden_states.dtype,
                      device=hidden_states.device)
    mamba_conv1d_tail(projected, attention_mask, conv1d_weight, conv1d_bias, out)
    return out, gate


def launch_count() -> int:
    return int(_so.lib.so_launch_count())
