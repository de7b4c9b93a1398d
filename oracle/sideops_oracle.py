"""CPU restatement of the side operators.  TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and
bench.py's CPU-baseline leg; never by the package.

* `rmsnorm_qk`: kernels/038_flux_multi_head_rmsnorm_qk/kernel.cu:143-196 — per (token, head) row of 128 fp32:
  scale = rsqrt(sum(x^2) / 128 + eps), out = (x * scale) * weight[head].  Floating point: the sum order and the
  reciprocal square root differ between implementations, so parity is a tolerance (stated in the tests).
* `mamba_conv1d_tail`: kernels/029_mamba_conv1d_with_gating/kernel.cu:196-258 — bf16 rounding after the masked
  multiply, after the convolution (fp32 accumulation in tap order, then bias), after the sigmoid and after the
  product; an output is kept where the mask is at least one half.  The products of two bf16 values are exact in
  fp32, so the fp32 accumulation below is bit-identical to a fused-multiply-add chain.
* `mamba_in_proj`: kernels/029_mamba_conv1d_with_gating/kernel.cu:36-64, 274-312 — a bf16 GEMM with fp32
  accumulation whose epilogue adds the bf16 bias in fp32 and rounds once to bf16.  Floating point: the order of the
  K sum differs between implementations, so parity is a tolerance of one bf16 rounding step (stated in the tests).

Pinned against outputs of the reference's own CUDA kernels run on a B200 (fixtures under tests/golden/, made by
tests/golden/make_sideops_golden.py).
"""
from __future__ import annotations

import torch


def rmsnorm_qk(query: torch.Tensor, key: torch.Tensor, weight_q: torch.Tensor, weight_k: torch.Tensor, eps: float):
    def one(x, w):
        x = x.float()
        scale = torch.rsqrt(x.pow(2).sum(-1, keepdim=True) * (1.0 / 128.0) + eps)
        return (x * scale) * w.float()

    return one(query, weight_q), one(key, weight_k)


def mamba_in_proj(hidden_states: torch.Tensor, in_proj_weight: torch.Tensor, in_proj_bias: torch.Tensor,
                  exact: bool = False) -> torch.Tensor:
    """bf16 [..., K], [N, K], [N] -> bf16 [..., N]; with `exact` the unrounded float64 result instead."""
    if exact:
        return hidden_states.double() @ in_proj_weight.double().t() + in_proj_bias.double()
    acc = hidden_states.float() @ in_proj_weight.float().t()
    return (acc + in_proj_bias.float()).to(torch.bfloat16)


def mamba_conv1d_tail(projected: torch.Tensor, attention_mask: torch.Tensor, conv1d_weight: torch.Tensor,
                      conv1d_bias: torch.Tensor) -> torch.Tensor:
    """bf16 [B, L, W], [B, L], [C, 1, 4], [C] -> bf16 [B, C, L]."""
    channels = conv1d_bias.shape[0]
    batch, sequence, _ = projected.shape
    mask = attention_mask.float()
    x = (projected[:, :, :channels].float() * mask[:, :, None]).to(torch.bfloat16).float()   # [B, L, C]
    pad = torch.zeros(batch, 3, channels, dtype=torch.float32, device=x.device)
    xp = torch.cat([pad, x], dim=1)                                                           # [B, L + 3, C]
    w = conv1d_weight.float().reshape(channels, 4)
    acc = xp[:, 0:sequence] * w[:, 0]
    for tap in (1, 2, 3):
        acc = acc + xp[:, tap:tap + sequence] * w[:, tap]
    acc = acc + conv1d_bias.float()
    conv = acc.to(torch.bfloat16)
    sig = torch.sigmoid(conv.float()).to(torch.bfloat16)
    act = (conv.float() * sig.float()).to(torch.bfloat16)
    keep = (attention_mask >= 0.5)[:, :, None]
    out = torch.where(keep, act, torch.zeros((), dtype=torch.bfloat16, device=act.device))
    return out.transpose(1, 2).contiguous()
