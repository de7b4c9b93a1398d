"""Seeded synthetic workloads for the FP8 gate/up + SwiGLU path.

The benchmark suite that the reference submission targets ships its own
workload list and input generator; neither is available offline, so every
shape here is synthetic: X ~ N(0, 1), W ~ N(0, 0.02), quantised to e4m3 with
1x128 activation block scales and 128x128 weight block scales, each scale
being amax / 448.  Tensor layouts are the ones the reference entry point
takes (kernels/179_fp8_mlp_gate_up_projection/kernel.py:345-383):

    x            e4m3 [M, K]          scale_x     f32 [M, K/128]
    gate / up    e4m3 [N, K]          scale_gate  f32 [N/128, K/128]  (same for up)
    output       bf16 [M, N]

Everything is plain torch and runs on whichever device it is given, so the
CPU checker and the CUDA kernels see identical bits.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch

BLOCK = 128
E4M3_MAX = 448.0

# Named shapes: (M, K, N).  "small" is CPU-checkable in full; the others are the
# single-GPU prefill / decode shapes and the shape that is column-sharded.
SHAPES: Dict[str, Tuple[int, int, int]] = {
    "small": (128, 2048, 5632),
    "prefill_8b": (4096, 4096, 14336),
    "decode_70b": (16, 8192, 28672),
    "prefill_sharded": (16384, 7168, 18432),
    "reference_native": (1024, 3584, 18944),
}
SWEEP_M = (1, 8, 32, 128, 512, 2048, 8192)
SWEEP_KN = (4096, 14336)


def quantize_activation_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 [M, K] -> (e4m3 [M, K], f32 scales [M, K/128]); scale = amax / 448 per 1x128 block."""
    m, k = x.shape
    if k % BLOCK:
        raise ValueError(f"K={k} is not a multiple of {BLOCK}")
    xb = x.float().reshape(m, k // BLOCK, BLOCK)
    amax = xb.abs().amax(dim=-1, keepdim=True).clamp_min(1e-12)
    scale = amax / E4M3_MAX
    q = (xb / scale).clamp_(-E4M3_MAX, E4M3_MAX).reshape(m, k).to(torch.float8_e4m3fn)
    return q.contiguous(), scale.reshape(m, k // BLOCK).contiguous()


def quantize_weight_128x128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 [N, K] -> (e4m3 [N, K], f32 scales [N/128, K/128]); scale = amax / 448 per 128x128 block."""
    n, k = w.shape
    if n % BLOCK or k % BLOCK:
        raise ValueError(f"N={n}, K={k} must be multiples of {BLOCK}")
    wb = w.float().reshape(n // BLOCK, BLOCK, k // BLOCK, BLOCK)
    amax = wb.abs().amax(dim=(1, 3), keepdim=True).clamp_min(1e-12)
    scale = amax / E4M3_MAX
    q = (wb / scale).clamp_(-E4M3_MAX, E4M3_MAX).reshape(n, k).to(torch.float8_e4m3fn)
    return q.contiguous(), scale.reshape(n // BLOCK, k // BLOCK).contiguous()


@dataclass
class GateUpInputs:
    """One workload in the reference's argument order."""

    x: torch.Tensor
    scale_x: torch.Tensor
    gate_proj_weight: torch.Tensor
    scale_gate: torch.Tensor
    up_proj_weight: torch.Tensor
    scale_up: torch.Tensor

    @property
    def shape(self) -> Tuple[int, int, int]:
        return self.x.shape[0], self.x.shape[1], self.gate_proj_weight.shape[0]

    def args(self):
        return (self.x, self.scale_x, self.gate_proj_weight, self.scale_gate,
                self.up_proj_weight, self.scale_up)

    def to(self, device) -> "GateUpInputs":
        return GateUpInputs(*(t.to(device) for t in self.args()))

    def rows(self, idx: torch.Tensor) -> "GateUpInputs":
        """Restriction to a subset of tokens (output rows depend on no other token)."""
        return GateUpInputs(self.x[idx].contiguous(), self.scale_x[idx].contiguous(),
                            self.gate_proj_weight, self.scale_gate,
                            self.up_proj_weight, self.scale_up)

    def column_blocks(self, blocks: torch.Tensor) -> "GateUpInputs":
        """Restriction to a subset of 128-wide output column blocks."""
        rows = (blocks[:, None] * BLOCK + torch.arange(BLOCK, device=blocks.device)[None, :]).reshape(-1)
        return GateUpInputs(self.x, self.scale_x,
                            self.gate_proj_weight[rows].contiguous(), self.scale_gate[blocks].contiguous(),
                            self.up_proj_weight[rows].contiguous(), self.scale_up[blocks].contiguous())

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.args())


def make_inputs(m: int, k: int, n: int, seed: int = 0, device="cpu",
                x_std: float = 1.0, w_std: float = 0.02) -> GateUpInputs:
    """Seeded workload.  The weights are drawn as one concatenated W[2N, K] (gate rows first)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    x = torch.randn(m, k, generator=gen, device=dev, dtype=torch.float32) * x_std
    xq, sx = quantize_activation_1x128(x)
    del x
    parts = []
    for _ in range(2):
        w = torch.randn(n, k, generator=gen, device=dev, dtype=torch.float32) * w_std
        parts.append(quantize_weight_128x128(w))
        del w
    (gq, sg), (uq, su) = parts
    return GateUpInputs(xq, sx, gq, sg, uq, su)


def algorithmic_flops(m: int, k: int, n: int) -> int:
    """Two GEMMs at 2 flop per multiply-add; scaling and SiLU are not counted."""
    return 4 * m * n * k


def algorithmic_bytes(m: int, k: int, n: int) -> int:
    """Every operand touched once: X, scale_x, both W, both W scale grids, bf16 output."""
    kb, nb = k // BLOCK, n // BLOCK
    return m * k + 4 * m * kb + 2 * n * k + 8 * nb * kb + 2 * m * n


# ---- side operators (problems 038 and 029 of the reference repository) --------------------------------------
# Seeded synthetic inputs, drawn on the CPU so that every machine sees the same bits.

RMSNORM_SHAPES = {  # name -> (tokens, heads); head width is 128
    "flux_128": (128, 48), "flux_2048": (2048, 48), "flux_4608": (4608, 48), "flux_16384": (16384, 48),
}
MAMBA_TAIL_SHAPES = {  # name -> (batch, sequence, channels, projected width)
    "mamba_b1_l128": (1, 128, 16384, 32768), "mamba_b1_l2048": (1, 2048, 16384, 32768),
    "mamba_b4_l2048": (4, 2048, 16384, 32768),
}


def make_rmsnorm_inputs(tokens: int, heads: int, seed: int = 0, device="cpu"):
    """(query, key, weight_q, weight_k, eps): fp32 [1, tokens, heads, 128] x2, [heads, 128] x2."""
    g = torch.Generator().manual_seed(seed)
    query = torch.randn(1, tokens, heads, 128, generator=g) * 1.5
    key = torch.randn(1, tokens, heads, 128, generator=g) * 0.7 + 0.1
    weight_q = 1.0 + 0.1 * torch.randn(heads, 128, generator=g)
    weight_k = 1.0 + 0.1 * torch.randn(heads, 128, generator=g)
    return query.to(device), key.to(device), weight_q.to(device), weight_k.to(device), 1e-6


def make_mamba_tail_inputs(batch: int, sequence: int, channels: int, width: int, seed: int = 0, device="cpu",
                           padded: bool = True):
    """(projected, attention_mask, conv1d_weight, conv1d_bias), all bf16.  With `padded`, every batch row but
    the first has a run of masked positions at its start and a few inside (left padding plus holes)."""
    g = torch.Generator().manual_seed(seed)
    projected = (torch.randn(batch, sequence, width, generator=g) * 2.0).to(torch.bfloat16)
    mask = torch.ones(batch, sequence)
    if padded:
        for b in range(1, batch):
            mask[b, : (b * 37) % max(1, sequence // 2)] = 0.0
        holes = torch.rand(batch, sequence, generator=g) < 0.02
        mask[holes] = 0.0
    conv_w = (torch.randn(channels, 1, 4, generator=g) * 0.5).to(torch.bfloat16)
    conv_b = (torch.randn(channels, generator=g) * 0.5).to(torch.bfloat16)
    return projected.to(device), mask.to(torch.bfloat16).to(device), conv_w.to(device), conv_b.to(device)
