"""CPU restatement of the activation quantiser in integer / byte arithmetic (numpy).  TEST INFRASTRUCTURE ONLY.

The quantiser produces the tensors the reference's entry point receives ready-made (`x` e4m3 with one fp32 scale per
1x128 block, kernels/179_fp8_mlp_gate_up_projection/kernel.py:356-357): scale = amax / 448 (IEEE fp32 division,
amax clamped to 1e-12), q = e4m3(clamp(x / scale, -448, 448)) with round-to-nearest-even.  `encode_e4m3fn` below
spells the e4m3fn rounding out on the bits of the fp32 quotient instead of calling a library cast, so that the
kernel, torch's cast and this restatement are three independent statements of the same bytes.

e4m3fn: 1 sign, 4 exponent (bias 7), 3 mantissa bits; no infinities; 0x7f / 0xff are NaN; largest finite 448 =
0x7e; smallest normal 2^-6; subnormals k * 2^-9, k = 1..7.

Pinned: `tests/test_oracle.py` checks `encode_e4m3fn` against torch's `float8_e4m3fn` cast on every fp32 value that
is a bf16 value in range, on all 256 decoded bytes, on exact ties and on random fp32 values, and the whole quantiser
against the torch quantiser of `workloads`.
"""
from __future__ import annotations

import numpy as np


def encode_e4m3fn(values: np.ndarray) -> np.ndarray:
    """fp32 array -> uint8 array of e4m3fn bytes; round to nearest even, |v| > 448 saturates to 448, NaN -> 0x7f."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    bits = v.view(np.uint32)
    sign = ((bits >> 24) & 0x80).astype(np.uint8)
    mag = np.abs(v)
    out = np.zeros(v.shape, dtype=np.uint8)

    # normal range of the target: 2^-6 <= |v|.  Keep 3 mantissa bits of the fp32 significand, rounding on the 20
    # dropped bits; a carry out of the mantissa moves into the exponent by itself because the fields are adjacent.
    m32 = bits & 0x7FFFFFFF
    lsb = (m32 >> 20) & 1
    rounded = (m32 + 0x7FFFF + lsb) >> 20                      # exponent(8) . mantissa(3), biased by 127
    normal = rounded.astype(np.int64) - ((127 - 7) << 3)       # rebias to 7
    # subnormal range: value = k * 2^-9; k = RNE(|v| * 2^9) (exact scaling, then ties-to-even on the integer)
    scaled = mag.astype(np.float64) * 512.0
    k = np.rint(np.where(scaled < 16.0, scaled, 0.0))          # half to even; larger or NaN inputs are not subnormal
    sub = k.astype(np.int64)                                    # k == 8 is the smallest normal: byte 0x08, same code

    is_sub = mag < np.float32(2.0 ** -6)
    code = np.where(is_sub, sub, normal)
    code = np.where(mag > np.float32(448.0), 0x7E, code)       # saturate (the rounding above cannot exceed 0x7e
    code = np.where(code > 0x7E, 0x7E, code)                   # otherwise, but a value just under 464 would round up)
    out = (code.astype(np.uint8) | sign)
    out = np.where(np.isnan(v), np.uint8(0x7F), out)
    return out.astype(np.uint8)


def decode_e4m3fn(codes: np.ndarray) -> np.ndarray:
    """uint8 e4m3fn bytes -> fp32 (NaN for 0x7f / 0xff)."""
    c = np.ascontiguousarray(codes, dtype=np.uint8).astype(np.int64)
    sign = np.where(c & 0x80, -1.0, 1.0)
    e = (c >> 3) & 0xF
    m = c & 7
    val = np.where(e == 0, m * 2.0 ** -9, (8 + m) * 2.0 ** (e - 10.0))
    val = np.where((c & 0x7F) == 0x7F, np.nan, val)
    return (sign * val).astype(np.float32)


def quantize_activation_1x128(x: np.ndarray):
    """fp32 [M, K] -> (uint8 e4m3fn bytes [M, K], fp32 scales [M, K/128])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    if k % 128:
        raise ValueError(f"K={k} is not a multiple of 128")
    xb = x.reshape(m, k // 128, 128)
    amax = np.maximum(np.abs(xb).max(axis=-1, keepdims=True), np.float32(1e-12)).astype(np.float32)
    scale = (amax / np.float32(448.0)).astype(np.float32)      # IEEE fp32 division
    quotient = (xb / scale).astype(np.float32)
    quotient = np.clip(quotient, np.float32(-448.0), np.float32(448.0))
    return encode_e4m3fn(quotient).reshape(m, k), scale.reshape(m, k // 128)
