"""Exhaustive small-shape sweep under the range-checked debug build of the library.

`compute-sanitizer` is not available on the machines these tests run on, so the library carries its own checker:
built with -DGU_BOUNDS=1 (libgateup_bounds.so) every kernel tests each computed TMA coordinate, global index and
ring / accumulator stage index against its extent before using it, records the first violation in the status word
(`gu_last_status` -> GU_EBOUNDS) and skips the access.  This test runs every token count M = 1 ... 129 at
K, N in {128, 256} through every plan that takes the shape — the lone-CTA tile kernel and its stream-K schedule, the
CTA-pair kernel (forced also where the second CTA of a pair has no rows) and the weight-streaming kernel — inside
that build, with canary rows and columns around the destination, against the CPU oracle; then a few larger shapes
through the pair kernel's stream-K schedule, its FP8-output epilogue and its plain-GEMM mode.  A process binds one build
of the library, so the sweep runs in a child process.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_SWEEP = r"""
import os, sys
sys.path.insert(0, os.environ["GU_ROOT"])
import sol_execbench_b200_kernels_b200.build as B
B.LIB_PATH = B.BOUNDS_LIB_PATH
import torch
import sol_execbench_b200_kernels_b200 as pkg
from sol_execbench_b200_kernels_b200 import _cabi, workloads as W
from oracle import gateup_oracle as O

assert _cabi.lib.gu_is_range_checked_build() == 1
dev = torch.device("cuda:0")
pkg.last_status(clear=True)
launches = 0
for k in (128, 256):
    for n in (128, 256):
        wide = torch.empty(129 + 2, n + 256, dtype=torch.bfloat16, device=dev)
        for m in range(1, 130):
            inp = W.make_inputs(m, k, n, seed=1000 * k + 10 * n + m)
            ref = O.gateup_blockwise(*inp.args())
            g = inp.to(dev)
            plans = ["tile_dp", "tile_pair", "tile_sk"] + (["stream"] if m <= 64 else [])
            for plan in plans:
                wide.fill_(7.0)
                view = wide[1:m + 1, 128:128 + n]
                pkg.run_with_plan(*g.args(), view, plan)
                launches += 1
                torch.cuda.synchronize()
                code, detail = pkg.last_status()
                assert code == 0, f"M={m} K={k} N={n} {plan}: device status {code}, detail {detail:#x}"
                got = view.float().cpu()
                st = O.error_stats(got, ref)
                # (a stream-K hand-off adds partial sums in another association: single roundings may differ)
                assert st["finite"] and st["rel_l2"] <= 1e-3 and st["max_abs"] <= 2e-2, (m, k, n, plan, st)
                mask = torch.ones_like(wide, dtype=torch.bool)
                mask[1:m + 1, 128:128 + n] = False
                assert bool((wide[mask] == 7.0).all()), f"M={m} K={k} N={n} {plan}: wrote outside the destination"
# larger shapes for what needs many tiles or other epilogues: the pair kernel's stream-K schedule (a tile per cluster
# at least), its FP8-output epilogue and its plain-GEMM mode
for shape in ((512, 128, 4864), (300, 256, 5120), (1100, 128, 2432)):
    inp = W.make_inputs(*shape, seed=sum(shape))
    ref = O.gateup_blockwise(*inp.args())
    g = inp.to(dev)
    m, k, n = shape
    wide = torch.full((m + 2, n + 256), 7.0, dtype=torch.bfloat16, device=dev)
    view = wide[1:m + 1, 128:128 + n]
    pkg.run_with_plan(*g.args(), view, "tile_pair_sk")
    launches += 1
    torch.cuda.synchronize()
    code, detail = pkg.last_status()
    assert code == 0, f"{shape} tile_pair_sk: device status {code}, detail {detail:#x}"
    st = O.error_stats(view.float().cpu(), ref)
    assert st["finite"] and st["rel_l2"] <= 1e-3, (shape, st)
    mask = torch.ones_like(wide, dtype=torch.bool)
    mask[1:m + 1, 128:128 + n] = False
    assert bool((wide[mask] == 7.0).all()), f"{shape} tile_pair_sk: wrote outside the destination"
for shape in ((300, 256, 256), (129, 128, 384)):
    m, k, n = shape
    g = W.make_inputs(*shape, seed=7 + m).to(dev)
    q = torch.zeros(m, n, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    sc = torch.zeros(m, n // 128, dtype=torch.float32, device=dev)
    pkg.run_fp8_output(*g.args(), q, sc)
    ref = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    pkg.run_with_plan(*g.args(), ref, "tile_dp")
    c = torch.empty(m, k, dtype=torch.bfloat16, device=dev)
    wq, ws = W.quantize_weight_128x128(torch.randn(k, n, device=dev) * 0.05)
    pkg.blockwise_gemm(q, sc, wq, ws, c)
    launches += 3
    torch.cuda.synchronize()
    code, detail = pkg.last_status()
    assert code == 0, f"{shape} fp8 output / plain GEMM: device status {code}, detail {detail:#x}"
    q_ref, s_ref = W.quantize_activation_1x128(ref.cpu().float())
    assert torch.equal(sc.cpu(), s_ref) and torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    want = O.gemm_blockwise(q.cpu(), sc.cpu(), wq.cpu(), ws.cpu())
    assert O.error_stats(c, want)["rel_l2"] <= 1e-3
print(f"swept {launches} launches under the range-checked build: status 0 throughout")
"""


def test_every_small_shape_through_every_plan_under_the_range_checked_build():
    lib = os.path.join(ROOT, "sol_execbench_b200_kernels_b200", "libgateup_bounds.so")
    assert os.path.exists(lib), "libgateup_bounds.so is missing: python -m sol_execbench_b200_kernels_b200.build --bounds"
    proc = subprocess.run([sys.executable, "-c", _SWEEP], env=dict(os.environ, GU_ROOT=ROOT), capture_output=True,
                          text=True, timeout=1500)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    assert "status 0 throughout" in proc.stdout


_PROJ_SWEEP = r"""
import os, sys
sys.path.insert(0, os.environ["GU_ROOT"])
import sol_execbench_b200_kernels_b200.build as B
B.SIDE_LIB_PATH = B.SIDE_BOUNDS_LIB_PATH
import torch
from sol_execbench_b200_kernels_b200 import _sideops_cabi, side_ops

assert _sideops_cabi.lib.so_is_range_checked_build() == 1
dev = torch.device("cuda:0")
side_ops.last_status()
launches = 0
g = torch.Generator().manual_seed(3)
for k in (8, 64, 72, 200):
    for n in (8, 248, 264, 520):
        weight = (torch.randn(n, k, generator=g) * 0.1).to(torch.bfloat16).to(dev)
        bias = (torch.randn(n, generator=g) * 0.2).to(torch.bfloat16).to(dev)
        for m in list(range(1, 131)) + [255, 256, 257, 300, 383, 384, 385, 511, 513]:
            hidden = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).to(dev)
            buf = torch.full((m + 2, n), 7.0, dtype=torch.bfloat16, device=dev)     # canary rows around the result
            out = buf[1:m + 1]
            side_ops.mamba_in_proj(hidden, weight, bias, out)
            launches += 1
            torch.cuda.synchronize()
            code, detail = side_ops.last_status()
            assert code == 0, f"M={m} K={k} N={n}: device status {code}, detail {detail:#x}"
            exact = hidden.double() @ weight.double().t() + bias.double()
            mags = hidden.double().abs() @ weight.double().abs().t() + bias.double().abs()
            err = (out.double() - exact).abs()
            assert bool((err <= exact.abs() * 2.0 ** -8 + mags * 2.0 ** -16 + 1e-30).all()), (m, k, n, float(err.max()))
            assert bool((buf[0] == 7.0).all()) and bool((buf[m + 1] == 7.0).all()), f"M={m} K={k} N={n}: wrote outside"
print(f"swept {launches} projection launches under the range-checked build: status 0 throughout")
"""


def test_projection_small_shapes_under_the_range_checked_build():
    """The bf16 projection GEMM relies on TMA's out-of-range behaviour for ragged M, K and N (reads give zero, stores
    are clipped): every M = 1 ... 130 and a few around the 256-row pair tile, at K and N that are and are not whole
    tiles, inside the range-checked build of libsideops, with canary rows around the destination."""
    lib = os.path.join(ROOT, "sol_execbench_b200_kernels_b200", "libsideops_bounds.so")
    assert os.path.exists(lib), "libsideops_bounds.so is missing: python -m sol_execbench_b200_kernels_b200.build --bounds"
    proc = subprocess.run([sys.executable, "-c", _PROJ_SWEEP], env=dict(os.environ, GU_ROOT=ROOT), capture_output=True,
                          text=True, timeout=1500)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    assert "status 0 throughout" in proc.stdout


def test_the_regular_library_is_not_the_range_checked_build():
    from sol_execbench_b200_kernels_b200 import _cabi, _sideops_cabi

    assert _cabi.lib.gu_is_range_checked_build() == 0
    assert _sideops_cabi.lib.so_is_range_checked_build() == 0
