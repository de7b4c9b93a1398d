"""gu_run_decode_static: the decode kernel with its stream-K scratch built into the library.

It exists for hosts that may not allocate device memory themselves — a serving runtime that
owns all of HBM and forbids cudaMalloc after start-up, or a decode loop that cannot take the
device-wide synchronisation an allocation brings — so they have no workspace to pass to gu_run.
The test calls it through the C ABI twice in a row and checks each result against gu_run (same
kernel, caller-supplied workspace) and against the CPU oracle, with the tolerances of the other GPU
tests, and that the device's free memory is the same before and after the second call (nothing was
allocated behind the caller's back).  The file sorts last
so that a run that stops at the first failure has already run every other test; it also passes
on its own in a fresh process (the first call does the per-device set-up).
"""
import ctypes

import pytest
import torch

from oracle import gateup_oracle as O
from sol_execbench_b200_kernels_b200 import workloads as W

pytestmark = pytest.mark.gpu

ATOL = 2e-2
REL_L2 = 1e-2


def _problem(_cabi, g, out, m, k, n, ws=None, nbytes=0, plan=0):
    return _cabi.GuProblem(g.x.data_ptr(), g.scale_x.data_ptr(), g.gate_proj_weight.data_ptr(),
                           g.scale_gate.data_ptr(), g.up_proj_weight.data_ptr(), g.scale_up.data_ptr(),
                           out.data_ptr(), m, k, n, out.stride(0), ws.data_ptr() if ws is not None else None,
                           nbytes, plan, 0)


@pytest.mark.parametrize("shape", [(16, 2048, 2304), (5, 1024, 18944)])
def test_static_scratch_entry_point_matches_workspace_entry_point(shape):
    from sol_execbench_b200_kernels_b200 import _cabi

    m, k, n = shape
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    lib = _cabi.lib

    nbytes = lib.gu_workspace_bytes(m, k, n, _cabi.PLAN_STREAM)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    assert lib.gu_workspace_init(ws.data_ptr(), nbytes, stream) == 0

    for call in range(2):                      # two calls in a row share the built-in array
        g = W.make_inputs(m, k, n, seed=30 + call, device=dev)
        want = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=dev)
        pr = _problem(_cabi, g, want, m, k, n, ws, nbytes, _cabi.PLAN_STREAM)
        assert lib.gu_run(ctypes.byref(pr), stream) == 0
        ps = _problem(_cabi, g, got, m, k, n)              # no workspace at all
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(dev)
        assert lib.gu_run_decode_static(ctypes.byref(ps), stream) == 0
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(dev)
        if call == 1:                                       # (the first call on a device may load the module)
            assert free_after == free_before, (free_before, free_after)
        detail = ctypes.c_int(0)
        assert lib.gu_last_status(ctypes.byref(detail), 1) == 0, hex(detail.value)
        assert torch.isfinite(got.float()).all() and not (got == 0).all()
        diff = (got.float() - want.float())
        assert diff.abs().max().item() <= ATOL
        assert (torch.linalg.vector_norm(diff) / torch.linalg.vector_norm(want.float())).item() <= REL_L2
        # and against the CPU restatement, on every token and a few column blocks
        blocks = torch.tensor(sorted({0, n // 256, n // 128 - 1}), device=dev)
        sub = g.column_blocks(blocks).to("cpu")
        cols = (blocks[:, None] * 128 + torch.arange(128, device=dev)[None]).reshape(-1)
        for oracle in (O.gateup_blockwise, O.gateup_dequant):
            st = O.error_stats(got[:, cols].cpu(), oracle(*sub.args()))
            assert st["rel_l2"] <= REL_L2 and (st["max_abs"] <= ATOL or st["min_abs_ref_over"] >= 2.0), st


def test_static_scratch_entry_point_rejects_more_than_16_tokens():
    from sol_execbench_b200_kernels_b200 import _cabi

    m, k, n = 17, 256, 256
    dev = torch.device("cuda:0")
    g = W.make_inputs(m, k, n, seed=32, device=dev)
    out = torch.full((m, n), 3.0, dtype=torch.bfloat16, device=dev)
    pr = _problem(_cabi, g, out, m, k, n)
    rc = _cabi.lib.gu_run_decode_static(ctypes.byref(pr), torch.cuda.current_stream().cuda_stream)
    assert rc == _cabi.GU_ESTATIC_LIMIT
    assert "16 tokens" in _cabi.error_string(rc)
    torch.cuda.synchronize()
    assert (out == 3.0).all()                  # nothing was launched
