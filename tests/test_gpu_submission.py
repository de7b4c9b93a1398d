"""The emitted SOL-ExecBench submissions, compiled the way the evaluator compiles them (one torch extension per
problem from the flat source directory) and called through their `run` entry points on a GPU: results must equal
the package's own entry points bit for bit, since both reach the same kernels through the same C ABI."""
import os

import pytest
import torch

from sol_execbench_b200_kernels_b200 import submission as S
from sol_execbench_b200_kernels_b200 import workloads as W

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILT = os.path.join(ROOT, "tests", "_built_submissions")


def _extension(problem):
    src = S.emit(problem, os.path.join(BUILT, f"src_{problem}"))
    so = S.build_extension(src, os.path.join(BUILT, f"build_{problem}"))    # incremental: a no-op when up to date
    return S.load_extension(so)


def test_problem_179_submission_equals_package_run():
    import sol_execbench_b200_kernels_b200 as pkg
    ext = _extension("179")
    dev = torch.device("cuda:0")
    for (m, k, n) in ((128, 2048, 1024), (16, 4096, 8192), (300, 512, 640)):
        inp = W.make_inputs(m, k, n, seed=m, device=dev)
        want = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        pkg.run(*inp.args(), want)
        for _ in range(2):          # twice: the second call reuses the cached scratch of the small-M plan
            got = torch.full_like(want, float("nan"))
            ext.run(*inp.args(), got)
            torch.cuda.synchronize()
            assert torch.equal(got, want), (m, k, n)
    with pytest.raises(RuntimeError, match="scale_x must have shape"):
        ext.run(inp.x, inp.scale_x[:, :1].contiguous(), inp.gate_proj_weight, inp.scale_gate, inp.up_proj_weight,
                inp.scale_up, got)
    with pytest.raises(RuntimeError, match="bfloat16"):
        ext.run(*inp.args(), got.float())


def test_problem_038_submission_equals_package_rmsnorm():
    from sol_execbench_b200_kernels_b200 import side_ops
    ext = _extension("38")
    dev = torch.device("cuda:0")
    q, k, wq, wk, eps = W.make_rmsnorm_inputs(333, 48, seed=1, device=dev)
    want_q, want_k = torch.empty_like(q), torch.empty_like(k)
    side_ops.rmsnorm_qk(q, k, wq, wk, eps, want_q, want_k)
    got_q, got_k = torch.empty_like(q), torch.empty_like(k)
    ext.run(q, k, wq, wk, eps, got_q, got_k)
    torch.cuda.synchronize()
    assert torch.equal(got_q, want_q) and torch.equal(got_k, want_k)
    with pytest.raises(RuntimeError, match="float32"):
        ext.run(q.half(), k, wq, wk, eps, got_q, got_k)


def test_problem_029_submission_equals_package_op():
    from sol_execbench_b200_kernels_b200 import side_ops
    ext = _extension("29")
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(2)
    hidden = (torch.randn(2, 150, 512, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    in_w = (torch.randn(256, 512, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    in_b = (torch.randn(256, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    _, mask, cw, cb = W.make_mamba_tail_inputs(2, 150, 128, 64, seed=2, device=dev)
    want_out, want_gate = side_ops.mamba_conv1d_with_gating(hidden, mask, in_w, in_b, cw, cb)
    got_out, got_gate = ext.run(hidden, mask, in_w, in_b, cw, cb)
    torch.cuda.synchronize()
    assert got_out.shape == (2, 128, 150) and got_gate.shape == (2, 128, 150)
    assert torch.equal(got_out, want_out) and torch.equal(got_gate, want_gate)
    assert got_gate.stride() == want_gate.stride()
