"""GPU parity of the side operators (problems 038 and 029) through the C ABI: against the CPU restatement on
seeded inputs, against fixtures made from the reference's own kernels, and — when the reference's extension was
built under oracle/_ref/ — against the reference kernel itself."""
import glob
import importlib.util
import json
import os

import pytest
import torch

from oracle import sideops_oracle as O
from sol_execbench_b200_kernels_b200 import workloads as W

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
# fp32 RMSNorm: the sum order and the hardware reciprocal square root (2 ulp) differ from the restatement
NORM_RTOL = NORM_ATOL = 4e-6


def _dev():
    return torch.device("cuda:0")


def _ref_ext(name):
    path = os.path.join(ROOT, "oracle", "_ref", name, name + ".so")
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("tokens,heads", [(1, 48), (3, 48), (128, 48), (129, 48), (1000, 48), (2048, 48), (77, 24),
                                          (33, 5), (5, 1)])
def test_rmsnorm_matches_oracle(tokens, heads):
    from sol_execbench_b200_kernels_b200 import side_ops
    q, k, wq, wk, eps = W.make_rmsnorm_inputs(tokens, heads, seed=tokens + heads, device=_dev())
    qn = torch.full_like(q, float("nan"))
    kn = torch.full_like(k, float("nan"))
    side_ops.rmsnorm_qk(q, k, wq, wk, eps, qn, kn)
    torch.cuda.synchronize()
    a, b = O.rmsnorm_qk(q.cpu(), k.cpu(), wq.cpu(), wk.cpu(), eps)
    torch.testing.assert_close(qn.cpu(), a, rtol=NORM_RTOL, atol=NORM_ATOL)
    torch.testing.assert_close(kn.cpu(), b, rtol=NORM_RTOL, atol=NORM_ATOL)


def test_rmsnorm_leading_dimensions_eps_and_empty_input():
    from sol_execbench_b200_kernels_b200 import side_ops
    g = torch.Generator().manual_seed(9)
    q = torch.randn(2, 7, 11, 48, 128, generator=g).to(_dev()) * 1e-3     # eps matters at this magnitude
    k = torch.randn(2, 7, 11, 48, 128, generator=g).to(_dev())
    wq = torch.randn(48, 128, generator=g).to(_dev())
    wk = torch.randn(48, 128, generator=g).to(_dev())
    qn, kn = torch.empty_like(q), torch.empty_like(k)
    side_ops.rmsnorm_qk(q, k, wq, wk, 1e-5, qn, kn)
    a, b = O.rmsnorm_qk(q.cpu(), k.cpu(), wq.cpu(), wk.cpu(), 1e-5)
    torch.testing.assert_close(qn.cpu(), a, rtol=NORM_RTOL, atol=NORM_ATOL)
    torch.testing.assert_close(kn.cpu(), b, rtol=NORM_RTOL, atol=NORM_ATOL)
    e = torch.empty(1, 0, 48, 128, device=_dev())
    side_ops.rmsnorm_qk(e, e, wq, wk, 1e-6, torch.empty_like(e), torch.empty_like(e))
    # rows of zeros stay zeros (rsqrt(eps) * 0)
    z = torch.zeros(1, 4, 48, 128, device=_dev())
    zn, zk = torch.full_like(z, 1.0), torch.full_like(z, 1.0)
    side_ops.rmsnorm_qk(z, z, wq, wk, 1e-6, zn, zk)
    assert float(zn.abs().max()) == 0.0 and float(zk.abs().max()) == 0.0


def test_rmsnorm_against_reference_kernel_outputs():
    from sol_execbench_b200_kernels_b200 import side_ops
    files = sorted(glob.glob(os.path.join(GOLDEN, "ref038_*.json")))
    assert files
    for jf in files:
        meta = json.load(open(jf))
        ref = torch.load(jf[:-5] + ".pt")
        q, k, wq, wk, eps = W.make_rmsnorm_inputs(meta["tokens"], meta["heads"], meta["seed"], _dev())
        qn, kn = torch.empty_like(q), torch.empty_like(k)
        side_ops.rmsnorm_qk(q, k, wq, wk, eps, qn, kn)
        rs = meta["row_stride"]
        torch.testing.assert_close(qn[0, ::rs].cpu(), ref["query_norm"], rtol=NORM_RTOL, atol=NORM_ATOL)
        torch.testing.assert_close(kn[0, ::rs].cpu(), ref["key_norm"], rtol=NORM_RTOL, atol=NORM_ATOL)


def test_rmsnorm_against_reference_kernel_when_built():
    ref = _ref_ext("ref038_rmsnorm_qk")
    if ref is None:
        pytest.skip("the reference's extension is not built under oracle/_ref/")
    from sol_execbench_b200_kernels_b200 import side_ops
    for tokens in (128, 640, 4608):
        q, k, wq, wk, eps = W.make_rmsnorm_inputs(tokens, 48, seed=tokens, device=_dev())
        qn, kn = torch.empty_like(q), torch.empty_like(k)
        rq, rk = torch.empty_like(q), torch.empty_like(k)
        side_ops.rmsnorm_qk(q, k, wq, wk, eps, qn, kn)
        ref.run(q, k, wq, wk, eps, rq, rk)
        torch.testing.assert_close(qn, rq, rtol=NORM_RTOL, atol=NORM_ATOL)
        torch.testing.assert_close(kn, rk, rtol=NORM_RTOL, atol=NORM_ATOL)


def _assert_tail_close(got, want, what=""):
    """bf16 result of four rounding steps, one of them after a sigmoid evaluated with hardware exp2 / reciprocal:
    bit-equal except where a rounding to bf16 falls the other way — at most 1e-3 of the elements, each by at
    most two bf16 steps of the result.  Magnitudes below 1e-30 are not compared: a sigmoid below the smallest
    normal fp32 (arguments under -87) is flushed to zero by the hardware exp2, as in the reference's kernel."""
    assert got.shape == want.shape and got.dtype == want.dtype
    g, w = got.float().cpu(), want.float().cpu()
    diff = (g - w).abs()
    bad = diff > 1e-30
    nbad = int(bad.sum())
    assert nbad <= max(2, 1e-3 * w.numel()), f"{what}: {nbad} of {w.numel()} differ"
    if nbad:
        assert bool((diff[bad] <= w.abs()[bad] * 2.0 ** -6).all()), f"{what}: a difference above two bf16 steps"


@pytest.mark.parametrize("batch,sequence,channels,width", [
    (1, 128, 64, 64), (1, 128, 128, 256), (2, 300, 128, 256), (3, 333, 64, 128), (2, 1000, 256, 512),
    (1, 1, 64, 128), (1, 3, 64, 128), (1, 4, 64, 128), (2, 129, 192, 200), (1, 256, 16384, 32768), (4, 131, 64, 64), (2, 1002, 64, 64), (1, 130, 128, 128)])
def test_mamba_tail_matches_oracle(batch, sequence, channels, width):
    from sol_execbench_b200_kernels_b200 import side_ops
    p, m, cw, cb = W.make_mamba_tail_inputs(batch, sequence, channels, width, seed=sequence + channels, device=_dev())
    out = torch.full((batch, channels, sequence), float("nan"), dtype=torch.bfloat16, device=_dev())
    side_ops.mamba_conv1d_tail(p, m, cw, cb, out)
    torch.cuda.synchronize()
    want = O.mamba_conv1d_tail(p.cpu(), m.cpu(), cw.cpu(), cb.cpu())
    _assert_tail_close(out, want, f"B{batch} L{sequence} C{channels}")
    masked = (m.cpu() < 0.5)[:, None, :].expand_as(want)
    assert bool((out.cpu()[masked] == 0).all())


def test_mamba_tail_extreme_values_and_empty_input():
    from sol_execbench_b200_kernels_b200 import side_ops
    p, m, cw, cb = W.make_mamba_tail_inputs(2, 200, 64, 64, seed=1, device=_dev(), padded=False)
    p = p * 40.0          # convolution results up to a few hundred either side: both sigmoid tails
    out = torch.empty(2, 64, 200, dtype=torch.bfloat16, device=_dev())
    side_ops.mamba_conv1d_tail(p, m, cw, cb, out)
    want = O.mamba_conv1d_tail(p.cpu(), m.cpu(), cw.cpu(), cb.cpu())
    assert bool(torch.isfinite(out.float()).all())
    _assert_tail_close(out, want, "large magnitudes")
    side_ops.mamba_conv1d_tail(p[:0], m[:0], cw, cb, out[:0])     # batch 0: nothing to launch
    # all masked: all zeros
    side_ops.mamba_conv1d_tail(p, torch.zeros_like(m), cw, cb, out)
    assert float(out.float().abs().max()) == 0.0


def test_mamba_tail_against_reference_kernel_outputs():
    from sol_execbench_b200_kernels_b200 import side_ops
    files = sorted(glob.glob(os.path.join(GOLDEN, "ref029_*.json")))
    assert files
    for jf in files:
        ref = torch.load(jf[:-5] + ".pt")
        px = ref["projected_x"]
        channels = px.shape[-1] // 64 * 64          # whole 64-channel tiles of the sampled channels
        p = px[:, :, :channels].contiguous().to(_dev())
        out = torch.empty(p.shape[0], channels, p.shape[1], dtype=torch.bfloat16, device=_dev())
        side_ops.mamba_conv1d_tail(p, ref["mask"].to(_dev()), ref["conv_w"][:channels].contiguous().to(_dev()),
                                   ref["conv_b"][:channels].contiguous().to(_dev()), out)
        _assert_tail_close(out, ref["output"][:, :channels], os.path.basename(jf))


def test_mamba_with_gating_matches_reference_op_when_built():
    ref = _ref_ext("ref029_mamba_conv1d")
    if ref is None:
        pytest.skip("the reference's extension is not built under oracle/_ref/")
    from sol_execbench_b200_kernels_b200 import side_ops
    g = torch.Generator().manual_seed(11)
    hidden = (torch.randn(2, 200, 8192, generator=g) * 0.5).to(torch.bfloat16).to(_dev())
    in_w = (torch.randn(32768, 8192, generator=g) * 0.02).to(torch.bfloat16).to(_dev())
    in_b = (torch.randn(32768, generator=g) * 0.1).to(torch.bfloat16).to(_dev())
    _, mask, cw, cb = W.make_mamba_tail_inputs(2, 200, 16384, 64, seed=11, device=_dev())
    want_out, want_gate = ref.run(hidden, mask, in_w, in_b, cw, cb)
    # same projection for both tails (the two GEMM libraries round differently): take the reference's
    projected = torch.empty(0, dtype=torch.bfloat16, device=_dev()).set_(
        want_gate.untyped_storage(), 0, (2, 200, 32768), (200 * 32768, 32768, 1))
    out = torch.empty(2, 16384, 200, dtype=torch.bfloat16, device=_dev())
    side_ops.mamba_conv1d_tail(projected, mask, cw, cb, out)
    _assert_tail_close(out, want_out, "reference tail")
    # whole op through this package's entry point: shapes, the gate view, and agreement within GEMM rounding
    got_out, got_gate = side_ops.mamba_conv1d_with_gating(hidden, mask, in_w, in_b, cw, cb)
    assert got_out.shape == want_out.shape and got_gate.shape == want_gate.shape
    assert got_gate.stride() == want_gate.stride()
    rel = float(torch.linalg.vector_norm(got_out.float() - want_out.float()) / torch.linalg.vector_norm(want_out.float()))
    assert rel <= 1e-2


# ------------------------------------------------------------------------------------------------------------
# Input projection of problem 029: bf16 GEMM + bias.  The exact (float64) result is rounded once to bf16 by an ideal
# implementation; fp32 accumulation over K in another order moves a value by far less than a rounding step, but can
# move it across a rounding boundary, so the bound is one bf16 step (2^-8 relative to the value) plus the
# accumulation error (a small multiple of 2^-24 of the sum of the products' magnitudes; 2^-16 of it is allowed).
# ------------------------------------------------------------------------------------------------------------
PROJ_SHAPES = [(1, 64, 8), (5, 8, 16), (127, 72, 264), (128, 256, 512), (129, 512, 256), (256, 64, 256),
               (300, 1024, 776), (257, 200, 1000), (1000, 520, 2048), (512, 8192, 1024), (2048, 1024, 4096)]


def _proj_inputs(m, k, n, seed):
    g = torch.Generator().manual_seed(seed)
    hidden = (torch.randn(m, k, generator=g) * 0.5).to(torch.bfloat16).to(_dev())
    weight = (torch.randn(n, k, generator=g) * 0.04).to(torch.bfloat16).to(_dev())
    bias = (torch.randn(n, generator=g) * 0.2).to(torch.bfloat16).to(_dev())
    return hidden, weight, bias


def _assert_proj_close(got, hidden, weight, bias, label):
    exact = O.mamba_in_proj(hidden, weight, bias, exact=True)              # float64, on the GPU
    mags = hidden.double().abs() @ weight.double().abs().t() + bias.double().abs()
    bound = exact.abs() * 2.0 ** -8 + mags * 2.0 ** -16 + 1e-30
    err = (got.double() - exact).abs()
    worst = float((err / bound).max())
    assert worst <= 1.0, f"{label}: error / bound = {worst}"
    # and the typical value is correctly rounded: most outputs equal the rounding of the exact result
    same = float((got == exact.to(torch.bfloat16)).double().mean())
    assert same >= 0.98, f"{label}: only {same:.4f} of the outputs equal the rounded exact result"


@pytest.mark.parametrize("shape", PROJ_SHAPES)
def test_mamba_in_proj_matches_exact_product(shape):
    from sol_execbench_b200_kernels_b200 import side_ops
    m, k, n = shape
    hidden, weight, bias = _proj_inputs(m, k, n, seed=m + k + n)
    got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=_dev())
    side_ops.mamba_in_proj(hidden, weight, bias, got)
    torch.cuda.synchronize()
    assert side_ops.last_status() == (0, 0)
    assert torch.isfinite(got.float()).all()
    _assert_proj_close(got, hidden, weight, bias, str(shape))
    # the CPU restatement (fp32 accumulation in the library's order) agrees within the same bound
    if m * k * n <= 300 * 1024 * 776:
        want = O.mamba_in_proj(hidden.cpu(), weight.cpu(), bias.cpu())
        _assert_proj_close(want.to(_dev()), hidden, weight, bias, f"oracle {shape}")
        assert float((got.cpu() == want).double().mean()) >= 0.98


def test_mamba_in_proj_is_deterministic_and_leaves_neighbours_alone():
    from sol_execbench_b200_kernels_b200 import side_ops
    m, k, n = 333, 512, 520
    hidden, weight, bias = _proj_inputs(m, k, n, seed=4)
    # the destination sits inside a larger allocation: rows before and after it must keep their contents
    buf = torch.full((m + 2, n), 7.0, dtype=torch.bfloat16, device=_dev())
    out = buf[1:m + 1]
    side_ops.mamba_in_proj(hidden, weight, bias, out)
    first = out.clone()
    side_ops.mamba_in_proj(hidden, weight, bias, out)
    torch.cuda.synchronize()
    assert torch.equal(out, first)
    assert (buf[0] == 7.0).all() and (buf[m + 1] == 7.0).all()
    # 3-D input as the operator passes it, and a row count of zero
    out3 = torch.empty(3, 111, n, dtype=torch.bfloat16, device=_dev())
    side_ops.mamba_in_proj(hidden.reshape(3, 111, k), weight, bias, out3)
    assert torch.equal(out3.reshape(m, n), first)
    side_ops.mamba_in_proj(hidden[:0], weight, bias, out[:0])


def test_mamba_in_proj_pair_and_lone_kernels_agree_on_shared_rows():
    """Rows are independent: the first 128 rows computed by the lone-CTA kernel (M = 128) equal the same rows of a
    larger problem computed by the pair kernel, bit for bit (same K order, same epilogue)."""
    from sol_execbench_b200_kernels_b200 import side_ops
    k, n = 1024, 768
    hidden, weight, bias = _proj_inputs(512, k, n, seed=6)
    big = torch.empty(512, n, dtype=torch.bfloat16, device=_dev())
    small = torch.empty(128, n, dtype=torch.bfloat16, device=_dev())
    side_ops.mamba_in_proj(hidden, weight, bias, big)
    side_ops.mamba_in_proj(hidden[:128], weight, bias, small)
    torch.cuda.synchronize()
    assert torch.equal(big[:128], small)


def test_mamba_in_proj_rejects_what_the_contract_excludes():
    from sol_execbench_b200_kernels_b200 import side_ops
    hidden, weight, bias = _proj_inputs(16, 64, 64, seed=8)
    out = torch.empty(16, 64, dtype=torch.bfloat16, device=_dev())
    with pytest.raises(ValueError, match="bfloat16"):
        side_ops.mamba_in_proj(hidden.float(), weight, bias, out)
    with pytest.raises(ValueError, match="in_proj_bias"):
        side_ops.mamba_in_proj(hidden, weight, bias[:32], out)
    with pytest.raises(ValueError, match="multiples of 8"):
        side_ops.mamba_in_proj(hidden[:, :60].contiguous(), weight[:, :60].contiguous(), bias, out)
    with pytest.raises(ValueError, match="contiguous"):
        side_ops.mamba_in_proj(hidden, weight.t().contiguous().t(), bias, out)
    with pytest.raises(ValueError, match="projected"):
        side_ops.mamba_in_proj(hidden, weight, bias, out[:8])
