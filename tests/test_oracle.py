"""CPU checks of the oracle itself: the two restatements against each other, against an
independent scalar evaluation, and against the committed golden fixtures."""
import glob
import json
import os

import numpy as np
import pytest
import torch

from oracle import gateup_oracle as O
from sol_execbench_b200_kernels_b200 import workloads as W

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_quantizers_scale_and_range():
    torch.manual_seed(3)
    x = torch.randn(5, 256)
    q, s = W.quantize_activation_1x128(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (5, 2)
    assert torch.allclose(s, x.reshape(5, 2, 128).abs().amax(-1) / 448.0)
    assert torch.isfinite(q.float()).all() and q.float().abs().max() <= 448
    # the largest element of every block lands exactly on +-448
    assert (q.float().reshape(5, 2, 128).abs().amax(-1) == 448).all()
    w = torch.randn(256, 384) * 0.02
    qw, sw = W.quantize_weight_128x128(w)
    assert sw.shape == (2, 3)
    deq = O.dequantize(qw, sw, 128)
    assert (deq - w).abs().max() <= sw.max() * 32  # half an e4m3 ulp at the top binade is 16 quanta


def test_quantizer_zero_block_is_finite():
    x = torch.zeros(2, 128)
    q, s = W.quantize_activation_1x128(x)
    assert torch.isfinite(s).all() and (q.float() == 0).all()


def test_quantizer_rejects_ragged_k():
    with pytest.raises(ValueError):
        W.quantize_activation_1x128(torch.zeros(2, 100))
    with pytest.raises(ValueError):
        W.quantize_weight_128x128(torch.zeros(100, 128))


def _scalar_oracle(inp):
    """Independent float64 evaluation, element by element in numpy (tiny shapes only)."""
    x = inp.x.float().double().numpy()
    sx = inp.scale_x.double().numpy()
    res = []
    for w, s in ((inp.gate_proj_weight, inp.scale_gate), (inp.up_proj_weight, inp.scale_up)):
        wd = w.float().double().numpy()
        sd = s.double().numpy()
        m, k = x.shape
        n = wd.shape[0]
        acc = np.zeros((m, n))
        for j in range(k // 128):
            part = x[:, j * 128:(j + 1) * 128] @ wd[:, j * 128:(j + 1) * 128].T
            acc += part * sx[:, j:j + 1] * np.repeat(sd[:, j], 128)[None, :]
        res.append(torch.from_numpy(acc).float())
    return O.swiglu_bf16(res[0], res[1])


@pytest.mark.parametrize("shape", [(3, 128, 128), (17, 384, 256), (128, 512, 384)])
def test_restatements_agree(shape):
    inp = W.make_inputs(*shape, seed=11)
    a = O.gateup_dequant(*inp.args())
    b = O.gateup_blockwise(*inp.args())
    c = _scalar_oracle(inp)
    for lhs, rhs in ((a, c), (b, c), (a, b)):
        st = O.error_stats(lhs, rhs)
        assert st["finite"] and st["rel_l2"] <= 1e-3 and st["max_abs"] <= 2e-2, st


def test_small_config_oracles_within_north_star_tolerance():
    m, k, n = W.SHAPES["small"]
    inp = W.make_inputs(m, k, n, seed=0)
    a = O.gateup_dequant(*inp.args())
    b = O.gateup_blockwise(*inp.args())
    st = O.error_stats(a, b)
    assert st["max_abs"] <= 2e-2 and st["rel_l2"] <= 1e-2, st
    assert a.dtype == torch.bfloat16 and tuple(a.shape) == (m, n)


def test_swiglu_rounding_boundaries():
    g = torch.tensor([[1.00390625, -3.0, 20.0, -100.0]])   # 1.00390625 is not a bf16 value
    u = torch.tensor([[2.0, 0.5, 1.0, 1.0]])
    out = O.swiglu_bf16(g, u)
    gb = g.to(torch.bfloat16).float()
    act = (gb * torch.sigmoid(gb)).to(torch.bfloat16)
    assert torch.equal(out, (act.float() * u.to(torch.bfloat16).float()).to(torch.bfloat16))
    assert out[0, 3] == 0


def test_row_and_column_restriction_are_exact():
    inp = W.make_inputs(40, 256, 384, seed=5)
    full = O.gateup_blockwise(*inp.args())
    rows = torch.tensor([3, 17, 39])
    assert torch.equal(O.gateup_blockwise(*inp.rows(rows).args()), full[rows])
    blocks = torch.tensor([2, 0])
    cols = (blocks[:, None] * 128 + torch.arange(128)[None]).reshape(-1)
    assert torch.equal(O.gateup_blockwise(*inp.column_blocks(blocks).args()), full[:, cols])


def _fixtures():
    return sorted(glob.glob(os.path.join(GOLDEN, "ref_*.json")))


@pytest.mark.parametrize("meta_path", _fixtures() or [None])
def test_golden_fixtures(meta_path):
    """Outputs of the reference submission's own GPU kernel on seeded inputs, regenerated here from the seed."""
    if meta_path is None:
        pytest.skip("no golden fixtures committed yet")
    with open(meta_path) as f:
        meta = json.load(f)
    data = torch.load(meta_path[:-5] + ".pt", weights_only=True)
    m, k, n = meta["shape"]
    inp = W.make_inputs(m, k, n, seed=meta["seed"])
    rows, cols = data["rows"], data["cols"]
    sub = inp.rows(rows)
    for name, fn in (("blockwise", O.gateup_blockwise), ("dequant", O.gateup_dequant)):
        got = fn(*sub.args())[:, cols]
        st = O.error_stats(got, data["out"])
        assert st["rel_l2"] <= 1e-2, (name, st)
        assert st["frac_over_atol"] <= 1e-4, (name, st)


# ---------------------------------------------------------------------------------------------
# the quantiser's integer / byte restatement (numpy) against torch's cast and the torch quantiser
# ---------------------------------------------------------------------------------------------
def _torch_e4m3_bytes(values):
    import numpy as np
    return torch.from_numpy(np.asarray(values, dtype=np.float32)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def test_e4m3_encoding_restatement_equals_the_library_cast():
    import numpy as np
    from oracle import quantize_oracle as Q

    # every bf16 value in range (both signs, zeros, subnormals of the target)
    v = (np.arange(0, 1 << 16, dtype=np.uint32) << 16).view(np.float32)
    v = v[np.isfinite(v) & (np.abs(v) <= 448)]
    assert np.array_equal(Q.encode_e4m3fn(v), _torch_e4m3_bytes(v))
    # all 256 bytes decode like the library type and encode back to themselves
    codes = np.arange(256, dtype=np.uint8)
    dec = Q.decode_e4m3fn(codes)
    lib = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.isnan(dec), np.isnan(lib)) and np.array_equal(dec[~np.isnan(dec)], lib[~np.isnan(lib)])
    fin = ~np.isnan(dec)
    assert np.array_equal(Q.encode_e4m3fn(dec[fin]), codes[fin])
    # exact ties between neighbouring codes go to the even code
    mag = dec[:0x7F].astype(np.float64)
    ties = ((mag[:-1] + mag[1:]) / 2).astype(np.float32)
    assert np.array_equal(Q.encode_e4m3fn(ties), _torch_e4m3_bytes(ties))
    assert np.array_equal(Q.encode_e4m3fn(-ties), _torch_e4m3_bytes(-ties))
    # random magnitudes over the whole range, NaN, saturation
    rng = np.random.default_rng(0)
    r = (rng.standard_normal(400_000) * rng.choice([1e-3, 0.02, 1.0, 50.0, 300.0], 400_000)).astype(np.float32)
    r = np.clip(r, -448, 448)
    assert np.array_equal(Q.encode_e4m3fn(r), _torch_e4m3_bytes(r))
    special = np.array([np.nan, 1e9, -1e9, 463.9, 464.0, 448.0, -448.0], dtype=np.float32)
    assert list(Q.encode_e4m3fn(special)) == [0x7F, 0x7E, 0xFE, 0x7E, 0x7E, 0x7E, 0xFE]


@pytest.mark.parametrize("m,k", [(3, 128), (17, 384), (64, 1024)])
def test_quantiser_restatement_equals_the_torch_quantiser(m, k):
    import numpy as np
    from oracle import quantize_oracle as Q

    g = torch.Generator().manual_seed(m * k)
    x = torch.randn(m, k, generator=g) * torch.rand(m, 1, generator=g) * 8
    x[0, :128] = 0.0                                   # an all-zero block: scale = 1e-12 / 448
    x[-1, 5] = 3e4
    want_q, want_s = W.quantize_activation_1x128(x)
    got_q, got_s = Q.quantize_activation_1x128(x.numpy())
    assert np.array_equal(got_s, want_s.numpy())
    assert np.array_equal(got_q, want_q.view(torch.uint8).numpy())
    # bf16 activations are quantised from their exact fp32 values
    xb = x.to(torch.bfloat16)
    want_q, want_s = W.quantize_activation_1x128(xb.float())
    got_q, got_s = Q.quantize_activation_1x128(xb.float().numpy())
    assert np.array_equal(got_s, want_s.numpy()) and np.array_equal(got_q, want_q.view(torch.uint8).numpy())


# ---------------------------------------------------------------------------------------------
# the plain C restatement (oracle/gateup_oracle.c): no tensor library underneath
# ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def c_oracle():
    from oracle import build_c
    return build_c.load()


def _run_c(lib, inp):
    m, k = inp.x.shape
    n = inp.gate_proj_weight.shape[0]
    out = torch.empty(m, n, dtype=torch.int16)
    keep = [t.contiguous() for t in (inp.x.view(torch.uint8), inp.scale_x, inp.gate_proj_weight.view(torch.uint8),
                                     inp.scale_gate, inp.up_proj_weight.view(torch.uint8), inp.scale_up)]
    assert lib.gateup_oracle_c(*[t.data_ptr() for t in keep], out.data_ptr(), m, k, n) == 0
    return out.view(torch.bfloat16)


@pytest.mark.parametrize("shape", [(1, 128, 128), (16, 256, 256), (40, 512, 384), (129, 384, 256)])
def test_c_restatement_equals_the_block_ordered_oracle(c_oracle, shape):
    inp = W.make_inputs(*shape, seed=3)
    got = _run_c(c_oracle, inp)
    want = O.gateup_blockwise(*inp.args())
    # same order, same rounding boundaries; the sigmoid comes from libm here and from torch there, so a rounding
    # to bf16 may, rarely, fall the other way
    diff = (got.float() - want.float()).abs()
    assert int((diff > 0).sum()) <= max(1, 1e-4 * got.numel())
    assert O.error_stats(got, want)["rel_l2"] <= 1e-4
    st = O.error_stats(got, O.gateup_dequant(*inp.args()))
    assert st["rel_l2"] <= 1e-2 and st["frac_over_atol"] <= 1e-4


def test_c_restatement_of_the_single_gemm(c_oracle):
    inp = W.make_inputs(24, 384, 256, seed=8)
    out = torch.empty(24, 256, dtype=torch.int16)
    keep = [inp.x.view(torch.uint8).contiguous(), inp.scale_x, inp.gate_proj_weight.view(torch.uint8).contiguous(),
            inp.scale_gate]
    assert c_oracle.gemm_oracle_c(*[t.data_ptr() for t in keep], out.data_ptr(), 24, 384, 256) == 0
    want = O.gemm_blockwise(inp.x, inp.scale_x, inp.gate_proj_weight, inp.scale_gate)
    assert torch.equal(out.view(torch.bfloat16), want)
    assert c_oracle.gemm_oracle_c(*[t.data_ptr() for t in keep], out.data_ptr(), 24, 100, 256) == -1


@pytest.mark.parametrize("name", ["ref_square_128x512x512", "ref_256x1024x1024"])
def test_c_restatement_against_reference_kernel_outputs(c_oracle, name):
    """The same fixtures as above (outputs of the reference's own GPU kernel), against the C statement."""
    meta_path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name + ".json")
    if not os.path.exists(meta_path):
        pytest.skip("fixture not committed")
    with open(meta_path) as f:
        meta = json.load(f)
    data = torch.load(meta_path[:-5] + ".pt", weights_only=True)
    m, k, n = meta["shape"]
    inp = W.make_inputs(m, k, n, seed=meta["seed"])
    got = _run_c(c_oracle, inp.rows(data["rows"]))[:, data["cols"]]
    st = O.error_stats(got, data["out"])
    assert st["rel_l2"] <= 1e-4 and st["frac_over_atol"] <= 1e-4, st
