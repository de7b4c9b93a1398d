"""Activation quantiser on the GPU against the torch implementation that generates every other test's
inputs (`workloads.quantize_activation_1x128`, run on the CPU): e4m3 bytes and fp32 scales must be
identical, for bf16 and fp32 inputs."""
import pytest
import torch

from sol_execbench_b200_kernels_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _compare(x_cpu):
    import sol_execbench_b200_kernels_b200 as pkg

    q_ref, s_ref = W.quantize_activation_1x128(x_cpu.float())
    q, s = pkg.quantize_activation(x_cpu.to("cuda:0"))
    torch.cuda.synchronize()
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float32
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    # third statement of the same bytes: the integer restatement of the e4m3 rounding (numpy)
    from oracle import quantize_oracle as Q
    q_np, s_np = Q.quantize_activation_1x128(x_cpu.float().numpy())
    assert (q.cpu().view(torch.uint8).numpy() == q_np).all() and (s.cpu().numpy() == s_np).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 128), (7, 384), (128, 4096), (1000, 7168), (4096, 512), (33, 128 * 61)])
def test_quantizer_bits_match_torch(shape, dtype):
    gen = torch.Generator().manual_seed(shape[0] * 7919 + shape[1])
    x = torch.randn(*shape, generator=gen).to(dtype)
    _compare(x)


def test_quantizer_edge_values():
    x = torch.zeros(4, 256)
    x[1, :128] = 1e-30            # amax below the clamp floor
    x[2, 5] = 3.0e38              # huge block maximum
    x[2, 6] = -3.0e38
    x[3] = torch.linspace(-5, 5, 256)
    _compare(x)
    _compare(x.to(torch.bfloat16))


def test_quantizer_keeps_the_sign_of_zero():
    # -0.0 in, and negatives so small that their quotient rounds to zero: e4m3 0x80, as the torch quantiser gives
    x = torch.randn(8, 256, generator=torch.Generator().manual_seed(5))
    x[0, 3] = -0.0
    x[1, 100:140] = -0.0
    x[2, 7] = -1e-12
    x[3, :128] = -0.0                # a whole block of negative zeros (amax 0: the clamp floor sets the scale)
    x[4, 130] = -1e-30
    for dtype in (torch.float32, torch.bfloat16):
        _compare(x.to(dtype))
    q, _ = W.quantize_activation_1x128(x)
    assert int(q.view(torch.uint8)[0, 3]) == 0x80    # (the reference quantiser itself keeps the sign)


def test_quantizer_pitched_rows_and_outputs_feed_run():
    import sol_execbench_b200_kernels_b200 as pkg

    m, k, n = 200, 512, 256
    wide = torch.randn(m, k + 128, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to("cuda:0")
    x = wide[:, :k]                                   # row pitch k + 128
    q, s = pkg.quantize_activation(x)
    q_ref, s_ref = W.quantize_activation_1x128(x.cpu().float())
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s.cpu(), s_ref)
    # the quantiser's outputs are exactly what `run` takes
    inp = W.make_inputs(m, k, n, seed=15).to("cuda:0")
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda:0")
    pkg.run(q, s, inp.gate_proj_weight, inp.scale_gate, inp.up_proj_weight, inp.scale_up, out)
    torch.cuda.synchronize()
    assert pkg.last_status()[0] == 0 and torch.isfinite(out.float()).all()


def test_quantizer_argument_errors():
    import sol_execbench_b200_kernels_b200 as pkg

    with pytest.raises(ValueError, match="CUDA"):
        pkg.quantize_activation(torch.zeros(2, 128))
    with pytest.raises(ValueError, match="multiple of 128"):
        pkg.quantize_activation(torch.zeros(2, 100, device="cuda:0"))
    with pytest.raises(ValueError, match="bf16 or fp32"):
        pkg.quantize_activation(torch.zeros(2, 128, device="cuda:0", dtype=torch.float16))
    with pytest.raises(ValueError, match="row-major"):
        pkg.quantize_activation(torch.zeros(128, 2, device="cuda:0").t())
