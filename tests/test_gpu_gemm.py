"""The tile kernel in single-projection mode (plain block-scaled FP8 GEMM, bf16 out) against the oracle."""
import pytest
import torch

from oracle import gateup_oracle as O
from sol_execbench_b200_kernels_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _operands(m, k, n, seed):
    gen = torch.Generator().manual_seed(seed)
    a, sa = W.quantize_activation_1x128(torch.randn(m, k, generator=gen))
    b, sb = W.quantize_weight_128x128(torch.randn(n, k, generator=gen) * 0.02)
    return a, sa, b, sb


@pytest.mark.parametrize("shape", [(128, 128, 128), (128, 256, 256), (100, 384, 384), (300, 512, 640), (257, 1024, 128),
                                   (512, 14336 // 4, 1024), (64, 2048, 4096)])
def test_blockwise_gemm_parity(shape):
    import sol_execbench_b200_kernels_b200 as pkg

    m, k, n = shape
    a, sa, b, sb = _operands(m, k, n, seed=40 + m)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    pkg.blockwise_gemm(a.cuda(), sa.cuda(), b.cuda(), sb.cuda(), out)
    torch.cuda.synchronize()
    assert pkg.last_status()[0] == 0
    for ref in (O.gemm_blockwise(a, sa, b, sb), O.gemm_dequant(a, sa, b, sb)):
        st = O.error_stats(out, ref)
        assert st["finite"] and not st["all_zero"], st
        assert st["rel_l2"] <= 1e-2, st
        # one bf16 ulp of the result is the worst a correct sum in another order can be off by
        assert st["max_abs"] <= max(2e-2, 2 ** -7 * float(ref.float().abs().max())), st
    assert torch.equal(out.cpu(), O.gemm_blockwise(a, sa, b, sb)) or O.error_stats(out, O.gemm_blockwise(a, sa, b, sb))["rel_l2"] < 1e-4


@pytest.mark.parametrize("shape", [(300, 512, 640), (513, 1024, 384), (1024, 2048, 128), (777, 256, 1152)])
def test_blockwise_gemm_on_cta_pairs_equals_the_lone_cta_kernel_row_block_by_row_block(shape):
    # more than 128 rows run on CTA pairs (256 x 256 tiles); token rows are independent, so the same rows fed in
    # blocks of at most 128 (the lone-CTA kernel) must give the same bits — including an odd number of column blocks
    import sol_execbench_b200_kernels_b200 as pkg

    m, k, n = shape
    a, sa, b, sb = (t.cuda() for t in _operands(m, k, n, seed=60 + m))
    whole = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    pkg.blockwise_gemm(a, sa, b, sb, whole)
    pieces = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    for lo in range(0, m, 128):
        hi = min(m, lo + 128)
        pkg.blockwise_gemm(a[lo:hi].contiguous(), sa[lo:hi].contiguous(), b, sb, pieces[lo:hi])
    torch.cuda.synchronize()
    assert pkg.last_status()[0] == 0
    assert torch.equal(whole, pieces)


def test_blockwise_gemm_pitched_output_and_errors():
    import sol_execbench_b200_kernels_b200 as pkg

    m, k, n = 130, 256, 384
    a, sa, b, sb = _operands(m, k, n, seed=41)
    wide = torch.full((m, n + 128), 5.0, dtype=torch.bfloat16, device="cuda:0")
    pkg.blockwise_gemm(a.cuda(), sa.cuda(), b.cuda(), sb.cuda(), wide[:, :n])
    torch.cuda.synchronize()
    assert (wide[:, n:] == 5.0).all()
    assert O.error_stats(wide[:, :n], O.gemm_blockwise(a, sa, b, sb))["rel_l2"] <= 1e-3
    with pytest.raises(ValueError, match="scale_b"):
        pkg.blockwise_gemm(a.cuda(), sa.cuda(), b.cuda(), sb.cuda()[:, :1], wide[:, :n])
    with pytest.raises(ValueError, match="CUDA"):
        pkg.blockwise_gemm(a, sa, b, sb, torch.empty(m, n, dtype=torch.bfloat16))


@pytest.mark.parametrize("shape", [(128, 256, 128), (129, 128, 128), (256, 256, 256), (300, 512, 384), (1000, 1024, 640),
                                   (2048, 512, 1792), (256, 128, 14336), (100, 128, 14336)])  # (the last two have -0.0 outputs)
def test_fp8_output_epilogue_equals_quantising_the_bf16_result(shape):
    """Fused re-quantisation: e4m3 bytes and scales identical to quantising `run`'s bf16 output afterwards."""
    import sol_execbench_b200_kernels_b200 as pkg

    m, k, n = shape
    inp = W.make_inputs(m, k, n, seed=50 + m).to("cuda:0")
    ref = torch.empty(m, n, dtype=torch.bfloat16, device="cuda:0")
    pkg.run_with_plan(*inp.args(), ref, "tile_dp")
    q = torch.zeros(m, n, dtype=torch.uint8, device="cuda:0").view(torch.float8_e4m3fn)
    s = torch.zeros(m, n // 128, dtype=torch.float32, device="cuda:0")
    pkg.run_fp8_output(*inp.args(), q, s)
    torch.cuda.synchronize()
    assert pkg.last_status()[0] == 0
    q_ref, s_ref = W.quantize_activation_1x128(ref.cpu().float())
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))


def test_mlp_block_against_oracle_chain():
    import sol_execbench_b200_kernels_b200 as pkg

    m, h, n = 200, 512, 1024
    gen = torch.Generator().manual_seed(60)
    x = torch.randn(m, h, generator=gen).to(torch.bfloat16)
    gq, sg = W.quantize_weight_128x128(torch.randn(n, h, generator=gen) * 0.02)
    uq, su = W.quantize_weight_128x128(torch.randn(n, h, generator=gen) * 0.02)
    dq, sd = W.quantize_weight_128x128(torch.randn(h, n, generator=gen) * 0.02)
    out = pkg.mlp_block(x.cuda(), gq.cuda(), sg.cuda(), uq.cuda(), su.cuda(), dq.cuda(), sd.cuda())
    torch.cuda.synchronize()
    assert pkg.last_status()[0] == 0
    # the same chain on the CPU: quantise, gate/up + SwiGLU (bf16), quantise, down projection
    xq, sx = W.quantize_activation_1x128(x.float())
    mid = O.gateup_blockwise(xq, sx, gq, sg, uq, su)
    mq, ms = W.quantize_activation_1x128(mid.float())
    ref = O.gemm_blockwise(mq, ms, dq, sd)
    st = O.error_stats(out, ref)
    assert st["finite"] and not st["all_zero"] and st["rel_l2"] <= 1e-2 and st["max_abs"] <= 2e-2, st
