"""The bounded-wait protocol, run to its limit on a GPU without faulting anything.

`gu_wait_probe` launches one CTA whose only wait is on a barrier that nothing ever arrives on — the same
`mbar_wait` / `WaitCtx::fail` / abort-flag code the real kernels wait with, with no copy or MMA in flight.  With the
limit lowered to a few milliseconds the launch must return by itself, `gu_last_status` must name the wait that
gave up, and the context must stay usable (a normal call afterwards is correct).  The reference has nothing of the
kind: its cluster wait spins without bound (variants/cute_fused_v1/blockwise_gemm_fused.py:85-91).
"""
import time

import pytest
import torch

from oracle import gateup_oracle as O
from sol_execbench_b200_kernels_b200 import workloads as W

pytestmark = pytest.mark.gpu

WAIT_PROBE_ID = 31


def test_bounded_wait_runs_out_reports_and_leaves_the_context_usable():
    import sol_execbench_b200_kernels_b200 as pkg
    from sol_execbench_b200_kernels_b200 import _cabi

    pkg.last_status(clear=True)
    stream = torch.cuda.current_stream().cuda_stream
    assert _cabi.lib.gu_set_wait_limit_ns(3_000_000) == 0          # 3 ms instead of 2 s
    try:
        t0 = time.perf_counter()
        assert _cabi.lib.gu_wait_probe(stream) == 0
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
        assert elapsed < 1.0, f"the wait did not give up at its limit ({elapsed:.3f} s)"
        code, detail = pkg.last_status(clear=True)
        assert code == _cabi.GU_ETIMEOUT
        assert (detail >> 24) & 0xFF == WAIT_PROBE_ID and (detail & 0xFFFFFF) == 0   # wait id, block 0
        assert pkg.last_status() == (0, 0)                          # cleared
    finally:
        assert _cabi.lib.gu_set_wait_limit_ns(0) == 0               # back to the default
    # the context is intact: both tile kernels and the streaming kernel still give the right bits
    for shape, plan in (((300, 512, 384), "tile"), ((100, 384, 256), "tile_dp"), ((16, 1024, 1024), "stream")):
        inp = W.make_inputs(*shape, seed=12)
        g = inp.to("cuda:0")
        out = torch.empty(shape[0], shape[2], dtype=torch.bfloat16, device="cuda:0")
        pkg.run_with_plan(*g.args(), out, plan)
        torch.cuda.synchronize()
        assert pkg.last_status() == (0, 0)
        st = O.error_stats(out, O.gateup_blockwise(*inp.args()))
        assert st["max_abs"] <= 2e-2 and st["rel_l2"] <= 1e-4, (shape, plan, st)


def test_wait_limit_setter_round_trip():
    from sol_execbench_b200_kernels_b200 import _cabi

    assert _cabi.lib.gu_set_wait_limit_ns(5_000_000_000) == 0
    assert _cabi.lib.gu_set_wait_limit_ns(0) == 0


def test_peer_barrier_gives_up_on_a_rank_that_never_arrives_and_passes_once_it_has():
    """`gu_peer_barrier` for rank 0 of 2 with nobody stamping for rank 1: the launch must return at its time limit
    and name the missing rank; rank 1's own barrier, launched afterwards, finds rank 0's stamp and passes at once.
    (The two ranks' flag arrays live on this one GPU; no kernel ever waits for a kernel launched after it to finish
    normally — the first launch is meant to run out.)"""
    import sol_execbench_b200_kernels_b200 as pkg
    from sol_execbench_b200_kernels_b200 import _cabi

    dev = torch.device("cuda:0")
    pkg.last_status(clear=True)
    flags = torch.zeros(2, 64, dtype=torch.int32, device=dev)
    ptrs = [flags[0].data_ptr(), flags[1].data_ptr()]
    t0 = time.perf_counter()
    pkg.peer_barrier(ptrs, 0, dev, limit_ns=3_000_000)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    code, detail = pkg.last_status(clear=True)
    assert code == _cabi.GU_ETIMEOUT and (detail >> 24) & 0xFF == 20 and (detail & 0xFF) == 1   # rank 1 is missing
    pkg.peer_barrier(ptrs, 1, dev, limit_ns=3_000_000)
    torch.cuda.synchronize()
    assert pkg.last_status() == (0, 0)
    f = flags.cpu()
    assert f[0, 0] == 1 and f[0, 1] == 1 and f[1, 0] == 1 and f[1, 1] == 1     # both ranks stamped both arrays
    assert f[0, 16] == 1 and f[1, 16] == 1                                     # both have passed barrier number 1
    # a barrier of one rank needs nobody else
    solo = torch.zeros(64, dtype=torch.int32, device=dev)
    for expect in (1, 2, 3):
        pkg.peer_barrier([solo.data_ptr()], 0, dev)
        torch.cuda.synchronize()
        assert pkg.last_status() == (0, 0) and int(solo[16]) == expect
