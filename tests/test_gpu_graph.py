"""A launch recorded in a CUDA graph must stay correct when it is replayed: the tile kernel keeps no state between
launches, and the weight-streaming kernel and the pair kernel's stream-K schedule (the last shape) take the epoch of
their hand-off flags from a counter in the workspace, not from the host.  Each replay runs on new activations written into the captured buffers."""
import pytest
import torch

from sol_execbench_b200_kernels_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(16, 4096, 8192), (8, 8192, 28672), (32, 8192, 28672), (256, 1024, 2048),
                                   (512, 384, 4864)])
def test_replayed_graph_equals_eager_calls(shape):
    import sol_execbench_b200_kernels_b200 as pkg

    m, k, n = shape
    dev = torch.device("cuda:0")
    base = W.make_inputs(m, k, n, seed=3, device=dev)
    x = base.x.clone()
    sx = base.scale_x.clone()
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    args = (x, sx, base.gate_proj_weight, base.scale_gate, base.up_proj_weight, base.scale_up, out)
    pkg.run(*args)                      # first call outside the capture: attributes, descriptors
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        pkg.run(*args)
    for trial in range(4):
        fresh = W.make_inputs(m, k, n, seed=10 + trial, device=dev)
        x.view(torch.uint8).copy_(fresh.x.view(torch.uint8))
        sx.copy_(fresh.scale_x)
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert pkg.last_status()[0] == 0
        want = torch.empty_like(out)
        pkg.run(x, sx, base.gate_proj_weight, base.scale_gate, base.up_proj_weight, base.scale_up, want)
        torch.cuda.synchronize()
        assert torch.equal(out, want), f"replay {trial} of {shape} (plan {pkg.select_plan(m, k, n)})"


def test_replays_and_eager_calls_may_interleave_on_one_workspace():
    import sol_execbench_b200_kernels_b200 as pkg

    m, k, n = 16, 4096, 8192
    dev = torch.device("cuda:0")
    inp = W.make_inputs(m, k, n, seed=5, device=dev)
    out_a = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    out_b = torch.empty_like(out_a)
    pkg.run(*inp.args(), out_a)
    torch.cuda.synchronize()
    want = out_a.clone()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        pkg.run(*inp.args(), out_b)     # the workspace of this stream exists before the capture
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            pkg.run(*inp.args(), out_b)
        for _ in range(3):
            out_b.zero_()
            graph.replay()
            pkg.run(*inp.args(), out_a)
            graph.replay()
        stream.synchronize()
    torch.cuda.synchronize()
    assert pkg.last_status()[0] == 0
    assert torch.equal(out_a, want) and torch.equal(out_b, want)
