"""Column-parallel sharding: index arithmetic and the gather layout, exercised with
world_size-2 (and 4) gloo ranks on CPU.  The per-rank arithmetic is done by the oracle here;
the GPU tests cover the kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gateup_oracle as O
from sol_execbench_b200_kernels_b200 import workloads as W
from sol_execbench_b200_kernels_b200.sharded import (assemble_gathered, gather_columns, shard_bounds,
                                                      shard_concat_weights, shard_down_weights, shard_weights)


def test_shard_bounds_cover_and_tile():
    n = 18432
    for world in (1, 2, 4, 8):
        edges = [shard_bounds(n, r, world) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
            assert a1 == b0
        assert all((hi - lo) % 128 == 0 and hi - lo == n // world for lo, hi in edges)


def test_shard_bounds_errors():
    with pytest.raises(ValueError):
        shard_bounds(128 * 3, 0, 2)        # 3 column blocks over 2 ranks
    with pytest.raises(ValueError):
        shard_bounds(1000, 0, 2)           # not a multiple of 128
    with pytest.raises(ValueError):
        shard_bounds(256, 2, 2)            # rank out of range
    with pytest.raises(ValueError):
        shard_bounds(256, 0, 0)


def test_shards_are_views_and_match_concat_form():
    inp = W.make_inputs(8, 256, 512, seed=4)
    w = torch.cat([inp.gate_proj_weight.view(torch.uint8), inp.up_proj_weight.view(torch.uint8)]).view(torch.float8_e4m3fn)
    sw = torch.cat([inp.scale_gate, inp.scale_up])
    for r in range(2):
        a = shard_weights(inp.gate_proj_weight, inp.scale_gate, inp.up_proj_weight, inp.scale_up, r, 2)
        b = shard_concat_weights(w, sw, r, 2)
        assert a[0].data_ptr() == inp.gate_proj_weight[r * 256:].data_ptr() and a[0].is_contiguous()
        for ta, tb in zip(a, b):
            assert torch.equal(ta.view(torch.uint8) if ta.dtype == torch.float8_e4m3fn else ta,
                               tb.view(torch.uint8) if tb.dtype == torch.float8_e4m3fn else tb)


def test_assemble_gathered_layout():
    r, m, ns = 4, 5, 6
    full = torch.arange(m * r * ns, dtype=torch.float32).reshape(m, r * ns)
    gathered = torch.stack([full[:, i * ns:(i + 1) * ns] for i in range(r)])
    assert torch.equal(assemble_gathered(gathered), full)
    out = torch.empty(m, r * ns)
    assert assemble_gathered(gathered, out) is out and torch.equal(out, full)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, shape, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        inp = W.make_inputs(*shape, seed=9)
        gw, sg, uw, su = shard_weights(inp.gate_proj_weight, inp.scale_gate, inp.up_proj_weight, inp.scale_up,
                                       rank, world)
        local = O.gateup_blockwise(inp.x, inp.scale_x, gw, sg, uw, su)
        full = gather_columns(local)
        if rank == 0:
            ref = O.gateup_blockwise(*inp.args())
            q.put(bool(torch.equal(full, ref)))
        # every rank ends up with the same contiguous result
        check = full.clone().float()
        dist.all_reduce(check, op=dist.ReduceOp.MAX)
        assert torch.equal(check, full.float())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_gather_matches_unsharded_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, (24, 256, 1024), q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get() is True


def test_row_parallel_down_projection_shards_sum_to_the_unsharded_result():
    """The K-shards of the down projection (each rank's intermediate columns) add up to the full product."""
    m, h, n, world = 24, 256, 1024, 4
    gen = torch.Generator().manual_seed(17)
    mid = torch.randn(m, n, generator=gen)
    mq, ms = W.quantize_activation_1x128(mid)
    dq, sd = W.quantize_weight_128x128(torch.randn(h, n, generator=gen) * 0.02)
    full = O._blockwise_gemm(mq, ms, dq, sd)
    acc = torch.zeros(m, h)
    for r in range(world):
        lo, hi = shard_bounds(n, r, world)
        dw, ds = shard_down_weights(dq, sd, r, world)
        assert dw.is_contiguous() and tuple(dw.shape) == (h, n // world) and tuple(ds.shape) == (h // 128, n // world // 128)
        acc += O._blockwise_gemm(mq.view(torch.uint8)[:, lo:hi].contiguous().view(torch.float8_e4m3fn),
                                 ms[:, lo // 128:hi // 128].contiguous(), dw, ds)
    assert torch.allclose(acc, full, rtol=1e-5, atol=1e-5)


def _reduce_rank_main(rank, world, port, m, h, q):
    """The exchange schedule of the fused row-parallel GEMM + all-reduce, with gloo standing in for the peer stores:
    every rank's bf16 partial result is cut into the owners' row runs and delivered into the owners' slots
    (slot = sending rank), each owner sums its slots in rank order in fp32 and rounds once, the reduced runs are
    delivered to everybody."""
    from sol_execbench_b200_kernels_b200.sharded import owned_rows

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100 + rank)
        partial = torch.randn(m, h, generator=g).to(torch.bfloat16)
        rows = m // world
        send = [partial[slice(*owned_rows(m, d, world))].contiguous() for d in range(world)]
        slots = [torch.empty(rows, h, dtype=torch.bfloat16) for _ in range(world)]
        # slot s of this rank = rank s's partial of my rows (point to point: gloo has no all-to-all)
        slots[rank].copy_(send[rank])
        work = [dist.isend(send[d], d) for d in range(world) if d != rank]
        work += [dist.irecv(slots[s], s) for s in range(world) if s != rank]
        for w in work:
            w.wait()
        acc = torch.zeros(rows, h, dtype=torch.float32)
        for s in range(world):
            acc += slots[s].float()
        mine = acc.to(torch.bfloat16)
        full = [torch.empty(rows, h, dtype=torch.bfloat16) for _ in range(world)]
        dist.all_gather(full, mine)
        # by value (numpy), so that nothing refers to this process's shared memory after it exits
        q.put((rank, partial.view(torch.int16).numpy().copy(), torch.cat(full).view(torch.int16).numpy().copy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_reduce_scatter_and_gather_schedule_gloo(world):
    import torch.multiprocessing as mp
    from sol_execbench_b200_kernels_b200.sharded import owned_rows

    m, h = 128 * world * 2, 64
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_reduce_rank_main, args=(r, world, port, m, h, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted((q.get(timeout=120) for _ in range(world)), key=lambda t: t[0])
    got = [(r, torch.from_numpy(a).view(torch.bfloat16), torch.from_numpy(b).view(torch.bfloat16)) for r, a, b in got]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = torch.zeros(m, h, dtype=torch.float32)
    for _, partial, _ in got:
        want += partial.float()                            # rank order, fp32, one rounding
    want = want.to(torch.bfloat16)
    for rank, _, full in got:
        assert torch.equal(full, want), f"rank {rank}"
    edges = [owned_rows(m, r, world) for r in range(world)]
    assert edges[0][0] == 0 and edges[-1][1] == m and all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
    with pytest.raises(ValueError):
        owned_rows(128 * world + 128, 0, world) if world > 1 else owned_rows(100, 0, 1)
