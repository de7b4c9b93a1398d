"""Column-parallel sharding of the intermediate dimension N across the GPUs of one box.

Output column n depends only on gate row n and up row n, so rank r of R owns
the row range [r*N/R, (r+1)*N/R) of both weight matrices and of both scale
grids, x and scale_x are replicated, and each rank produces output[:, its
columns] with no reduction and no data-path collective.  The reference is
single-GPU only; this is the multi-GPU layer added on top of its entry point.

An all-gather over NCCL (NVLink / NVSwitch) runs only when a contiguous [M, N]
result is asked for.  NCCL gathers contiguous buffers, so ranks exchange their
[M, N/R] slices into a rank-major [R, M, N/R] buffer that is then permuted into
row-major [M, N] locally.

One process per GPU; `group=None` means the default process group.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

BLOCK = 128


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """[start, stop) of the output columns rank `rank` owns; shards are whole 128-column scale blocks."""
    if n % BLOCK:
        raise ValueError(f"N={n} is not a multiple of {BLOCK}")
    nb = n // BLOCK
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    if nb % world:
        raise ValueError(f"N/128 = {nb} column blocks do not divide over {world} ranks")
    per = nb // world
    return rank * per * BLOCK, (rank + 1) * per * BLOCK


def shard_weights(gate_w: torch.Tensor, scale_gate: torch.Tensor, up_w: torch.Tensor, scale_up: torch.Tensor,
                  rank: int, world: int):
    """This rank's row ranges of the four weight-side tensors (contiguous views, no copy)."""
    n = gate_w.shape[0]
    lo, hi = shard_bounds(n, rank, world)
    blo, bhi = lo // BLOCK, hi // BLOCK
    return gate_w[lo:hi], scale_gate[blo:bhi], up_w[lo:hi], scale_up[blo:bhi]


def shard_concat_weights(w: torch.Tensor, scale_w: torch.Tensor, rank: int, world: int):
    """Same for concatenated W[2N, K]: the shard is two row ranges, returned as (gate, sg, up, su) views."""
    n = w.shape[0] // 2
    nb = n // BLOCK
    return shard_weights(w[:n], scale_w[:nb], w[n:], scale_w[nb:], rank, world)


def shard_down_weights(down_w: torch.Tensor, scale_down: torch.Tensor, rank: int, world: int):
    """Row-parallel shard of the down projection: the K range (intermediate columns) this rank produced.

    `down_w` is e4m3 [H, N], `scale_down` fp32 [H/128, N/128]; returns contiguous copies of
    down_w[:, lo:hi] and scale_down[:, lo/128:hi/128] (do this once, when the weights are loaded).
    """
    n = down_w.shape[1]
    lo, hi = shard_bounds(n, rank, world)
    w8 = down_w.view(torch.uint8)[:, lo:hi].contiguous().view(down_w.dtype)
    return w8, scale_down[:, lo // BLOCK:hi // BLOCK].contiguous()


def assemble_gathered(gathered: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rank-major [R, M, N/R] -> row-major [M, N]."""
    r, m, ns = gathered.shape
    if out is None:
        out = torch.empty(m, r * ns, dtype=gathered.dtype, device=gathered.device)
    out.view(m, r, ns).copy_(gathered.transpose(0, 1))
    return out


def gather_columns(local: torch.Tensor, group=None, out: Optional[torch.Tensor] = None,
                   scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather every rank's [M, N/R] slice and return the contiguous [M, N] result."""
    world = dist.get_world_size(group)
    m, ns = local.shape
    if scratch is None:
        scratch = torch.empty(world, m, ns, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(scratch.view(world * m, ns), local.contiguous(), group=group)
    return assemble_gathered(scratch, out)


class PeerBarrier:
    """The library's own cross-rank barrier for the fused gather / reduce paths (`gu_peer_barrier`): a 64-word flag
    array per rank in symmetric memory, stamped by plain peer stores and polled locally with a time limit, so a
    rank that never arrives costs its peers the limit and an error status instead of a kernel that spins forever
    (torch's symmetric-memory barrier has no such bound).  Collective to construct; `__call__` enqueues one barrier
    on the current stream."""

    def __init__(self, device, group=None, limit_ns: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device(device)
        self.flags = symm_mem.empty((64,), dtype=torch.int32, device=self.device)
        self.flags.zero_()
        self.handle = symm_mem.rendezvous(self.flags, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.limit_ns = int(limit_ns)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every rank's flags are zero before anyone stamps them

    def __call__(self) -> None:
        from .kernel import peer_barrier

        peer_barrier(self.ptrs, self.rank, self.device, self.limit_ns)


class GatherBuffers:
    """One bf16 [M, N] result buffer per rank, each mapped into every rank of the group.

    Built on torch's symmetric memory (CUDA peer mappings over NVLink / NVSwitch).  `out` is this rank's
    buffer; `ptrs[r]` the address of rank r's buffer in this process; `barrier()` enqueues the library's bounded
    cross-rank barrier (`PeerBarrier`) on the current stream.  Allocate once and reuse: the rendezvous is collective and slow.
    """

    def __init__(self, m: int, n: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.out = symm_mem.empty((m, n), dtype=torch.bfloat16, device=device)
        self.handle = symm_mem.rendezvous(self.out, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.shape = (m, n)
        self._barrier = PeerBarrier(device, self.group)

    def barrier(self) -> None:
        self._barrier()


@torch.no_grad()
def run_sharded_fused(x: torch.Tensor, scale_x: torch.Tensor, gate_shard: torch.Tensor,
                      scale_gate_shard: torch.Tensor, up_shard: torch.Tensor, scale_up_shard: torch.Tensor,
                      buffers: GatherBuffers) -> torch.Tensor:
    """Column-parallel op with the all-gather fused into the kernel epilogue.

    Each rank computes its N/R columns and TMA-stores every output tile straight into all ranks' [M, N]
    buffers (its own and, over NVLink, its peers'), so the transfer overlaps the math tile by tile and no
    NCCL all-gather or permute follows.  A cross-rank barrier orders the stores before anyone reads.
    Returns this rank's contiguous [M, N] result.
    """
    from .kernel import run_gather

    # nobody may still be reading the buffers of the previous call when the first tile lands
    buffers.barrier()
    run_gather(x, scale_x, gate_shard, scale_gate_shard, up_shard, scale_up_shard, buffers.ptrs, buffers.rank,
               buffers.shape, buffers.out.stride(0))
    buffers.barrier()
    return buffers.out


@torch.no_grad()
def mlp_block_sharded(x: torch.Tensor, gate_shard: torch.Tensor, scale_gate_shard: torch.Tensor,
                      up_shard: torch.Tensor, scale_up_shard: torch.Tensor, down_shard: torch.Tensor,
                      scale_down_shard: torch.Tensor, group=None) -> torch.Tensor:
    """Tensor-parallel MLP block: column-parallel gate/up, row-parallel down projection, one all-reduce.

    Every rank quantises the replicated activations, computes its N/R intermediate columns (kept as e4m3 +
    scales, never exchanged), multiplies them with its K-shard of the down weights (`shard_down_weights`) and
    the bf16 partial results [M, H] are summed over the ranks with an NCCL all-reduce (the one exchange step
    this block has).  Returns the full bf16 [M, H] on every rank.
    """
    from .kernel import BLOCK as _B, blockwise_gemm, quantize_activation, run_fp8_output

    m = x.shape[0]
    n_local = gate_shard.shape[0]
    xq, sx = quantize_activation(x)
    mid_q = torch.empty(m, n_local, dtype=torch.float8_e4m3fn, device=x.device)
    mid_s = torch.empty(m, n_local // _B, dtype=torch.float32, device=x.device)
    run_fp8_output(xq, sx, gate_shard, scale_gate_shard, up_shard, scale_up_shard, mid_q, mid_s)
    partial = torch.empty(m, down_shard.shape[0], dtype=torch.bfloat16, device=x.device)
    blockwise_gemm(mid_q, mid_s, down_shard, scale_down_shard, partial)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


def owned_rows(m: int, rank: int, world: int) -> Tuple[int, int]:
    """[start, stop) of the token rows whose reduced sum rank `rank` produces in the fused row-parallel GEMM +
    all-reduce: equal runs of whole 128-row tiles, so that every output tile of the GEMM has one owner."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    if m % (BLOCK * world):
        raise ValueError(f"M={m} must be a multiple of {BLOCK} * world ({world})")
    rows = m // world
    return rank * rows, (rank + 1) * rows


class ReduceBuffers:
    """Symmetric buffers of the fused row-parallel GEMM + all-reduce: per rank a bf16 slot buffer
    [world, M/world, H] (one partial result per sending rank, for the token rows this rank owns) and a bf16
    [M, H] result, both mapped into every rank of the group.  Allocate once and reuse."""

    def __init__(self, m: int, h: int, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        world = dist.get_world_size(self.group)
        owned_rows(m, 0, world)  # raises when the rows do not split into whole tiles per rank
        self.slots = symm_mem.empty((world, m // world, h), dtype=torch.bfloat16, device=device)
        self.slots_handle = symm_mem.rendezvous(self.slots, self.group)
        self.out = symm_mem.empty((m, h), dtype=torch.bfloat16, device=device)
        self.handle = symm_mem.rendezvous(self.out, self.group)
        self.rank = self.handle.rank
        self.world = self.handle.world_size
        self.slot_ptrs = [int(p) for p in self.slots_handle.buffer_ptrs]
        self.out_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.shape = (m, h)
        self._barrier = PeerBarrier(device, self.group)

    def barrier(self) -> None:
        self._barrier()


@torch.no_grad()
def mlp_block_sharded_fused(x: torch.Tensor, gate_shard: torch.Tensor, scale_gate_shard: torch.Tensor,
                            up_shard: torch.Tensor, scale_up_shard: torch.Tensor, down_shard: torch.Tensor,
                            scale_down_shard: torch.Tensor, buffers: ReduceBuffers, gather: bool = True) -> torch.Tensor:
    """`mlp_block_sharded` with the all-reduce done by the library's own kernels over peer memory.

    The down projection's epilogue TMA-stores each bf16 partial tile into the slot buffer of the rank that
    owns those token rows (reduce-scatter, overlapped with the math tile by tile); after a barrier each rank
    sums its slots in rank order and writes the reduced rows into every rank's [M, H] result (all-gather by
    peer stores).  Two cross-rank barriers, no NCCL call.  All ranks return identical bits.  With
    `gather=False` each rank keeps only the rows it owns ([M/R, H], the reduce-scatter form) and nothing is sent back.  Consume the
    result on the stream this was called on (or synchronise with it) before the next call on `buffers`.
    """
    from .kernel import BLOCK as _B, blockwise_gemm_scatter, quantize_activation, reduce_gather, run_fp8_output

    m, h = buffers.shape
    n_local = gate_shard.shape[0]
    xq, sx = quantize_activation(x)
    mid_q = torch.empty(m, n_local, dtype=torch.float8_e4m3fn, device=x.device)
    mid_s = torch.empty(m, n_local // _B, dtype=torch.float32, device=x.device)
    run_fp8_output(xq, sx, gate_shard, scale_gate_shard, up_shard, scale_up_shard, mid_q, mid_s)
    # No barrier in front of the scatter: the barrier that ended the previous call on these buffers already ordered
    # every rank's reads of its slots before this point, and `out` is not written before the next barrier, by
    # which every rank has enqueued (on this stream) whatever reads the previous result.
    blockwise_gemm_scatter(mid_q, mid_s, down_shard, scale_down_shard, buffers.slot_ptrs, buffers.rank)
    buffers.barrier()  # all partial tiles have landed in their owners' slots
    if gather:
        reduce_gather(buffers.slots, buffers.out_ptrs, buffers.rank, m, h)
        buffers.barrier()  # every rank's rows have landed in every result
        return buffers.out
    # reduce-scatter form (sequence-parallel consumers): only this rank's rows, written locally.  The closing barrier
    # stays: it is what lets the next call's scatter overwrite the slots.
    own = [p if r == buffers.rank else None for r, p in enumerate(buffers.out_ptrs)]
    reduce_gather(buffers.slots, own, buffers.rank, m, h)
    buffers.barrier()
    rows = m // buffers.world
    return buffers.out[buffers.rank * rows:(buffers.rank + 1) * rows]


@torch.no_grad()
def run_sharded(x: torch.Tensor, scale_x: torch.Tensor, gate_shard: torch.Tensor, scale_gate_shard: torch.Tensor,
                up_shard: torch.Tensor, scale_up_shard: torch.Tensor, output_shard: torch.Tensor,
                group=None, gather: bool = False, gathered_out: Optional[torch.Tensor] = None,
                scratch: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """One rank's part of the column-parallel op.

    `*_shard` are this rank's slices (see `shard_weights`), `output_shard` is bf16
    [M, N/R].  With `gather=True` returns the contiguous [M, N] tensor (NCCL
    all-gather + local permute); otherwise returns None and nothing is exchanged.
    """
    from .kernel import run  # needs the CUDA library; kept out of the index helpers above

    run(x, scale_x, gate_shard, scale_gate_shard, up_shard, scale_up_shard, output_shard)
    if not gather:
        return None
    return gather_columns(output_shard, group=group, out=gathered_out, scratch=scratch)
