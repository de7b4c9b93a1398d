"""End-to-end call for callers whose activations and results live in host memory.

`HostPipeline.run` takes pinned-host `x` / `scale_x` and a pinned-host bf16 destination; the weights
stay resident on the GPU, as model parameters do.  The token rows are cut into chunks and three
streams are kept busy at once: host-to-device copy of chunk i+1, the fused kernel on chunk i,
device-to-host copy of chunk i-1 (PCIe is full duplex), so the call costs about as much as the
slowest of the three instead of their sum.  Calls made one after another overlap too: a call only
waits, chunk by chunk, for what the call before it still needs (its kernel before the chunk's device
input is overwritten, its copy-out before the chunk's device result is), so in a loop the slowest of
the three streams never idles between steps.  The result is complete after `synchronize()`; the
caller's stream is not made to wait for it.  Rows are independent and the kernel is asked for whole tiles
(no tile cut along K, see `run_with_plan`), so chunking changes no bit of the result of the unsplit
whole-tile call.  PyTorch provides the streams, events and pinned memory; the arithmetic is `run`.
"""
from __future__ import annotations

from typing import List

import torch

from .kernel import run_with_plan


class HostPipeline:
    def __init__(self, m: int, k: int, n: int, device, chunks: int = 4):
        if k % 128 or n % 128 or m < 1:
            raise ValueError("need M >= 1 and K, N multiples of 128")
        self.m, self.k, self.n = m, k, n
        self.device = torch.device(device)
        # chunk boundaries on multiples of 128 rows (whole tiles), at least one chunk
        blocks = (m + 127) // 128
        chunks = max(1, min(chunks, blocks))
        per = (blocks + chunks - 1) // chunks
        self.bounds: List[tuple] = []
        for c in range(chunks):
            lo, hi = c * per * 128, min(m, (c + 1) * per * 128)
            if lo < hi:
                self.bounds.append((lo, hi))
        self.x = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=self.device)
        self.scale_x = torch.empty(m, k // 128, dtype=torch.float32, device=self.device)
        self.out = torch.empty(m, n, dtype=torch.bfloat16, device=self.device)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.bytes_h2d = m * k + m * (k // 128) * 4
        self.bytes_d2h = m * n * 2
        # per chunk, from the call before: its kernel has read the device input / its copy-out has read the device result
        self.ev_computed: List[torch.cuda.Event] = [None] * len(self.bounds)
        self.ev_copied_out: List[torch.cuda.Event] = [None] * len(self.bounds)

    @torch.no_grad()
    def run(self, x_host: torch.Tensor, scale_x_host: torch.Tensor, gate_w: torch.Tensor, scale_gate: torch.Tensor,
            up_w: torch.Tensor, scale_up: torch.Tensor, out_host: torch.Tensor) -> None:
        """Asynchronous with respect to the host and to the caller's stream; call `synchronize()` before reading
        `out_host` (or before changing `x_host` / `scale_x_host` for the next call)."""
        for t, name in ((x_host, "x_host"), (scale_x_host, "scale_x_host"), (out_host, "out_host")):
            if t.is_cuda or not t.is_pinned():
                raise ValueError(f"{name} must be a pinned host tensor")
        if tuple(x_host.shape) != (self.m, self.k) or tuple(out_host.shape) != (self.m, self.n):
            raise ValueError("host tensors do not match the pipeline's shape")
        x8 = x_host.view(torch.uint8)
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(start)  # what the caller queued before this call (e.g. the weights' producer) is ordered first
        for c, (lo, hi) in enumerate(self.bounds):
            with torch.cuda.stream(self.s_in):
                if self.ev_computed[c] is not None:
                    self.s_in.wait_event(self.ev_computed[c])  # the call before has read this chunk's device input
                self.x[lo:hi].view(torch.uint8).copy_(x8[lo:hi], non_blocking=True)
                self.scale_x[lo:hi].copy_(scale_x_host[lo:hi], non_blocking=True)
                copied = torch.cuda.Event()
                copied.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(copied)
                if self.ev_copied_out[c] is not None:
                    self.s_run.wait_event(self.ev_copied_out[c])  # ... and copied this chunk's device result out
                run_with_plan(self.x[lo:hi], self.scale_x[lo:hi], gate_w, scale_gate, up_w, scale_up, self.out[lo:hi],
                              "auto", whole_tiles=True)
                computed = torch.cuda.Event()
                computed.record(self.s_run)
                self.ev_computed[c] = computed
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(computed)
                out_host[lo:hi].copy_(self.out[lo:hi], non_blocking=True)
                copied_out = torch.cuda.Event()
                copied_out.record(self.s_out)
                self.ev_copied_out[c] = copied_out

    def synchronize(self) -> None:
        """Blocks the host until every call made so far has delivered its result."""
        self.s_out.synchronize()


class ShardedHostPipeline:
    """End-to-end call of the column-sharded op for host-memory callers on the R GPUs of one box.

    With the plain `HostPipeline` on every rank the replicated activations would cross PCIe R times per step, all
    through one host.  Here every rank keeps in pinned host memory only ITS row block of `x` / `scale_x` (rows
    [r M/R, (r+1) M/R)), copies that to its GPU, and the ranks exchange the blocks over NVLink (an NCCL all-gather:
    plumbing, not arithmetic) so that every rank holds all M rows; each rank then computes its N/R output columns for
    all rows and copies its [M, N/R] slice back to pinned host memory.  Per step a rank moves M K / R bytes in and
    2 M N / R bytes out over its own PCIe link.  The rows are cut into chunks (the same sub-range of every rank's
    block at a time) and three streams are kept busy: copy-in + exchange of chunk i+1, the kernel on chunk i, copy-out
    of chunk i-1.  Rows are independent, so neither the sharding of the rows nor the chunking changes a bit of the
    result.  Needs an initialised NCCL process group (one process per GPU)."""

    def __init__(self, m: int, k: int, n_local: int, device, group=None, chunks: int = 4):
        import torch.distributed as dist

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if k % 128 or n_local % 128 or m < 1 or m % (128 * self.world):
            raise ValueError("need K, N/R multiples of 128 and M a multiple of 128 x the number of ranks")
        self.m, self.k, self.n = m, k, n_local
        self.device = torch.device(device)
        self.block_rows = m // self.world
        blocks = self.block_rows // 128
        chunks = max(1, min(chunks, blocks))
        per = (blocks + chunks - 1) // chunks
        self.bounds: List[tuple] = [(c * per * 128, min(self.block_rows, (c + 1) * per * 128))
                                    for c in range(chunks) if c * per * 128 < self.block_rows]
        r = self.world
        # per chunk: this rank's rows, every rank's rows after the exchange ([R, rows, K]), the result for them
        self.x_own = [torch.empty(hi - lo, k, dtype=torch.uint8, device=self.device) for lo, hi in self.bounds]
        self.sx_own = [torch.empty(hi - lo, k // 128, dtype=torch.float32, device=self.device) for lo, hi in self.bounds]
        self.x_all = [torch.empty(r * (hi - lo), k, dtype=torch.uint8, device=self.device) for lo, hi in self.bounds]
        self.sx_all = [torch.empty(r * (hi - lo), k // 128, dtype=torch.float32, device=self.device) for lo, hi in self.bounds]
        self.out = [torch.empty(r * (hi - lo), n_local, dtype=torch.bfloat16, device=self.device) for lo, hi in self.bounds]
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.bytes_h2d = self.block_rows * k + self.block_rows * (k // 128) * 4
        self.bytes_d2h = m * n_local * 2
        self.bytes_nvlink_in = (r - 1) * self.bytes_h2d   # what this rank receives from its peers per step
        self.ev_computed: List[torch.cuda.Event] = [None] * len(self.bounds)
        self.ev_copied_out: List[torch.cuda.Event] = [None] * len(self.bounds)

    @torch.no_grad()
    def run(self, x_block_host: torch.Tensor, scale_x_block_host: torch.Tensor, gate_shard: torch.Tensor,
            scale_gate_shard: torch.Tensor, up_shard: torch.Tensor, scale_up_shard: torch.Tensor,
            out_host: torch.Tensor) -> None:
        """`x_block_host` e4m3 [M/R, K] and `scale_x_block_host` fp32 [M/R, K/128]: this rank's rows, pinned;
        `out_host` bf16 [M, N/R] pinned: this rank's columns of all rows.  Asynchronous with respect to the host and to
        the caller's stream; consecutive calls overlap as in `HostPipeline`; `synchronize()` before reading `out_host`."""
        import torch.distributed as dist

        for t, name in ((x_block_host, "x_block_host"), (scale_x_block_host, "scale_x_block_host"), (out_host, "out_host")):
            if t.is_cuda or not t.is_pinned():
                raise ValueError(f"{name} must be a pinned host tensor")
        if tuple(x_block_host.shape) != (self.block_rows, self.k) or tuple(out_host.shape) != (self.m, self.n):
            raise ValueError("host tensors do not match the pipeline's shape")
        x8 = x_block_host.view(torch.uint8)
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(start)
        for c, (lo, hi) in enumerate(self.bounds):
            rows = hi - lo
            with torch.cuda.stream(self.s_in):
                if self.ev_computed[c] is not None:
                    self.s_in.wait_event(self.ev_computed[c])  # the call before has read this chunk's gathered rows
                self.x_own[c].copy_(x8[lo:hi], non_blocking=True)
                self.sx_own[c].copy_(scale_x_block_host[lo:hi], non_blocking=True)
                dist.all_gather_into_tensor(self.x_all[c], self.x_own[c], group=self.group)
                dist.all_gather_into_tensor(self.sx_all[c], self.sx_own[c], group=self.group)
                gathered = torch.cuda.Event()
                gathered.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(gathered)
                if self.ev_copied_out[c] is not None:
                    self.s_run.wait_event(self.ev_copied_out[c])  # ... and copied this chunk's device result out
                run_with_plan(self.x_all[c].view(torch.float8_e4m3fn), self.sx_all[c], gate_shard, scale_gate_shard,
                              up_shard, scale_up_shard, self.out[c], "auto", whole_tiles=True)
                computed = torch.cuda.Event()
                computed.record(self.s_run)
                self.ev_computed[c] = computed
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(computed)
                for r in range(self.world):  # rank r's rows of this chunk sit at r * M/R + [lo, hi) of the result
                    out_host[r * self.block_rows + lo:r * self.block_rows + hi].copy_(
                        self.out[c][r * rows:(r + 1) * rows], non_blocking=True)
                copied_out = torch.cuda.Event()
                copied_out.record(self.s_out)
                self.ev_copied_out[c] = copied_out

    def synchronize(self) -> None:
        """Blocks the host until every call made so far has delivered its result."""
        self.s_out.synchronize()
