"""End-to-end call for callers whose activations and results live in host memory.

`HostPipeline.run` takes pinned-host `x` / `scale_x` and a pinned-host bf16 destination; the weights
stay resident on the GPU, as model parameters do.  The token rows are cut into chunks and three
streams are kept busy at once: host-to-device copy of chunk i+1, the fused kernel on chunk i,
device-to-host copy of chunk i-1 (PCIe is full duplex), so the call costs about as much as the
slowest of the three instead of their sum.  Rows are independent, so chunking changes no bit of the
result.  PyTorch provides the streams, events and pinned memory; the arithmetic is `run`.
"""
from __future__ import annotations

from typing import List

import torch

from .kernel import run


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

    @torch.no_grad()
    def run(self, x_host: torch.Tensor, scale_x_host: torch.Tensor, gate_w: torch.Tensor, scale_gate: torch.Tensor,
            up_w: torch.Tensor, scale_up: torch.Tensor, out_host: torch.Tensor) -> None:
        """Asynchronous with respect to the host; call `synchronize()` before reading `out_host`."""
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
            s.wait_event(start)  # everything queued before this call (earlier readers of the buffers) is ordered first
        for lo, hi in self.bounds:
            with torch.cuda.stream(self.s_in):
                self.x[lo:hi].view(torch.uint8).copy_(x8[lo:hi], non_blocking=True)
                self.scale_x[lo:hi].copy_(scale_x_host[lo:hi], non_blocking=True)
                copied = torch.cuda.Event()
                copied.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(copied)
                run(self.x[lo:hi], self.scale_x[lo:hi], gate_w, scale_gate, up_w, scale_up, self.out[lo:hi])
                computed = torch.cuda.Event()
                computed.record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(computed)
                out_host[lo:hi].copy_(self.out[lo:hi], non_blocking=True)
        done = torch.cuda.Event()
        done.record(self.s_out)
        cur.wait_event(done)

    def synchronize(self) -> None:
        torch.cuda.current_stream(self.device).synchronize()
