#!/usr/bin/env python
"""Benchmark of the FP8 gate/up + SwiGLU hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--gather]
    python bench.py --sweep            # M in {1,8,32,128,512,2048,8192} at K=4096, N=14336: plan crossover

A step is one pass of the fused op over one synthetic workload (seeded
N(0,1) activations, N(0,0.02) weights, e4m3 block quantisation).

  N = 1   workload "prefill_8b"  (M=4096, K=4096, N=14336; tensor-bound), plus the
          decode shape (M=16, K=8192, N=28672; HBM-bound) reported under "also".
  N > 1   workload "prefill_sharded" (M=16384, K=7168, N=18432) with the intermediate
          dimension column-sharded over the ranks (torchrun, one process per GPU);
          no data-path collective unless --gather asks for the contiguous output.

Prints ONE JSON line on rank 0.  `--impl reference` times the CPU restatement of
the reference's definition (dequantise, fp32 matmul, SwiGLU) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "FP8 gate/up+SwiGLU TFLOP/s & HBM GB/s vs roofline at 1/2/4/8 B200"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_FLUSH_BYTES = 256 << 20  # written, then read back, between timed iterations; B200 L2 is 126 MB


def flush_l2(buf: torch.Tensor) -> None:
    """Evicts the workload from L2: writes a buffer larger than L2, then reads it back so the lines it
    leaves behind are clean (dirty lines would be written back during the timed kernel and charge it
    with DRAM traffic that is not its own)."""
    buf.zero_()
    buf.sum()

def ncu_traffic_bytes(workload: str):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel on `workload`,
    as recorded by the ncu summary committed under profiles/ (a line `traffic_bytes[<workload>] = <integer>`);
    None when no capture of that workload is on record."""
    import glob
    import re

    pat = re.compile(r"traffic_bytes\[" + re.escape(workload) + r"\]\s*=\s*(\d+)")
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))):
        try:
            with open(path) as f:
                hit = pat.search(f.read())
        except OSError:
            continue
        if hit:
            return int(hit.group(1))
    return None


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _loop(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([c.strip() for c in out.splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[1]))
                mx.append(float(s[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, s[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
def time_device_steps(fn, steps: int, warmup: int, flush: torch.Tensor, barrier=None):
    """Per-step CUDA-event timing on the current stream, L2 flushed before every step."""
    for _ in range(warmup):
        flush_l2(flush)
        fn()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush_l2(flush)
        starts[i].record()
        fn()
        stops[i].record()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    per = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    return sum(per), per


def roofline_for(m, k, n, ms, peaks, W):
    flops = W.algorithmic_flops(m, k, n)
    nbytes = W.algorithmic_bytes(m, k, n)
    fp8_peak = 2.0 * peaks["bf16_tflops"]       # dense FP8 = 2x the measured dense bf16 burst rate
    t_tensor = flops / (fp8_peak * 1e12)
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9)
    src = "of measured" if peaks["_source"] == "measured" else "of fallback"
    if t_tensor >= t_hbm:
        achieved = flops / (ms * 1e-3) / 1e12
        return {"bound": "tensor", "achieved": round(achieved, 2), "peak": round(fp8_peak, 1), "unit": "TFLOP/s",
                "frac": round(achieved / fp8_peak, 4), "traffic": None,
                "peak_source": f"2 x bf16_tflops burst, {src}", "algorithmic_flops": flops}
    achieved = nbytes / (ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": None,
            "peak_source": f"hbm_gbs, {src}", "algorithmic_bytes": nbytes}


def cpu_baseline(inp_cpu, oracle, max_flops: float = 2.0e12):
    """Oracle (dequant, fp32 matmul, SwiGLU) on the host cores over a bounded row sample of the workload."""
    m, k, n = inp_cpu.shape
    rows = int(min(m, max(64, max_flops // (4 * k * n))))
    oracle.gateup_dequant(*inp_cpu.rows(torch.arange(min(m, 16))).args())  # untimed warm pass (thread pool, pages)
    sub = inp_cpu if rows == m else inp_cpu.rows(torch.arange(rows))
    timings = {}
    oracle.gateup_dequant(*sub.args(), timings=timings)
    flops = 4.0 * rows * k * n
    return {
        "value": round(flops / timings["total_s"] / 1e12, 4), "unit": "TFLOP/s",
        "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(), "kind": "port",
        "sample": f"rows 0..{rows - 1} of M={m} (K={k}, N={n}), one timed pass, weights dequantised inside the pass",
        "seconds": round(timings["total_s"], 3),
        "phases_s": {p: round(timings[p], 3) for p in ("dequant_s", "matmul_s", "swiglu_s")},
    }


def parity_of(out, inp, W, oracle, label):
    """Sampled parity of a device result against both CPU restatements (16 token rows x 3 column blocks of 128):
    the numbers the tolerance of the path is stated in (max-abs 2e-2, relative L2 1e-2 on the bf16 output)."""
    m, k, n = inp.shape
    dev = out.device
    rows = torch.arange(0, m, max(1, m // 16), device=dev)[:16]
    nb = n // 128
    blocks = torch.tensor(sorted({0, nb // 2, nb - 1}), device=dev)
    sub = inp.rows(rows).column_blocks(blocks).to("cpu")
    cols = (blocks[:, None] * 128 + torch.arange(128, device=dev)[None]).reshape(-1)
    got = out[rows][:, cols].cpu()
    res = {"config": label, "sample": f"{len(rows)} token rows x {len(blocks)} column blocks of 128", "atol": 2e-2}
    for name, fn in (("gateup_dequant", oracle.gateup_dequant), ("gateup_blockwise", oracle.gateup_blockwise)):
        st = oracle.error_stats(got, fn(*sub.args()))
        entry = {"max_abs": round(st["max_abs"], 6), "rel_l2": float(f"{st['rel_l2']:.3e}"),
                 "n_over_atol": st["n_over_atol"], "frac_over_atol": st["frac_over_atol"],
                 "max_ulp_over": st["max_ulp_over"]}
        if name == "gateup_dequant":
            res.update(entry)
            res["vs"] = name
        else:
            entry["bit_equal"] = bool(torch.equal(got, fn(*sub.args()).to(torch.bfloat16)))
            res["vs_" + name] = entry
    return res


def sustained_leg(fn, flops, peaks, gpu_index, seconds=2.5):
    """The same launch back to back for `seconds` (no flush: the operands exceed L2), CUDA events around the whole
    run, against twice the measured SUSTAINED bf16 rate; the median SM clock under load is sampled beside it."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(20):
        fn()
    b.record()
    torch.cuda.synchronize()
    count = max(50, int(seconds * 1e3 / max(a.elapsed_time(b) / 20, 1e-3)))
    with ClockSampler(gpu_index) as clocks:
        a.record()
        for _ in range(count):
            fn()
        b.record()
        torch.cuda.synchronize()
    ms = a.elapsed_time(b) / count
    peak = 2.0 * peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"])
    ach = flops / (ms * 1e-3) / 1e12
    c = clocks.summary()
    return {"launches": count, "seconds": round(ms * count * 1e-3, 3), "ms_per_step": round(ms, 5),
            "tflops": round(ach, 2), "peak": round(peak, 1), "frac": round(ach / peak, 4),
            "peak_source": "2 x bf16_tflops_sustained, " + ("of measured" if peaks["_source"] == "measured" else "of fallback"),
            "clocks": c, "ms_x_mhz": round(ms * c["sm_mhz"], 2) if c.get("sm_mhz") else None}


def pcie_rates(dev, nbytes=64 << 20):
    """Pinned-host copy bandwidth each way (GB/s), the ceiling of the end-to-end leg."""
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    devb = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    res = {}
    for name, (dst, src) in {"h2d_gbs": (devb, host), "d2h_gbs": (host, devb)}.items():
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            dst.copy_(src, non_blocking=True)
        b.record()
        torch.cuda.synchronize()
        res[name] = round(3 * nbytes / (a.elapsed_time(b) * 1e-3) / 1e9, 1)
    return res


def run_sweep(args):
    """M sweep at K=4096, N=14336: every plan that can run each M, the heuristic's pick and the roofline fraction."""
    import sol_execbench_b200_kernels_b200 as pkg
    from sol_execbench_b200_kernels_b200 import workloads as W

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    peaks = load_peaks()
    flush = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.float32, device=dev)
    k, n = W.SWEEP_KN
    rows = []
    for m in W.SWEEP_M:
        inp = W.make_inputs(m, k, n, seed=0, device=dev)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        entry = {"m": m, "auto_plan": pkg.select_plan(m, k, n), "plans": {}}
        # "tile" is the heuristic's tile kernel (CTA pairs above 128 tokens, their stream-K schedule where whole tiles
        # would idle 5 % of the device), "tile_pair" the pair kernel with whole tiles forced, "tile_dp" the lone-CTA kernel
        for plan in (("stream", "tile") if m <= 64 else (("tile",) if m <= 128 else ("tile", "tile_pair", "tile_dp"))):
            ms, _ = time_device_steps(lambda: pkg.run_with_plan(*inp.args(), out, plan), args.steps, args.warmup, flush)
            ms /= args.steps
            roof = roofline_for(m, k, n, ms, peaks, W)
            entry["plans"][plan] = {"us": round(ms * 1e3, 2), "bound": roof["bound"], "achieved": roof["achieved"],
                                    "unit": roof["unit"], "frac": roof["frac"],
                                    "tflops": round(W.algorithmic_flops(m, k, n) / (ms * 1e-3) / 1e12, 1),
                                    "gbs": round(W.algorithmic_bytes(m, k, n) / (ms * 1e-3) / 1e9, 1)}
        best = min(entry["plans"], key=lambda q: entry["plans"][q]["us"])
        entry["fastest"] = best
        rows.append(entry)
        del inp, out
    code, detail = pkg.last_status()
    if code != 0:
        raise SystemExit(f"bench.py: device status {code} detail {detail:#x}")
    print(json.dumps({"metric": METRIC, "sweep": {"k": k, "n": n, "rows": rows}, "steps": args.steps,
                      "warmup": args.warmup, "data": "synthetic",
                      "peaks": {"fp8_tflops": 2.0 * peaks["bf16_tflops"], "hbm_gbs": peaks["hbm_gbs"],
                                "source": peaks["_source"]}}), flush=True)


def run_ours(args):
    import torch.distributed as dist

    import sol_execbench_b200_kernels_b200 as pkg
    from sol_execbench_b200_kernels_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this library has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_gpus = world
    peaks = load_peaks()

    workload = args.workload or ("prefill_8b" if n_gpus == 1 else "prefill_sharded")
    m, k, n = W.SHAPES[workload]
    # every rank draws the same seeded workload on its GPU and keeps its own column shard
    full = W.make_inputs(m, k, n, seed=0, device=dev)
    if n_gpus > 1:
        gw, sg, uw, su = pkg.shard_weights(full.gate_proj_weight, full.scale_gate, full.up_proj_weight,
                                           full.scale_up, rank, world)
        gw, sg, uw, su = (t.clone() for t in (gw, sg, uw, su))
        local = W.GateUpInputs(full.x, full.scale_x, gw, sg, uw, su)
        del full
        torch.cuda.empty_cache()
    else:
        local = full
    n_local = local.gate_proj_weight.shape[0]
    out = torch.empty(m, n_local, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.float32, device=dev)
    gathered = torch.empty(m, n, dtype=torch.bfloat16, device=dev) if (args.gather and n_gpus > 1) else None
    scratch = torch.empty(world, m, n_local, dtype=torch.bfloat16, device=dev) if gathered is not None else None

    buffers = pkg.GatherBuffers(m, n, dev) if (args.fused_gather and n_gpus > 1) else None

    def step():
        if buffers is not None:
            pkg.run_sharded_fused(*local.args(), buffers)
        elif n_gpus > 1:
            pkg.run_sharded(*local.args(), out, gather=gathered is not None, gathered_out=gathered, scratch=scratch)
        else:
            pkg.run(*local.args(), out)

    barrier = (lambda: dist.barrier()) if n_gpus > 1 else None
    with ClockSampler(local_rank) as clocks:
        launches0 = pkg.launch_count()
        total_ms, per = time_device_steps(step, args.steps, args.warmup, flush, barrier)
        launches_timed = (pkg.launch_count() - launches0) * args.steps // (args.steps + args.warmup)
        # keep the GPU busy long enough for a few clock samples when the steps are very short
        t_end = time.perf_counter() + max(0.0, 0.4 - total_ms * 1e-3)
        while time.perf_counter() < t_end:
            step()
        torch.cuda.synchronize()
    assert launches_timed >= args.steps  # at least one kernel of this library per step
    code, detail = pkg.last_status()
    if code != 0:
        raise SystemExit(f"bench.py: device status {code} detail {detail:#x}")

    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if n_gpus > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    flops_job = W.algorithmic_flops(m, k, n)
    value = flops_job / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the public host-memory entry point: pinned host activations in, host result out ----
    from sol_execbench_b200_kernels_b200.host_pipeline import HostPipeline

    out_host = torch.empty(m, n_local, dtype=torch.bfloat16).pin_memory()
    if n_gpus > 1:
        # every rank holds only its row block of the activations in host memory; the blocks are exchanged over NVLink
        from sol_execbench_b200_kernels_b200.host_pipeline import ShardedHostPipeline

        pipe = ShardedHostPipeline(m, k, n_local, dev, chunks=max(1, args.e2e_chunks))
        lo, hi = rank * pipe.block_rows, (rank + 1) * pipe.block_rows
        x_host = local.x[lo:hi].cpu().view(torch.uint8).pin_memory().view(torch.float8_e4m3fn)
        sx_host = local.scale_x[lo:hi].cpu().pin_memory()
    else:
        pipe = HostPipeline(m, k, n_local, dev, chunks=args.e2e_chunks)
        x_host = local.x.cpu().view(torch.uint8).pin_memory().view(torch.float8_e4m3fn)
        sx_host = local.scale_x.cpu().pin_memory()

    def e2e_step():
        pipe.run(x_host, sx_host, local.gate_proj_weight, local.scale_gate, local.up_proj_weight, local.scale_up,
                 out_host)

    for _ in range(max(1, args.warmup // 2)):
        e2e_step()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    e2e_steps = max(30, args.steps)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_ok = bool(torch.equal(out_host[:: max(1, m // 64)].to(dev), out[:: max(1, m // 64)])) if buffers is None else True
    te = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if n_gpus > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_s = float(te.item())
    pcie = pcie_rates(dev)
    # what the copies alone allow: both directions run at once, so the slower of the two bounds a step
    copy_s = max(pipe.bytes_h2d / (pcie["h2d_gbs"] * 1e9), pipe.bytes_d2h / (pcie["d2h_gbs"] * 1e9))
    e2e = {"value": round(flops_job / (e2e_s / e2e_steps) / 1e12, 3), "unit": "TFLOP/s",
           "h2d_bytes_per_step": pipe.bytes_h2d, "d2h_bytes_per_step": pipe.bytes_d2h, "steps": e2e_steps,
           "ms_per_step": round(e2e_s / e2e_steps * 1e3, 4), "matches_device_run": e2e_ok,
           "pcie": {**pcie, "copy_bound_ms": round(copy_s * 1e3, 4),
                    "ceiling": round(flops_job / max(copy_s, ms_per_step * 1e-3) / 1e12, 1),
                    "note": "ceiling = the metric if a step took only the slower of its host copies (or the kernel)"},
           "note": ("HostPipeline.run: weights resident in HBM; x and scale_x copied from pinned host memory and the "
                    f"bf16 output copied back to pinned host memory every step, in {len(pipe.bounds)} row chunks on three "
                    "streams, consecutive steps overlapping chunk by chunk; wall clock over all steps") if n_gpus == 1 else
                   ("ShardedHostPipeline.run: every rank copies its M/R row block of x and scale_x from pinned host "
                    "memory, the blocks are exchanged over NVLink (NCCL all-gather), every rank copies its [M, N/R] slice "
                    f"of the bf16 output back to pinned host memory, in {len(pipe.bounds)} row chunks on three streams, "
                    "consecutive steps overlapping chunk by chunk; bytes are per rank; wall clock over all steps, max over ranks")}
    if n_gpus > 1:
        e2e["nvlink_bytes_in_per_step"] = pipe.bytes_nvlink_in

    result = None
    parity = None
    if rank == 0 and buffers is None:
        from oracle import gateup_oracle as oracle  # checker only: parity of the timed configuration

        step()
        torch.cuda.synchronize()
        parity = parity_of(out, local, W, oracle, f"{workload}" + (f", rank 0 shard of {n_gpus}" if n_gpus > 1 else ""))
    scaling_base = None
    if n_gpus > 1 and not (args.gather or args.fused_gather):
        # the same workload, unsharded, on rank 0's GPU in this very run: the base the N-GPU value is compared with
        if rank == 0:
            whole = W.make_inputs(m, k, n, seed=0, device=dev)
            wout = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            bsteps = 5
            bms, _ = time_device_steps(lambda: pkg.run(*whole.args(), wout), bsteps, 3, flush)
            base_ms = bms / bsteps
            base_tf = flops_job / (base_ms * 1e-3) / 1e12
            scaling_base = {"workload": f"{workload}: M={m} K={k} N={n}, unsharded on one GPU (rank 0, same run)",
                            "one_gpu_ms": round(base_ms, 5), "one_gpu_tflops": round(base_tf, 2), "steps": bsteps,
                            "efficiency": round(value / (n_gpus * base_tf), 4)}
            del whole, wout
            torch.cuda.empty_cache()
        dist.barrier()
    if rank == 0:
        roof = roofline_for(m, k, n_local, ms_per_step, peaks, W)
        roof["traffic"] = ncu_traffic_bytes(workload)
        result = {
            "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": n_gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True, "scaling": "strong" if n_gpus > 1 or workload == "prefill_sharded" else "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32 accumulate -> bf16", "data": "synthetic",
            "config": {"workload": f"{workload}: M={m} K={k} N={n}", "sharding": f"N column-sharded over {n_gpus}" if n_gpus > 1 else "none",
                       "per_rank_n": n_local, "plan": pkg.select_plan(m, k, n_local),
                       "gather": "fused peer stores" if buffers is not None else ("nccl" if gathered is not None else False),
                       "l2": f"flushed before every timed step by writing, then reading back, a {L2_FLUSH_BYTES >> 20} MiB buffer"},
            "roofline": roof, "e2e": e2e, "gpu_launches": launches_timed,
            "clocks": clocks.summary(), "parity": parity,
        }
        if scaling_base is not None:
            result["scaling_base"] = scaling_base

    # ---- decode shape (HBM-bound) and CPU baseline: rank 0, single-GPU runs only ----
    if n_gpus == 1 and not args.workload:
        from oracle import gateup_oracle as oracle  # checker and CPU baseline legs: the only uses of it here

        result["also"] = []
        dm, dk, dn = W.SHAPES["decode_70b"]
        del out, pipe
        torch.cuda.empty_cache()
        dec = W.make_inputs(dm, dk, dn, seed=0, device=dev)
        dout = torch.empty(dm, dn, dtype=torch.bfloat16, device=dev)
        dsteps = max(args.steps, 20)
        dms, _ = time_device_steps(lambda: pkg.run(*dec.args(), dout), dsteps, max(args.warmup, 3), flush)
        droof = roofline_for(dm, dk, dn, dms / dsteps, peaks, W)
        droof["traffic"] = ncu_traffic_bytes("decode_70b")
        result["also"].append({
            "workload": f"decode_70b: M={dm} K={dk} N={dn}", "plan": pkg.select_plan(dm, dk, dn),
            "ms_per_step": round(dms / dsteps, 5), "steps": dsteps,
            "tflops": round(W.algorithmic_flops(dm, dk, dn) / (dms / dsteps * 1e-3) / 1e12, 2),
            "roofline": droof, "parity": parity_of(dout, dec, W, oracle, "decode_70b")})
        del dec, dout
        torch.cuda.empty_cache()
        sm_, sk_, sn_ = W.SHAPES["prefill_sharded"]
        big = W.make_inputs(sm_, sk_, sn_, seed=0, device=dev)
        bout = torch.empty(sm_, sn_, dtype=torch.bfloat16, device=dev)
        bsteps = 5
        bms, _ = time_device_steps(lambda: pkg.run(*big.args(), bout), bsteps, 3, flush)
        result["also"].append({
            "workload": f"prefill_sharded on one GPU: M={sm_} K={sk_} N={sn_}", "plan": pkg.select_plan(sm_, sk_, sn_),
            "ms_per_step": round(bms / bsteps, 5), "steps": bsteps,
            "tflops": round(W.algorithmic_flops(sm_, sk_, sn_) / (bms / bsteps * 1e-3) / 1e12, 2),
            "roofline": roofline_for(sm_, sk_, sn_, bms / bsteps, peaks, W)})
        del big, bout
        torch.cuda.empty_cache()
        # the step in front of the path: bf16 activations -> e4m3 + 1x128 scales (pure streaming)
        qx = torch.randn(sm_, sk_, device=dev, dtype=torch.bfloat16)
        qq = torch.empty(sm_, sk_, dtype=torch.float8_e4m3fn, device=dev)
        qs = torch.empty(sm_, sk_ // 128, dtype=torch.float32, device=dev)
        qsteps = 20
        qms, _ = time_device_steps(lambda: pkg.quantize_activation(qx, qq, qs), qsteps, 3, flush)
        qbytes = sm_ * sk_ * 3 + sm_ * (sk_ // 128) * 4
        qach = qbytes / (qms / qsteps * 1e-3) / 1e9
        result["also"].append({
            "workload": f"quantize_activation bf16 -> e4m3: M={sm_} K={sk_}", "ms_per_step": round(qms / qsteps, 5),
            "steps": qsteps,
            "roofline": {"bound": "hbm", "achieved": round(qach, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(qach / peaks["hbm_gbs"], 4), "traffic": None, "algorithmic_bytes": qbytes,
                         "peak_source": "hbm_gbs, " + ("of measured" if peaks["_source"] == "measured" else "of fallback")}})
        del qx, qq, qs
        torch.cuda.empty_cache()
        # the step behind the path: the down projection as a plain block-scaled GEMM on the re-quantised result,
        # and the three-launch MLP block (quantise, gate/up + SwiGLU with e4m3 output, down projection)
        hm, hh, hn = W.SHAPES["prefill_8b"]          # tokens, hidden, intermediate
        blk = W.make_inputs(hm, hh, hn, seed=0, device=dev)
        dq, dsc = W.quantize_weight_128x128(torch.randn(hh, hn, device=dev) * 0.02)
        mid_q = torch.empty(hm, hn, dtype=torch.float8_e4m3fn, device=dev)
        mid_s = torch.empty(hm, hn // 128, dtype=torch.float32, device=dev)
        pkg.run_fp8_output(*blk.args(), mid_q, mid_s)
        yout = torch.empty(hm, hh, dtype=torch.bfloat16, device=dev)
        gsteps = 10
        gms, _ = time_device_steps(lambda: pkg.blockwise_gemm(mid_q, mid_s, dq, dsc, yout), gsteps, 3, flush)
        gfl = 2.0 * hm * hh * hn
        gach = gfl / (gms / gsteps * 1e-3) / 1e12
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        result["also"].append({
            "workload": f"down projection (blockwise_gemm): M={hm} K={hn} N={hh}", "ms_per_step": round(gms / gsteps, 5),
            "steps": gsteps, "tflops": round(gach, 2),
            "roofline": {"bound": "tensor", "achieved": round(gach, 2), "peak": round(fp8_peak, 1), "unit": "TFLOP/s",
                         "frac": round(gach / fp8_peak, 4), "traffic": None, "algorithmic_flops": gfl}})
        xb = torch.randn(hm, hh, device=dev, dtype=torch.bfloat16)
        bms, _ = time_device_steps(lambda: pkg.mlp_block(xb, blk.gate_proj_weight, blk.scale_gate, blk.up_proj_weight,
                                                          blk.scale_up, dq, dsc, yout), gsteps, 3, flush)
        bfl = 6.0 * hm * hh * hn
        result["also"].append({
            "workload": f"mlp_block bf16 in -> bf16 out (3 launches): M={hm} H={hh} N={hn}",
            "ms_per_step": round(bms / gsteps, 5), "steps": gsteps,
            "tflops": round(bfl / (bms / gsteps * 1e-3) / 1e12, 2)})
        del blk, dq, dsc, mid_q, mid_s, yout, xb
        torch.cuda.empty_cache()
        # an awkward tile count: 512 tokens are 3.03 rounds of tiles (the tile plan's stream-K schedule runs here)
        wm, wk, wn = 512, W.SWEEP_KN[0], W.SWEEP_KN[1]
        wav = W.make_inputs(wm, wk, wn, seed=0, device=dev)
        wout = torch.empty(wm, wn, dtype=torch.bfloat16, device=dev)
        wsteps = 20
        wrow = {}
        for plan in ("tile", "tile_pair"):
            wms, _ = time_device_steps(lambda: pkg.run_with_plan(*wav.args(), wout, plan), wsteps, 3, flush)
            wrow[plan] = wms / wsteps
        result["also"].append({
            "workload": f"sweep row M={wm} K={wk} N={wn}", "plan": "tile (heuristic schedule)",
            "ms_per_step": round(wrow["tile"], 5), "steps": wsteps, "whole_tiles_ms_per_step": round(wrow["tile_pair"], 5),
            "tflops": round(W.algorithmic_flops(wm, wk, wn) / (wrow["tile"] * 1e-3) / 1e12, 2),
            "roofline": roofline_for(wm, wk, wn, wrow["tile"], peaks, W)})
        del wav, wout
        # the repository's other operators (problems 038 and 029) behind the second C ABI, one shape each
        from sol_execbench_b200_kernels_b200 import side_ops
        side = {}
        q_, k_, wq_, wk_, eps_ = W.make_rmsnorm_inputs(*W.RMSNORM_SHAPES["flux_4608"], 0, dev)
        qn_, kn_ = torch.empty_like(q_), torch.empty_like(k_)
        sms, _ = time_device_steps(lambda: side_ops.rmsnorm_qk(q_, k_, wq_, wk_, eps_, qn_, kn_), 10, 3, flush)
        nb_ = 4 * q_.numel() * 4
        side["rmsnorm_qk flux_4608"] = {"us": round(sms / 10 * 1e3, 2), "bound": "hbm",
                                        "frac": round(nb_ / (sms / 10) / 1e6 / peaks["hbm_gbs"], 4)}
        del q_, k_, qn_, kn_
        pb, pl, pc, pw = W.MAMBA_TAIL_SHAPES["mamba_b1_l2048"]
        pp, pmask, pcw, pcb = W.make_mamba_tail_inputs(pb, pl, pc, pw, 0, dev)
        pout = torch.empty(pb, pc, pl, dtype=torch.bfloat16, device=dev)
        sms, _ = time_device_steps(lambda: side_ops.mamba_conv1d_tail(pp, pmask, pcw, pcb, pout), 10, 3, flush)
        side["mamba_conv1d_tail b1_l2048"] = {"us": round(sms / 10 * 1e3, 2), "bound": "hbm",
                                              "frac": round(2 * pb * pl * pc * 2 / (sms / 10) / 1e6 / peaks["hbm_gbs"], 4)}
        gen_ = torch.Generator().manual_seed(0)
        ph = (torch.randn(pb * pl, 8192, generator=gen_) * 0.5).to(torch.bfloat16).to(dev)
        pwt = (torch.randn(pw, 512, generator=gen_) * 0.02).to(torch.bfloat16).to(dev).repeat(1, 16)
        pbias = (torch.randn(pw, generator=gen_) * 0.1).to(torch.bfloat16).to(dev)
        sms, _ = time_device_steps(lambda: side_ops.mamba_in_proj(ph, pwt, pbias, pp.view(pb * pl, pw)), 5, 3, flush)
        side["mamba_in_proj M=2048 K=8192 N=32768"] = {
            "us": round(sms / 5 * 1e3, 2), "bound": "tensor (bf16)",
            "frac": round(2.0 * pb * pl * 8192 * pw / (sms / 5) / 1e9 / peaks["bf16_tflops"], 4)}
        scode, sdetail = side_ops.last_status()
        if scode != 0:
            raise SystemExit(f"bench.py: side-ops device status {scode} detail {sdetail:#x}")
        result["also"].append({"workload": "side operators (problems 038, 029)", "rows": side,
                               "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"]}})
        del pp, pmask, pcw, pcb, pout, ph, pwt, pbias
        torch.cuda.empty_cache()
        # last, because seconds under the power cap leave the part hot and slow for whatever is timed next
        sout = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        result["also"].append({"workload": f"{workload} back to back (sustained)",
                               **sustained_leg(lambda: pkg.run(*local.args(), sout), flops_job, peaks, local_rank)})
        del sout, local
        torch.cuda.empty_cache()
        cpu_inp = W.make_inputs(m, k, n, seed=0, device="cpu")
        result["cpu_baseline"] = cpu_baseline(cpu_inp, oracle)
    if rank == 0:
        print(json.dumps(result), flush=True)
    if n_gpus > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------
# reference arm: the CPU definition (dequantise, fp32 matmul, SwiGLU) on the host cores
# --------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from oracle import gateup_oracle as oracle
    from sol_execbench_b200_kernels_b200 import workloads as W

    # a launcher for several ranks pins every rank to one OpenMP thread; this arm is the host cores' number
    torch.set_num_threads(os.cpu_count() or 1)
    n_gpus = max(world, args.gpus)
    workload = args.workload or ("prefill_8b" if n_gpus == 1 else "prefill_sharded")
    m, k, n = W.SHAPES[workload]
    # bounded sample: a row block of the workload, sized so warmup + steps stay within minutes
    rows = min(m, 1024)
    inp = W.make_inputs(rows, k, n, seed=0, device="cpu")
    for _ in range(args.warmup):
        oracle.gateup_dequant(*inp.args())
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.gateup_dequant(*inp.args())
    dt = (time.perf_counter() - t0) / args.steps
    value = 4.0 * rows * k * n / dt / 1e12
    sample = (f"{rows} token rows of {workload} (M={m}, K={k}, N={n}) per step; weights dequantised inside every "
              f"step as the CPU definition does; throughput is per-row-proportional for the matmul part")
    # The reference itself has no CPU code for this path (its CPU definition lives in a dataset that is fetched at
    # set-up); what it does ship is a single-GPU kernel.  Where that kernel can run (one GPU, the reference copy
    # present) its time on this box is reported beside the CPU number, measured in a child process.
    reference_gpu = {"unavailable": "the reference is single-GPU"}
    if n_gpus == 1:
        if not torch.cuda.is_available():
            reference_gpu = {"unavailable": "no CUDA device"}
        elif not os.path.exists(os.path.join(REF_KERNEL_DIR, "kernel.py")):
            reference_gpu = {"unavailable": "no copy of the reference's kernel directory on this machine"}
        else:
            gpu_rows, failures = ref_gpu_groups(["prefill_8b"] if workload == "prefill_8b" else [], 10, 3, timeout_s=420)
            reference_gpu = gpu_rows[0] if gpu_rows else {"unavailable": "; ".join(failures) or f"no group for {workload}"}
            reference_gpu["what"] = ("the reference's kernel.py::run (two CuTe-DSL GEMMs + Triton SwiGLU) and this "
                                     "library timed alternately on the same operands, CUDA events, L2 flushed")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": "TFLOP/s", "n_gpus": n_gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "strong" if n_gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32 (dequantised e4m3)",
        "data": "synthetic", "config": {"workload": f"{workload}: M={m} K={k} N={n}", "sample_rows": rows},
        "cpu_baseline": {"value": round(value, 4), "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                         "host_cpus": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "reference_gpu": reference_gpu,
    }), flush=True)


# --------------------------------------------------------------------------------------
# same-harness GPU comparison with the reference's own default variant (one GPU only)
# --------------------------------------------------------------------------------------
REF_KERNEL_DIR = os.path.join(ROOT, "baseline", "_ref", "179_fp8_mlp_gate_up_projection")
# the M values of the reference's own micro-benchmark at its native K = 3584, N = 18944 (tools/bench_179_epilogue.py:15-16)
REF_NATIVE_M = (384, 512, 768, 1152, 1280, 1792, 2048, 2304, 2816, 3072, 3584, 3840, 5120, 5632, 6144, 8704)
REF_GPU_GROUPS = {"prefill_8b": (4096, 14336, (4096,)), "reference_native": (3584, 18944, REF_NATIVE_M)}


def _load_reference_kernel():
    """The unmodified kernels/179_fp8_mlp_gate_up_projection/kernel.py of the reference, from the git-ignored copy
    under baseline/_ref (it loads NVIDIA's CuTe-DSL blockwise GEMM example from $CUTLASS_DIR: the image's tree)."""
    import importlib.util

    path = os.path.join(REF_KERNEL_DIR, "kernel.py")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{os.path.relpath(path, ROOT)} is not on this machine")
    fi = importlib.util.find_spec("flashinfer")
    if fi is None:
        raise FileNotFoundError("no CUTLASS tree on this machine (flashinfer's vendored copy)")
    os.environ.setdefault("CUTLASS_DIR", os.path.join(os.path.dirname(fi.origin), "data", "cutlass"))
    spec = importlib.util.spec_from_file_location("_reference_179_kernel", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def run_ref_gpu_one(args):
    """Child of --ref-gpu: one (K, N) per process, because the reference caches its compiled kernel under a key
    that omits K and N (kernel.py:263).  Times the reference's `run` (kernel.py:398-503: two CuTe-DSL GEMMs + a
    Triton SwiGLU) and this library's `run` alternately on the same operands, same L2 flush, same CUDA events."""
    import sol_execbench_b200_kernels_b200 as pkg
    from sol_execbench_b200_kernels_b200 import workloads as W

    k, n, ms_list = args.ref_gpu_one.split(",")
    k, n = int(k), int(n)
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    ref = _load_reference_kernel()
    flush = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.float32, device=dev)
    rows = []
    for m in (int(v) for v in ms_list.split(":")):
        inp = W.make_inputs(m, k, n, seed=0, device=dev)
        out_ref = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        out_own = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        fns = {"reference": lambda: ref.run(*inp.args(), out_ref), "this_library": lambda: pkg.run(*inp.args(), out_own)}
        for fn in fns.values():
            for _ in range(max(3, args.warmup)):
                fn()
        torch.cuda.synchronize()
        times = {name: [] for name in fns}
        for _ in range(args.steps):
            for name, fn in fns.items():
                flush_l2(flush)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                times[name].append(a.elapsed_time(b))
        med = {name: sorted(t)[len(t) // 2] for name, t in times.items()}
        diff = (out_ref.float() - out_own.float()).abs()
        flops = W.algorithmic_flops(m, k, n)
        rows.append({"m": m, "k": k, "n": n, "reference_ms": round(med["reference"], 5),
                     "this_library_ms": round(med["this_library"], 5),
                     "reference_tflops": round(flops / (med["reference"] * 1e-3) / 1e12, 1),
                     "this_library_tflops": round(flops / (med["this_library"] * 1e-3) / 1e12, 1),
                     "speedup": round(med["reference"] / med["this_library"], 3),
                     "max_abs_between": float(diff.max()), "frac_bit_equal": float((out_ref == out_own).float().mean())})
        del inp, out_ref, out_own
        torch.cuda.empty_cache()
    code, detail = pkg.last_status()
    print(json.dumps({"k": k, "n": n, "rows": rows, "device_status": code}), flush=True)


def ref_gpu_groups(groups, steps, warmup, timeout_s=900):
    """Runs run_ref_gpu_one in a child process per (K, N); returns (rows, failures)."""
    rows, failures = [], []
    for name in groups:
        k, n, ms = REF_GPU_GROUPS[name]
        cmd = [sys.executable, os.path.abspath(__file__), "--ref-gpu-one", f"{k},{n},{':'.join(map(str, ms))}",
               "--steps", str(steps), "--warmup", str(warmup)]
        try:
            proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s)
            line = [l for l in proc.stdout.splitlines() if l.startswith("{")]
            if proc.returncode != 0 or not line:
                tail = (proc.stderr or proc.stdout).strip().splitlines()[-1:] or ["no output"]
                failures.append(f"{name}: exit {proc.returncode}: {tail[0][:200]}")
                continue
            rows += json.loads(line[-1])["rows"]
        except subprocess.TimeoutExpired:
            failures.append(f"{name}: no result within {timeout_s} s")
    return rows, failures


def run_ref_gpu(args):
    """Study line: the reference's default variant against this library on one B200, same harness, on prefill_8b
    and on the reference's native shape over its own list of M."""
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 or args.gpus > 1:
        raise SystemExit("bench.py --ref-gpu: one GPU only (the reference is single-GPU)")
    rows, failures = ref_gpu_groups(list(REF_GPU_GROUPS), max(5, min(args.steps, 10)), args.warmup)
    print(json.dumps({"study": "reference default variant (kernel.py::run) against this library, one B200, CUDA events, "
                               f"L2 flushed (write then read of {L2_FLUSH_BYTES >> 20} MiB) before every timed call, medians",
                      "rows": rows, "failures": failures}), flush=True)


def run_trace(args):
    """Study line: where the roles of the CTA-pair kernel spend their time.  Needs the library built with
    -DGU_TRACE (`python -m sol_execbench_b200_kernels_b200.build --trace`, or --lib for another study build);
    prints, per K block and for the first CTA pair, the cycles each role waited for the others, and the time
    stamps of sixteen consecutive K blocks of the first tile (issuer and one consumer warp)."""
    import ctypes

    import sol_execbench_b200_kernels_b200 as pkg
    from sol_execbench_b200_kernels_b200 import _cabi
    from sol_execbench_b200_kernels_b200 import workloads as W

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    workload = args.workload or "prefill_8b"
    m, k, n = W.SHAPES[workload]
    inp = W.make_inputs(m, k, n, seed=0, device=dev)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.float32, device=dev)
    buf = (ctypes.c_uint64 * 288)()
    for _ in range(3):
        pkg.run_with_plan(*inp.args(), out, "tile_pair")
    torch.cuda.synchronize()
    _cabi.lib.gu_trace_read(buf, 288, 1)
    total_ms, _ = time_device_steps(lambda: pkg.run_with_plan(*inp.args(), out, "tile_pair"), args.steps, 0, flush)
    words = _cabi.lib.gu_trace_read(buf, 288, 1)
    if words < 288:
        raise SystemExit("bench.py --trace: this library was built without -DGU_TRACE (see --lib)")
    names = ["producer_wait_slot", "issuer_wait_operands_and_stage", None, "consumer_wait_partial", None, "consumer_k_loop",
             "consumer_hand_over", "epilogue_busy", "epilogue_wait", "cta_total", "k_blocks"]
    roles = {}
    for r in range(2):
        v = [int(buf[16 * r + i]) for i in range(11)]
        kbn = max(v[10], 1)
        roles[f"cta{r}"] = {nm: round(x / kbn, 1) for nm, x in zip(names, v) if nm and nm != "k_blocks"}
    ev = lambda r, role, i: int(buf[32 + (r * 2 + role) * 64 + i])
    base = ev(0, 0, 0)
    stamps = [{"k_block": 8 + i,
               "issuer_polls_passed": ev(0, 0, 4 * i) - base, "issuer_mmas_issued": ev(0, 0, 4 * i + 2) - base,
               "issuer_commits_issued": ev(0, 0, 4 * i + 3) - base, "consumer_partial_seen": ev(0, 1, 4 * i) - base,
               "consumer_stage_handed_back": ev(0, 1, 4 * i + 3) - base} for i in range(16)]
    print(json.dumps({"study": "CTA-pair kernel: cycles per K block each role of the first pair spent (trace build; the "
                               "counters cost the traced threads some cycles themselves)",
                      "workload": f"{workload}: M={m} K={k} N={n}", "ms_per_step": round(total_ms / args.steps, 5),
                      "steps": args.steps, "cycles_per_k_block": roles,
                      "time_stamps_even_cta_cycles": stamps}), flush=True)


def run_mlp(args):
    """Tensor-parallel MLP block (quantise -> gate/up + SwiGLU -> down projection -> sum over ranks) on N GPUs:
    the NCCL all-reduce form against the form whose reduction runs in this library's kernels over peer memory.
    A study line, not the headline metric."""
    import torch.distributed as dist

    import sol_execbench_b200_kernels_b200 as pkg
    from sol_execbench_b200_kernels_b200 import workloads as W

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("bench.py --mlp: launch under torch.distributed.run with 2 or more ranks")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    m, h, n = W.SHAPES["prefill_8b"]
    full = W.make_inputs(m, h, n, seed=0, device=dev)
    gw, sg, uw, su = (t.clone() for t in pkg.shard_weights(full.gate_proj_weight, full.scale_gate,
                                                           full.up_proj_weight, full.scale_up, rank, world))
    del full
    torch.manual_seed(1)
    dq, sd = W.quantize_weight_128x128(torch.randn(h, n, device=dev) * 0.02)
    dw, ds = pkg.shard_down_weights(dq, sd, rank, world)
    del dq, sd
    xb = torch.randn(m, h, device=dev).to(torch.bfloat16)
    flush = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.float32, device=dev)
    bufs = pkg.ReduceBuffers(m, h, dev)
    forms = {
        "nccl_all_reduce": lambda: pkg.mlp_block_sharded(xb, gw, sg, uw, su, dw, ds),
        "fused_peer_stores": lambda: pkg.mlp_block_sharded_fused(xb, gw, sg, uw, su, dw, ds, bufs),
    }
    res = {}
    for name, fn in forms.items():
        total_ms, _ = time_device_steps(fn, args.steps, args.warmup, flush, lambda: dist.barrier())
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name] = round(float(t.item()) / args.steps, 5)
    code, detail = pkg.last_status()
    if code != 0:
        raise SystemExit(f"bench.py: device status {code} detail {detail:#x}")
    if rank == 0:
        flops = 2.0 * m * h * n * 3
        print(json.dumps({"study": "tensor-parallel MLP block", "n_gpus": world, "m": m, "hidden": h, "intermediate": n,
                          "ms_per_step": res, "tflops": {k: round(flops / (v * 1e-3) / 1e12, 1) for k, v in res.items()},
                          "steps": args.steps, "warmup": args.warmup}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def run_side(args):
    """The side operators on one GPU, CUDA-event time per launch with L2 flushed: the two HBM-bound ones (per-head
    RMSNorm of query / key; Mamba conv1d tail) as achieved algorithmic GB/s against the measured copy bandwidth, the
    Mamba input projection as TFLOP/s against the measured bf16 GEMM rate.  A study line, not the headline metric."""
    from sol_execbench_b200_kernels_b200 import side_ops
    from sol_execbench_b200_kernels_b200 import workloads as W

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    flush = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.float32, device=dev)
    rows = {}
    for name, (tokens, heads) in W.RMSNORM_SHAPES.items():
        if args.workload and args.workload != name:
            continue
        q, k, wq, wk, eps = W.make_rmsnorm_inputs(tokens, heads, 0, dev)
        qn, kn = torch.empty_like(q), torch.empty_like(k)
        total, _ = time_device_steps(lambda: side_ops.rmsnorm_qk(q, k, wq, wk, eps, qn, kn), args.steps, args.warmup, flush)
        nbytes = 4 * q.numel() * 4          # two tensors, read and written once, fp32
        rows[name] = (total / args.steps, nbytes)
    for name, (b, l, c, w) in W.MAMBA_TAIL_SHAPES.items():
        if args.workload and args.workload != name:
            continue
        p, mask, cw, cb = W.make_mamba_tail_inputs(b, l, c, w, 0, dev)
        out = torch.empty(b, c, l, dtype=torch.bfloat16, device=dev)
        total, _ = time_device_steps(lambda: side_ops.mamba_conv1d_tail(p, mask, cw, cb, out), args.steps, args.warmup, flush)
        nbytes = 2 * b * l * c * 2          # the convolved half read once, the result written once, bf16
        rows[name] = (total / args.steps, nbytes)
    # the Mamba input projection (tensor-bound): this library's tcgen05 kernel and, as the library baseline on the same
    # inputs, torch's linear (cuBLAS); K = 8192, N = 32768 as the reference fixes them
    proj = {}
    for name, (b, l, c, w) in W.MAMBA_TAIL_SHAPES.items():
        if args.workload and args.workload != name:
            continue
        m, kdim = b * l, 8192
        g = torch.Generator().manual_seed(0)
        hidden = (torch.randn(m, kdim, generator=g) * 0.5).to(torch.bfloat16).to(dev)
        weight = (torch.randn(w, 512, generator=g) * 0.02).to(torch.bfloat16).to(dev).repeat(1, kdim // 512)
        bias = (torch.randn(w, generator=g) * 0.1).to(torch.bfloat16).to(dev)
        out = torch.empty(m, w, dtype=torch.bfloat16, device=dev)
        total, _ = time_device_steps(lambda: side_ops.mamba_in_proj(hidden, weight, bias, out), args.steps, args.warmup, flush)
        lib_total, _ = time_device_steps(lambda: torch.nn.functional.linear(hidden, weight, bias), args.steps, args.warmup, flush)
        want = torch.nn.functional.linear(hidden, weight, bias)
        rel = float(torch.linalg.vector_norm(out.float() - want.float()) / torch.linalg.vector_norm(want.float()))
        flops = 2.0 * m * kdim * w
        proj[name + "_in_proj"] = {
            "m": m, "k": kdim, "n": w, "us": round(total / args.steps * 1e3, 2),
            "tflops": round(flops / (total / args.steps) / 1e9, 1),
            "frac": round(flops / (total / args.steps) / 1e9 / peaks["bf16_tflops"], 4),
            "torch_linear_us": round(lib_total / args.steps * 1e3, 2),
            "torch_linear_tflops": round(flops / (lib_total / args.steps) / 1e9, 1),
            "rel_l2_vs_torch_linear": rel}
        del hidden, weight, bias, out, want
    code, detail = side_ops.last_status()
    if code != 0:
        raise SystemExit(f"bench.py: side-ops device status {code} detail {detail:#x}")
    src = "of measured" if peaks["_source"] == "measured" else "of fallback"
    print(json.dumps({
        "study": "side operators", "steps": args.steps, "warmup": args.warmup, "peak_gbs": peaks["hbm_gbs"],
        "peak_source": f"hbm_gbs, {src}", "gpu_launches": side_ops.launch_count(),
        "rows": {k: {"us": round(ms * 1e3, 2), "algorithmic_bytes": nb, "gbs": round(nb / ms / 1e6, 1),
                     "frac": round(nb / ms / 1e6 / peaks["hbm_gbs"], 4)} for k, (ms, nb) in rows.items()},
        "projection": {"peak_tflops": peaks["bf16_tflops"], "peak_source": f"bf16_tflops burst, {src}", "rows": proj}}),
        flush=True)


def run_graph(args):
    """Decode-sized calls issued one after another, as a token loop does: eager calls through the Python entry point
    against replays of one CUDA graph that recorded the call.  Wall clock per call over a few hundred calls (the GPU
    is never flushed here: the point is the host cost per launch).  A study line, not the headline metric."""
    import sol_execbench_b200_kernels_b200 as pkg
    from sol_execbench_b200_kernels_b200 import workloads as W

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    rows = {}
    calls = 300
    for name, (m, k, n) in {"m1_k4096_n14336": (1, 4096, 14336), "m16_k4096_n14336": (16, 4096, 14336),
                            "decode_70b": W.SHAPES["decode_70b"]}.items():
        inp = W.make_inputs(m, k, n, seed=0, device=dev)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        for _ in range(5):
            pkg.run(*inp.args(), out)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(calls):
            pkg.run(*inp.args(), out)
        torch.cuda.synchronize()
        eager = (time.perf_counter() - t0) / calls
        want = out.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            pkg.run(*inp.args(), out)
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(calls):
            graph.replay()
        torch.cuda.synchronize()
        replay = (time.perf_counter() - t0) / calls
        rows[name] = {"plan": pkg.select_plan(m, k, n), "eager_us_per_call": round(eager * 1e6, 2),
                      "graph_replay_us_per_call": round(replay * 1e6, 2), "replay_equals_eager": bool(torch.equal(out, want))}
    code, detail = pkg.last_status()
    if code != 0:
        raise SystemExit(f"bench.py: device status {code} detail {detail:#x}")
    print(json.dumps({"study": "decode loop: eager calls against CUDA-graph replays", "calls": calls, "rows": rows,
                      "gpu_launches": pkg.launch_count()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default=None, help="override: one of workloads.SHAPES")
    ap.add_argument("--gather", action="store_true", help="N>1: also all-gather the contiguous [M, N] output")
    ap.add_argument("--fused-gather", action="store_true",
                    help="N>1: contiguous [M, N] output on every rank through peer stores in the kernel epilogue")
    ap.add_argument("--e2e-chunks", type=int, default=4,
                    help="row chunks of the host-memory pipeline in the e2e leg (measured on prefill_8b: 2 chunks 2.31 ms, "
                         "4 2.13, 8 2.21, 16 2.22 per step)")
    ap.add_argument("--mlp", action="store_true",
                    help="N>1: tensor-parallel MLP block, NCCL all-reduce against the fused peer-store reduction")
    ap.add_argument("--graph", action="store_true",
                    help="one GPU: decode-sized call loop, eager against CUDA-graph replay (host cost per launch)")
    ap.add_argument("--side", action="store_true",
                    help="one GPU: the side operators (RMSNorm of query/key, Mamba conv1d tail) against the HBM roofline")
    ap.add_argument("--sweep", action="store_true", help="M sweep at K=4096, N=14336 on one GPU (plan crossover study)")
    ap.add_argument("--ref-gpu", action="store_true",
                    help="one GPU: the reference's default variant against this library, same harness (needs baseline/_ref)")
    ap.add_argument("--ref-gpu-one", default=None, help=argparse.SUPPRESS)
    ap.add_argument("--trace", action="store_true", help="one GPU: role counters of the CTA-pair kernel (trace build)")
    ap.add_argument("--lib", default=None,
                    help="study runs: load this build of the library (e.g. libgateup_trace.so) instead of libgateup.so")
    args = ap.parse_args()
    if args.lib or args.trace:
        from pathlib import Path

        import sol_execbench_b200_kernels_b200.build as _build

        _build.LIB_PATH = Path(args.lib).resolve() if args.lib else _build.TRACE_LIB_PATH
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.trace:
        run_trace(args)
    elif args.ref_gpu_one:
        run_ref_gpu_one(args)
    elif args.ref_gpu:
        run_ref_gpu(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.mlp:
        run_mlp(args)
    elif args.side:
        run_side(args)
    elif args.graph:
        run_graph(args)
    elif args.sweep:
        run_sweep(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
