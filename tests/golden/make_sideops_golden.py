"""Generates the side-operator fixtures in this directory by running the reference's own CUDA kernels of
problems 038 and 029 (compiled unmodified by oracle/build_ref.py into oracle/_ref/) on seeded inputs.

Needs a B200.  Usage, from the repository root:

    python tests/golden/make_sideops_golden.py --out <directory> [--time]

Writes `<name>.pt` (sampled outputs of the reference) and `<name>.json` (shape, seed, sampling, sha256 of the
full output, error of the CPU restatement against it); copy them into tests/golden/ to commit them.  The inputs
are not stored: `workloads.make_rmsnorm_inputs` / `make_mamba_tail_inputs` regenerate them bit for bit.
With --time also writes `reference_gpu_time_sideops.json` (CUDA events, L2 flushed between calls).
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import sideops_oracle as O  # noqa: E402
from sol_execbench_b200_kernels_b200 import workloads as W  # noqa: E402

# name -> (tokens, heads, seed, row stride)
RMSNORM_CASES = {"ref038_t128": (128, 48, 3, 16), "ref038_t2048": (2048, 48, 4, 259), "ref038_t4608": (4608, 48, 5, 585)}
# name -> (batch, sequence, seed, channel stride, sampled channels kept); channels 16384 / width 32768 are fixed
# by the reference
MAMBA_CASES = {"ref029_b1_l128": (1, 128, 6, 16, 256), "ref029_b2_l1000": (2, 1000, 7, 128, 64),
               "ref029_b3_l333": (3, 333, 8, 64, 128)}


def load_ref(name: str):
    path = os.path.join(ROOT, "oracle", "_ref", name, name + ".so")
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest()


def time_fn(fn, iters=20):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        flush.sum()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--time", action="store_true")
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    dev = torch.device("cuda:0")
    times = {}

    ref038 = load_ref("ref038_rmsnorm_qk")
    if ref038 is not None:
        for name, (tokens, heads, seed, rs) in RMSNORM_CASES.items():
            q, k, wq, wk, eps = W.make_rmsnorm_inputs(tokens, heads, seed, dev)
            qn, kn = torch.empty_like(q), torch.empty_like(k)
            ref038.run(q, k, wq, wk, eps, qn, kn)
            torch.cuda.synchronize()
            oq, ok = O.rmsnorm_qk(q.cpu(), k.cpu(), wq.cpu(), wk.cpu(), eps)
            err = max(float((oq - qn.cpu()).abs().max()), float((ok - kn.cpu()).abs().max()))
            torch.save({"query_norm": qn[0, ::rs].cpu().clone(), "key_norm": kn[0, ::rs].cpu().clone()},
                       os.path.join(args.out, name + ".pt"))
            json.dump({"op": "rmsnorm_qk", "tokens": tokens, "heads": heads, "seed": seed, "row_stride": rs,
                       "sha256_query_norm": sha(qn), "sha256_key_norm": sha(kn), "oracle_max_abs_err": err},
                      open(os.path.join(args.out, name + ".json"), "w"), indent=1)
            print(name, "oracle max abs err", err)
        if args.time:
            for wl, (tokens, heads) in W.RMSNORM_SHAPES.items():
                q, k, wq, wk, eps = W.make_rmsnorm_inputs(tokens, heads, 0, dev)
                qn, kn = torch.empty_like(q), torch.empty_like(k)
                times["rmsnorm_qk/" + wl] = time_fn(lambda: ref038.run(q, k, wq, wk, eps, qn, kn))
                from sol_execbench_b200_kernels_b200 import side_ops
                times["rmsnorm_qk_this_package/" + wl] = time_fn(lambda: side_ops.rmsnorm_qk(q, k, wq, wk, eps, qn, kn))
    else:
        print("oracle/_ref/ref038_rmsnorm_qk missing: skipped")

    ref029 = load_ref("ref029_mamba_conv1d")
    if ref029 is not None:
        # the extension exports the whole op (projection + tail); the projection it computed is read back from
        # the storage behind `gate`, which the reference returns as a view of it (binding.cpp:88-92)
        for name, (batch, sequence, seed, cs, keep) in MAMBA_CASES.items():
            g = torch.Generator().manual_seed(seed)
            hidden = (torch.randn(batch, sequence, 8192, generator=g) * 0.5).to(torch.bfloat16).to(dev)
            in_w = (torch.randn(32768, 8192, generator=g) * 0.02).to(torch.bfloat16).to(dev)
            in_b = (torch.randn(32768, generator=g) * 0.1).to(torch.bfloat16).to(dev)
            _, mask, cw, cb = W.make_mamba_tail_inputs(batch, sequence, 16384, 64, seed, dev)
            out, gate = ref029.run(hidden, mask, in_w, in_b, cw, cb)
            torch.cuda.synchronize()
            projected = torch.empty(0, dtype=torch.bfloat16, device=dev).set_(
                gate.untyped_storage(), 0, (batch, sequence, 32768), (sequence * 32768, 32768, 1))
            want = O.mamba_conv1d_tail(projected.cpu(), mask.cpu(), cw.cpu(), cb.cpu())
            diff = (want.float() - out.cpu().float()).abs()
            nz = int((diff > 0).sum())
            torch.save({"projected_x": projected[:, :, :16384:cs][:, :, :keep].cpu().clone(), "mask": mask.cpu(),
                        "conv_w": cw[::cs][:keep].cpu().clone(), "conv_b": cb[::cs][:keep].cpu().clone(),
                        "output": out[:, ::cs][:, :keep].cpu().clone()}, os.path.join(args.out, name + ".pt"))
            json.dump({"op": "mamba_conv1d_tail", "batch": batch, "sequence": sequence, "seed": seed,
                       "channel_stride": cs, "channels_kept": keep, "sha256_output": sha(out), "oracle_mismatches": nz,
                       "oracle_max_abs_err": float(diff.max()), "numel": out.numel()},
                      open(os.path.join(args.out, name + ".json"), "w"), indent=1)
            print(name, "oracle mismatches", nz, "of", out.numel(), "max", float(diff.max()))
        if args.time:
            # whole op (projection GEMM + tail) of the reference; run this script under a profiler's launch list
            # to read the reference's tail kernel and this package's side by side on the same projection
            from sol_execbench_b200_kernels_b200 import side_ops
            batch, sequence = 4, 2048
            g = torch.Generator().manual_seed(1)
            hidden = (torch.randn(batch, sequence, 8192, generator=g) * 0.5).to(torch.bfloat16).to(dev)
            in_w = (torch.randn(32768, 8192, generator=g) * 0.02).to(torch.bfloat16).to(dev)
            in_b = (torch.randn(32768, generator=g) * 0.1).to(torch.bfloat16).to(dev)
            _, mask, cw, cb = W.make_mamba_tail_inputs(batch, sequence, 16384, 64, 1, dev)
            times["mamba_conv1d_with_gating/reference_whole_op_b4_l2048"] = time_fn(
                lambda: ref029.run(hidden, mask, in_w, in_b, cw, cb), iters=5)
            times["mamba_conv1d_with_gating/this_package_whole_op_b4_l2048"] = time_fn(
                lambda: side_ops.mamba_conv1d_with_gating(hidden, mask, in_w, in_b, cw, cb), iters=5)
    else:
        print("oracle/_ref/ref029_mamba_conv1d missing: skipped")

    if args.time:
        json.dump({"unit": "ms, median of 20, L2 flushed", "times": times},
                  open(os.path.join(args.out, "reference_gpu_time_sideops.json"), "w"), indent=1)
        print(times)


if __name__ == "__main__":
    main()
