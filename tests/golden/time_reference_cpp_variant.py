"""Times the reference's C++ variant of problem 179 (variants/cuda_cpp_v4, compiled unmodified by
oracle/build_ref.py) beside this package on the variant's fixed K = 3584, N = 18944, in one process and one harness
(CUDA events, L2 flushed before every launch, median of 20).  Needs a B200.

    python tests/golden/time_reference_cpp_variant.py --out <directory>

Writes `reference_gpu_time_cuda_cpp_v4.json`; copy it into tests/golden/ to commit it.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import sol_execbench_b200_kernels_b200 as pkg  # noqa: E402
from sol_execbench_b200_kernels_b200 import workloads as W  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    name = "ref179_cuda_cpp_v4"
    path = os.path.join(ROOT, "oracle", "_ref", name, name + ".so")
    if not os.path.exists(path):
        raise SystemExit(f"{path} missing: run oracle/build_ref.py first")
    spec = importlib.util.spec_from_file_location(name, path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def time_fn(fn, iters=20):
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

    rows = {}
    k, n = 3584, 18944
    for m in (512, 1152, 4096, 8704):
        inp = W.make_inputs(m, k, n, seed=0, device=dev)
        want = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        got = torch.empty_like(want)
        t_ref = time_fn(lambda: ref.run(*inp.args(), want))
        t_own = time_fn(lambda: pkg.run(*inp.args(), got))
        diff = (got.float() - want.float()).abs()
        flops = W.algorithmic_flops(m, k, n)
        rows[f"M={m}"] = {"reference_cpp_ms": round(t_ref, 4), "this_package_ms": round(t_own, 4),
                          "reference_cpp_tflops": round(flops / t_ref / 1e9, 1),
                          "this_package_tflops": round(flops / t_own / 1e9, 1),
                          "max_abs_diff": float(diff.max()), "elements_over_2e-2": int((diff > 2e-2).sum())}
        print(m, rows[f"M={m}"], flush=True)
    os.makedirs(args.out, exist_ok=True)
    json.dump({"shape": {"K": k, "N": n}, "unit": "ms, median of 20, L2 flushed", "rows": rows},
              open(os.path.join(args.out, "reference_gpu_time_cuda_cpp_v4.json"), "w"), indent=1)


if __name__ == "__main__":
    main()
