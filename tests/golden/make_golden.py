"""Generates the golden fixtures in this directory by running the reference submission's own
GPU kernel (kernels/179_fp8_mlp_gate_up_projection/kernel.py::run, unmodified) on seeded inputs.

Needs a B200, the image's CUTLASS tree (the reference loads NVIDIA's CuTe-DSL blockwise GEMM
example from $CUTLASS_DIR) and an unmodified copy of the reference's kernel directory at
baseline/_ref/179_fp8_mlp_gate_up_projection (git-ignored).  Usage, from the repository root:

    python tests/golden/make_golden.py --out <directory> [--only NAME[,NAME...]]

Each shape runs in a fresh process because the reference caches its compiled kernel under a key
that omits K and N (kernel.py:263).  For every shape a `<name>.pt` (sampled rows/columns of the
reference output) and a `<name>.json` (shape, seed, sampling, sha256 of the full output, and the
error of both CPU oracles against it) are written; copy them into tests/golden/ to commit them.
The inputs are not stored: `workloads.make_inputs(M, K, N, seed)` regenerates them bit for bit.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF_DIR = os.path.join(ROOT, "baseline", "_ref", "179_fp8_mlp_gate_up_projection")

# name -> (M, K, N, seed, row stride, column stride)
SHAPES = {
    "ref_small_128x2048x5632": (128, 2048, 5632, 0, 1, 11),
    "ref_square_128x512x512": (128, 512, 512, 21, 1, 1),
    "ref_native_256x3584x18944": (256, 3584, 18944, 22, 4, 37),
    "ref_256x1024x1024": (256, 1024, 1024, 23, 2, 2),
    # the two large configurations of the benchmark line (tensor-bound prefill, and the shape that is column-sharded)
    "ref_prefill_8b_4096x4096x14336": (4096, 4096, 14336, 0, 157, 37),
    "ref_prefill_sharded_16384x7168x18432": (16384, 7168, 18432, 0, 1021, 37),
}


def _load_reference():
    spec = importlib.util.find_spec("flashinfer")
    cutlass_dir = os.path.join(os.path.dirname(spec.origin), "data", "cutlass")
    os.environ.setdefault("CUTLASS_DIR", cutlass_dir)
    path = os.path.join(REF_DIR, "kernel.py")
    if not os.path.exists(path):
        raise SystemExit(f"{path} missing: copy the reference's kernel directory there first")
    spec = importlib.util.spec_from_file_location("_reference_179_kernel", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _one(name: str, out_dir: str) -> None:
    import torch

    sys.path.insert(0, ROOT)
    from oracle import gateup_oracle as O
    from sol_execbench_b200_kernels_b200 import workloads as W

    ref = _load_reference()
    m, k, n, seed, rs, cs = SHAPES[name]
    inp = W.make_inputs(m, k, n, seed=seed)
    g = inp.to("cuda:0")
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda:0")
    ref.run(*g.args(), out)
    torch.cuda.synchronize()
    out = out.cpu()
    rows = torch.arange(0, m, rs)
    cols = torch.arange(0, n, cs)
    stats = {}
    for oname, fn in (("blockwise", O.gateup_blockwise), ("dequant", O.gateup_dequant)):
        stats[oname] = O.error_stats(fn(*inp.args()), out)
    meta = {
        "shape": [m, k, n], "seed": seed, "row_stride": rs, "col_stride": cs,
        "generator": "reference kernels/179_fp8_mlp_gate_up_projection/kernel.py::run (default policy), "
                     f"torch {torch.__version__}, {torch.cuda.get_device_name(0)}",
        "sha256_full_output": hashlib.sha256(out.view(torch.int16).numpy().tobytes()).hexdigest(),
        "oracle_vs_reference": stats,
    }
    os.makedirs(out_dir, exist_ok=True)
    torch.save({"rows": rows, "cols": cols, "out": out[rows][:, cols].clone()}, os.path.join(out_dir, name + ".pt"))
    with open(os.path.join(out_dir, name + ".json"), "w") as f:
        json.dump(meta, f, indent=1)
    print(name, json.dumps(stats), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden", "_generated"))
    ap.add_argument("--only", default=None, help="comma-separated fixture names to (re)generate instead of all")
    ap.add_argument("--one", default=None)
    args = ap.parse_args()
    if args.one:
        return _one(args.one, args.out)
    names = [n for n in SHAPES if not args.only or n in args.only.split(",")]
    jobs = [["--one", n] for n in names]
    failed = 0
    for job in jobs:
        rc = subprocess.run([sys.executable, os.path.abspath(__file__), "--out", args.out, *job], timeout=900).returncode
        failed += rc != 0
    sys.exit(1 if failed else 0)


if __name__ == "__main__":
    main()
