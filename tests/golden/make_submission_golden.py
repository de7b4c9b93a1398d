"""Generates the packaging fixtures in this directory with the reference's own tooling
(tools/extra_kernels.py of a checkout of the reference repository, imported, not copied):

* `toy_submission/manifest.compact.json` — a manifest (compact form; its canonical form is what gets packaged);
* `toy_submission_artifact.sha256` — sha256 of the artifact the reference's `build_artifact` makes of it;
* `traces_trial{1,2,3}.jsonl` + `trace_summary_expected.json` — seeded synthetic evaluator traces (16 workloads, the count the
  reference's lock file gives problem 29) and the summary the reference's `command_summarize` writes for them.

    python tests/golden/make_submission_golden.py /path/to/reference/checkout
"""
from __future__ import annotations

import importlib.util
import json
import random
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TOY = HERE / "toy_submission"


def main(reference_root: str) -> None:
    spec = importlib.util.spec_from_file_location("_reference_extra_kernels",
                                                  str(Path(reference_root) / "tools" / "extra_kernels.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)

    manifest = {
        "author": "fixture", "definition": "000_toy_scale",
        "description": "Packaging fixture — not a kernel. It exists so that the manifest rules, the forbidden-API audit, "
                       "the embedding of several sources (two of them headers, one plain text, one with non-ASCII "
                       "characters) and the canonical byte form can be checked against the reference's own packager "
                       "without depending on any real kernel source, which changes from commit to commit.",
        "name": "toy_scale_v1",
        "sources": [{"path": "binding.cpp"}, {"path": "kernel.cu"}, {"path": "scale.h"}, {"path": "config.h"},
                    {"path": "notes.txt"}],
        "spec": {"binding": "torch",
                 "compile_options": {"cflags": ["-O3"], "cuda_cflags": ["-O3", "-std=c++17"], "ld_flags": ["-lcuda"]},
                 "dependencies": [], "destination_passing_style": True, "entry_point": "binding.cpp::run",
                 "languages": ["cuda_cpp"], "target_hardware": ["B200", "LOCAL"]},
    }
    # the manifest is kept in compact form beside the toy sources; the canonical `solution.json` the packager wants is
    # written into a scratch copy (the tests do the same)
    (TOY / "manifest.compact.json").write_text(json.dumps(manifest, separators=(",", ":"), ensure_ascii=False) + "\n",
                                                encoding="utf-8")
    import shutil
    import tempfile
    scratch = Path(tempfile.mkdtemp()) / "toy_submission"
    shutil.copytree(TOY, scratch)
    (scratch / "solution.json").write_bytes(ref.canonical_json_bytes(manifest))
    ref.ROOT = scratch.parent
    ref.variant_dir = lambda config, variant=None: scratch
    config = {"name": "000_toy_scale", "directory": "toy_submission"}
    ref.load_source_manifest(config)
    artifact = ref.build_artifact(config, "B200", None, ["-DFIXTURE=1"])
    (HERE / "toy_submission_artifact.sha256").write_text(ref.sha256_bytes(artifact) + "\n")

    # traces: 16 workloads (problem 29 of the reference's lock file) x 3 trials, summarised by the reference's own
    # command_summarize
    load_lock = ref.load_lock  # reads the checkout's kernels/benchmark.lock.json
    ref.ROOT = Path(reference_root)
    lock = load_lock()
    config = ref.problem_config(lock, "29")
    workloads = config["workloads"]
    rng = random.Random(20260101)
    base = [rng.uniform(0.02, 3.0) for _ in range(workloads)]
    for trial in range(3):
        lines = []
        for w in range(workloads):
            latency = round(base[w] * rng.uniform(0.97, 1.03), 6)
            lines.append(json.dumps({"workload": {"uuid": f"w{w}"},
                                     "evaluation": {"status": "PASSED", "environment": {"hardware": "NVIDIA B200"},
                                                    "performance": {"latency_ms": latency}}}))
        (HERE / f"traces_trial{trial + 1}.jsonl").write_text("\n".join(lines) + "\n")
    import argparse
    ref.command_summarize(argparse.Namespace(
        problem_id=29, traces=[str(HERE / f"traces_trial{t}.jsonl") for t in (1, 2, 3)],
        output=str(HERE / "trace_summary_expected.json")))
    print("fixtures written")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
