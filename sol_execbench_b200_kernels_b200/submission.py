"""Benchmark-format side of the kernels: emit, check, package and summarise SOL-ExecBench submissions.

The reference repository ships each kernel as a directory with a `solution.json` manifest and its sources, checks
it (`tools/extra_kernels.py:291-393`, `load_source_manifest`), embeds the sources into one JSON artifact for the
evaluator (`:396-486`, `build_artifact`) and condenses three evaluator traces into a summary (`:699-746`,
`command_summarize`).  This module does the same for this package's kernels: `emit` writes a flat submission
directory (a torch binding + the CUDA sources + manifest, language `cuda_cpp`, binding `torch`), `validate` applies
the manifest rules and the forbidden-API audit, `package` produces the artifact bytes, `summarize` the trace summary.
Pure Python, no GPU and no network; the evaluator itself is not part of this repository.

    python -m sol_execbench_b200_kernels_b200.submission emit 179 <dir>
    python -m sol_execbench_b200_kernels_b200.submission lint <dir>
    python -m sol_execbench_b200_kernels_b200.submission package <dir> <artifact.json> [--target B200]
    python -m sol_execbench_b200_kernels_b200.submission build <dir> <build dir>      (torch extension, sm_100a)
    python -m sol_execbench_b200_kernels_b200.submission summarize <problem> <t1> <t2> <t3> --workloads N -o out.json
"""
from __future__ import annotations

import argparse
import hashlib
import json
import statistics
import sys
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BINDINGS = PKG_DIR / "submission_src"

# vocabulary of the manifest (tools/extra_kernels.py:29-40)
ALLOWED_LANGUAGES = {"cuda_cpp", "cublas", "cudnn", "cutlass", "cute_dsl", "pytorch", "triton"}
ALLOWED_DEPENDENCIES = {"cublas", "cudnn", "cutlass", "torch", "triton"}
CPP_LANGUAGES = {"cuda_cpp", "cublas", "cudnn", "cutlass"}
PYTHON_LANGUAGES = {"cute_dsl", "pytorch", "triton"}
TOP_LEVEL_FIELDS = {"author", "definition", "description", "name", "sources", "spec"}
SPEC_FIELDS = {"binding", "compile_options", "dependencies", "destination_passing_style", "entry_point", "languages",
               "target_hardware"}

# Source text a submission may not contain, lower-cased substring match (tools/extra_kernels.py:46-84): APIs that
# time, leave the current stream, start threads, touch the process / network / file system, delay, patch the
# runtime, reach the profiler or keep numeric tensors across calls.
FORBIDDEN_FRAGMENTS: Dict[str, tuple] = {
    "benchmark or evaluator timing": ("cudaeventcreate", "cudaeventrecord", "cudaeventelapsedtime", "clock_gettime",
                                      "std::chrono", "time.perf_counter", "torch.cuda.event"),
    "non-current CUDA stream or graph": ("cudastreamcreate", "getdefaultcudastream", "getstreamfrompool", "cudagraph"),
    "thread injection": ("std::thread", "pthread_create", "import threading"),
    "process, network, or filesystem access": ("std::getenv", "getenv(", "std::system", "system(", "popen(",
                                               "subprocess", "urllib", "requests.", "socket(", "fopen(", "ifstream",
                                               "/proc/"),
    "deliberate delay": ("sleep(", "usleep("),
    "Python runtime mutation": ("monkeypatch", "setattr(torch"),
    "profiler access": ("cupti", "nvtxrange"),
    "persistent numeric workspace": ("thread_local at::tensor", "thread_local torch::tensor"),
}


class SubmissionError(RuntimeError):
    """A manifest, source or trace that breaks the submission rules."""


# problem id -> what `emit` writes.  `sources` maps the name inside the submission to the file in this repository;
# the first entry is the torch binding that holds the entry point.
PROBLEMS: Dict[str, Dict[str, Any]] = {
    "179": {
        "definition": "003_fp8_mlp_gate_up_projection",
        "name": "fp8_mlp_gate_up_tcgen05_fused_swiglu",
        "description": "One-launch FP8 gate/up projection with SwiGLU for sm_100a: TMA-fed tcgen05 MMA over both "
                       "weight tiles per activation tile, fp32 per-128-block scale promotion from TMEM, bf16 rounding "
                       "after both GEMMs, SiLU and the product; weight-streaming stream-K plan for M <= 32.",
        "destination_passing_style": True,
        "sources": [("binding.cpp", BINDINGS / "binding_179.cpp"), ("gateup.cu", CSRC / "gateup.cu"),
                    ("gateup_tile.cuh", CSRC / "gateup_tile.cuh"), ("gateup_stream.cuh", CSRC / "gateup_stream.cuh"),
                    ("quantize_act.cuh", CSRC / "quantize_act.cuh"), ("reduce_gather.cuh", CSRC / "reduce_gather.cuh"),
                    ("ptx_sm100.cuh", CSRC / "ptx_sm100.cuh"), ("gateup.h", INCLUDE / "gateup.h")],
    },
    "38": {
        "definition": "038_flux_multi_head_rmsnorm_qk",
        "name": "flux_rmsnorm_qk_warp_rows",
        "description": "Per-head RMSNorm of query and key in one launch: four 512-byte rows per warp, all loads "
                       "issued before the reduction, HBM-bound.",
        "destination_passing_style": True,
        "sources": [("binding.cpp", BINDINGS / "binding_038.cpp"), ("sideops.cu", CSRC / "sideops.cu"),
                    ("sideops.h", INCLUDE / "sideops.h")],
    },
    "29": {
        "definition": "029_mamba_conv1d_with_gating",
        "name": "mamba_conv1d_tail_packed_f32x2",
        "description": "Mamba input projection through the vendor GEMM, then one kernel for mask, depthwise causal "
                       "conv1d, SiLU, mask and the [L, C] -> [C, L] transposition with packed f32x2 arithmetic.",
        "destination_passing_style": False,
        "sources": [("binding.cpp", BINDINGS / "binding_029.cpp"), ("sideops.cu", CSRC / "sideops.cu"),
                    ("sideops.h", INCLUDE / "sideops.h")],
    },
}

# in-repository include paths that become flat inside a submission directory
_INCLUDE_REWRITES = (('#include "../../include/gateup.h"', '#include "gateup.h"'),
                     ('#include "../../include/sideops.h"', '#include "sideops.h"'))


def canonical_json_bytes(value: Any) -> bytes:
    """The byte form the reference requires of a manifest: 2-space indent, sorted keys, one trailing newline
    (tools/extra_kernels.py:91-94)."""
    return (json.dumps(value, ensure_ascii=False, indent=2, sort_keys=True) + "\n").encode("utf-8")


def sha256_bytes(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def manifest_for(problem: str, author: str = "sol-execbench-b200-kernels") -> Dict[str, Any]:
    cfg = PROBLEMS[str(problem)]
    return {
        "author": author,
        "definition": cfg["definition"],
        "description": cfg["description"],
        "name": cfg["name"],
        "sources": [{"path": name} for name, _ in cfg["sources"]],
        "spec": {
            "binding": "torch",
            "compile_options": {"cflags": ["-O3", "-std=c++17"], "cuda_cflags": ["-O3", "-std=c++17"], "ld_flags": []},
            "dependencies": [],
            "destination_passing_style": cfg["destination_passing_style"],
            "entry_point": "binding.cpp::run",
            "languages": ["cuda_cpp"],
            "target_hardware": ["B200"],
        },
    }


def _write_if_changed(path: Path, data: bytes) -> None:
    # an unchanged file keeps its time stamp, so that an incremental build of the directory stays a no-op
    if not path.is_file() or path.read_bytes() != data:
        path.write_bytes(data)


def emit(problem: str, out_dir, author: str = "sol-execbench-b200-kernels") -> Path:
    """Write the submission directory of `problem` ("179", "38" or "29"): manifest, binding and sources, flat."""
    problem = str(int(problem))
    if problem not in PROBLEMS:
        raise SubmissionError(f"no submission recipe for problem {problem}")
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    for name, src in PROBLEMS[problem]["sources"]:
        text = Path(src).read_text(encoding="utf-8")
        for old, new in _INCLUDE_REWRITES:
            text = text.replace(old, new)
        _write_if_changed(out / name, text.encode("utf-8"))
    _write_if_changed(out / "solution.json", canonical_json_bytes(manifest_for(problem, author)))
    validate(out, definition=PROBLEMS[problem]["definition"])
    return out


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise SubmissionError(message)


def audit_source(text: str, where: str = "source") -> None:
    lowered = text.lower()
    for category, fragments in FORBIDDEN_FRAGMENTS.items():
        for fragment in fragments:
            if fragment in lowered:
                raise SubmissionError(f"forbidden {category} API {fragment!r} in {where}")


def validate(directory, definition: Optional[str] = None) -> Dict[str, Any]:
    """Apply the reference's manifest rules to `directory/solution.json` and audit the listed sources.
    Returns the manifest; raises SubmissionError with the first rule that fails."""
    directory = Path(directory)
    path = directory / "solution.json"
    _need(path.is_file(), f"{path} is missing")
    raw = path.read_bytes()
    try:
        manifest = json.loads(raw.decode("utf-8"))
    except ValueError as exc:
        raise SubmissionError(f"{path} is not JSON: {exc}") from exc
    _need(isinstance(manifest, dict), "solution.json must hold an object")
    _need(raw == canonical_json_bytes(manifest), "solution.json is not canonical JSON")
    unknown = set(manifest) - TOP_LEVEL_FIELDS
    _need(not unknown, f"unsupported solution field(s): {', '.join(sorted(unknown))}")
    if definition is not None:
        _need(manifest.get("definition") == definition, f"solution definition does not match {definition}")
    _need(bool(manifest.get("name")) and bool(manifest.get("author")), "solution name and author must be nonempty")
    spec = manifest.get("spec")
    _need(isinstance(spec, dict), "solution spec must be an object")
    _need(set(spec) == SPEC_FIELDS, f"solution spec fields mismatch (missing={sorted(SPEC_FIELDS - set(spec))}, "
                                    f"extra={sorted(set(spec) - SPEC_FIELDS)})")
    languages = spec["languages"]
    _need(isinstance(languages, list) and bool(languages) and all(l in ALLOWED_LANGUAGES for l in languages),
          "solution languages are missing or unsupported")
    uses_cpp = any(l in CPP_LANGUAGES for l in languages)
    uses_python = any(l in PYTHON_LANGUAGES for l in languages)
    _need(not (uses_cpp and uses_python), "C++ and Python solution languages cannot be mixed")
    expected_binding = "torch" if uses_cpp else None
    _need(spec["binding"] == expected_binding, f"solution binding must be {expected_binding!r} for its languages")
    deps = spec["dependencies"]
    _need(isinstance(deps, list) and all(d in ALLOWED_DEPENDENCIES for d in deps),
          "solution dependencies are malformed or unsupported")
    _need(isinstance(spec["destination_passing_style"], bool), "destination_passing_style must be a boolean")
    entry = spec["entry_point"]
    _need(isinstance(entry, str) and entry.count("::") == 1 and all(entry.split("::", 1)),
          "solution entry point must be <source>::<symbol>")
    options = spec["compile_options"]
    expected_options = {"cflags", "cuda_cflags", "ld_flags"} if uses_cpp else set()
    _need(isinstance(options, dict) and set(options) == expected_options,
          f"compile_options fields must be {sorted(expected_options)}")
    for key, values in options.items():
        _need(isinstance(values, list) and all(isinstance(v, str) for v in values),
              f"compile option {key} must be a list of strings")
    targets = spec["target_hardware"]
    _need(isinstance(targets, list) and "B200" in targets, "source solution must include B200 target hardware")
    sources = manifest.get("sources")
    _need(isinstance(sources, list) and bool(sources), "solution sources must be a nonempty list")
    seen = set()
    for source in sources:
        _need(isinstance(source, dict) and set(source) == {"path"}, "source manifest entries must contain only path")
        rel = Path(source["path"])
        _need(not rel.is_absolute() and ".." not in rel.parts, f"unsafe source path: {rel}")
        _need(rel.as_posix() not in seen, f"duplicate source path: {rel}")
        seen.add(rel.as_posix())
        local = directory / rel
        _need(not local.is_symlink() and local.is_file(), f"missing kernel source: {rel}")
        audit_source(local.read_text(encoding="utf-8"), rel.as_posix())
    _need(entry.split("::", 1)[0] in seen, "entry point file is not listed in sources")
    return manifest


def package(directory, target: str = "B200", extra_cuda_cflags: Optional[Iterable[str]] = None) -> bytes:
    """The artifact the evaluator takes: the manifest with every source's text embedded as `content` and the
    target hardware narrowed to `target` (tools/extra_kernels.py:396-486)."""
    directory = Path(directory)
    manifest = validate(directory)
    packaged = json.loads(json.dumps(manifest))
    packaged["spec"]["target_hardware"] = [target]
    if extra_cuda_cflags:
        _need(any(l in CPP_LANGUAGES for l in packaged["spec"]["languages"]),
              "extra CUDA flags require a C++/CUDA source variant")
        packaged["spec"]["compile_options"]["cuda_cflags"].extend(extra_cuda_cflags)
    for source in packaged["sources"]:
        source["content"] = (directory / source["path"]).read_text(encoding="utf-8")
    return canonical_json_bytes(packaged)


def read_traces(path) -> List[Dict[str, Any]]:
    """One JSON object per non-empty line (tools/extra_kernels.py:136-145)."""
    traces = []
    for number, line in enumerate(Path(path).read_text(encoding="utf-8").splitlines(), 1):
        if not line.strip():
            continue
        value = json.loads(line)
        _need(isinstance(value, dict), f"{path}: line {number} is not an object")
        traces.append(value)
    return traces


def summarize(trace_paths, workloads: int, problem_id: int, problem_name: str, contract_sha256: str) -> Dict[str, Any]:
    """Condense exactly three evaluator traces (one per trial, `workloads` lines each) into the summary the
    reference publishes: per-trial mean latency and per-workload mean / median; any workload that did not pass
    makes the whole summary fail (tools/extra_kernels.py:699-746)."""
    trace_paths = list(trace_paths)
    _need(len(trace_paths) == 3, "exactly three trace files are required")
    trials = [read_traces(p) for p in trace_paths]
    _need(all(len(t) == workloads for t in trials), f"each trace must contain {workloads} workloads")
    latencies: List[List[float]] = [[] for _ in range(workloads)]
    hardware = set()
    for trial_index, trial in enumerate(trials):
        for workload_index, trace in enumerate(trial):
            evaluation = trace.get("evaluation") or {}
            _need(evaluation.get("status") == "PASSED",
                  f"trial {trial_index + 1}, workload {workload_index} did not pass: {evaluation.get('status')}")
            hardware.add(str((evaluation.get("environment") or {}).get("hardware", "unknown")))
            latency = (evaluation.get("performance") or {}).get("latency_ms")
            _need(isinstance(latency, (float, int)) and not isinstance(latency, bool) and latency > 0,
                  "passed trace is missing a positive latency")
            latencies[workload_index].append(float(latency))
    trial_means = [statistics.fmean(latencies[w][t] for w in range(workloads)) for t in range(3)]
    return {
        "contract_sha256": contract_sha256,
        "hardware": sorted(hardware),
        "problem_id": int(problem_id),
        "problem_name": problem_name,
        "trial_mean_latency_ms": [round(v, 9) for v in trial_means],
        "workloads": [{"latency_ms_mean": round(statistics.fmean(v), 9),
                       "latency_ms_median": round(statistics.median(v), 9)} for v in latencies],
    }


def build_extension(directory, build_dir, name: Optional[str] = None, verbose: bool = False) -> Path:
    """Compile a `cuda_cpp` submission directory the way the evaluator does — one torch extension from the listed
    .cpp / .cu sources with the manifest's flags, here for sm_100a — and return the path of the shared object.
    nvcc cross-compiles without a GPU.  The module exports the manifest's entry symbol (`run`)."""
    import os

    directory, build_dir = Path(directory), Path(build_dir)
    manifest = validate(directory)
    spec = manifest["spec"]
    _need(any(l in CPP_LANGUAGES for l in spec["languages"]), "only C++/CUDA submissions are compiled")
    name = name or f"submission_{manifest['definition']}"
    build_dir.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils import cpp_extension

    sources = [str(directory / s["path"]) for s in manifest["sources"] if s["path"].endswith((".cpp", ".cu", ".cc"))]
    cpp_extension.load(name=name, sources=sources, build_directory=str(build_dir),
                       extra_cflags=list(spec["compile_options"]["cflags"]),
                       extra_cuda_cflags=list(spec["compile_options"]["cuda_cflags"]) +
                       ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo"],
                       extra_include_paths=[str(directory)], extra_ldflags=list(spec["compile_options"]["ld_flags"]),
                       is_python_module=False, verbose=verbose)
    return build_dir / f"{name}.so"


def load_extension(shared_object, name: Optional[str] = None):
    """Import a shared object made by `build_extension` (torch must be imported first: it provides the symbols)."""
    import importlib.util

    import torch  # noqa: F401

    shared_object = Path(shared_object)
    name = name or shared_object.stem
    spec = importlib.util.spec_from_file_location(name, str(shared_object))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="submission", description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="command", required=True)
    p = sub.add_parser("emit")
    p.add_argument("problem")
    p.add_argument("directory")
    p.add_argument("--author", default="sol-execbench-b200-kernels")
    p = sub.add_parser("lint")
    p.add_argument("directory")
    p = sub.add_parser("package")
    p.add_argument("directory")
    p.add_argument("output")
    p.add_argument("--target", default="B200")
    p.add_argument("--cuda-cflag", action="append", default=[])
    p = sub.add_parser("build")
    p.add_argument("directory")
    p.add_argument("build_dir")
    p = sub.add_parser("summarize")
    p.add_argument("problem")
    p.add_argument("traces", nargs=3)
    p.add_argument("--workloads", type=int, required=True)
    p.add_argument("--contract-sha256", default="")
    p.add_argument("-o", "--output", required=True)
    args = ap.parse_args(argv)
    try:
        if args.command == "emit":
            out = emit(args.problem, args.directory, args.author)
            print(f"problem {int(args.problem)}: submission written to {out}")
        elif args.command == "lint":
            manifest = validate(args.directory)
            print(f"{manifest['definition']}: source manifest and files are valid")
        elif args.command == "build":
            print(build_extension(args.directory, args.build_dir))
        elif args.command == "package":
            data = package(args.directory, args.target, args.cuda_cflag)
            Path(args.output).write_bytes(data)
            print(f"staged {args.target} artifact: {args.output}\nSHA-256: {sha256_bytes(data)}")
        else:
            problem = str(int(args.problem))
            name = PROBLEMS.get(problem, {}).get("definition", f"problem_{problem}")
            summary = summarize(args.traces, args.workloads, int(problem), name, args.contract_sha256)
            Path(args.output).write_bytes(canonical_json_bytes(summary))
            print(json.dumps(summary, indent=2, sort_keys=True))
    except SubmissionError as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
