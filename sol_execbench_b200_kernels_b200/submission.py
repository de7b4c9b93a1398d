"""Benchmark-format side of the kernels: emit, check, package and summarise SOL-ExecBench submissions.

The reference repository ships each kernel as a directory with a `solution.json` manifest and its sources, checks
it (`tools/extra_kernels.py:291-393`, `load_source_manifest`), embeds the sources into one JSON artifact for the
evaluator (`:396-486`, `build_artifact`) and condenses three evaluator traces into a summary (`:699-746`,
`command_summarize`).  This module serves the same file formats for this package's kernels: `emit` writes a flat
submission directory (a torch binding + the CUDA sources + manifest, language `cuda_cpp`, binding `torch`), `validate`
evaluates a table of manifest rules plus the forbidden-API audit and reports every broken rule at once, `package`
produces the artifact bytes, `summarize` the trace summary.
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
                    ("gateup_tile.cuh", CSRC / "gateup_tile.cuh"), ("gateup_pair.cuh", CSRC / "gateup_pair.cuh"),
                    ("gateup_stream.cuh", CSRC / "gateup_stream.cuh"),
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
                    ("proj_gemm.cuh", CSRC / "proj_gemm.cuh"), ("ptx_sm100.cuh", CSRC / "ptx_sm100.cuh"),
                    ("sideops.h", INCLUDE / "sideops.h")],
    },
    "29": {
        "definition": "029_mamba_conv1d_with_gating",
        "name": "mamba_in_proj_tcgen05_conv1d_tail_packed_f32x2",
        "description": "Mamba input projection as a persistent tcgen05 bf16 GEMM on CTA pairs with the bias in its "
                       "epilogue, then one kernel for mask, depthwise causal conv1d, SiLU, mask and the "
                       "[L, C] -> [C, L] transposition with packed f32x2 arithmetic.",
        "destination_passing_style": False,
        "sources": [("binding.cpp", BINDINGS / "binding_029.cpp"), ("sideops.cu", CSRC / "sideops.cu"),
                    ("proj_gemm.cuh", CSRC / "proj_gemm.cuh"), ("ptx_sm100.cuh", CSRC / "ptx_sm100.cuh"),
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


def audit_source(text: str, where: str = "source") -> None:
    """Raise if `text` names an API a submission may not use (FORBIDDEN_FRAGMENTS); `where` labels the complaint."""
    lowered = text.lower()
    hits = [(category, fragment) for category, fragments in FORBIDDEN_FRAGMENTS.items()
            for fragment in fragments if fragment in lowered]
    if hits:
        raise SubmissionError("; ".join(f"{where} uses {fragment!r} ({category})" for category, fragment in hits))


# ---------------------------------------------------------------------------------------------------------------
# Manifest rules.  The format is the reference's (tools/extra_kernels.py:291-393 checks the same manifest); here the
# rules are data: each entry looks at a parsed view of the manifest and returns a complaint or nothing, every rule is
# evaluated, and one exception carries all complaints, so a broken manifest is fixed in one pass instead of rule by rule.
# ---------------------------------------------------------------------------------------------------------------
class _ManifestView:
    """What the rules look at: the manifest, its `spec` (an empty dict when it is not an object), the directory and
    the language family the manifest declares."""

    def __init__(self, manifest: Dict[str, Any], directory: Path, expected_definition: Optional[str]):
        self.manifest = manifest
        self.directory = directory
        self.expected_definition = expected_definition
        spec = manifest.get("spec")
        self.spec: Dict[str, Any] = spec if isinstance(spec, dict) else {}
        langs = self.spec.get("languages")
        self.languages: List[str] = langs if isinstance(langs, list) and all(isinstance(l, str) for l in langs) else []
        compiled = [l for l in self.languages if l in CPP_LANGUAGES]
        scripted = [l for l in self.languages if l in PYTHON_LANGUAGES]
        self.family = "mixed" if compiled and scripted else ("compiled" if compiled else ("python" if scripted else None))
        srcs = manifest.get("sources")
        self.sources: List[Any] = srcs if isinstance(srcs, list) else []

    def source_paths(self) -> List[str]:
        return [s["path"] for s in self.sources if isinstance(s, dict) and isinstance(s.get("path"), str)]


def _listing(values) -> str:
    return ", ".join(sorted(map(str, values))) or "none"


def _rule_known_keys(v):
    extra = set(v.manifest) - TOP_LEVEL_FIELDS
    return f"solution.json has top-level keys this format does not know: {_listing(extra)}" if extra else None


def _rule_identity(v):
    ok = all(isinstance(v.manifest.get(k), str) and v.manifest.get(k) for k in ("name", "author"))
    return None if ok else "`name` and `author` must both be non-empty strings"


def _rule_definition(v):
    want, got = v.expected_definition, v.manifest.get("definition")
    return None if want is None or got == want else f"the manifest is for definition {got!r}, this directory must hold {want!r}"


def _rule_spec_keys(v):
    if not isinstance(v.manifest.get("spec"), dict):
        return "`spec` must be an object"
    have = set(v.spec)
    if have == SPEC_FIELDS:
        return None
    return f"`spec` must have exactly its seven keys: absent {_listing(SPEC_FIELDS - have)}; not allowed {_listing(have - SPEC_FIELDS)}"


def _rule_languages(v):
    langs = v.spec.get("languages")
    ok = isinstance(langs, list) and langs and all(l in ALLOWED_LANGUAGES for l in langs)
    return None if ok or "languages" not in v.spec else f"`spec.languages` must be a non-empty list drawn from {_listing(ALLOWED_LANGUAGES)}"


def _rule_one_family(v):
    return "`spec.languages` combines compiled and Python languages; a submission is one or the other" if v.family == "mixed" else None


def _rule_binding(v):
    if v.family not in ("compiled", "python") or "binding" not in v.spec:
        return None
    want = "torch" if v.family == "compiled" else None
    return None if v.spec["binding"] == want else f"`spec.binding` has to be {want!r} when the languages are {v.family}"


def _rule_dependencies(v):
    deps = v.spec.get("dependencies")
    ok = isinstance(deps, list) and all(d in ALLOWED_DEPENDENCIES for d in deps)
    return None if ok or "dependencies" not in v.spec else f"`spec.dependencies` must be a list drawn from {_listing(ALLOWED_DEPENDENCIES)}"


def _rule_destination_passing(v):
    ok = isinstance(v.spec.get("destination_passing_style"), bool)
    return None if ok or "destination_passing_style" not in v.spec else "`spec.destination_passing_style` must be true or false"


def _entry_parts(v):
    entry = v.spec.get("entry_point")
    if isinstance(entry, str):
        parts = entry.split("::")
        if len(parts) == 2 and all(parts):
            return parts
    return None


def _rule_entry_shape(v):
    return None if _entry_parts(v) or "entry_point" not in v.spec else "`spec.entry_point` must have the form file::symbol"


def _rule_compile_options(v):
    if v.family not in ("compiled", "python") or "compile_options" not in v.spec:
        return None
    options = v.spec["compile_options"]
    want = {"cflags", "cuda_cflags", "ld_flags"} if v.family == "compiled" else set()
    if not isinstance(options, dict) or set(options) != want:
        return f"`spec.compile_options` must have exactly the keys {{{_listing(want)}}} for {v.family} languages"
    bad = [k for k, flags in options.items() if not (isinstance(flags, list) and all(isinstance(f, str) for f in flags))]
    return f"`spec.compile_options.{bad[0]}` must be a list of strings" if bad else None


def _rule_target(v):
    hw = v.spec.get("target_hardware")
    ok = isinstance(hw, list) and "B200" in hw
    return None if ok or "target_hardware" not in v.spec else "`spec.target_hardware` must be a list that names B200"


def _rule_sources(v):
    if not v.sources:
        return "`sources` must be a non-empty list"
    complaints, seen = [], set()
    for index, entry in enumerate(v.sources):
        if not (isinstance(entry, dict) and set(entry) == {"path"} and isinstance(entry["path"], str)):
            complaints.append(f"`sources[{index}]` may carry the key `path` and nothing else")
            continue
        rel = Path(entry["path"])
        posix = rel.as_posix()
        if rel.is_absolute() or ".." in rel.parts:
            complaints.append(f"`sources[{index}].path` points outside the submission directory: {posix}")
            continue
        if posix in seen:
            complaints.append(f"`sources` lists {posix} twice")
            continue
        seen.add(posix)
        local = v.directory / rel
        if local.is_symlink() or not local.is_file():
            complaints.append(f"{posix} is listed in `sources` but is not a regular file of the directory")
            continue
        try:
            audit_source(local.read_text(encoding="utf-8"), posix)
        except SubmissionError as exc:
            complaints.append(str(exc))
    return "; ".join(complaints) or None


def _rule_entry_listed(v):
    parts = _entry_parts(v)
    if not parts or not v.sources:
        return None
    return None if parts[0] in v.source_paths() else f"`spec.entry_point` names {parts[0]}, which `sources` does not list"


MANIFEST_RULES = (
    _rule_known_keys, _rule_identity, _rule_definition, _rule_spec_keys, _rule_languages, _rule_one_family,
    _rule_binding, _rule_dependencies, _rule_destination_passing, _rule_entry_shape, _rule_compile_options,
    _rule_target, _rule_sources, _rule_entry_listed,
)


def validate(directory, definition: Optional[str] = None) -> Dict[str, Any]:
    """Check `directory/solution.json` and the sources it lists against MANIFEST_RULES.  Returns the manifest;
    raises SubmissionError naming every rule that is broken."""
    directory = Path(directory)
    path = directory / "solution.json"
    if not path.is_file():
        raise SubmissionError(f"{path}: no manifest")
    raw = path.read_bytes()
    try:
        manifest = json.loads(raw.decode("utf-8"))
    except ValueError as exc:
        raise SubmissionError(f"{path} does not parse as JSON: {exc}") from exc
    if not isinstance(manifest, dict):
        raise SubmissionError(f"{path} must hold one JSON object")
    complaints = []
    if raw != canonical_json_bytes(manifest):
        complaints.append("solution.json is not in canonical form (two-space indent, sorted keys, one final newline)")
    view = _ManifestView(manifest, directory, definition)
    complaints += [c for c in (rule(view) for rule in MANIFEST_RULES) if c]
    if complaints:
        raise SubmissionError(f"{path}: " + "; ".join(complaints))
    return manifest


def package(directory, target: str = "B200", extra_cuda_cflags: Optional[Iterable[str]] = None) -> bytes:
    """The single-file artifact the evaluator takes (the format `build_artifact` of the reference produces,
    tools/extra_kernels.py:396-486): the checked manifest, with `target_hardware` narrowed to `target`, any extra
    CUDA flags appended, and the text of every listed source stored beside its path as `content`."""
    directory = Path(directory)
    manifest = validate(directory)
    spec = dict(manifest["spec"])
    spec["target_hardware"] = [target]
    extra = list(extra_cuda_cflags or ())
    if extra:
        options = spec["compile_options"]
        if "cuda_cflags" not in options:
            raise SubmissionError("extra CUDA flags only apply to a compiled (C++/CUDA) submission")
        spec["compile_options"] = {**options, "cuda_cflags": [*options["cuda_cflags"], *extra]}
    embedded = [{"path": entry["path"], "content": (directory / entry["path"]).read_text(encoding="utf-8")}
                for entry in manifest["sources"]]
    return canonical_json_bytes({**manifest, "spec": spec, "sources": embedded})


def read_traces(path) -> List[Dict[str, Any]]:
    """The evaluator's trace file: one JSON object per line, blank lines ignored."""
    records = []
    for number, line in enumerate(Path(path).read_text(encoding="utf-8").splitlines(), 1):
        if line.strip():
            record = json.loads(line)
            if not isinstance(record, dict):
                raise SubmissionError(f"{path}, line {number}: expected a JSON object")
            records.append(record)
    return records


def _passed_latency(record: Dict[str, Any], trial: int, workload: int):
    """(latency in ms, hardware label) of one trace record that must have passed."""
    evaluation = record.get("evaluation") or {}
    status = evaluation.get("status")
    if status != "PASSED":
        raise SubmissionError(f"trial {trial}, workload {workload} did not pass: {status}")
    latency = (evaluation.get("performance") or {}).get("latency_ms")
    if isinstance(latency, bool) or not isinstance(latency, (int, float)) or latency <= 0:
        raise SubmissionError(f"trial {trial}, workload {workload} passed but carries no positive latency")
    return float(latency), str((evaluation.get("environment") or {}).get("hardware", "unknown"))


def summarize(trace_paths, workloads: int, problem_id: int, problem_name: str, contract_sha256: str) -> Dict[str, Any]:
    """Three evaluator trace files (one per trial, `workloads` records each) condensed into the summary record the
    reference's `command_summarize` writes (tools/extra_kernels.py:699-746; the keys and the 9-digit rounding are that
    format): mean latency per trial, mean and median per workload over the trials.  A record that did not pass, or
    has no positive latency, fails the whole summary."""
    trace_paths = list(trace_paths)
    if len(trace_paths) != 3:
        raise SubmissionError(f"a summary takes exactly three trace files, got {len(trace_paths)}")
    table, hardware = [], set()      # table[trial][workload] = latency
    for trial, path in enumerate(trace_paths, 1):
        records = read_traces(path)
        if len(records) != workloads:
            raise SubmissionError(f"{path}: a trace must contain {workloads} records, this one has {len(records)}")
        row = []
        for workload, record in enumerate(records):
            latency, label = _passed_latency(record, trial, workload)
            row.append(latency)
            hardware.add(label)
        table.append(row)
    per_workload = list(zip(*table))  # columns: one workload over the three trials
    digits = 9
    return {
        "contract_sha256": contract_sha256,
        "hardware": sorted(hardware),
        "problem_id": int(problem_id),
        "problem_name": problem_name,
        "trial_mean_latency_ms": [round(statistics.fmean(row), digits) for row in table],
        "workloads": [{"latency_ms_mean": round(statistics.fmean(col), digits),
                       "latency_ms_median": round(statistics.median(col), digits)} for col in per_workload],
    }


def build_extension(directory, build_dir, name: Optional[str] = None, verbose: bool = False) -> Path:
    """Compile a `cuda_cpp` submission directory the way the evaluator does — one torch extension from the listed
    .cpp / .cu sources with the manifest's flags, here for sm_100a — and return the path of the shared object.
    nvcc cross-compiles without a GPU.  The module exports the manifest's entry symbol (`run`)."""
    import os

    directory, build_dir = Path(directory), Path(build_dir)
    manifest = validate(directory)
    spec = manifest["spec"]
    if not any(l in CPP_LANGUAGES for l in spec["languages"]):
        raise SubmissionError("only compiled (C++/CUDA) submissions can be built")
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
