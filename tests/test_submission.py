"""Benchmark-format side (manifest, audit, artifact, trace summary), on CPU.  The fixtures under tests/golden/
were produced by the reference's own tooling (tests/golden/make_submission_golden.py)."""
import json
import os
import shutil

import pytest

from sol_execbench_b200_kernels_b200 import submission as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
TOY = os.path.join(GOLDEN, "toy_submission")


@pytest.fixture()
def toy(tmp_path):
    """A scratch copy of the toy submission with its manifest written in canonical form as `solution.json`."""
    d = tmp_path / "toy_submission"
    shutil.copytree(TOY, d)
    manifest = json.load(open(d / "manifest.compact.json", encoding="utf-8"))
    (d / "solution.json").write_bytes(S.canonical_json_bytes(manifest))
    return d


def test_toy_manifest_is_valid_and_packages_to_the_reference_artifact_bytes(toy):
    TOY = toy  # noqa: N806 - shadows the module constant on purpose
    manifest = S.validate(TOY, definition="000_toy_scale")
    assert manifest["spec"]["entry_point"] == "binding.cpp::run"
    data = S.package(TOY, "B200", ["-DFIXTURE=1"])
    want = open(os.path.join(GOLDEN, "toy_submission_artifact.sha256")).read().strip()
    assert S.sha256_bytes(data) == want          # byte-identical to the reference's build_artifact
    art = json.loads(data)
    assert art["spec"]["target_hardware"] == ["B200"]
    assert art["spec"]["compile_options"]["cuda_cflags"][-1] == "-DFIXTURE=1"
    assert all("content" in s for s in art["sources"]) and "µs → ok" in art["sources"][1]["content"]
    assert [s["path"] for s in art["sources"]] == ["binding.cpp", "kernel.cu", "scale.h", "config.h", "notes.txt"]
    assert S.canonical_json_bytes(art) == data


def test_trace_summary_equals_the_reference_summary():
    traces = [os.path.join(GOLDEN, f"traces_trial{t}.jsonl") for t in (1, 2, 3)]
    want = json.load(open(os.path.join(GOLDEN, "trace_summary_expected.json")))
    got = S.summarize(traces, want and len(want["workloads"]), want["problem_id"], want["problem_name"],
                      want["contract_sha256"])
    assert got == want
    assert S.canonical_json_bytes(got) == open(os.path.join(GOLDEN, "trace_summary_expected.json"), "rb").read()


def test_trace_summary_rejects_failed_missing_and_miscounted_traces(tmp_path):
    src = [os.path.join(GOLDEN, f"traces_trial{t}.jsonl") for t in (1, 2, 3)]
    with pytest.raises(S.SubmissionError, match="exactly three"):
        S.summarize(src[:2], 16, 29, "x", "")
    with pytest.raises(S.SubmissionError, match="must contain 15 records, this one has 16"):
        S.summarize(src, 15, 29, "x", "")
    lines = open(src[0]).read().splitlines()
    bad = json.loads(lines[3])
    bad["evaluation"]["status"] = "INCORRECT_NUMERICAL"
    p = tmp_path / "t1.jsonl"
    p.write_text("\n".join(lines[:3] + [json.dumps(bad)] + lines[4:]) + "\n\n")
    with pytest.raises(S.SubmissionError, match="trial 1, workload 3 did not pass: INCORRECT_NUMERICAL"):
        S.summarize([str(p), src[1], src[2]], 16, 29, "x", "")
    bad["evaluation"]["status"] = "PASSED"
    bad["evaluation"]["performance"]["latency_ms"] = 0
    p.write_text("\n".join(lines[:3] + [json.dumps(bad)] + lines[4:]) + "\n")
    with pytest.raises(S.SubmissionError, match="no positive latency"):
        S.summarize([str(p), src[1], src[2]], 16, 29, "x", "")


@pytest.mark.parametrize("problem", ["179", "38", "29"])
def test_emitted_submissions_pass_the_manifest_rules(tmp_path, problem):
    out = S.emit(problem, tmp_path / "sub")
    manifest = S.validate(out, definition=S.PROBLEMS[problem]["definition"])
    names = sorted(s["path"] for s in manifest["sources"])
    assert "binding.cpp" in names and sorted(os.listdir(out)) == sorted(names + ["solution.json"])
    assert manifest["spec"]["destination_passing_style"] is (problem != "29")
    # flat directory: no include reaches outside it
    for n in names:
        assert "../" not in (out / n).read_text()
    art = json.loads(S.package(out))
    assert [s["path"] for s in art["sources"]] == [s["path"] for s in manifest["sources"]]
    assert S.main(["lint", str(out)]) == 0


def _toy_copy(tmp_path):
    d = tmp_path / "toy"
    shutil.copytree(TOY, d)
    manifest = json.load(open(d / "manifest.compact.json", encoding="utf-8"))
    (d / "solution.json").write_bytes(S.canonical_json_bytes(manifest))
    return d


def _rewrite(d, mutate):
    m = json.load(open(d / "solution.json"))
    mutate(m)
    (d / "solution.json").write_bytes(S.canonical_json_bytes(m))


@pytest.mark.parametrize("mutate,message", [
    (lambda m: m.update(extra=1), "top-level keys this format does not know: extra"),
    (lambda m: m.update(name=""), "`name` and `author` must both be non-empty"),
    (lambda m: m["spec"].pop("binding"), "exactly its seven keys: absent binding"),
    (lambda m: m["spec"].update(languages=["cuda_cpp", "triton"]), "combines compiled and Python languages"),
    (lambda m: m["spec"].update(languages=["fortran"]), "`spec.languages` must be a non-empty list drawn from"),
    (lambda m: m["spec"].update(binding=None), "`spec.binding` has to be 'torch'"),
    (lambda m: m["spec"].update(dependencies=["numpy"]), "dependencies"),
    (lambda m: m["spec"].update(destination_passing_style="yes"), "must be true or false"),
    (lambda m: m["spec"].update(entry_point="binding.cpp"), "form file::symbol"),
    (lambda m: m["spec"]["compile_options"].pop("ld_flags"), "`spec.compile_options` must have exactly the keys"),
    (lambda m: m["spec"]["compile_options"].update(cflags="-O3"), "list of strings"),
    (lambda m: m["spec"].update(target_hardware=["LOCAL"]), "must be a list that names B200"),
    (lambda m: m.update(sources=[]), "`sources` must be a non-empty list"),
    (lambda m: m["sources"].append({"path": "../x.cu"}), "points outside the submission directory"),
    (lambda m: m["sources"].append({"path": "kernel.cu"}), "lists kernel.cu twice"),
    (lambda m: m["sources"].append({"path": "absent.cu"}), "absent.cu is listed in `sources` but is not a regular file"),
    (lambda m: m["sources"][0].update(content="x"), "may carry the key `path` and nothing else"),
    (lambda m: m["spec"].update(entry_point="other.cpp::run"), "names other.cpp, which `sources` does not list"),
])
def test_manifest_rules(tmp_path, mutate, message):
    d = _toy_copy(tmp_path)
    _rewrite(d, mutate)
    with pytest.raises(S.SubmissionError, match=message):
        S.validate(d)


def test_non_canonical_bytes_wrong_definition_and_forbidden_sources(tmp_path):
    d = _toy_copy(tmp_path)
    with pytest.raises(S.SubmissionError, match="this directory must hold '038_flux_multi_head_rmsnorm_qk'"):
        S.validate(d, definition="038_flux_multi_head_rmsnorm_qk")
    text = (d / "solution.json").read_text()
    (d / "solution.json").write_text(text.replace("  ", "    ", 1))
    with pytest.raises(S.SubmissionError, match="not in canonical form"):
        S.validate(d)
    (tmp_path / "second_parent").mkdir()
    d2 = _toy_copy(tmp_path / "second_parent")
    for fragment, category in (("cudaEventRecord(e, s);", "timing"), ("std::getenv(\"X\")", "process"),
                               ("usleep(5);", "delay"), ("cudaStreamCreate(&s);", "stream"),
                               ("std::thread t;", "thread"), ("#include <cupti.h>", "profiler")):
        (d2 / "kernel.cu").write_text(open(os.path.join(TOY, "kernel.cu")).read() + "\n// " + fragment + "\n")
        with pytest.raises(S.SubmissionError, match=category):
            S.validate(d2)


def test_package_sources_of_this_repository_are_audit_clean():
    for problem, cfg in S.PROBLEMS.items():
        for name, path in cfg["sources"]:
            S.audit_source(open(path).read(), f"{problem}:{name}")


def test_cli_package_and_summarize(tmp_path, capsys, toy):
    out = tmp_path / "artifact.json"
    assert S.main(["package", str(toy), str(out), "--cuda-cflag=-DFIXTURE=1"]) == 0
    assert S.sha256_bytes(out.read_bytes()) == open(os.path.join(GOLDEN, "toy_submission_artifact.sha256")).read().strip()
    summary = tmp_path / "summary.json"
    traces = [os.path.join(GOLDEN, f"traces_trial{t}.jsonl") for t in (1, 2, 3)]
    contract = json.load(open(os.path.join(GOLDEN, "trace_summary_expected.json")))["contract_sha256"]
    assert S.main(["summarize", "29", *traces, "--workloads", "16", "--contract-sha256", contract, "-o", str(summary)]) == 0
    assert summary.read_bytes() == open(os.path.join(GOLDEN, "trace_summary_expected.json"), "rb").read()
    assert S.main(["lint", str(tmp_path)]) == 1      # no manifest there
    capsys.readouterr()


@pytest.mark.parametrize("problem,module", [("179", "submission_003_fp8_mlp_gate_up_projection"),
                                            ("38", "submission_038_flux_multi_head_rmsnorm_qk"),
                                            ("29", "submission_029_mamba_conv1d_with_gating")])
def test_built_extensions_load_and_reject_host_tensors(problem, module):
    """The torch extensions that `submission.build_extension` makes of the emitted directories (built beside the
    tests by the repository's build entry point) import without a GPU and refuse CPU tensors before any CUDA call."""
    import torch

    so = os.path.join(ROOT, "tests", "_built_submissions", f"build_{problem}", module + ".so")
    if not os.path.exists(so):
        pytest.skip("the submission extensions are not built")
    ext = S.load_extension(so)
    bf = torch.bfloat16
    if problem == "179":
        x = torch.zeros(128, 128).to(torch.float8_e4m3fn)
        args = (x, torch.zeros(128, 1), x, torch.zeros(1, 1), x, torch.zeros(1, 1), torch.zeros(128, 128, dtype=bf))
    elif problem == "38":
        q = torch.zeros(1, 2, 48, 128)
        args = (q, q, torch.zeros(48, 128), torch.zeros(48, 128), 1e-6, q.clone(), q.clone())
    else:
        args = (torch.zeros(1, 4, 128, dtype=bf), torch.zeros(1, 4, dtype=bf), torch.zeros(128, 128, dtype=bf),
                torch.zeros(128, dtype=bf), torch.zeros(64, 1, 4, dtype=bf), torch.zeros(64, dtype=bf))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ext.run(*args)
