"""The benchmark script's output contract, as far as it can be checked without a GPU: the reference arm prints one
JSON line with the agreed keys, the roofline helper picks the bound and reports algorithmic work, the peaks fall back
when the measured file is absent, and the device arm refuses to run without a GPU instead of falling back."""
import importlib.util
import json
import os
import subprocess
import sys

import pytest
import torch

from sol_execbench_b200_kernels_b200 import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("_bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_the_contract_line():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in d, key
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["value"] > 0 and d["vs_baseline"] is None
    assert d["config"]["workload"].startswith("prefill_8b") and "model" not in d["config"]
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0


def test_reference_arm_is_silent_on_other_ranks():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                           "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=120, cwd=ROOT,
                          env=env)
    assert proc.returncode == 0 and proc.stdout.strip() == ""


def test_roofline_helper_picks_the_bound(bench):
    peaks = {"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "_source": "measured"}
    m, k, n = W.SHAPES["prefill_8b"]
    r = bench.roofline_for(m, k, n, 0.5, peaks, W)
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and r["peak"] == 3200.0
    assert r["algorithmic_flops"] == 4 * m * k * n
    assert abs(r["achieved"] - 4 * m * k * n / 0.5e-3 / 1e12) < 0.01 and abs(r["frac"] - r["achieved"] / 3200.0) < 1e-3
    assert "of measured" in r["peak_source"]
    m, k, n = W.SHAPES["decode_70b"]
    r = bench.roofline_for(m, k, n, 0.08, dict(peaks, _source="fallback"), W)
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and r["peak"] == 6500.0
    assert r["algorithmic_bytes"] == W.algorithmic_bytes(m, k, n) and "of fallback" in r["peak_source"]


def test_peaks_fall_back_when_the_measured_file_is_absent(bench, tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    p = bench.load_peaks()
    assert p["_source"] == "fallback" and p["hbm_gbs"] > 0 and p["bf16_tflops"] > 0
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps({"hbm_gbs": 1.0, "bf16_tflops": 2.0}))
    p = bench.load_peaks()
    assert p["_source"] == "measured" and p["hbm_gbs"] == 1.0


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the refusal on a machine without a GPU")
def test_device_arm_refuses_to_run_without_a_gpu():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1"], capture_output=True,
                          text=True, timeout=300, cwd=ROOT)
    assert proc.returncode != 0 and "no CUDA device" in (proc.stderr + proc.stdout)
