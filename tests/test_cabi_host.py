"""Host-side checks that need no GPU: the library loads, exports what include/gateup.h
declares, validates arguments before touching CUDA, and the Python entry point refuses CPU tensors."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "gateup.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gu_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_all_exported(gateup_lib):
    declared = _declared_symbols()
    assert "gu_run" in declared and len(declared) >= 9
    for name in declared:
        assert hasattr(gateup_lib.lib, name), f"{name} declared in gateup.h but not exported"
    assert sorted(gateup_lib.EXPORTS) == declared


def test_version_and_error_strings(gateup_lib):
    assert gateup_lib.lib.gu_version() == 1
    for code in range(0, -9, -1):
        msg = gateup_lib.error_string(code)
        assert msg and msg != "unknown error"
    assert gateup_lib.error_string(-99) == "unknown error"


def test_struct_layout_matches_header(gateup_lib):
    # 7 pointers, 4 int64, pointer, size_t, 2 int32 -> 8-byte fields throughout
    assert ctypes.sizeof(gateup_lib.GuProblem) == 7 * 8 + 4 * 8 + 8 + 8 + 8


@pytest.mark.parametrize("shape,plan", [
    ((16, 8192, 28672), "stream"), ((1, 4096, 14336), "stream"), ((32, 8192, 28672), "stream"),
    ((32, 4096, 14336), "tile"), ((64, 8192, 28672), "tile"), ((16, 2048, 5632), "tile"),
    ((65, 4096, 14336), "tile"), ((128, 2048, 5632), "tile"), ((4096, 4096, 14336), "tile"),
    ((16384, 7168, 18432), "tile"),
])
def test_plan_heuristic(gateup_lib, shape, plan):
    code = gateup_lib.lib.gu_select_plan(*shape)
    assert gateup_lib.PLAN_NAMES[code] == plan


@pytest.mark.parametrize("shape", [(0, 128, 128), (4, 100, 128), (4, 128, 200), (4, 0, 128), (-1, 128, 128)])
def test_plan_rejects_bad_shapes(gateup_lib, shape):
    assert gateup_lib.lib.gu_select_plan(*shape) == gateup_lib.GU_EINVAL_SHAPE
    assert gateup_lib.lib.gu_workspace_bytes(*shape, 0) == 0


def test_workspace_sizes(gateup_lib):
    lib = gateup_lib.lib
    assert lib.gu_workspace_bytes(4096, 4096, 14336, gateup_lib.PLAN_AUTO) == 0      # 3584 tiles: data-parallel
    assert lib.gu_workspace_bytes(4096, 4096, 14336, gateup_lib.PLAN_TILE) == 0
    assert lib.gu_workspace_bytes(4096, 4096, 14336, gateup_lib.PLAN_TILE_DP) == 0
    sk = 4096 + 256 * 128 * 256 * 4
    assert lib.gu_workspace_bytes(4096, 4096, 14336, gateup_lib.PLAN_TILE_SK) == sk
    # 224 pair tiles on 74 clusters are 3.03 rounds: the pair kernel's stream-K schedule is chosen and needs scratch
    assert lib.gu_workspace_bytes(512, 4096, 14336, gateup_lib.PLAN_AUTO) == sk
    assert lib.gu_workspace_bytes(512, 4096, 14336, gateup_lib.PLAN_TILE_PAIR_SK) == sk
    assert lib.gu_workspace_bytes(512, 4096, 14336, gateup_lib.PLAN_TILE_PAIR) == 0
    assert lib.gu_workspace_bytes(256, 4096, 14336, gateup_lib.PLAN_AUTO) == 0        # 1.51 rounds: whole tiles
    assert lib.gu_workspace_bytes(512, 4096, 9472, gateup_lib.PLAN_AUTO) == 0         # two rounds exactly
    assert lib.gu_workspace_bytes(128, 4096, 14336, gateup_lib.PLAN_TILE_SK) == sk
    # three 128-token blocks: the lone-CTA kernel with whole tiles (3 rounds) beats two 256-token pair blocks
    assert lib.gu_workspace_bytes(384, 4096, 14336, gateup_lib.PLAN_AUTO) == 0
    assert lib.gu_workspace_bytes(384, 2048, 5632, gateup_lib.PLAN_AUTO) == 0
    assert lib.gu_workspace_bytes(1024, 4096, 14336, gateup_lib.PLAN_AUTO) == sk       # 6.05 rounds of pairs
    w16 = lib.gu_workspace_bytes(16, 8192, 28672, gateup_lib.PLAN_AUTO)
    w64 = lib.gu_workspace_bytes(64, 8192, 28672, gateup_lib.PLAN_STREAM)
    assert w16 == 4096 + 256 * 2 * 16 * 128 * 4
    assert w64 == 4096 + 256 * 2 * 64 * 128 * 4


# (op, (M, K, N), kernel) rows of the B200 measurements the choice was fitted on: the fastest of the three kernels there
_MEASURED_CHOICES = [
    ("gateup", (256, 4096, 14336), "tile_pair"),        # 44.4 us against 47.2 lone
    ("gateup", (384, 4096, 14336), "tile_dp"),          # three 128-token blocks: 65.4 lone against 71.6 / 73.7
    ("gateup", (512, 4096, 14336), "tile_pair_sk"),     # 3.03 rounds: 71.7 cut, 73.8 whole, 83.9 lone
    ("gateup", (640, 4096, 14336), "tile_dp"),          # 86.0 lone against 90.1
    ("gateup", (768, 4096, 14336), "tile_pair"),        # 90.2 against 104.4 lone
    ("gateup", (1024, 4096, 14336), "tile_pair_sk"),
    ("gateup", (4096, 4096, 14336), "tile_pair"),       # the headline shape: whole tiles on pairs
    ("gateup", (16384, 7168, 18432), "tile_pair"),
    ("gateup", (16384, 7168, 2304), "tile_pair"),       # the 8-GPU shard of it
    ("gateup", (384, 8192, 28672), "tile_dp"),          # 197.6 lone against 221 - 233
    ("gateup", (512, 8192, 28672), "tile_pair_sk"),
    ("gateup", (384, 2048, 5632), "tile_dp"),           # 18.4 lone against 30.7
    ("gateup", (1024, 2048, 5632), "tile_dp"),          # 38.9 lone against 43.0
    ("gateup", (1536, 2048, 5632), "tile_dp"),          # 49.1 lone against 53.2 whole, 55.8 cut
    ("gateup", (1024, 7168, 2304), "tile_pair"),
    ("gateup", (128, 4096, 14336), "tile_dp"),
    ("gateup", (4096, 1024, 4096), "tile_dp"),          # 8 K blocks per tile: 51.1 lone against 73.7
    ("gateup", (256, 2560, 6912), "tile_dp"),           # 20.9 lone against 22.5
    ("gateup", (2048, 2560, 6912), "tile_pair"),        # 75.8 against 81.9 lone
    ("gateup", (4096, 3072, 8192), "tile_pair"),        # 180.2 against 206.8 lone
    ("gateup_fp8", (4096, 4096, 14336), "tile_pair"),
    ("gateup_fp8", (384, 4096, 14336), "tile_dp"),      # 68.1 lone against 79.9
    ("gateup_fp8", (512, 4096, 14336), "tile_pair"),    # 80.8 against 86.0 lone
    ("gateup_fp8", (4096, 2048, 5632), "tile_dp"),      # short K: the pair epilogue outlasts the K loop, 118.8 against 144.3
    ("gateup_fp8", (256, 2048, 5632), "tile_dp"),
    ("gemm", (4096, 14336, 4096), "tile_pair"),         # the down projection
    ("gemm", (1024, 14336, 4096), "tile_pair"),         # 60.4 against 69.7 lone
    ("gemm", (1152, 14336, 4096), "tile_dp"),           # nine blocks fit one round of lone CTAs: 71.8 against 105.5
    ("gemm", (1152, 4096, 4096), "tile_dp"),            # 28.5 against 38.9
    ("gemm", (768, 4096, 4096), "tile_pair"),           # 24.6 against 27.0 lone
    ("gemm", (1152, 5632, 2048), "tile_pair"),          # 29.6 against 32.8 lone
]


@pytest.mark.parametrize("op,shape,kernel", _MEASURED_CHOICES)
def test_tile_kernel_choice_matches_the_measurements(gateup_lib, op, shape, kernel):
    ops = {"gateup": gateup_lib.OP_GATEUP, "gateup_fp8": gateup_lib.OP_GATEUP_FP8, "gemm": gateup_lib.OP_GEMM}
    code = gateup_lib.lib.gu_select_tile_kernel(ops[op], *shape, 1)
    assert gateup_lib.PLAN_NAMES[code] == kernel
    # without scratch nothing is cut along K
    bare = gateup_lib.PLAN_NAMES[gateup_lib.lib.gu_select_tile_kernel(ops[op], *shape, 0)]
    assert bare in ("tile_dp", "tile_pair")


def test_tile_kernel_choice_rejects_bad_arguments(gateup_lib):
    lib = gateup_lib.lib
    assert lib.gu_select_tile_kernel(gateup_lib.OP_GATEUP, 4, 100, 128, 1) == gateup_lib.GU_EINVAL_SHAPE
    assert lib.gu_select_tile_kernel(3, 256, 128, 128, 1) == gateup_lib.GU_EINVAL_PLAN
    # scratch is asked for exactly where a stream-K schedule would run
    for shape in [(512, 4096, 14336), (384, 4096, 14336), (4096, 4096, 14336), (1024, 8192, 28672)]:
        cut = gateup_lib.PLAN_NAMES[lib.gu_select_tile_kernel(gateup_lib.OP_GATEUP, *shape, 1)].endswith("_sk")
        assert (lib.gu_workspace_bytes(*shape, gateup_lib.PLAN_TILE) > 0) == cut, shape


def _problem(gateup_lib, **over):
    base = dict(x=0x1000, scale_x=0x2000, gate_w=0x3000, scale_gate=0x4000, up_w=0x5000, scale_up=0x6000,
                output=0x7000, m=128, k=128, n=128, ld_output=128, workspace=None, workspace_bytes=0,
                plan=gateup_lib.PLAN_TILE, reserved=0)
    base.update(over)
    return gateup_lib.GuProblem(**base)


def test_argument_validation_precedes_any_cuda_call(gateup_lib):
    lib = gateup_lib.lib
    assert lib.gu_run(None, None) == gateup_lib.GU_EINVAL_NULL
    for field in ("x", "scale_x", "gate_w", "scale_gate", "up_w", "scale_up", "output"):
        pr = _problem(gateup_lib, **{field: None})
        assert lib.gu_run(ctypes.byref(pr), None) == gateup_lib.GU_EINVAL_NULL, field
    assert lib.gu_run(ctypes.byref(_problem(gateup_lib, k=130)), None) == gateup_lib.GU_EINVAL_SHAPE
    assert lib.gu_run(ctypes.byref(_problem(gateup_lib, n=64)), None) == gateup_lib.GU_EINVAL_SHAPE
    assert lib.gu_run(ctypes.byref(_problem(gateup_lib, m=0)), None) == gateup_lib.GU_EINVAL_SHAPE
    assert lib.gu_run(ctypes.byref(_problem(gateup_lib, ld_output=64)), None) == gateup_lib.GU_EINVAL_SHAPE
    assert lib.gu_run(ctypes.byref(_problem(gateup_lib, x=0x1001)), None) == gateup_lib.GU_EINVAL_ALIGN
    assert lib.gu_run(ctypes.byref(_problem(gateup_lib, ld_output=132)), None) == gateup_lib.GU_EINVAL_ALIGN
    assert lib.gu_run(ctypes.byref(_problem(gateup_lib, plan=7)), None) == gateup_lib.GU_EINVAL_PLAN
    assert lib.gu_run_concat(0x1000, 0x2000, None, 0x4000, 0x7000, 128, 128, 128, 128, None, 0, 0, None) \
        == gateup_lib.GU_EINVAL_NULL


def test_gather_entry_point_validates_before_any_cuda_call(gateup_lib):
    lib = gateup_lib.lib
    pr = _problem(gateup_lib)
    ptrs = (ctypes.c_void_p * 2)(0x7000, 0x9000)
    assert lib.gu_run_gather(None, ptrs, 2, 0, 256, None) == gateup_lib.GU_EINVAL_NULL
    assert lib.gu_run_gather(ctypes.byref(pr), None, 2, 0, 256, None) == gateup_lib.GU_EINVAL_NULL
    assert lib.gu_run_gather(ctypes.byref(pr), ptrs, 9, 0, 9 * 128, None) == gateup_lib.GU_EINVAL_SHAPE   # more than 8 ranks
    assert lib.gu_run_gather(ctypes.byref(pr), ptrs, 2, 2, 256, None) == gateup_lib.GU_EINVAL_SHAPE       # rank out of range
    assert lib.gu_run_gather(ctypes.byref(pr), ptrs, 2, 0, 128, None) == gateup_lib.GU_EINVAL_SHAPE       # pitch < N * world
    assert lib.gu_run_gather(ctypes.byref(pr), ptrs, 2, 0, 260, None) == gateup_lib.GU_EINVAL_ALIGN
    bad = (ctypes.c_void_p * 2)(0x7000, None)
    assert lib.gu_run_gather(ctypes.byref(pr), bad, 2, 0, 256, None) == gateup_lib.GU_EINVAL_NULL
    odd = (ctypes.c_void_p * 2)(0x7000, 0x9004)
    assert lib.gu_run_gather(ctypes.byref(pr), odd, 2, 0, 256, None) == gateup_lib.GU_EINVAL_ALIGN


@pytest.mark.skipif(torch.cuda.is_available(), reason="CPU-only check")
def test_valid_problem_without_a_gpu_fails_loudly(gateup_lib):
    # nothing to fall back to: a well-formed call on a machine without a device is an error, not a CPU result
    code = gateup_lib.lib.gu_run(ctypes.byref(_problem(gateup_lib)), None)
    assert code in (gateup_lib.GU_ECUDA, gateup_lib.GU_EDEVICE)


def test_python_entry_point_refuses_cpu_tensors(gateup_lib):
    import sol_execbench_b200_kernels_b200 as pkg
    from sol_execbench_b200_kernels_b200 import workloads as W

    inp = W.make_inputs(4, 128, 128, seed=0)
    out = torch.empty(4, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        pkg.run(*inp.args(), out)


def test_python_entry_point_shape_and_dtype_errors(gateup_lib):
    import sol_execbench_b200_kernels_b200 as pkg
    from sol_execbench_b200_kernels_b200 import workloads as W

    inp = W.make_inputs(4, 128, 128, seed=0)
    out = torch.empty(4, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="output"):
        pkg.run(*inp.args(), out.float())
    with pytest.raises(ValueError, match="scale_x"):
        pkg.run(inp.x, inp.scale_x[:, :0], *inp.args()[2:], out)
    with pytest.raises(ValueError, match="Unsupported contract shape"):
        pkg.run(inp.x[:, :100], *inp.args()[1:], out)
    with pytest.raises(ValueError):
        pkg.run_concat(inp.x, inp.scale_x, torch.empty(100, 128, dtype=torch.float8_e4m3fn), inp.scale_gate, out)
    with pytest.raises(ValueError, match="unknown plan"):
        pkg.run_with_plan(*inp.args(), out, "fastest")
