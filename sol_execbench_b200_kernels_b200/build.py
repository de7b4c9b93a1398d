"""Builds libgateup.so and libsideops.so (sm_100a only) next to this file, one nvcc call each.

Run as ``python -m sol_execbench_b200_kernels_b200.build``; nvcc cross-compiles
without a GPU.  The library is kept in-tree so it travels with the sources.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libgateup.so"
SOURCES = [CSRC / "gateup.cu"]
HEADERS = [CSRC / "ptx_sm100.cuh", CSRC / "gateup_tile.cuh", CSRC / "gateup_pair.cuh", CSRC / "gateup_stream.cuh",
           CSRC / "quantize_act.cuh", CSRC / "reduce_gather.cuh", PKG_DIR.parent / "include" / "gateup.h"]
# the same library with the pair kernel's per-role cycle counters compiled in (gu_trace_read); a profiling aid
TRACE_LIB_PATH = PKG_DIR / "libgateup_trace.so"

SIDE_LIB_PATH = PKG_DIR / "libsideops.so"
SIDE_SOURCES = [CSRC / "sideops.cu"]
SIDE_HEADERS = [PKG_DIR.parent / "include" / "sideops.h", CSRC / "proj_gemm.cuh", CSRC / "ptx_sm100.cuh"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-cudart", "static",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libgateup.so cannot be built")
    return nvcc


def _stale(lib: Path, deps) -> bool:
    if not lib.exists():
        return True
    built = lib.stat().st_mtime
    return any(p.stat().st_mtime > built for p in deps)


def is_stale() -> bool:
    return _stale(LIB_PATH, SOURCES + HEADERS) or _stale(SIDE_LIB_PATH, SIDE_SOURCES + SIDE_HEADERS)


def _compile(lib: Path, sources, verbose: bool, defines=()) -> None:
    cmd = [find_nvcc(), *NVCC_FLAGS, *[f"-D{d}" for d in defines]]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(lib), *map(str, sources)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write(proc.stderr)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile each library that is missing or older than its sources; returns the path of libgateup.so."""
    if force or _stale(LIB_PATH, SOURCES + HEADERS):
        _compile(LIB_PATH, SOURCES, verbose)
    if force or _stale(SIDE_LIB_PATH, SIDE_SOURCES + SIDE_HEADERS):
        _compile(SIDE_LIB_PATH, SIDE_SOURCES, verbose)
    return LIB_PATH


def build_trace(force: bool = False, verbose: bool = False) -> Path:
    """Compile libgateup_trace.so (-DGU_TRACE): same entry points, cycle counters of the pair kernel's roles."""
    if force or _stale(TRACE_LIB_PATH, SOURCES + HEADERS):
        _compile(TRACE_LIB_PATH, SOURCES, verbose, defines=("GU_TRACE",))
    return TRACE_LIB_PATH


# the range-checked debug build (-DGU_BOUNDS=1): same entry points, every computed coordinate and index tested
BOUNDS_LIB_PATH = PKG_DIR / "libgateup_bounds.so"


SIDE_BOUNDS_LIB_PATH = PKG_DIR / "libsideops_bounds.so"


def build_bounds(force: bool = False, verbose: bool = False) -> Path:
    if force or _stale(BOUNDS_LIB_PATH, SOURCES + HEADERS):
        _compile(BOUNDS_LIB_PATH, SOURCES, verbose, defines=("GU_BOUNDS=1",))
    if force or _stale(SIDE_BOUNDS_LIB_PATH, SIDE_SOURCES + SIDE_HEADERS):
        _compile(SIDE_BOUNDS_LIB_PATH, SIDE_SOURCES, verbose, defines=("GU_BOUNDS=1",))
    return BOUNDS_LIB_PATH


def build_study(name: str, defines, verbose: bool = False) -> Path:
    """Compile libgateup_<name>.so with extra -D switches (the study builds listed in csrc/gateup_pair.cuh)."""
    lib = PKG_DIR / f"libgateup_{name}.so"
    _compile(lib, SOURCES, verbose, defines=tuple(defines))
    return lib


if __name__ == "__main__":
    # python -m sol_execbench_b200_kernels_b200.build [--force] [-v] [--trace] [--bounds] [--study NAME DEFINE[,DEFINE...]]
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--trace" in sys.argv:
        print(build_trace(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--bounds" in sys.argv:
        print(build_bounds(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--study" in sys.argv:
        at = sys.argv.index("--study")
        print(build_study(sys.argv[at + 1], sys.argv[at + 2].split(","), verbose="-v" in sys.argv))
