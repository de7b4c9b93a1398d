"""Compiles oracle/gateup_oracle.c with gcc into oracle/_build/libgateup_oracle.so (git-ignored) and loads it.
Test infrastructure only.

    python oracle/build_c.py            # build if stale, print the path
"""
from __future__ import annotations

import ctypes
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCE = HERE / "gateup_oracle.c"
LIB = HERE / "_build" / "libgateup_oracle.so"


def build(force: bool = False) -> Path:
    if not force and LIB.exists() and LIB.stat().st_mtime >= SOURCE.stat().st_mtime:
        return LIB
    gcc = shutil.which("gcc") or shutil.which("cc")
    if gcc is None:
        raise RuntimeError("no C compiler found for the oracle's C restatement")
    LIB.parent.mkdir(parents=True, exist_ok=True)
    # -ffp-contract=off: the only fused multiply-add is the explicit fmaf of the promotion step
    cmd = [gcc, "-O2", "-std=c11", "-ffp-contract=off", "-fPIC", "-shared", "-o", str(LIB), str(SOURCE), "-lm"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"gcc failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB


def load() -> ctypes.CDLL:
    lib = ctypes.CDLL(str(build()))
    sig = [ctypes.c_void_p] * 7 + [ctypes.c_int64] * 3
    lib.gateup_oracle_c.restype = ctypes.c_int
    lib.gateup_oracle_c.argtypes = sig
    lib.gemm_oracle_c.restype = ctypes.c_int
    lib.gemm_oracle_c.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int64] * 3
    return lib


if __name__ == "__main__":
    print(build())
