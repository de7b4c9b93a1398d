"""Compiles the reference's own CUDA sources of problems 038 and 029, where they lie in a checkout of the
reference repository, into torch extensions under oracle/_ref/ (git-ignored).  Test infrastructure only: the GPU
parity tests load these libraries, when present, as a second check beside the CPU restatement; nothing in the
package imports them.  Nothing is copied: the compiler reads the sources in place.

    python oracle/build_ref.py /path/to/reference/checkout

Problem 029 includes CUTLASS headers when built for sm_100a; the header tree vendored by flashinfer is passed as
an include path, and a failure to compile is reported, not fatal.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

PROBLEMS = {
    "ref038_rmsnorm_qk": ("kernels/038_flux_multi_head_rmsnorm_qk", ["binding.cpp", "kernel.cu"], []),
    "ref029_mamba_conv1d": ("kernels/029_mamba_conv1d_with_gating", ["binding.cpp", "kernel.cu"], []),
    # Not built: the C++ variant of problem 179 (variants/cuda_cpp_v4).  It compiles against the CUTLASS tree of
    # this image, but its first launch returns "invalid configuration argument" from CUTLASS's cluster launch (the
    # variant was written against another CUTLASS release), so it cannot serve as a checker here.
}


def cutlass_include() -> list[str]:
    try:
        import flashinfer
    except Exception:
        return []
    root = Path(flashinfer.__file__).parent / "data" / "cutlass"
    return [str(root / "include"), str(root / "tools" / "util" / "include")] if root.exists() else []


def build(reference_root: str, only: str | None = None) -> dict:
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    from torch.utils import cpp_extension

    results = {}
    for name, (subdir, files, defines) in PROBLEMS.items():
        if only and only != name:
            continue
        src = Path(reference_root) / subdir
        build_dir = OUT / name
        build_dir.mkdir(parents=True, exist_ok=True)
        try:
            cpp_extension.load(
                name=name, sources=[str(src / f) for f in files], build_directory=str(build_dir),
                extra_cflags=["-O3", "-std=c++17"],
                extra_cuda_cflags=["-O3", "--use_fast_math", "-std=c++17"] + defines,
                extra_include_paths=[str(src)] + cutlass_include(), extra_ldflags=["-lcuda"],
                is_python_module=False, verbose=False)
            results[name] = "built"
        except Exception as exc:  # noqa: BLE001 - report and go on with the next problem
            results[name] = f"failed: {str(exc)[-400:]}"
    return results


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    root = sys.argv[1]
    for k, v in build(root, sys.argv[2] if len(sys.argv) > 2 else None).items():
        print(k, "->", v)
