"""Builds ``libb200mk.so`` (the C-ABI CUDA library) in-tree with nvcc.

sm_100a only; nvcc cross-compiles, so this works on a machine without a GPU.
Run as ``python -m thor_megakernels_b200.build`` or call ``build_library()``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIBRARY = PACKAGE_DIR / "libb200mk.so"
SOURCES = ["megakernel.cu", "nvfp4.cu", "gemv.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return nvcc


def is_stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    inputs = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PACKAGE_DIR.parent / "include" / "b200_megakernel.h"]
    return any(f.stat().st_mtime > built for f in inputs)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIBRARY
    sources = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    # Build beside the target and rename: several ranks may find the library stale at the same moment,
    # and none of them must ever load a half-written file.
    scratch = LIBRARY.with_name(f"{LIBRARY.name}.{os.getpid()}.tmp")
    cmd = [find_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", str(scratch), *sources]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        scratch.unlink(missing_ok=True)
        raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    os.replace(scratch, LIBRARY)
    if verbose:
        print(proc.stderr)
    return LIBRARY


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
