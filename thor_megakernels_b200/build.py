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
SOURCES = ["megakernel.cu", "nvfp4.cu", "gemv.cu", "linear_batched.cu", "batched_ops.cu", "batched_step.cu", "fp4_chain.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
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
    sources = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    nvcc = find_nvcc()
    # Build beside the target and rename: several ranks may find the library stale at the same moment,
    # and none of them must ever load a half-written file.  Sources compile side by side.
    tag = f"{os.getpid()}.tmp"
    objects = [PACKAGE_DIR / f"{src.stem}.{tag}.o" for src in sources]
    scratch = LIBRARY.with_name(f"{LIBRARY.name}.{tag}")
    procs = [(subprocess.Popen([nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", str(src), "-o", str(obj)],
                               stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True), src)
             for src, obj in zip(sources, objects)]
    logs, failed = [], []
    for proc, src in procs:
        out, _ = proc.communicate()
        logs.append(out)
        if proc.returncode != 0:
            failed.append(f"{src.name}:\n{out}")
    try:
        if failed:
            raise RuntimeError("nvcc failed:\n" + "\n".join(failed))
        link = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(scratch),
                               *map(str, objects)], capture_output=True, text=True)
        if link.returncode != 0:
            scratch.unlink(missing_ok=True)
            raise RuntimeError(f"link failed:\n{link.stdout}\n{link.stderr}")
        os.replace(scratch, LIBRARY)
    finally:
        for obj in objects:
            obj.unlink(missing_ok=True)
    if verbose:
        print("\n".join(logs))
    return LIBRARY


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
