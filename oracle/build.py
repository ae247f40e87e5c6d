"""TEST INFRASTRUCTURE ONLY - compiles oracle/nvfp4_ref.cpp into
oracle/_ref/libnvfp4_ref.so with g++ (needs the CUDA toolkit headers, no GPU)."""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "libnvfp4_ref.so"


def cuda_include() -> str:
    for root in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if root and (Path(root) / "include" / "cuda_fp4.h").exists():
            return str(Path(root) / "include")
    raise RuntimeError("CUDA toolkit headers (cuda_fp4.h) not found")


def build_oracle(force: bool = False) -> Path:
    src = HERE / "nvfp4_ref.cpp"
    if OUT.exists() and not force and OUT.stat().st_mtime >= src.stat().st_mtime:
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-I{cuda_include()}", "-o", str(OUT), str(src)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{proc.stderr}")
    return OUT


if __name__ == "__main__":
    print(build_oracle(force=True))
