"""In-tree build of libgrouped_mm_b200.so with nvcc for sm_100a.

The library is built next to the sources (``grouped_mm_bf16_b200/lib``) so that it travels with a
snapshot of the tree; nothing is cached outside the repository. ``python -m
grouped_mm_bf16_b200.build`` builds it, ``build_library()`` does the same from Python.

Plain ``-arch=sm_100a`` is not used: the family-specific target has to be named as
``-gencode arch=compute_100a,code=sm_100a`` for ptxas to accept tcgen05 instructions.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC_DIR = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libgrouped_mm_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc")
    if exe:
        return exe
    cand = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
    if cand.exists():
        return str(cand)
    raise RuntimeError("nvcc not found: cannot build libgrouped_mm_b200.so")


def sources() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cu")) + sorted(CSRC_DIR.glob("*.cuh")) + [PKG_DIR.parent / "include" / "grouped_mm_b200.h"]


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(src.exists() and src.stat().st_mtime > built for src in sources())


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compiles the CUDA library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    cu_files = [str(p) for p in sorted(CSRC_DIR.glob("*.cu"))]
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB_PATH), *cu_files]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
