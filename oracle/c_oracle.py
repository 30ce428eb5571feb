"""ctypes loader for the plain-C oracle (oracle/gmm_oracle.c) — TEST INFRASTRUCTURE."""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path
from typing import Optional

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
LIB = HERE / "libgmm_oracle.so"


def build(force: bool = False) -> Path:
    src = HERE / "gmm_oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-o", str(LIB), str(src)], check=True)
    return LIB


def grouped_mm_c(mat_a: torch.Tensor, mat_b: torch.Tensor, offs: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Runs the C oracle on CPU copies of the inputs; elements owned by no group come back as 0."""
    lib = ctypes.CDLL(str(build()))
    fn = lib.gmm_oracle_f32
    fn.restype = ctypes.c_int
    a = np.ascontiguousarray(mat_a.detach().cpu().float().numpy())
    b = np.ascontiguousarray(mat_b.detach().cpu().float().numpy())
    a2, b2 = a.ndim == 2, b.ndim == 2
    if not a2 and not b2:
        form, (G, M, K), N = 0, a.shape, b.shape[2]
        out = np.zeros((G, M, N), np.float32)
    elif a2 and not b2:
        form, (M, K), (G, _, N) = 1, a.shape, b.shape
        out = np.zeros((M, N), np.float32)
    elif not a2 and b2:
        form, (G, M, K), N = 2, a.shape, b.shape[1]
        out = np.zeros((M, N), np.float32)
    else:
        form, (M, K), N, G = 3, a.shape, b.shape[1], int(offs.numel())
        out = np.zeros((G, M, N), np.float32)
    offs_np = None if offs is None else np.ascontiguousarray(offs.detach().cpu().numpy().astype(np.int32))
    fp = ctypes.POINTER(ctypes.c_float)
    rc = fn(form, int(G), int(M), int(N), int(K), a.ctypes.data_as(fp), b.ctypes.data_as(fp),
            None if offs_np is None else offs_np.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
            out.ctypes.data_as(fp))
    if rc != 0:
        raise RuntimeError("gmm_oracle_f32 rejected its arguments")
    return torch.from_numpy(out)
