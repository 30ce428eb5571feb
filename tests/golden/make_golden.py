"""Generates tests/golden/grouped_mm_golden.pt — run once in a container that has the reference.

Two independent sources pin the CPU oracle (the reference itself stores no golden vectors):
  1. the reference's own kernel-level forward functions (grouped_mm_bf16/kernels.py:524-717),
     executed on CPU tensors by Triton's interpreter (TRITON_INTERPRET=1) in fp32 — this pins the
     group ownership, masking and shape logic of the real reference code;
  2. ``torch.nn.functional.grouped_mm`` on CPU in bf16 for 16-byte aligned shapes — this pins the
     bf16 semantics the reference mirrors (its README: "matches PyTorch grouped_mm shape
     semantics").
Inputs are seeded; inputs, offsets and outputs are stored so the test needs neither source.

Usage (the reference tree is read-only and is only put on sys.path):
    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")

import torch
import torch.nn.functional as F

OUT = Path(__file__).resolve().parent / "grouped_mm_golden.pt"

# Group-size patterns taken from the reference's tests (tests/test_grouped_mm.py:37, 75, 355-371).
M_PATTERNS = [[0, 7, 1, 13, 0, 11], [32, 32, 32], [10, 10, 10, 2], [31, 1, 31], [40, 30, 10, 7],
              [32, 16, 0, 0, 0], [1, 0] * 6, [5, 0, 7, 0, 3, 9]]
KN_PATTERNS = [[7, 0, 1, 13, 11], [8, 0, 16, 24, 8]]


def _offs(sizes):
    return torch.tensor(sizes, dtype=torch.int32).cumsum(0).to(torch.int32)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from grouped_mm_bf16 import kernels as ref  # the unmodified reference

    gen = torch.Generator().manual_seed(1234)
    cases = []

    def rnd(*shape):
        return torch.randn(*shape, generator=gen, dtype=torch.float32)

    # ---- source 1: reference kernels under the interpreter, fp32, odd K/N as its tests use
    for sizes in M_PATTERNS:
        k, n = 33, 29
        a, b, offs = rnd(sum(sizes), k), rnd(len(sizes), k, n), _offs(sizes)
        out = torch.zeros(sum(sizes), n)
        ref.grouped_mm_2d3d(a, b, offs, out)
        cases.append(dict(source="reference-interpreter", form="2d3d", a=a, b=b, offs=offs, out=out))
    for sizes in KN_PATTERNS:
        m, n = 16, 24
        a, b, offs = rnd(m, sum(sizes)), rnd(sum(sizes), n), _offs(sizes)
        out = torch.zeros(len(sizes), m, n)
        ref.grouped_mm_2d2d(a, b, offs, out)
        cases.append(dict(source="reference-interpreter", form="2d2d", a=a, b=b, offs=offs, out=out))
        m, k = 32, 48
        a, b = rnd(len(sizes), m, k), rnd(k, sum(sizes))
        out = torch.zeros(m, sum(sizes))
        ref.grouped_mm_3d2d(a, b, offs, out)
        cases.append(dict(source="reference-interpreter", form="3d2d", a=a, b=b, offs=offs, out=out))
    a, b = rnd(3, 17, 19), rnd(3, 19, 23)
    out = torch.zeros(3, 17, 23)
    ref.grouped_mm_3d3d(a, b, out)
    cases.append(dict(source="reference-interpreter", form="3d3d", a=a, b=b, offs=None, out=out))
    # offs[-1] below the extent: trailing rows belong to no group and stay untouched (zeros here).
    a, b, offs = rnd(40, 16), rnd(3, 16, 8), _offs([5, 9, 11])
    out = torch.zeros(40, 8)
    ref.grouped_mm_2d3d(a, b, offs, out)
    cases.append(dict(source="reference-interpreter", form="2d3d", a=a, b=b, offs=offs, out=out))

    # ---- source 2: torch.nn.functional.grouped_mm on CPU, bf16, aligned shapes
    sizes = [0, 7, 1, 13, 0, 11]
    a, b, offs = rnd(32, 64).bfloat16(), rnd(6, 64, 48).bfloat16(), _offs(sizes)
    cases.append(dict(source="torch-cpu", form="2d3d", a=a, b=b, offs=offs, out=F.grouped_mm(a, b, offs=offs)))
    bt = rnd(6, 48, 64).bfloat16().transpose(-2, -1)  # column-major B
    cases.append(dict(source="torch-cpu", form="2d3d", a=a, b=bt, offs=offs, out=F.grouped_mm(a, bt, offs=offs)))
    sizes = [8, 0, 16, 24, 8]
    at, b, offs = rnd(56, 16).bfloat16().t(), rnd(56, 24).bfloat16(), _offs(sizes)  # column-major A
    cases.append(dict(source="torch-cpu", form="2d2d", a=at, b=b, offs=offs, out=F.grouped_mm(at, b, offs=offs)))
    a, bt = rnd(5, 32, 48).bfloat16(), rnd(56, 48).bfloat16().t()
    cases.append(dict(source="torch-cpu", form="3d2d", a=a, b=bt, offs=offs, out=F.grouped_mm(a, bt, offs=offs)))
    a, b = rnd(4, 32, 64).bfloat16(), rnd(4, 64, 48).bfloat16()
    cases.append(dict(source="torch-cpu", form="3d3d", a=a, b=b, offs=None, out=F.grouped_mm(a, b)))

    for c in cases:
        for key in ("a", "b", "out"):
            c[key] = c[key].contiguous() if key == "out" else c[key]
        c["a_strides"], c["b_strides"] = tuple(c["a"].stride()), tuple(c["b"].stride())
    torch.save(dict(torch=str(torch.__version__), cases=cases), OUT)
    print(f"wrote {len(cases)} cases to {OUT} ({OUT.stat().st_size} bytes)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
