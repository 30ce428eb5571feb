"""CPU oracle for grouped_mm — TEST INFRASTRUCTURE, not part of the product.

A restatement, on CPU tensors, of what the reference computes on the GPU. Only tests,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import this module; the
product package never does and has no CPU path.

What it follows in the reference (lostmsu/grouped_mm_bf16):
  * group ownership: index i belongs to group ``upper_bound(offs, i)``, i.e. group g owns
    ``[offs[g-1], offs[g])`` with ``offs`` int32 END indices (grouped_mm_bf16/kernels.py:162-172);
    ``offs[-1]`` may be smaller than the extent, and is clamped to it (kernels.py:339);
  * output shapes of the four forms (grouped_mm_bf16/api.py:134-149);
  * fp32 accumulation with a single rounding at the store (kernels.py:226-245, 282-301, 343-360),
    so the oracle keeps its result in fp32 and the comparison allows for the final rounding;
  * 2D x 2D: an empty K range yields an all-zero block (kernels.py:282, 300-301; relied on by
    tests/test_grouped_mm.py:102-103);
  * 3D x 2D column ownership (kernels.py:496-521);
  * the per-group loops the reference's tests use as their own check
    (tests/test_grouped_mm.py:55-66, 93-105, 133-144).
The reference has no CPU compute path (api.py:93-94 raises for CPU tensors), so this is a port.

Parity pinning: the reference stores no golden vectors. The oracle is pinned against fixtures
generated in a GPU-less container by running the reference's own kernel-level functions under
Triton's interpreter in fp32 and ``torch.nn.functional.grouped_mm`` on CPU in bf16
(tests/golden/make_golden.py writes them; tests/test_oracle.py checks them).
"""

from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch


def group_bounds(offs, extent: int) -> List[Tuple[int, int]]:
    """[start, end) of every group along the ragged dimension, clamped into [0, extent]."""
    ends = [max(0, min(int(e), extent)) for e in (offs.tolist() if hasattr(offs, "tolist") else offs)]
    out, start = [], 0
    for e in ends:
        out.append((start, e) if e > start else (start, start))
        start = e
    return out


def grouped_mm_oracle(mat_a: torch.Tensor, mat_b: torch.Tensor, offs: Optional[torch.Tensor] = None):
    """Returns (ref, defined): fp32 result on CPU and a bool mask of the elements the op defines.

    Elements outside every group (rows/columns at or past ``offs[-1]``) are not written by the
    operator; they are zero in ``ref`` and False in ``defined``.
    """
    a = mat_a.detach().cpu()
    b = mat_b.detach().cpu()
    a_is_2d, b_is_2d = a.dim() == 2, b.dim() == 2
    if not a_is_2d and not b_is_2d:
        ref = torch.stack([a[g].float() @ b[g].float() for g in range(a.size(0))]) if a.size(0) else \
            torch.zeros((0, a.size(1), b.size(2)))
        return ref, torch.ones_like(ref, dtype=torch.bool)
    assert offs is not None
    offs_cpu = offs.detach().cpu()
    if a_is_2d and not b_is_2d:
        m_total, n = a.size(0), b.size(2)
        ref = torch.zeros((m_total, n), dtype=torch.float32)
        defined = torch.zeros((m_total, n), dtype=torch.bool)
        for g, (s, e) in enumerate(group_bounds(offs_cpu, m_total)):
            if e > s:
                ref[s:e] = a[s:e].float() @ b[g].float()
                defined[s:e] = True
        return ref, defined
    if a_is_2d and b_is_2d:
        m, k_total, n = a.size(0), a.size(1), b.size(1)
        g_count = offs_cpu.numel()
        ref = torch.zeros((g_count, m, n), dtype=torch.float32)
        for g, (s, e) in enumerate(group_bounds(offs_cpu, k_total)):
            if e > s:
                ref[g] = a[:, s:e].float() @ b[s:e].float()
        return ref, torch.ones_like(ref, dtype=torch.bool)
    m, n_total = a.size(1), b.size(1)
    ref = torch.zeros((m, n_total), dtype=torch.float32)
    defined = torch.zeros((m, n_total), dtype=torch.bool)
    for g, (s, e) in enumerate(group_bounds(offs_cpu, n_total)):
        if e > s:
            ref[:, s:e] = a[g].float() @ b[:, s:e].float()
            defined[:, s:e] = True
    return ref, defined


RTOL = 8e-3
ATOL_COEF = 1e-2


def atol_for(k: int, sigma_a: float, sigma_b: float) -> float:
    """Absolute tolerance 1e-2 * sqrt(K) * sigma_a * sigma_b for contraction length K."""
    return ATOL_COEF * math.sqrt(max(int(k), 0)) * sigma_a * sigma_b


def max_violation(out: torch.Tensor, ref: torch.Tensor, defined: torch.Tensor, atol: float,
                  rtol: float = RTOL) -> float:
    """max over defined elements of |out - ref| / (atol + rtol * |ref|); <= 1 means within tolerance."""
    o = out.detach().float().cpu()
    if not bool(defined.any()):
        return 0.0
    err = (o - ref).abs()
    bound = atol + rtol * ref.abs()
    ratio = torch.where(defined, err / bound.clamp_min(1e-30), torch.zeros_like(err))
    if not bool(torch.isfinite(o[defined]).all()):
        return float("inf")
    return float(ratio.max())


def kragged_atol(offs, k_total: int, sigma_a: float, sigma_b: float) -> torch.Tensor:
    """Per-group absolute tolerance for the 2D x 2D form (K is the group's own length); an empty
    group gets 0, i.e. its block must be exactly zero."""
    return torch.tensor([atol_for(e - s, sigma_a, sigma_b) for s, e in group_bounds(offs.cpu(), k_total)])
