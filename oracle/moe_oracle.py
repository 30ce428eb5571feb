"""CPU oracle for the MoE routing helpers — TEST INFRASTRUCTURE, not part of the product.

Restates on the host what the reference's benchmark does for the offsets
(bench/bench_2d3d.py:131-138: ``torch.bincount(expert_ids, minlength=experts)`` then
``cumsum`` to int32 end offsets) and extends it with the stable permutation a caller needs to
build ``mat_a``: a stable argsort of the assignments by expert. Integer results are compared
bit for bit.
"""

from __future__ import annotations

from typing import Optional

import torch


def route_oracle(expert_ids: torch.Tensor, num_experts: int):
    ids = expert_ids.detach().cpu().reshape(-1).long()
    valid = (ids >= 0) & (ids < num_experts)
    counts = torch.bincount(ids[valid], minlength=num_experts)
    offs = counts.cumsum(0).to(torch.int32)
    key = torch.where(valid, ids, torch.full_like(ids, num_experts))  # unrouted assignments sort last
    order = torch.sort(key, stable=True).indices
    n_valid = int(valid.sum())
    perm = torch.full((ids.numel(),), -1, dtype=torch.int32)
    perm[:n_valid] = order[:n_valid].to(torch.int32)
    inv = torch.full((ids.numel(),), -1, dtype=torch.int32)
    inv[order[:n_valid]] = torch.arange(n_valid, dtype=torch.int32)
    return offs, perm, inv


def permute_oracle(x: torch.Tensor, perm: torch.Tensor, topk: int) -> torch.Tensor:
    p = perm.detach().cpu().long()
    return x.detach().cpu()[p.clamp_min(0) // topk]


def combine_oracle(y: torch.Tensor, inv_perm: torch.Tensor, weights: Optional[torch.Tensor], topk: int) -> torch.Tensor:
    inv = inv_perm.detach().cpu().long().view(-1, topk)
    yy = y.detach().cpu().float()
    w = torch.ones(inv.shape) if weights is None else weights.detach().cpu().float().view(-1, topk)
    w = torch.where(inv >= 0, w, torch.zeros_like(w))
    return (yy[inv.clamp_min(0)] * w.unsqueeze(-1)).sum(1)


def gated_up_oracle(x: torch.Tensor, gate_up: torch.Tensor, offs: torch.Tensor):
    """``silu(x_g @ gate_g) * (x_g @ up_g)`` per group in fp32 on the CPU, with ``gate_up[g]`` holding
    ``[gate | up]`` side by side. No counterpart in the reference (its callers apply the activation
    after ``grouped_mm``, whose per-group product this restates as in grouped_mm_oracle). Returns
    ``(out [M_total, N] fp32, defined [M_total] bool)``: rows at or past ``offs[-1]`` are undefined."""
    xx, ww = x.detach().cpu().float(), gate_up.detach().cpu().float()
    n = ww.size(2) // 2
    ends = [max(0, min(int(e), xx.size(0))) for e in offs.detach().cpu().tolist()]
    out = torch.zeros((xx.size(0), n), dtype=torch.float32)
    defined = torch.zeros(xx.size(0), dtype=torch.bool)
    start = 0
    for g, end in enumerate(ends):
        if end > start:
            both = xx[start:end] @ ww[g]
            out[start:end] = torch.nn.functional.silu(both[:, :n]) * both[:, n:]
            defined[start:end] = True
        start = max(start, end)
    return out, defined
