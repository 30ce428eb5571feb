"""Caller-side MoE steps around ``grouped_mm``: routing to group order, row gather, weighted scatter.

``route`` turns per-token expert choices into the int32 END offsets ``grouped_mm`` takes as
``offs`` plus the row permutation; ``permute`` gathers token rows into group-contiguous order;
``combine`` sums each token's ``topk`` expert outputs back, weighted. The reference shows only the
offsets half of ``route``, on the host, in its benchmark (bench/bench_2d3d.py:131-138:
``bincount`` then ``cumsum``). Everything here runs in CUDA kernels of the same library, on the
current stream, with no host synchronisation; there is no CPU path.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._op import _DTYPES


def _check(lib, rc: int) -> None:
    if rc != 0:
        raise RuntimeError(_lib.error_message(lib, rc))


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def route(expert_ids: torch.Tensor, num_experts: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Stable grouping of routed assignments by expert.

    ``expert_ids``: int32 CUDA tensor ``[tokens, topk]`` (or flat ``[tokens * topk]``); entry
    ``i`` is the expert of assignment ``i`` = (token ``i // topk``, choice ``i % topk``).
    Returns ``(offs, perm, inv_perm)``: ``offs`` int32 ``[num_experts]`` END offsets,
    ``perm[p]`` the assignment at sorted position ``p``, ``inv_perm[i]`` the position of
    assignment ``i`` (-1 where the id is outside ``[0, num_experts)``).
    """
    if not expert_ids.is_cuda:
        raise RuntimeError("grouped_mm_b200.moe is GPU-only; CPU tensors are not supported")
    if expert_ids.dtype != torch.int32:
        raise RuntimeError("expert_ids have to be int32")
    lib = _lib.load()
    ids = expert_ids.reshape(-1).contiguous()
    n = ids.numel()
    dev = ids.device
    ws_bytes = int(lib.gmm_route_workspace_bytes(n, num_experts))
    if ws_bytes == 0:
        raise RuntimeError("Can't process more than 1024 groups" if num_experts >= 1024 else "invalid routing arguments")
    with torch.cuda.device(dev):
        ws = torch.empty(ws_bytes // 4, dtype=torch.int32, device=dev)
        offs = torch.empty(num_experts, dtype=torch.int32, device=dev)
        perm = torch.empty(n, dtype=torch.int32, device=dev)
        inv = torch.empty(n, dtype=torch.int32, device=dev)
        _check(lib, lib.gmm_route_build(ids.data_ptr(), n, num_experts, offs.data_ptr(), perm.data_ptr(),
                                        inv.data_ptr(), ws.data_ptr(), ws_bytes, _stream(dev)))
    return offs, perm, inv


def permute(x: torch.Tensor, perm: torch.Tensor, topk: int, n_rows: Optional[int] = None) -> torch.Tensor:
    """Gathers token rows into group order: ``out[r] = x[perm[r] // topk]`` (``[n_rows, K]``)."""
    if not (x.is_cuda and perm.is_cuda) or x.dim() != 2 or x.stride(1) != 1:
        raise RuntimeError("permute expects a CUDA [tokens, K] tensor with a contiguous last dimension")
    lib = _lib.load()
    n_rows = perm.numel() if n_rows is None else n_rows
    out = torch.empty((n_rows, x.size(1)), dtype=x.dtype, device=x.device)
    es = x.element_size()
    with torch.cuda.device(x.device):
        _check(lib, lib.gmm_permute_rows(x.data_ptr(), x.size(0), x.size(1) * es, x.stride(0) * es, perm.data_ptr(),
                                         topk, out.data_ptr(), out.stride(0) * es, n_rows, _stream(x.device)))
    return out


def combine(y: torch.Tensor, inv_perm: torch.Tensor, weights: Optional[torch.Tensor], topk: int,
            out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Weighted sum of each token's expert outputs: ``out[t] = sum_k w[t,k] * y[inv_perm[t*topk+k]]``."""
    if not (y.is_cuda and inv_perm.is_cuda) or y.dim() != 2 or y.stride(1) != 1:
        raise RuntimeError("combine expects a CUDA [rows, N] tensor with a contiguous last dimension")
    lib = _lib.load()
    n_tokens = inv_perm.numel() // topk
    out_dtype = out_dtype or y.dtype
    out = torch.empty((n_tokens, y.size(1)), dtype=out_dtype, device=y.device)
    w_ptr = None
    if weights is not None:
        weights = weights.reshape(-1).to(torch.float32).contiguous()
        if weights.numel() != n_tokens * topk:
            raise RuntimeError("weights must have one entry per assignment")
        w_ptr = weights.data_ptr()
    with torch.cuda.device(y.device):
        _check(lib, lib.gmm_combine_rows(y.data_ptr(), _DTYPES[y.dtype], y.stride(0), inv_perm.data_ptr(), w_ptr, topk,
                                         n_tokens, y.size(1), out.data_ptr(), _DTYPES[out_dtype], out.stride(0),
                                         _stream(y.device)))
    return out
