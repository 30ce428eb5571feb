"""Caller-side MoE steps around ``grouped_mm``: routing to group order, row gather, weighted scatter.

``route`` turns per-token expert choices into the int32 END offsets ``grouped_mm`` takes as
``offs`` plus the row permutation; ``permute`` gathers token rows into group-contiguous order;
``combine`` sums each token's ``topk`` expert outputs back, weighted; ``gated_up_projection`` is the
feed-forward block's first half, ``silu(x @ gate) * (x @ up)``, with the activation fused into the
grouped GEMM's epilogue, and ``feed_forward`` chains all of them with the down-projection into
one routed block. The reference shows only the
offsets half of ``route``, on the host, in its benchmark (bench/bench_2d3d.py:131-138:
``bincount`` then ``cumsum``). Everything here runs in CUDA kernels of the same library, on the
current stream, with no host synchronisation; there is no CPU path.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib, _op
from ._op import _DTYPES
from .api import forward_into, grouped_mm, output_geometry


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


def _gated_up_forward(x: torch.Tensor, gate_up: torch.Tensor, offs: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    n = gate_up.size(2) // 2
    size, strides = output_geometry((x.size(0), x.size(1)), (gate_up.size(0), x.size(1), n), offs.numel(),
                                    out_dtype.itemsize)
    out = torch.empty_strided(size, strides, device=x.device, dtype=out_dtype)
    if out.numel() == 0:
        return out
    if x.size(1) == 0:
        return out.zero_()  # silu(0) * 0
    if _op.grouped_mm_2d3d_swiglu(x, gate_up, offs, out):
        return out
    both = torch.empty((x.size(0), 2 * n), dtype=torch.float32, device=x.device)
    forward_into(x, gate_up, offs, both)
    torch.mul(torch.nn.functional.silu(both[:, :n]), both[:, n:], out=out)
    return out


class _GatedUp(torch.autograd.Function):
    """Keeps only the inputs: the backward pass recomputes both products (one grouped GEMM with an
    fp32 result) instead of storing the ``[M_total, 2N]`` pre-activations the forward never wrote."""

    @staticmethod
    def forward(ctx, x, gate_up, offs, out_dtype):  # type: ignore[override]
        ctx.save_for_backward(x, gate_up, offs)
        return _gated_up_forward(x, gate_up, offs, out_dtype)

    @staticmethod
    def backward(ctx, grad_out):  # type: ignore[override]
        x, gate_up, offs = ctx.saved_tensors
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if grad_out.numel() == 0 or x.size(1) == 0:
            return (torch.zeros_like(x) if need_x else None, torch.zeros_like(gate_up) if need_w else None, None, None)
        n = gate_up.size(2) // 2
        # Rows at or past offs[-1] belong to no group: zeros there give zero gradients.
        both = torch.zeros((x.size(0), 2 * n), dtype=torch.float32, device=x.device)
        forward_into(x, gate_up, offs, both)
        gate, up = both[:, :n], both[:, n:]
        sig = torch.sigmoid(gate)
        dy = grad_out.float()
        d_both = torch.empty((x.size(0), 2 * n), dtype=x.dtype, device=x.device)
        d_both[:, :n] = dy * up * sig * (1.0 + gate * (1.0 - sig))  # d silu(g)/dg = s (1 + g (1 - s))
        d_both[:, n:] = dy * gate * sig
        del both, sig, dy
        grad_x = grad_w = None
        if need_x:  # dX[rows_g] = dBoth[rows_g] @ W[g]^T  (2D x 3D)
            grad_x = torch.zeros_like(x)
            forward_into(d_both, gate_up.transpose(-2, -1), offs, grad_x)
        if need_w:  # dW[g] = X[rows_g]^T @ dBoth[rows_g]  (2D x 2D; empty groups give zeros)
            grad_w = torch.empty_like(gate_up)
            forward_into(x.transpose(-2, -1), d_both, offs, grad_w)
        return grad_x, grad_w, None, None


def gated_up_projection(x: torch.Tensor, gate_up: torch.Tensor, offs: torch.Tensor,
                        out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``out[rows_g] = silu(x[rows_g] @ gate[g]) * (x[rows_g] @ up[g])`` for every group ``g``.

    ``x`` ``[M_total, K]`` holds the token rows in group order (see ``permute``), ``gate_up``
    ``[G, K, 2N]`` each expert's gate weights in columns ``[0, N)`` and up weights in ``[N, 2N)``,
    ``offs`` the int32 END offsets. Returns ``[M_total, N]`` of ``out_dtype`` (default: ``x.dtype``;
    float32 also allowed); rows at or past ``offs[-1]`` are left uninitialised, as with ``grouped_mm``.

    Both products accumulate in fp32 and the activation is applied to the fp32 accumulators inside
    the GEMM kernel, so the ``[M_total, 2N]`` intermediate is neither written nor read back and the
    result is rounded once. Differentiable: the backward pass recomputes the two products rather
    than keeping them (three more grouped GEMMs: the recompute, dX and dW). The reference has no such
    op; its users call ``grouped_mm`` and an element-wise kernel.

    Operands the tensor-core path cannot address (fp32, unaligned pitches, odd ``N`` with a row-major
    ``gate_up``) are multiplied by the ordinary grouped GEMM into an fp32 intermediate and activated by
    torch kernels on the GPU instead: same values, one more pass over memory.
    """
    if not (x.is_cuda and gate_up.is_cuda and offs.is_cuda):
        raise RuntimeError("grouped_mm_b200.moe is GPU-only; CPU tensors are not supported")
    if x.dim() != 2 or gate_up.dim() != 3 or x.size(1) != gate_up.size(1):
        raise RuntimeError("gated_up_projection expects x [M_total, K] and gate_up [G, K, 2N]")
    if gate_up.size(2) % 2:
        raise RuntimeError("gate_up needs an even number of columns: [gate | up]")
    if x.dtype != gate_up.dtype:
        raise RuntimeError("x and gate_up must have the same dtype")
    if x.dtype not in _DTYPES:
        raise RuntimeError(f"Expected x to be Float32, BFloat16 or Float16 matrix, got {x.dtype}")
    if offs.dtype != torch.int32 or offs.dim() != 1 or offs.numel() != gate_up.size(0):
        raise RuntimeError("offs has to be a 1D int32 tensor with one END offset per group")
    if offs.numel() >= 1024:
        raise RuntimeError("Can't process more than 1024 groups")
    out_dtype = out_dtype or x.dtype
    if out_dtype not in (x.dtype, torch.float32):
        raise RuntimeError("out_dtype must be the input dtype or float32")
    return _GatedUp.apply(x, gate_up, offs, out_dtype)


def feed_forward(x: torch.Tensor, expert_ids: torch.Tensor, weights: Optional[torch.Tensor],
                 gate_up: torch.Tensor, down: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """A routed gated feed-forward block, token rows in and token rows out:

        out[t] = sum_k weights[t, k] * (silu(x[t] @ gate[e]) * (x[t] @ up[e])) @ down[e],   e = expert_ids[t, k]

    ``x`` ``[tokens, hidden]``, ``expert_ids`` int32 ``[tokens, topk]``, ``weights`` ``[tokens, topk]``
    (``None``: all ones), ``gate_up`` ``[experts, hidden, 2 * inter]`` (``[gate | up]``), ``down``
    ``[experts, inter, hidden]``. Five launches on the current stream, none of which waits for the
    host: ``route``, ``permute``, ``gated_up_projection``, ``grouped_mm`` and ``combine``. Assignments
    whose expert id lies outside ``[0, experts)`` contribute nothing.
    """
    if expert_ids.dim() != 2 or expert_ids.size(0) != x.size(0):
        raise RuntimeError("expert_ids has to be [tokens, topk]")
    if gate_up.dim() != 3 or down.dim() != 3 or gate_up.size(0) != down.size(0) or \
            gate_up.size(2) != 2 * down.size(1) or down.size(2) != x.size(1):
        raise RuntimeError("expected gate_up [experts, hidden, 2 * inter] and down [experts, inter, hidden]")
    topk, experts = expert_ids.size(1), gate_up.size(0)
    offs, perm, inv = route(expert_ids, experts)
    rows = permute(x, perm, topk)
    hidden = gated_up_projection(rows, gate_up, offs)
    y = grouped_mm(hidden, down, offs=offs)
    return combine(y, inv, weights, topk, out_dtype=out_dtype)
