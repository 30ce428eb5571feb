"""Expert-parallel routed feed-forward block: tokens on every rank, each rank's own experts.

One process per GPU; rank ``r`` of ``world`` holds the weights of experts
``[r * E_local, (r + 1) * E_local)`` and a batch of token rows of its own. ``feed_forward`` sends
every routed row to the rank that owns its expert, runs the grouped GEMMs there, and brings the
results back:

    route (by global expert id)  ->  gather rows in that order      local CUDA kernels (moe.py)
    all-to-all of per-expert row counts, then of the rows           NCCL, into the receiver's own memory
    regroup the received rows by local expert                       local CUDA kernels
    gated up-projection, down-projection                            grouped GEMM kernels, local memory only
    undo the regrouping, all-to-all back, weighted combine          NCCL + local CUDA kernels

The reference has no multi-GPU code; its operator, like this package's, never communicates. The
exchange is NCCL's all-to-all with per-peer split sizes (over NVLink on one node); the row counts
have to reach the host for those split sizes, which is the one host synchronisation of the block.
The GEMM kernels only ever read this GPU's memory: received rows land in a local buffer first.

The local steps are taken from an ``ops`` namespace so that the index arithmetic and the exchange
can be checked on CPU ranks over gloo with host stand-ins for the kernels; the default is the CUDA
implementation, and there is no CPU fallback inside it.
"""

from __future__ import annotations

from types import SimpleNamespace
from typing import Optional

import torch
import torch.distributed as dist


def cuda_ops() -> SimpleNamespace:
    """The CUDA implementation of the local steps (this package's kernels)."""
    from . import moe
    from .api import grouped_mm

    return SimpleNamespace(route=moe.route, permute=moe.permute, combine=moe.combine,
                           gated_up_projection=moe.gated_up_projection, grouped_mm=grouped_mm)


def split_sizes(counts: torch.Tensor, recv_counts: torch.Tensor):
    """Per-peer row counts for the two all-to-alls, from the ``[world, E_local]`` count matrices
    (rows this rank sends to / receives from each peer, by the peer's / this rank's local expert)."""
    return [int(v) for v in counts.sum(1).tolist()], [int(v) for v in recv_counts.sum(1).tolist()]


def received_expert_ids(recv_counts: torch.Tensor, total: int) -> torch.Tensor:
    """Local expert id of every received row. Rows arrive ordered by source rank, then by expert:
    ``recv_counts[s, e]`` rows of expert ``e`` from rank ``s``."""
    world, e_local = recv_counts.shape
    ids = torch.arange(e_local, device=recv_counts.device, dtype=torch.int32).repeat(world)
    return torch.repeat_interleave(ids, recv_counts.reshape(-1).long(), output_size=total)


def feed_forward(x: torch.Tensor, expert_ids: torch.Tensor, weights: Optional[torch.Tensor],
                 gate_up_local: torch.Tensor, down_local: torch.Tensor, group=None,
                 out_dtype: Optional[torch.dtype] = None, ops: Optional[SimpleNamespace] = None) -> torch.Tensor:
    """``moe.feed_forward`` with the experts spread over the ranks of ``group``.

    ``x`` ``[tokens, hidden]`` and ``expert_ids`` int32 ``[tokens, topk]`` (GLOBAL expert ids) are this
    rank's tokens; ``gate_up_local`` ``[E_local, hidden, 2 * inter]`` and ``down_local``
    ``[E_local, inter, hidden]`` the weights of this rank's experts. Returns this rank's
    ``[tokens, hidden]`` result. Every rank of the group has to call it (collective).
    """
    ops = ops or cuda_ops()
    world = dist.get_world_size(group)
    e_local = gate_up_local.size(0)
    experts = e_local * world
    topk = expert_ids.size(1)
    dev = x.device

    # rows in global expert order = ordered by destination rank, then by that rank's local expert
    offs, perm, inv = ops.route(expert_ids, experts)
    counts = torch.diff(offs, prepend=offs.new_zeros(1)).view(world, e_local)
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=group)
    send_split, recv_split = split_sizes(counts, recv_counts)  # the block's one host synchronisation
    n_send, n_recv = sum(send_split), sum(recv_split)

    rows = ops.permute(x, perm, topk, n_send)
    recv_rows = torch.empty((n_recv, x.size(1)), dtype=x.dtype, device=dev)
    dist.all_to_all_single(recv_rows, rows, recv_split, send_split, group=group)

    # received rows are grouped by source rank first: regroup them by local expert
    local_ids = received_expert_ids(recv_counts, n_recv)
    offs_l, perm_l, inv_l = ops.route(local_ids, e_local)
    grouped = ops.permute(recv_rows, perm_l, 1, n_recv)
    hidden = ops.gated_up_projection(grouped, gate_up_local, offs_l)
    y = ops.grouped_mm(hidden, down_local, offs=offs_l)

    # back into arrival order, back to the ranks the rows came from, and summed per token
    y_arrival = ops.permute(y, inv_l, 1, n_recv)
    y_back = torch.empty((n_send, y.size(1)), dtype=y.dtype, device=dev)
    dist.all_to_all_single(y_back, y_arrival, send_split, recv_split, group=group)
    return ops.combine(y_back, inv, weights, topk, out_dtype=out_dtype)
