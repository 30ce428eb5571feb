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

``feed_forward_peer`` (second half of this file) is the same block without the all-to-alls and
without the host synchronisation: the rows are stored into, and the results loaded from, the
peers' buffers by this package's own kernels.
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


# ---------------------------------------------------------------------------------------------
# The same block with the rows moved by this package's own kernels over peer memory.
#
# Every rank can work out, from the all-gathered per-expert row counts, where each of its routed
# rows belongs in the buffer of the GPU that owns the row's expert: that buffer holds the rows of
# local expert 0 first, then of local expert 1, ..., and inside an expert the rows of source rank 0,
# then of rank 1, ... . So the rows are written straight to their final, expert-grouped position
# with stores over NVLink (no pack, no unpack, no regrouping pass), the grouped GEMMs run on local
# memory, and every token pulls its result rows back from the peers' output buffers. No step
# needs a number on the host, so nothing here waits for the host.


def exchange_plan(offs: torch.Tensor, perm: torch.Tensor, inv: torch.Tensor, counts_all: torch.Tensor, rank: int,
                  e_local: int):
    """Index tables of one rank's part of the exchange (plain torch ops on ``offs.device``).

    ``offs`` ``[E]``, ``perm``, ``inv``: this rank's ``route`` result over the GLOBAL expert ids;
    ``counts_all`` ``[world, E]``: every rank's per-expert row counts (``counts_all[rank]`` is this
    rank's). Returns int32 tensors

      ``dst_rank``, ``dst_row``  per sorted position: owner of the row's expert and the row's place
                                 in the owner's buffer (-1 where the position holds no routed row)
      ``src_rank``, ``src_row``  the same two per assignment ``t * topk + k`` (for the way back)
      ``offs_local`` ``[e_local]``  END offsets of the rows this rank receives, by local expert
    """
    world, experts = counts_all.shape
    counts_all = counts_all.long()
    total = counts_all.sum(0).view(world, e_local)                      # rows per expert, by owner
    first_row = (total.cumsum(1) - total).reshape(-1)                   # where an expert starts in its owner's buffer
    earlier = counts_all[:rank].sum(0)                                  # rows of lower-ranked sources, per expert
    base = first_row + earlier                                          # this rank's first row of every expert
    starts = offs.long() - counts_all[rank]                             # first sorted position of every expert
    pos = torch.arange(perm.numel(), device=offs.device)
    g = torch.searchsorted(offs.long().contiguous(), pos, right=True)   # expert of sorted position p
    routed = g < experts
    gc = g.clamp_max(experts - 1)
    minus1 = torch.full_like(pos, -1)
    dst_rank = torch.where(routed, gc // e_local, minus1)
    dst_row = torch.where(routed, base[gc] + (pos - starts[gc]), minus1)
    back = inv.long().clamp_min(0)
    src_rank = torch.where(inv >= 0, dst_rank[back], minus1)
    src_row = torch.where(inv >= 0, dst_row[back], minus1)
    offs_local = total[rank].cumsum(0)
    i32 = torch.int32
    return dst_rank.to(i32), dst_row.to(i32), src_rank.to(i32), src_row.to(i32), offs_local.to(i32)


class PeerBuffers:
    """Symmetric receive and result buffers of one process group (``torch.distributed``'s symmetric
    memory: the same allocation on every rank, each mapped into every peer). Collective to create."""

    def __init__(self, capacity_rows: int, hidden: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.capacity, self.hidden = int(capacity_rows), int(hidden)
        self.rows = symm_mem.empty((self.capacity, self.hidden), dtype=dtype, device=device)   # dispatched rows
        self.result = symm_mem.empty((self.capacity, self.hidden), dtype=dtype, device=device)  # down-projection
        self._rows_hdl = symm_mem.rendezvous(self.rows, self.group)
        self._result_hdl = symm_mem.rendezvous(self.result, self.group)
        self.world = self._rows_hdl.world_size
        self.rank = self._rows_hdl.rank
        # device arrays of the peers' base pointers (entry r = rank r's buffer as mapped here)
        self.rows_ptrs = torch.tensor(list(self._rows_hdl.buffer_ptrs), dtype=torch.int64, device=device)
        self.result_ptrs = torch.tensor(list(self._result_hdl.buffer_ptrs), dtype=torch.int64, device=device)
        self._token = torch.zeros(1, dtype=torch.int32, device=device)

    def fence(self) -> None:
        """Orders, on the current stream, everything every rank did before against everything any
        rank does after: a one-element all-reduce."""
        dist.all_reduce(self._token, group=self.group)


def feed_forward_peer(x: torch.Tensor, expert_ids: torch.Tensor, weights: Optional[torch.Tensor],
                      gate_up_local: torch.Tensor, down_local: torch.Tensor, buffers: PeerBuffers,
                      out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``feed_forward`` with the rows moved by stores to and loads from the peers' buffers.

    Same arguments and result; ``buffers`` (created once, collectively) must hold at least as many
    rows as any rank can receive - ``world * tokens * topk`` is always enough. Enqueues on the
    current stream and returns without waiting for the host. Rows that would not fit are dropped
    and ``GMM_STATUS_BAD_PEER_INDEX`` appears in the device status word (``_op.check_status``).
    """
    import ctypes

    from . import _lib, _op, moe
    from .api import forward_into

    lib = _lib.load()
    dev = x.device
    world, rank = buffers.world, buffers.rank
    e_local = gate_up_local.size(0)
    experts = e_local * world
    topk = expert_ids.size(1)
    if x.size(1) != buffers.hidden or down_local.size(2) != buffers.hidden or x.dtype != buffers.rows.dtype:
        raise RuntimeError("buffers were created for another hidden size or dtype")
    if x.stride(1) != 1:
        raise RuntimeError("x needs a contiguous last dimension")

    offs, perm, inv = moe.route(expert_ids, experts)
    counts = torch.diff(offs, prepend=offs.new_zeros(1))
    counts_all = torch.empty((world, experts), dtype=torch.int32, device=dev)
    dist.all_gather_into_tensor(counts_all, counts, group=buffers.group)
    dst_rank, dst_row, src_rank, src_row, offs_local = exchange_plan(offs, perm, inv, counts_all, rank, e_local)

    stream = torch.cuda.current_stream(dev).cuda_stream
    status = _op.workspace(dev)
    es = x.element_size()
    with torch.cuda.device(dev):
        rc = lib.gmm_scatter_rows_to_peers(x.data_ptr(), x.size(0), x.size(1) * es, x.stride(0) * es, perm.data_ptr(),
                                           topk, dst_rank.data_ptr(), dst_row.data_ptr(), buffers.rows_ptrs.data_ptr(),
                                           world, buffers.rows.stride(0) * es, buffers.capacity, perm.numel(),
                                           status.data_ptr(), stream)
        if rc != 0:
            raise RuntimeError(_lib.error_message(lib, rc))
    buffers.fence()  # every rank's rows have arrived everywhere

    hidden_act = moe.gated_up_projection(buffers.rows, gate_up_local, offs_local)
    forward_into(hidden_act, down_local, offs_local, buffers.result)
    buffers.fence()  # every rank's results are complete

    n_tokens = x.size(0)
    out_dtype = out_dtype or x.dtype
    out = torch.empty((n_tokens, buffers.hidden), dtype=out_dtype, device=dev)
    w_ptr = None
    if weights is not None:
        weights = weights.reshape(-1).to(torch.float32).contiguous()
        w_ptr = weights.data_ptr()
    with torch.cuda.device(dev):
        rc = lib.gmm_combine_rows_from_peers(buffers.result_ptrs.data_ptr(), world, _op._DTYPES[buffers.result.dtype],
                                             buffers.result.stride(0), buffers.capacity, src_rank.data_ptr(),
                                             src_row.data_ptr(), w_ptr, topk, n_tokens, buffers.hidden, out.data_ptr(),
                                             _op._DTYPES[out_dtype], out.stride(0), status.data_ptr(), stream)
        if rc != 0:
            raise RuntimeError(_lib.error_message(lib, rc))
    return out
