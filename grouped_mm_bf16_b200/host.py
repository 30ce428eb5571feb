"""``grouped_mm`` for operands that live in host memory (expert weights kept off the GPU).

``grouped_mm_host`` computes the 2D x 3D form from pinned host tensors into a pinned host result.
The operator itself is GPU-only, as in the reference (grouped_mm_bf16/api.py:93-94); what this adds
is the transfer schedule around it: the groups are cut into chunks, and for chunk ``c`` the
host-to-device copy of its rows and weights (copy stream 1), the grouped GEMM of chunk ``c-1``
(compute stream) and the device-to-host copy of chunk ``c-2``'s result (copy stream 2) run at the
same time. PCIe is full duplex, so a step costs about max(bytes in, bytes out) / link speed instead
of their sum plus the compute.

Everything is enqueued asynchronously; the function returns after the last copy has been queued,
and the current stream is made to wait for it (``torch.cuda.current_stream().synchronize()`` or an
event on it completes the result).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .api import forward_into, output_geometry

_DEPTH = 5    # device staging slots for rows and results: filling, multiplying, draining, and two of slack
_B_DEPTH = 2  # device staging slots for weights: the ones in use and the ones being uploaded


class _Staging:
    """Per-device staging buffers and streams, grown on demand and reused across calls."""

    def __init__(self, device: torch.device):
        self.device = device
        self.h2d = torch.cuda.Stream(device)
        self.d2h = torch.cuda.Stream(device)
        self.bufs: List[Dict[str, Optional[torch.Tensor]]] = [dict(a=None, c=None) for _ in range(_DEPTH)]
        self.free_evt: List[Optional[torch.cuda.Event]] = [None] * _DEPTH  # slot reusable after this event
        self.b_bufs: List[Optional[torch.Tensor]] = [None] * _B_DEPTH
        self.b_free_evt: List[Optional[torch.cuda.Event]] = [None] * _B_DEPTH  # last GEMM that read the slot

    def take(self, slot: int, key: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        buf = self.bufs[slot][key]
        if buf is None or buf.numel() < numel or buf.dtype != dtype:
            buf = torch.empty(numel, dtype=dtype, device=self.device)
            self.bufs[slot][key] = buf
        return buf[:numel]

    def take_b(self, slot: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        buf = self.b_bufs[slot]
        if buf is None or buf.numel() < numel or buf.dtype != dtype:
            buf = torch.empty(numel, dtype=dtype, device=self.device)
            self.b_bufs[slot] = buf
        return buf[:numel]


_staging: Dict[int, _Staging] = {}


def _chunks(sizes: List[int], row_bytes: int, group_bytes: int, target_bytes: int) -> List[Tuple[int, int]]:
    """Contiguous group ranges [lo, hi) of roughly ``target_bytes`` of input each."""
    out, lo, acc = [], 0, 0
    for g, s in enumerate(sizes):
        acc += s * row_bytes + group_bytes
        if acc >= target_bytes:
            out.append((lo, g + 1))
            lo, acc = g + 1, 0
    if lo < len(sizes):
        out.append((lo, len(sizes)))
    return out


def plan_items(sizes: List[int], starts: List[int], row_bytes: int, group_bytes: int, chunk_bytes: int):
    """The work items of one call, in execution order: ``(lo, hi, r0, r1, new_b)`` = groups [lo, hi), rows
    [r0, r1) of ``mat_a`` / the result, and whether the groups' weights have to be uploaded (False for the
    second and later row pieces of one tall group, which reuse the weights already on the device).

    ``row_bytes`` counts a row's way up and its result's way down. A group whose rows move more than
    ``chunk_bytes`` is cut into row pieces, so that its first results start down the link while its later
    rows are still going up; the other groups are taken in contiguous runs of about ``chunk_bytes``. Tall
    groups go first, tallest first (the download stream has work from early on), then the runs by falling
    size, so that the un-overlapped tail, the last item's multiply and download, is the smallest.
    """
    piece_rows = max(256, (chunk_bytes // max(1, row_bytes)) // 256 * 256)
    tall = [g for g, sz in enumerate(sizes) if sz * row_bytes > chunk_bytes and sz > piece_rows]
    items = []
    for g in sorted(tall, key=lambda g: -sizes[g]):
        for r in range(0, sizes[g], piece_rows):
            items.append((g, g + 1, starts[g] + r, starts[g] + min(sizes[g], r + piece_rows), r == 0))
    runs, lo = [], 0
    for g in tall + [len(sizes)]:  # the short groups between two tall ones, in runs of about chunk_bytes
        if g > lo:
            for a, b in _chunks(sizes[lo:g], row_bytes, group_bytes, chunk_bytes):
                if sum(sizes[lo + a:lo + b]) > 0:
                    runs.append((lo + a, lo + b))
        lo = g + 1
    runs.sort(key=lambda c: -sum(sizes[c[0]:c[1]]))
    for a, b in runs:
        items.append((a, b, starts[a], max(starts[a], starts[b - 1] + sizes[b - 1]), True))
    return items


def grouped_mm_host(mat_a: torch.Tensor, mat_b: torch.Tensor, offs: torch.Tensor, out: Optional[torch.Tensor] = None,
                    device: Optional[torch.device] = None, chunk_bytes: int = 192 << 20) -> torch.Tensor:
    """``out[rows_g] = mat_a[rows_g] @ mat_b[g]`` with host-resident operands.

    ``mat_a`` ``[M_total, K]`` and ``mat_b`` ``[G, K, N]`` are CPU tensors (pinned memory makes the
    copies asynchronous and fast), ``offs`` a CPU int32 tensor of END offsets. Returns a pinned CPU
    tensor ``[M_total, N]`` of ``mat_a``'s dtype (``out`` if given). Rows at or past ``offs[-1]`` are
    left untouched.
    """
    if mat_a.is_cuda or mat_b.is_cuda or offs.is_cuda:
        raise RuntimeError("grouped_mm_host takes host tensors; use grouped_mm for device tensors")
    if mat_a.dim() != 2 or mat_b.dim() != 3 or mat_a.size(1) != mat_b.size(1):
        raise RuntimeError("grouped_mm_host implements the 2D x 3D form: [M_total, K] @ [G, K, N]")
    if offs.dtype != torch.int32 or offs.dim() != 1 or offs.numel() != mat_b.size(0):
        raise RuntimeError("offs has to be a 1D int32 tensor with one END offset per group")
    if not mat_a.is_contiguous() or not mat_b.is_contiguous():
        raise RuntimeError("grouped_mm_host expects contiguous host tensors")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    m_total, k = mat_a.shape
    n_groups, _, n = mat_b.shape
    if out is None:
        out = torch.empty((m_total, n), dtype=mat_a.dtype).pin_memory()
    ends = [max(0, min(int(e), m_total)) for e in offs.tolist()]
    starts = [0] + ends[:-1]
    sizes = [max(0, e - s) for s, e in zip(starts, ends)]
    es = mat_a.element_size()
    st = _staging.setdefault(dev.index, _Staging(dev))
    compute = torch.cuda.current_stream(dev)
    _, out_strides = output_geometry((1, k), (1, k, n), 1, es)  # padded leading stride of a device result
    n_pad = out_strides[0]

    items = plan_items(sizes, starts, (k + n) * es, k * n * es, chunk_bytes)
    # END offsets of every item's groups, rebased to the item's first row, uploaded once.
    rebased: List[int] = []
    for lo, hi, r0, r1, _ in items:
        rebased += [min(max(ends[g], r0), r1) - r0 for g in range(lo, hi)]
    offs_dev = torch.tensor(rebased, dtype=torch.int32).pin_memory().to(dev, non_blocking=True) if rebased else None
    start_evt = torch.cuda.Event()
    start_evt.record(compute)
    st.h2d.wait_event(start_evt)
    st.d2h.wait_event(start_evt)

    cursor, b_slot, b_d = 0, -1, None
    last_d2h = None
    for i, (lo, hi, r0, r1, new_b) in enumerate(items):
        slot = i % _DEPTH
        rows, g = r1 - r0, hi - lo
        with torch.cuda.stream(st.h2d):
            if st.free_evt[slot] is not None:
                st.h2d.wait_event(st.free_evt[slot])  # the slot's previous result has left the device
            a_d = st.take(slot, "a", rows * k, mat_a.dtype).view(rows, k)
            a_d.copy_(mat_a[r0:r1], non_blocking=True)
            if new_b:
                b_slot = (b_slot + 1) % _B_DEPTH
                if st.b_free_evt[b_slot] is not None:
                    st.h2d.wait_event(st.b_free_evt[b_slot])  # the last multiply that read these weights is done
                b_d = st.take_b(b_slot, g * k * n, mat_b.dtype).view(g, k, n)
                b_d.copy_(mat_b[lo:hi], non_blocking=True)
            loaded = torch.cuda.Event()
            loaded.record(st.h2d)
        compute.wait_event(loaded)
        c_d = torch.as_strided(st.take(slot, "c", rows * n_pad, mat_a.dtype), (rows, n), (n_pad, 1))
        forward_into(a_d, b_d, offs_dev[cursor:cursor + g], c_d)
        cursor += g
        done = torch.cuda.Event()
        done.record(compute)
        st.b_free_evt[b_slot] = done
        with torch.cuda.stream(st.d2h):
            st.d2h.wait_event(done)
            out[r0:r1].copy_(c_d, non_blocking=True)
            drained = torch.cuda.Event()
            drained.record(st.d2h)
        st.free_evt[slot] = drained
        last_d2h = drained
    if last_d2h is not None:
        compute.wait_event(last_d2h)
    return out
