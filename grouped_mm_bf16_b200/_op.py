"""The four kernel-level forward functions, bound to the C-ABI library.

Mirrors the functions the reference's ``api.py`` imports from ``kernels.py``
(grouped_mm_bf16/api.py:8-17; definitions kernels.py:524, 553, 583, 689): same names, same
arguments, ``out`` pre-allocated by the caller and written in place, ``None`` returned, launch on
the current CUDA stream without any host synchronisation. The work is registered as the torch
custom op ``grouped_mm_b200::forward`` whose CUDA implementation passes raw pointers, sizes and
strides to ``libgrouped_mm_b200.so`` through ctypes.
"""

from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.GMM_BF16, torch.float16: _lib.GMM_F16, torch.float32: _lib.GMM_F32}

_ws_lock = threading.Lock()
_workspaces: dict[int, torch.Tensor] = {}


def workspace(device: torch.device) -> torch.Tensor:
    """Per-device scratch (zero-filled once); its first int32 is the device status word."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None:
        with _ws_lock:
            ws = _workspaces.get(idx)
            if ws is None:
                nbytes = int(_lib.load().gmm_workspace_bytes())
                ws = torch.zeros((nbytes + 3) // 4, dtype=torch.int32, device=torch.device("cuda", idx))
                _workspaces[idx] = ws
    return ws


def _desc(t: torch.Tensor) -> _lib.GmmTensor:
    d = _lib.GmmTensor()
    d.data = t.data_ptr()
    d.dtype = _DTYPES[t.dtype]
    d.ndim = t.dim()
    for i in range(t.dim()):
        d.size[i] = t.size(i)
        d.stride[i] = t.stride(i)
    return d


def _tf32_allowed() -> bool:
    """fp32 operands may be multiplied as TF32 when torch's matmul knob says so, the setting the
    reference passes to its kernels as ALLOW_TF32 (grouped_mm_bf16/kernels.py:185-194). The
    reference reads the knob once per process; here it is read on every call."""
    return bool(torch.backends.cuda.matmul.allow_tf32)


def _flags(dtype: Optional[torch.dtype] = None) -> int:
    flags = _lib.GMM_FLAG_FORCE_GENERIC if os.environ.get("GROUPED_MM_B200_FORCE_GENERIC", "0") == "1" else 0
    if dtype == torch.float32 and _tf32_allowed():
        flags |= _lib.GMM_FLAG_ALLOW_TF32
    return flags


# ---------------------------------------------------------------------------------------------
# Re-laying out operands the TMA path cannot address.
#
# The tensor-core kernels need operands (16-bit, or fp32 when TF32 is allowed) whose rows start on
# 16-byte boundaries, and the ragged dimension must not be the contiguous one. The reference accepts any row- or column-major
# operand with any (odd) K and N, and so does this package: such calls run on the generic FMA
# kernel, which is one to two orders of magnitude slower. For problems large enough to notice, the
# operands are first copied into a layout the tensor-core kernels take (row pitch padded to a
# multiple of 16 bytes, ragged dimension made non-contiguous); the copy costs one pass over A and
# B, the GEMM then runs at tensor-core speed. Values and results are unchanged.

RELAYOUT_MIN_FLOPS = float(os.environ.get("GROUPED_MM_B200_RELAYOUT_MIN_FLOPS", 1.6e9))


def _aligned_rows(t: torch.Tensor) -> bool:
    """Row pitch, batch pitch and base address are multiples of 16 bytes."""
    q = 16 // t.element_size()
    lead = t.stride(-2) if t.stride(-1) == 1 else t.stride(-1)
    if t.data_ptr() % 16 or lead % q:
        return False
    return t.dim() == 2 or t.size(0) <= 1 or (t.stride(0) % q == 0 and t.stride(0) > 0)


def _relayout(t: torch.Tensor, row_major: bool) -> torch.Tensor:
    """Same values and shape; last two dims row-major (or column-major) with a padded pitch."""
    rows, cols = t.size(-2), t.size(-1)
    batch = tuple(t.shape[:-2])
    q = 16 // t.element_size()
    if row_major:
        buf = torch.empty(batch + (rows, -(-cols // q) * q), dtype=t.dtype, device=t.device)
        view = buf[..., :cols]
    else:
        buf = torch.empty(batch + (cols, -(-rows // q) * q), dtype=t.dtype, device=t.device)
        view = buf[..., :rows].transpose(-2, -1)
    view.copy_(t)
    return view


def _fix_operand(t: torch.Tensor, must_be_row_major: Optional[bool]) -> torch.Tensor:
    is_row = t.stride(-1) == 1 and t.stride(-2) >= max(1, t.size(-1))
    if must_be_row_major is None:
        return t if _aligned_rows(t) else _relayout(t, is_row)
    if is_row == must_be_row_major and _aligned_rows(t):
        return t
    return _relayout(t, must_be_row_major)


def tensor_core_layouts(form: int, mat_a: torch.Tensor, mat_b: torch.Tensor):
    """Returns (mat_a, mat_b), re-laid out where needed so that the tensor-core path applies.

    Per form, the ragged dimension must not be contiguous: 2D x 3D needs a row-major A, 3D x 2D a
    column-major B, 2D x 2D a column-major A and a row-major B; 3D x 3D takes either layout.
    """
    if form == _lib.FORM_2D3D:
        return _fix_operand(mat_a, True), _fix_operand(mat_b, None)
    if form == _lib.FORM_3D2D:
        return _fix_operand(mat_a, None), _fix_operand(mat_b, False)
    if form == _lib.FORM_2D2D:
        return _fix_operand(mat_a, False), _fix_operand(mat_b, True)
    return _fix_operand(mat_a, None), _fix_operand(mat_b, None)


def _worth_relayout(form: int, mat_a: torch.Tensor, mat_b: torch.Tensor, out: torch.Tensor) -> bool:
    if os.environ.get("GROUPED_MM_B200_FORCE_GENERIC", "0") == "1":
        return False
    if mat_a.dtype == torch.float32 and not (_tf32_allowed() and out.dtype == torch.float32):
        return False
    if form == _lib.FORM_2D3D:
        flops = 2.0 * mat_a.size(0) * mat_a.size(1) * mat_b.size(2)
    elif form == _lib.FORM_3D3D:
        flops = 2.0 * mat_a.size(0) * mat_a.size(1) * mat_a.size(2) * mat_b.size(2)
    elif form == _lib.FORM_3D2D:
        flops = 2.0 * mat_a.size(1) * mat_a.size(2) * mat_b.size(1)
    else:
        flops = 2.0 * mat_a.size(0) * mat_a.size(1) * mat_b.size(1)
    return flops >= RELAYOUT_MIN_FLOPS


# ---------------------------------------------------------------------------------------------
# Splitting the contraction of the K-ragged form.
#
# A 2D x 2D call has G * ceil(M / 256) * ceil(N / 256) output tiles, however long the groups are: a
# weight gradient of small experts (say M = N = 256, 4 groups, tens of thousands of rows each) would
# keep 4 of the GPU's 74 CTA pairs busy. Such a call is run as G * S groups instead: every group's
# range [ks, ke) is cut into S consecutive pieces (computed on the device from `offs`, no host
# wait), the kernel writes the S partial products to an fp32 scratch tensor, and they are added in a
# fixed order, so results stay run-to-run reproducible. The reference's kernel has the same shortage
# of parallelism (one program per output tile looping over all of K, kernels.py:248-301).

_SM_COUNT: dict[int, int] = {}


def _split_k_factor(mat_a: torch.Tensor, mat_b: torch.Tensor, offs: torch.Tensor) -> int:
    if os.environ.get("GROUPED_MM_B200_SPLIT_K", "1") == "0":
        return 1
    groups, m, k_total, n = offs.numel(), mat_a.size(0), mat_a.size(1), mat_b.size(1)
    if groups == 0 or m == 0 or n == 0:
        return 1
    idx = mat_a.device.index if mat_a.device.index is not None else torch.cuda.current_device()
    sms = _SM_COUNT.get(idx)
    if sms is None:
        sms = _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    units = max(1, sms // 2)
    tiles = groups * (-(-m // 256)) * (-(-n // 256))
    mean_k = k_total // groups
    if 2 * tiles > units or mean_k < 2048:
        return 1
    return max(1, min(-(-units // tiles), mean_k // 1024, (_lib_max_groups() - 1) // groups, 32))


def _lib_max_groups() -> int:
    return 1024  # the library rejects n_groups >= 1024


def _split_offsets(offs: torch.Tensor, k_total: int, splits: int) -> torch.Tensor:
    """END offsets of the G * S pieces: piece s of group g ends at ks + (ke - ks) * (s + 1) // S."""
    ends = offs.long().clamp(0, k_total)
    starts = torch.cat([ends.new_zeros(1), ends[:-1]])
    lens = (ends - starts).clamp_min(0)
    steps = torch.arange(1, splits + 1, device=offs.device)
    return (starts[:, None] + (lens[:, None] * steps) // splits).reshape(-1).to(torch.int32)


def _launch(form: int, mat_a: torch.Tensor, mat_b: torch.Tensor, offs: Optional[torch.Tensor], out: torch.Tensor,
            may_split: bool = True) -> None:
    lib = _lib.load()
    if not (mat_a.is_cuda and mat_b.is_cuda and out.is_cuda):
        raise RuntimeError("grouped_mm_b200 is GPU-only; CPU tensors are not supported")
    if _worth_relayout(form, mat_a, mat_b, out):
        mat_a, mat_b = tensor_core_layouts(form, mat_a, mat_b)
    if may_split and form == _lib.FORM_2D2D and mat_a.dtype != torch.float32:
        splits = _split_k_factor(mat_a, mat_b, offs)
        if splits > 1 and selected_kernel(form, mat_a, mat_b, out) in _lib.TCGEN05_KINDS:
            groups = offs.numel()
            partial = torch.empty((groups * splits, out.size(1), out.size(2)), dtype=torch.float32, device=out.device)
            _launch(form, mat_a, mat_b, _split_offsets(offs, mat_a.size(1), splits), partial, may_split=False)
            parts = partial.view(groups, splits, out.size(1), out.size(2))
            if out.dtype == torch.float32 and out.is_contiguous():
                torch.sum(parts, dim=1, out=out)
            else:
                out.copy_(parts.sum(1))
            return
    if offs is not None:
        offs = offs.contiguous()  # the library reads n_groups consecutive int32 values
    dev = mat_a.device
    # The library launches on the current device: switch only when the tensors live elsewhere.
    switch = dev.index is not None and dev.index != torch.cuda.current_device()
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        ws = workspace(dev)
        launch = _lib.GmmLaunch()
        launch.stream = torch.cuda.current_stream(dev).cuda_stream
        launch.workspace = ws.data_ptr()
        launch.workspace_bytes = ws.numel() * 4
        launch.flags = _flags(mat_a.dtype)
        maps = None
        if form == _lib.FORM_2D2D and offs.numel() > 0:
            # Scratch for the per-group tensor maps of the K-ragged tensor-core kernels: taken from
            # torch's caching allocator per call, so that calls on different streams never share it
            # and the block is not handed out again before this stream has finished with it.
            maps = torch.empty(int(lib.gmm_group_maps_bytes(offs.numel())), dtype=torch.uint8, device=dev)
            launch.group_maps = maps.data_ptr()
            launch.group_maps_bytes = maps.numel()
        a, b, c = _desc(mat_a), _desc(mat_b), _desc(out)
        if form == _lib.FORM_3D3D:
            rc = lib.grouped_mm_3d3d(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), ctypes.byref(launch))
        else:
            fn = (lib.grouped_mm_2d3d if form == _lib.FORM_2D3D else
                  lib.grouped_mm_3d2d if form == _lib.FORM_3D2D else lib.grouped_mm_2d2d)
            rc = fn(ctypes.byref(a), ctypes.byref(b), offs.data_ptr(), offs.numel(), ctypes.byref(c),
                    ctypes.byref(launch))
    finally:
        if switch:
            torch.cuda.set_device(prev)
    if rc != 0:
        raise RuntimeError(_lib.error_message(lib, rc))


@torch.library.custom_op("grouped_mm_b200::forward", mutates_args=("out",), device_types="cuda")
def _forward_op(mat_a: torch.Tensor, mat_b: torch.Tensor, offs: Optional[torch.Tensor], out: torch.Tensor,
                form: int) -> None:
    _launch(form, mat_a, mat_b, offs, out)


@_forward_op.register_fake
def _(mat_a, mat_b, offs, out, form):
    return None


def _dispatch(form: int, mat_a, mat_b, offs, out) -> None:
    """Eager calls go straight to the library; under torch.compile the registered custom op is
    used so that the call is traceable (the op's dispatcher round trip costs ~15 us per call)."""
    if torch.compiler.is_compiling():
        _forward_op(mat_a, mat_b, offs, out, form)
    else:
        _launch(form, mat_a, mat_b, offs, out)


def grouped_mm_3d3d(mat_a: torch.Tensor, mat_b: torch.Tensor, out: torch.Tensor) -> None:
    """out[g] = mat_a[g] @ mat_b[g] (reference: kernels.py:524-550)."""
    _dispatch(_lib.FORM_3D3D, mat_a, mat_b, None, out)


def grouped_mm_2d2d(mat_a: torch.Tensor, mat_b: torch.Tensor, offs: torch.Tensor, out: torch.Tensor) -> None:
    """out[g] = mat_a[:, ks:ke] @ mat_b[ks:ke, :], zeros for an empty range (reference: kernels.py:553-580)."""
    _dispatch(_lib.FORM_2D2D, mat_a, mat_b, offs, out)


def grouped_mm_2d3d(mat_a: torch.Tensor, mat_b: torch.Tensor, offs: torch.Tensor, out: torch.Tensor) -> None:
    """out[rows_g] = mat_a[rows_g] @ mat_b[g] (reference: kernels.py:583-686)."""
    _dispatch(_lib.FORM_2D3D, mat_a, mat_b, offs, out)


def grouped_mm_3d2d(mat_a: torch.Tensor, mat_b: torch.Tensor, offs: torch.Tensor, out: torch.Tensor) -> None:
    """out[:, cols_g] = mat_a[g] @ mat_b[:, cols_g] (reference: kernels.py:689-717)."""
    if mat_a.size(0) != offs.numel():
        raise RuntimeError("matrix batch sizes have to match")
    _dispatch(_lib.FORM_3D2D, mat_a, mat_b, offs, out)


def grouped_mm_2d3d_swiglu(mat_a: torch.Tensor, gate_up: torch.Tensor, offs: torch.Tensor, out: torch.Tensor) -> bool:
    """out[rows_g] = silu(mat_a[rows_g] @ gate_up[g][:, :N]) * (mat_a[rows_g] @ gate_up[g][:, N:]) in one
    kernel. Returns False, having launched nothing, when the operands are not addressable by the
    tensor-core path (the caller then multiplies and activates separately). No counterpart in the reference."""
    lib = _lib.load()
    if not (mat_a.is_cuda and gate_up.is_cuda and out.is_cuda):
        raise RuntimeError("grouped_mm_b200 is GPU-only; CPU tensors are not supported")
    dev = mat_a.device
    offs = offs.contiguous()
    with torch.cuda.device(dev):
        ws = workspace(dev)
        launch = _lib.GmmLaunch()
        launch.stream = torch.cuda.current_stream(dev).cuda_stream
        launch.workspace = ws.data_ptr()
        launch.workspace_bytes = ws.numel() * 4
        launch.flags = _flags(mat_a.dtype)
        a, b, c = _desc(mat_a), _desc(gate_up), _desc(out)
        rc = lib.grouped_mm_2d3d_swiglu(ctypes.byref(a), ctypes.byref(b), offs.data_ptr(), offs.numel(),
                                        ctypes.byref(c), ctypes.byref(launch))
    if rc == _lib.GMM_ERR_NOT_FUSABLE:
        return False
    if rc != 0:
        raise RuntimeError(_lib.error_message(lib, rc))
    return True


def _zero_past_offsets(t: torch.Tensor, dim: int, offs: torch.Tensor) -> None:
    lib = _lib.load()
    if not (t.is_cuda and offs.is_cuda):
        raise RuntimeError("grouped_mm_b200 is GPU-only; CPU tensors are not supported")
    if t.dim() != 2 or t.element_size() not in (2, 4):
        raise RuntimeError("zero_past_offsets takes a 2-D tensor of 2- or 4-byte elements")
    if t.numel() == 0:
        return
    offs = offs.contiguous()
    other = 1 - dim
    with torch.cuda.device(t.device):
        rc = lib.gmm_zero_past_offsets(ctypes.c_void_p(t.data_ptr()), t.element_size(), t.size(dim), t.size(other),
                                       t.stride(dim), t.stride(other), ctypes.c_void_p(offs.data_ptr()),
                                       offs.numel(), ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream))
    if rc != 0:
        raise RuntimeError(_lib.error_message(lib, rc))


@torch.library.custom_op("grouped_mm_b200::zero_past_offsets", mutates_args=("t",), device_types="cuda")
def _zero_past_offsets_op(t: torch.Tensor, dim: int, offs: torch.Tensor) -> None:
    _zero_past_offsets(t, dim, offs)


@_zero_past_offsets_op.register_fake
def _(t, dim, offs):
    return None


def zero_past_offsets(t: torch.Tensor, dim: int, offs: torch.Tensor) -> None:
    """Zero-fills ``t`` (2-D) at indices >= offs[-1] along ``dim``: the part of a ragged output that no
    group owns and the kernels leave untouched. The offset is read on the device (no host wait), and
    nothing is written when it equals the extent. A registered custom op under torch.compile."""
    if torch.compiler.is_compiling():
        _zero_past_offsets_op(t, dim, offs)
    else:
        _zero_past_offsets(t, dim, offs)


def selected_kernel(form: int, mat_a: torch.Tensor, mat_b: torch.Tensor, out: torch.Tensor) -> int:
    """Which kernel a call with these tensors is routed to (0 none, 1 tcgen05 single-CTA, 2 generic,
    3 tcgen05 CTA-pair)."""
    lib = _lib.load()
    a, b, c = _desc(mat_a), _desc(mat_b), _desc(out)
    rc = lib.gmm_select_kernel(form, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), _flags(mat_a.dtype))
    if rc < 0:
        raise RuntimeError(_lib.error_message(lib, rc))
    return rc


def check_status(device: torch.device) -> int:
    """Synchronises the current stream and returns the device status word (0 = no wait gave up)."""
    lib = _lib.load()
    with torch.cuda.device(device):
        ws = workspace(device)
        raw = ctypes.c_int32(0)
        rc = lib.gmm_check_status(ctypes.c_void_p(ws.data_ptr()),
                                  ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream), ctypes.byref(raw))
    if rc not in (0, _lib.GMM_ERR_DEVICE_WAIT):
        raise RuntimeError(_lib.error_message(lib, rc))
    return int(raw.value)
