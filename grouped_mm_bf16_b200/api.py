"""Public operator: ``grouped_mm(mat_a, mat_b, offs=None, bias=None, out_dtype=None)``.

Same contract as the reference's ``grouped_mm_bf16.grouped_mm`` (grouped_mm_bf16/api.py:275-287),
which mirrors ``torch._grouped_mm``: argument checks in the reference's order and with its
messages (api.py:61-122), output shape and 16-byte padded leading stride (api.py:125-163), the
early-outs for empty outputs and K == 0 (api.py:188-212), GPU-only, ``bias`` rejected. The
arithmetic is done by the CUDA library behind ``_op`` instead of Triton kernels.

Two deliberate differences:
  * ``out_dtype=torch.float32`` is accepted for 16-bit inputs (the reference raises for any
    ``out_dtype != mat_a.dtype``, api.py:54-58); every other mismatch raises the same error.
  * 16-byte alignment decides which kernel runs rather than whether the call is accepted,
    because the reference accepts odd K and N (tests/test_grouped_mm.py:378, 421). Setting
    ``GROUPED_MM_B200_STRICT_ALIGN=1`` turns misalignment into an error instead.

Backward is expressed with the same forward kernels on transposed views (the reference has
seven separate kernels for it, kernels.py:720-1090).
"""

from __future__ import annotations

import os
from typing import Optional, Sequence, Tuple

import torch

from . import _op

_FLOAT_DTYPES = (torch.bfloat16, torch.float16, torch.float32)
MAX_GROUPS = 1024


def is_row_major(mat: torch.Tensor) -> bool:
    """True for a row-major matrix (last dim contiguous), False for column-major, else raises.

    Same rule as the reference (api.py:31-51): only the last two dimensions are inspected and the
    leading stride may exceed the dense size.
    """
    if mat.dim() not in (2, 3):
        raise RuntimeError(f"mat must be 2D or 3D, got dim={mat.dim()}")
    rows, cols = mat.size(-2), mat.size(-1)
    s_row, s_col = mat.stride(-2), mat.stride(-1)
    if s_col == 1 and s_row >= max(1, cols):
        return True
    if s_row == 1 and s_col >= max(1, rows):
        return False
    raise RuntimeError(
        f"Invalid strides/sizes, got {tuple(mat.stride())} for strides and {tuple(mat.size())} for sizes"
    )


def _resolve_out_dtype(mat_a: torch.Tensor, out_dtype: Optional[torch.dtype]) -> torch.dtype:
    if out_dtype is None or out_dtype == mat_a.dtype:
        return mat_a.dtype
    if out_dtype == torch.float32 and mat_a.dtype in (torch.bfloat16, torch.float16):
        return torch.float32
    raise RuntimeError("Grouped gemm output dtype must match `mat_a` dtype")


def _check_strict_alignment(name: str, mat: torch.Tensor) -> None:
    esize = mat.element_size()
    lead = mat.stride(-2) if mat.stride(-1) == 1 else mat.stride(-1)
    if mat.data_ptr() % 16 != 0 or (lead * esize) % 16 != 0:
        raise RuntimeError(f"{name}: strides should be multiple of 16 bytes")


def validate_inputs(mat_a, mat_b, offs, bias, out_dtype) -> Tuple[bool, bool, torch.dtype]:
    """Checks the arguments; returns (a_is_2d, b_is_2d, resolved output dtype)."""
    for name, mat in (("mat_a", mat_a), ("mat_b", mat_b)):
        if mat.dtype not in _FLOAT_DTYPES:
            raise RuntimeError(f"Expected {name} to be Float32, BFloat16 or Float16 matrix, got {mat.dtype}")
    if mat_a.dim() not in (2, 3):
        raise RuntimeError("mat_a has to be 2 or 3d")
    if mat_b.dim() not in (2, 3):
        raise RuntimeError("mat_b has to be 2 or 3d")
    if mat_a.dtype != mat_b.dtype:
        raise RuntimeError("mat_a and mat_b must have the same dtype")

    a_is_2d, b_is_2d = mat_a.dim() == 2, mat_b.dim() == 2
    k_of_b = mat_b.size(0) if (a_is_2d and b_is_2d) else mat_b.size(-2)
    if mat_a.size(-1) != k_of_b:
        raise RuntimeError("contraction dimension of mat_a and mat_b must match")

    if not (mat_a.is_cuda and mat_b.is_cuda):
        raise RuntimeError("grouped_mm_bf16 is GPU-only (CUDA/HIP); CPU tensors are not supported")
    if mat_a.device != mat_b.device:
        raise RuntimeError("mat_a and mat_b must be on the same device")

    is_row_major(mat_a)
    is_row_major(mat_b)

    needs_offs = a_is_2d or b_is_2d
    if (offs is not None) != needs_offs:
        raise RuntimeError("Have to provide offsets if there is a 2d matrix, or no offset if both matrices are 3d")
    if offs is not None:
        if not offs.is_cuda:
            raise RuntimeError("offs must be a CUDA/HIP tensor (CPU offs are not supported)")
        if offs.device != mat_a.device:
            raise RuntimeError("offs must be on the same device as inputs")
        if offs.dim() != 1:
            raise RuntimeError("offs has to be 1D")
        if offs.dtype != torch.int32:
            raise RuntimeError("Offsets have to be int32")
        if offs.numel() >= MAX_GROUPS:
            raise RuntimeError("Can't process more than 1024 groups")
    if bias is not None:
        raise RuntimeError("Bias not supported yet")

    resolved = _resolve_out_dtype(mat_a, out_dtype)
    if os.environ.get("GROUPED_MM_B200_STRICT_ALIGN", "0") == "1":
        _check_strict_alignment("mat_a", mat_a)
        _check_strict_alignment("mat_b", mat_b)
    return a_is_2d, b_is_2d, resolved


def output_geometry(a_shape: Sequence[int], b_shape: Sequence[int], n_groups: Optional[int],
                    elem_size: int) -> Tuple[Tuple[int, ...], Tuple[int, ...]]:
    """Output size and strides for the four shape forms (reference: api.py:134-163).

    The last-dimension stride is padded up to a multiple of 16 bytes, as PyTorch's CUDA
    ``_grouped_mm`` does, so a 2-D result has strides (N_pad, 1) and a 3-D one (M*N_pad, N_pad, 1).
    """
    a_is_2d, b_is_2d = len(a_shape) == 2, len(b_shape) == 2
    if a_is_2d and b_is_2d:
        size = (n_groups, a_shape[0], b_shape[1])
    elif a_is_2d:
        if n_groups != b_shape[0]:
            raise RuntimeError("matrix batch sizes have to match")
        size = (a_shape[0], b_shape[-1])
    elif b_is_2d:
        if n_groups != a_shape[0]:
            raise RuntimeError("matrix batch sizes have to match")
        size = (a_shape[1], b_shape[1])
    else:
        if a_shape[0] != b_shape[0]:
            raise RuntimeError("batched dimension has to match")
        size = (a_shape[0], a_shape[1], b_shape[-1])
    align = 16 // elem_size
    padded = -(-size[-1] // align) * align
    strides = (padded, 1) if len(size) == 2 else (size[1] * padded, padded, 1)
    return tuple(size), strides


def create_output(mat_a, mat_b, offs, out_dtype: torch.dtype) -> torch.Tensor:
    esize = out_dtype.itemsize
    size, strides = output_geometry(tuple(mat_a.shape), tuple(mat_b.shape),
                                    None if offs is None else offs.size(0), esize)
    return torch.empty_strided(size, strides, device=mat_a.device, dtype=out_dtype)


def forward_into(mat_a, mat_b, offs, out) -> None:
    """Dispatches to the kernel-level function of the shape form; zero-fills when K == 0."""
    if out.numel() == 0:
        return
    if mat_a.size(-1) == 0:
        out.zero_()
        return
    a_is_2d, b_is_2d = mat_a.dim() == 2, mat_b.dim() == 2
    if not a_is_2d and not b_is_2d:
        _op.grouped_mm_3d3d(mat_a, mat_b, out)
    elif a_is_2d and b_is_2d:
        _op.grouped_mm_2d2d(mat_a, mat_b, offs, out)
    elif a_is_2d:
        _op.grouped_mm_2d3d(mat_a, mat_b, offs, out)
    else:
        _op.grouped_mm_3d2d(mat_a, mat_b, offs, out)


def _stride_valid(t: torch.Tensor) -> torch.Tensor:
    try:
        is_row_major(t)
        return t
    except RuntimeError:
        return t.contiguous()


def _grad_operand(grad_out: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """``grad_out`` in a layout and dtype the forward kernels take as an operand."""
    g = _stride_valid(grad_out)
    return g if g.dtype == like.dtype else g.to(like.dtype)


# Kernel-level backward functions with the reference's names and signatures
# (grouped_mm_bf16/kernels.py:1093, 1155, 1264, 1332): ``grad_a`` / ``grad_b`` are pre-allocated (or
# None when not needed) and fully written, zeros included. Each gradient is one forward call on
# transposed views, so the reference's fp32 scratch buffers and atomics (kernels.py:1232, 1303, 986)
# have no counterpart.


def grouped_mm_3d3d_backward(mat_a, mat_b, grad_out, grad_a, grad_b) -> None:
    """C[g] = A[g] B[g]:  dA[g] = dC[g] B[g]^T,  dB[g] = A[g]^T dC[g]."""
    g = _grad_operand(grad_out, mat_a)
    if grad_a is not None:
        forward_into(g, mat_b.transpose(-2, -1), None, grad_a)
    if grad_b is not None:
        forward_into(mat_a.transpose(-2, -1), g, None, grad_b)


def grouped_mm_2d3d_backward(mat_a, mat_b, offs, grad_out, grad_a, grad_b) -> None:
    """C[rows_g] = A[rows_g] B[g]:  dA[rows_g] = dC[rows_g] B[g]^T (2D x 3D), dB[g] = A[rows_g]^T dC[rows_g]
    (2D x 2D; empty groups give zeros). Rows past offs[-1] belong to no group: their gradient is zero."""
    g = _grad_operand(grad_out, mat_a)
    if grad_a is not None:
        _op.zero_past_offsets(grad_a, 0, offs)
        forward_into(g, mat_b.transpose(-2, -1), offs, grad_a)
    if grad_b is not None:
        forward_into(mat_a.transpose(-2, -1), g, offs, grad_b)


def grouped_mm_2d2d_backward(mat_a, mat_b, offs, grad_out, grad_a, grad_b) -> None:
    """C[g] = A[:,ks:ke] B[ks:ke,:]:  dA[:,ks:ke] = dC[g] B[ks:ke,:]^T (3D x 2D),
    dB[ks:ke,:] = A[:,ks:ke]^T dC[g] (2D x 3D). Indices past offs[-1] get zero gradient."""
    g = _grad_operand(grad_out, mat_a)
    if grad_a is not None:
        _op.zero_past_offsets(grad_a, 1, offs)
        forward_into(g, mat_b.transpose(-2, -1), offs, grad_a)
    if grad_b is not None:
        _op.zero_past_offsets(grad_b, 0, offs)
        forward_into(mat_a.transpose(-2, -1), g, offs, grad_b)


def grouped_mm_3d2d_backward(mat_a, mat_b, offs, grad_out, grad_a, grad_b) -> None:
    """C[:,ns:ne] = A[g] B[:,ns:ne]:  dA[g] = dC[:,ns:ne] B[:,ns:ne]^T (2D x 2D),
    dB[:,ns:ne] = A[g]^T dC[:,ns:ne] (3D x 2D). Columns past offs[-1] get zero gradient."""
    if mat_a.size(0) != offs.numel():
        raise RuntimeError("matrix batch sizes have to match")
    g = _grad_operand(grad_out, mat_a)
    if grad_a is not None:
        forward_into(g, mat_b.transpose(-2, -1), offs, grad_a)
    if grad_b is not None:
        _op.zero_past_offsets(grad_b, 1, offs)
        forward_into(mat_a.transpose(-2, -1), g, offs, grad_b)


class _GroupedMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mat_a, mat_b, offs, bias, out_dtype):  # type: ignore[override]
        a_is_2d, b_is_2d, resolved = validate_inputs(mat_a, mat_b, offs, bias, out_dtype)
        out = create_output(mat_a, mat_b, offs, resolved)
        ctx.forms = (a_is_2d, b_is_2d)
        ctx.has_offs = offs is not None
        ctx.save_for_backward(mat_a, mat_b, *([offs] if offs is not None else []))
        forward_into(mat_a, mat_b, offs, out)
        return out

    @staticmethod
    def backward(ctx, grad_out):  # type: ignore[override]
        saved = ctx.saved_tensors
        mat_a, mat_b = saved[0], saved[1]
        offs = saved[2] if ctx.has_offs else None
        need_a, need_b = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if grad_out.numel() == 0 or mat_a.size(-1) == 0:
            return (torch.zeros_like(mat_a) if need_a else None, torch.zeros_like(mat_b) if need_b else None,
                    None, None, None)
        a_is_2d, b_is_2d = ctx.forms
        grad_a = torch.empty_like(mat_a) if need_a else None
        grad_b = torch.empty_like(mat_b) if need_b else None
        if not a_is_2d and not b_is_2d:
            grouped_mm_3d3d_backward(mat_a, mat_b, grad_out, grad_a, grad_b)
        elif a_is_2d and not b_is_2d:
            grouped_mm_2d3d_backward(mat_a, mat_b, offs, grad_out, grad_a, grad_b)
        elif a_is_2d and b_is_2d:
            grouped_mm_2d2d_backward(mat_a, mat_b, offs, grad_out, grad_a, grad_b)
        else:
            grouped_mm_3d2d_backward(mat_a, mat_b, offs, grad_out, grad_a, grad_b)
        return grad_a, grad_b, None, None, None


def grouped_mm(
    mat_a: torch.Tensor,
    mat_b: torch.Tensor,
    offs: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """Grouped matrix multiply with ``torch.nn.functional.grouped_mm`` semantics, on B200.

    Shape forms (``offs`` = int32 end indices along the ragged dimension):
      * 3D x 3D: ``[G,M,K] @ [G,K,N] -> [G,M,N]`` (no ``offs``)
      * 2D x 3D: ``[M_total,K] @ [G,K,N] -> [M_total,N]``, rows grouped by ``offs``
      * 3D x 2D: ``[G,M,K] @ [K,N_total] -> [M,N_total]``, columns grouped by ``offs``
      * 2D x 2D: ``[M,K_total] @ [K_total,N] -> [G,M,N]``, contraction grouped by ``offs``
    """
    return _GroupedMM.apply(mat_a, mat_b, offs, bias, out_dtype)
