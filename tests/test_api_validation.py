"""Argument rules of grouped_mm that can be checked without a GPU.

The reference checks, in order: dtypes, ranks, dtype equality, contraction match, then
"GPU-only" (grouped_mm_bf16/api.py:68-96). CPU tensors therefore reach every check before the
GPU-only one; the later checks (offs, bias, out_dtype) are covered by the GPU tests.
"""

import pytest
import torch

from grouped_mm_bf16_b200 import grouped_mm
from grouped_mm_bf16_b200.api import _resolve_out_dtype, is_row_major, output_geometry


def test_drop_in_import_name():
    import grouped_mm_bf16
    from grouped_mm_bf16.kernels import grouped_mm_2d2d, grouped_mm_2d3d, grouped_mm_3d2d, grouped_mm_3d3d  # noqa: F401

    assert grouped_mm_bf16.grouped_mm is grouped_mm


def test_rejects_integer_dtype():
    with pytest.raises(RuntimeError, match="Expected mat_a to be Float32, BFloat16 or Float16 matrix"):
        grouped_mm(torch.zeros(4, 4, dtype=torch.int32), torch.zeros(4, 4))
    with pytest.raises(RuntimeError, match="Expected mat_b to be Float32, BFloat16 or Float16 matrix"):
        grouped_mm(torch.zeros(4, 4), torch.zeros(4, 4, dtype=torch.float64))


def test_rejects_bad_rank():
    with pytest.raises(RuntimeError, match="mat_a has to be 2 or 3d"):
        grouped_mm(torch.zeros(4), torch.zeros(4, 4))
    with pytest.raises(RuntimeError, match="mat_b has to be 2 or 3d"):
        grouped_mm(torch.zeros(4, 4), torch.zeros(1, 1, 4, 4))


def test_rejects_mixed_dtypes_and_contraction_mismatch():
    with pytest.raises(RuntimeError, match="must have the same dtype"):
        grouped_mm(torch.zeros(4, 4), torch.zeros(4, 4).bfloat16())
    with pytest.raises(RuntimeError, match="contraction dimension"):
        grouped_mm(torch.zeros(4, 5), torch.zeros(2, 4, 4))
    with pytest.raises(RuntimeError, match="contraction dimension"):
        grouped_mm(torch.zeros(4, 5), torch.zeros(4, 5))


def test_cpu_tensors_are_rejected_after_shape_checks():
    with pytest.raises(RuntimeError, match="GPU-only"):
        grouped_mm(torch.zeros(2, 4, 8).bfloat16(), torch.zeros(2, 8, 4).bfloat16())


def test_row_and_column_major_rule():
    assert is_row_major(torch.zeros(4, 8)) is True
    assert is_row_major(torch.zeros(8, 4).t()) is False
    assert is_row_major(torch.zeros(4, 16)[:, :8]) is True  # padded leading stride
    with pytest.raises(RuntimeError, match="Invalid strides/sizes"):
        is_row_major(torch.zeros(4, 16)[:, ::2])


def test_out_dtype_rule():
    a = torch.zeros(2, 2).bfloat16()
    assert _resolve_out_dtype(a, None) == torch.bfloat16
    assert _resolve_out_dtype(a, torch.bfloat16) == torch.bfloat16
    assert _resolve_out_dtype(a, torch.float32) == torch.float32  # superset of the reference
    with pytest.raises(RuntimeError, match="output dtype must match"):
        _resolve_out_dtype(a, torch.float16)
    with pytest.raises(RuntimeError, match="output dtype must match"):
        _resolve_out_dtype(torch.zeros(2, 2), torch.bfloat16)


def test_output_geometry_pads_leading_stride_to_16_bytes():
    # 2D x 3D, bf16: N = 29 pads to 32 elements
    assert output_geometry((32, 33), (6, 33, 29), 6, 2) == ((32, 29), (32, 1))
    # 3D x 3D, fp32: N = 23 pads to 24
    assert output_geometry((3, 17, 19), (3, 19, 23), None, 4) == ((3, 17, 23), (17 * 24, 24, 1))
    # 2D x 2D
    assert output_geometry((16, 32), (32, 24), 5, 2) == ((5, 16, 24), (16 * 24, 24, 1))
    # 3D x 2D
    assert output_geometry((5, 32, 48), (48, 32), 5, 2) == ((32, 32), (32, 1))
    with pytest.raises(RuntimeError, match="matrix batch sizes have to match"):
        output_geometry((32, 8), (6, 8, 4), 5, 2)
    with pytest.raises(RuntimeError, match="matrix batch sizes have to match"):
        output_geometry((5, 32, 48), (48, 32), 4, 2)
    with pytest.raises(RuntimeError, match="batched dimension has to match"):
        output_geometry((3, 4, 8), (2, 8, 4), None, 2)


def test_kernels_module_has_the_eight_names_the_reference_api_imports():
    """grouped_mm_bf16/api.py:8-17 imports four forward and four backward functions from kernels."""
    import inspect

    from grouped_mm_bf16 import kernels

    for form in ("3d3d", "2d3d", "2d2d", "3d2d"):
        fwd = getattr(kernels, f"grouped_mm_{form}")
        bwd = getattr(kernels, f"grouped_mm_{form}_backward")
        n_fwd, n_bwd = len(inspect.signature(fwd).parameters), len(inspect.signature(bwd).parameters)
        assert (n_fwd, n_bwd) == ((3, 5) if form == "3d3d" else (4, 6))
    a = torch.zeros((4, 8), dtype=torch.bfloat16)
    b = torch.zeros((2, 8, 8), dtype=torch.bfloat16)
    offs = torch.tensor([2, 4], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="GPU-only"):
        kernels.grouped_mm_2d3d_backward(a, b, offs, torch.zeros((4, 8), dtype=torch.bfloat16),
                                         torch.empty_like(a), torch.empty_like(b))
