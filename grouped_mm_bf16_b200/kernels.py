"""Kernel-level entry points under the module name the reference uses.

``from grouped_mm_bf16.kernels import grouped_mm_2d3d, grouped_mm_2d3d_backward`` style imports
(the eight names grouped_mm_bf16/api.py:8-17 takes from the reference's ``kernels.py``) keep
working: forward functions write into a pre-allocated ``out``, backward functions into
pre-allocated ``grad_a`` / ``grad_b`` (either may be ``None``), and all return ``None``.
"""

from ._op import grouped_mm_2d2d, grouped_mm_2d3d, grouped_mm_3d2d, grouped_mm_3d3d
from .api import (grouped_mm_2d2d_backward, grouped_mm_2d3d_backward, grouped_mm_3d2d_backward,
                  grouped_mm_3d3d_backward)

__all__ = [
    "grouped_mm_3d3d", "grouped_mm_2d2d", "grouped_mm_2d3d", "grouped_mm_3d2d",
    "grouped_mm_3d3d_backward", "grouped_mm_2d2d_backward", "grouped_mm_2d3d_backward", "grouped_mm_3d2d_backward",
]
