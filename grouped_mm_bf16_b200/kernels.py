"""Kernel-level forward entry points under the module name the reference uses.

``from grouped_mm_bf16.kernels import grouped_mm_2d3d`` style imports of forward functions
(grouped_mm_bf16/api.py:8-17 in the reference) keep working; each function writes into a
pre-allocated ``out`` and returns ``None``.
"""

from ._op import grouped_mm_2d2d, grouped_mm_2d3d, grouped_mm_3d2d, grouped_mm_3d3d

__all__ = ["grouped_mm_3d3d", "grouped_mm_2d2d", "grouped_mm_2d3d", "grouped_mm_3d2d"]
