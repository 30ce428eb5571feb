"""Drop-in import name: ``from grouped_mm_bf16 import grouped_mm`` resolves to the B200 build.

Code written against lostmsu/grouped_mm_bf16 imports ``grouped_mm_bf16``; this shim forwards that
name (and ``grouped_mm_bf16.kernels``) to ``grouped_mm_bf16_b200`` so nothing else has to change.
"""

import sys as _sys

import grouped_mm_bf16_b200 as _impl
from grouped_mm_bf16_b200 import grouped_mm, kernels

_sys.modules[__name__ + ".kernels"] = kernels
__all__ = ["grouped_mm", "kernels"]
__version__ = _impl.__version__
