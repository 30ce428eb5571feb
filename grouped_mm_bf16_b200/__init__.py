"""B200-native grouped GEMM with ``torch.nn.functional.grouped_mm`` semantics.

``grouped_mm`` is the operator; ``kernels`` exposes the four kernel-level forward functions with
the names and signatures of the reference package's ``kernels.py``. Importing the package does
not load the CUDA library; the first call does, and fails loudly if it has not been built.
"""

from .api import grouped_mm

__all__ = ["grouped_mm"]
__version__ = "0.1.0"
