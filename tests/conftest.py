"""Shared pytest configuration: the ``gpu`` marker, import path, and the in-tree library build."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

REPO_ROOT = Path(__file__).resolve().parents[1]
if str(REPO_ROOT) not in sys.path:
    sys.path.insert(0, str(REPO_ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def built_library():
    """Path of libgrouped_mm_b200.so, compiled first if it is missing or stale (needs nvcc)."""
    from grouped_mm_bf16_b200.build import build_library

    return build_library()


@pytest.fixture(scope="session")
def golden_cases():
    import torch

    return torch.load(REPO_ROOT / "tests" / "golden" / "grouped_mm_golden.pt")["cases"]
