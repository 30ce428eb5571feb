"""The C-ABI library: it loads, exports every declared symbol, and routes shapes as documented.

No compute call is made here, so no GPU is needed; gmm_select_kernel only inspects its arguments.
"""

import ctypes
import re
from pathlib import Path

import pytest

from grouped_mm_bf16_b200 import _lib

HEADER = Path(__file__).resolve().parents[1] / "include" / "grouped_mm_b200.h"


@pytest.fixture(scope="module")
def lib(built_library):
    return _lib.load()


def _declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return set(re.findall(r"\b(g(?:mm|rouped_mm)_\w+)\s*\(", text))


def test_every_declared_symbol_is_exported(lib):
    declared = _declared_functions()
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    for name in declared:
        assert getattr(lib, name) is not None


def test_version_and_error_strings(lib):
    assert lib.gmm_abi_version() == 2
    assert lib.gmm_error_string(0) == b"ok"
    assert b"1024 groups" in lib.gmm_error_string(-3)
    assert lib.gmm_workspace_bytes() >= 4


def _tensor(shape, strides, dtype=_lib.GMM_BF16, ptr=0x10000):
    t = _lib.GmmTensor()
    t.data, t.dtype, t.ndim = ptr, dtype, len(shape)
    for i, (s, st) in enumerate(zip(shape, strides)):
        t.size[i], t.stride[i] = s, st
    return t


def _select(lib, form, a, b, c, flags=0):
    return lib.gmm_select_kernel(form, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), flags)


def test_aligned_bf16_shapes_take_the_tcgen05_kernel(lib):
    a = _tensor((32, 64), (64, 1))
    b = _tensor((6, 64, 48), (64 * 48, 48, 1))
    c = _tensor((32, 48), (48, 1))
    assert _select(lib, _lib.FORM_2D3D, a, b, c) == _lib.GMM_KERNEL_TCGEN05
    assert _select(lib, _lib.FORM_2D3D, a, b, c, _lib.GMM_FLAG_FORCE_GENERIC) == _lib.GMM_KERNEL_GENERIC
    bt = _tensor((6, 64, 48), (64 * 48, 1, 64))  # column-major B
    assert _select(lib, _lib.FORM_2D3D, a, bt, c) == _lib.GMM_KERNEL_TCGEN05
    a3 = _tensor((4, 32, 64), (32 * 64, 64, 1))
    b3 = _tensor((4, 64, 48), (64 * 48, 48, 1))
    c3 = _tensor((4, 32, 48), (32 * 48, 48, 1))
    assert _select(lib, _lib.FORM_3D3D, a3, b3, c3) == _lib.GMM_KERNEL_TCGEN05


def test_unaligned_or_fp32_shapes_take_the_generic_kernel(lib):
    a = _tensor((32, 33), (33, 1))
    b = _tensor((6, 33, 29), (33 * 29, 29, 1))
    c = _tensor((32, 29), (32, 1))
    assert _select(lib, _lib.FORM_2D3D, a, b, c) == _lib.GMM_KERNEL_GENERIC
    a = _tensor((32, 64), (64, 1), _lib.GMM_F32)
    b = _tensor((6, 64, 48), (64 * 48, 48, 1), _lib.GMM_F32)
    c = _tensor((32, 48), (48, 1), _lib.GMM_F32)
    assert _select(lib, _lib.FORM_2D3D, a, b, c) == _lib.GMM_KERNEL_GENERIC
    a = _tensor((32, 64), (64, 1), ptr=0x10002)  # base not 16-byte aligned
    b = _tensor((6, 64, 48), (64 * 48, 48, 1))
    c = _tensor((32, 48), (48, 1))
    assert _select(lib, _lib.FORM_2D3D, a, b, c) == _lib.GMM_KERNEL_GENERIC


def test_fp32_takes_the_tcgen05_kernel_only_when_tf32_is_allowed(lib):
    a = _tensor((32, 64), (64, 1), _lib.GMM_F32)
    b = _tensor((6, 64, 48), (64 * 48, 48, 1), _lib.GMM_F32)
    c = _tensor((32, 48), (48, 1), _lib.GMM_F32)
    assert _select(lib, _lib.FORM_2D3D, a, b, c, _lib.GMM_FLAG_ALLOW_TF32) == _lib.GMM_KERNEL_TCGEN05
    assert _select(lib, _lib.FORM_2D3D, a, b, c, 0) == _lib.GMM_KERNEL_GENERIC
    both = _lib.GMM_FLAG_ALLOW_TF32 | _lib.GMM_FLAG_FORCE_GENERIC
    assert _select(lib, _lib.FORM_2D3D, a, b, c, both) == _lib.GMM_KERNEL_GENERIC
    # a 16-bit result of fp32 operands stays on the generic kernel
    c16 = _tensor((32, 48), (48, 1), _lib.GMM_BF16)
    assert _select(lib, _lib.FORM_2D3D, a, b, c16, _lib.GMM_FLAG_ALLOW_TF32) == _lib.GMM_KERNEL_GENERIC
    # rows of fp32 must start on 16-byte boundaries: a pitch of 4 elements is enough, 6 is not
    a4 = _tensor((32, 60), (60, 1), _lib.GMM_F32)
    b4 = _tensor((6, 60, 44), (60 * 44, 44, 1), _lib.GMM_F32)
    c4 = _tensor((32, 44), (44, 1), _lib.GMM_F32)
    assert _select(lib, _lib.FORM_2D3D, a4, b4, c4, _lib.GMM_FLAG_ALLOW_TF32) == _lib.GMM_KERNEL_TCGEN05
    a6 = _tensor((32, 62), (62, 1), _lib.GMM_F32)
    b6 = _tensor((6, 62, 44), (62 * 44, 44, 1), _lib.GMM_F32)
    assert _select(lib, _lib.FORM_2D3D, a6, b6, c4, _lib.GMM_FLAG_ALLOW_TF32) == _lib.GMM_KERNEL_GENERIC
    # tall groups take the CTA-pair kernel, as with 16-bit operands
    at = _tensor((8192, 64), (64, 1), _lib.GMM_F32)
    bt = _tensor((2, 64, 512), (64 * 512, 512, 1), _lib.GMM_F32)
    ct = _tensor((8192, 512), (512, 1), _lib.GMM_F32)
    assert _select(lib, _lib.FORM_2D3D, at, bt, ct, _lib.GMM_FLAG_ALLOW_TF32) == _lib.GMM_KERNEL_TCGEN05_PAIR
    flags = _lib.GMM_FLAG_ALLOW_TF32 | _lib.GMM_FLAG_NO_PAIR
    assert _select(lib, _lib.FORM_2D3D, at, bt, ct, flags) == _lib.GMM_KERNEL_TCGEN05
    # the flag changes nothing for 16-bit operands
    a = _tensor((32, 64), (64, 1))
    b = _tensor((6, 64, 48), (64 * 48, 48, 1))
    c = _tensor((32, 48), (48, 1))
    assert _select(lib, _lib.FORM_2D3D, a, b, c, _lib.GMM_FLAG_ALLOW_TF32) == _lib.GMM_KERNEL_TCGEN05


def test_ragged_dimension_must_not_be_the_contiguous_one(lib):
    # 2D x 3D with column-major A: rows (ragged) are contiguous -> generic
    a = _tensor((32, 64), (1, 32))
    b = _tensor((6, 64, 48), (64 * 48, 48, 1))
    c = _tensor((32, 48), (48, 1))
    assert _select(lib, _lib.FORM_2D3D, a, b, c) == _lib.GMM_KERNEL_GENERIC
    # 2D x 2D: column-major A and row-major B (the weight-gradient layout) -> tcgen05
    a = _tensor((16, 64), (1, 16))
    b = _tensor((64, 24), (24, 1))
    c = _tensor((5, 16, 24), (16 * 24, 24, 1), _lib.GMM_F32)
    assert _select(lib, _lib.FORM_2D2D, a, b, c) == _lib.GMM_KERNEL_TCGEN05
    a = _tensor((16, 64), (64, 1))  # row-major A: K (ragged) contiguous -> generic
    assert _select(lib, _lib.FORM_2D2D, a, b, c) == _lib.GMM_KERNEL_GENERIC
    # 3D x 2D: needs column-major B (K contiguous)
    a3 = _tensor((5, 32, 48), (32 * 48, 48, 1))
    b2 = _tensor((48, 56), (1, 48))
    c2 = _tensor((32, 56), (56, 1))
    assert _select(lib, _lib.FORM_3D2D, a3, b2, c2) == _lib.GMM_KERNEL_TCGEN05
    b2 = _tensor((48, 56), (56, 1))
    assert _select(lib, _lib.FORM_3D2D, a3, b2, c2) == _lib.GMM_KERNEL_GENERIC


def test_argument_errors(lib):
    a = _tensor((32, 64), (64, 1))
    b = _tensor((6, 60, 48), (60 * 48, 48, 1))  # contraction mismatch
    c = _tensor((32, 48), (48, 1))
    assert _select(lib, _lib.FORM_2D3D, a, b, c) == -1
    b = _tensor((6, 64, 48), (64 * 48, 48, 1), dtype=7)
    assert _select(lib, _lib.FORM_2D3D, a, b, c) == -2
    b = _tensor((1024, 64, 48), (64 * 48, 48, 1))
    assert _select(lib, _lib.FORM_2D3D, a, b, c) == -3
    empty = _tensor((0, 48), (48, 1))
    a0 = _tensor((0, 64), (64, 1))
    b = _tensor((6, 64, 48), (64 * 48, 48, 1))
    assert _select(lib, _lib.FORM_2D3D, a0, b, empty) == _lib.GMM_KERNEL_NONE
    # a launch without a workspace is refused before any CUDA call
    launch = _lib.GmmLaunch()
    rc = lib.grouped_mm_2d3d(ctypes.byref(a), ctypes.byref(b), ctypes.c_void_p(0x1000), 6, ctypes.byref(c),
                             ctypes.byref(launch))
    assert rc == -4


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="has not been built"):
        _lib.load()
