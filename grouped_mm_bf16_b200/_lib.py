"""ctypes binding of libgrouped_mm_b200.so (declared in include/grouped_mm_b200.h).

There is no fallback: if the library is missing or a call fails, a RuntimeError is raised.
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path
from typing import Optional

# GROUPED_MM_B200_LIB points at another build of the library (for example to compare two builds).
LIB_PATH = Path(os.environ.get("GROUPED_MM_B200_LIB") or Path(__file__).resolve().parent / "lib" / "libgrouped_mm_b200.so")

GMM_BF16, GMM_F16, GMM_F32 = 0, 1, 2
GMM_KERNEL_NONE, GMM_KERNEL_TCGEN05, GMM_KERNEL_GENERIC, GMM_KERNEL_TCGEN05_PAIR = 0, 1, 2, 3
TCGEN05_KINDS = (GMM_KERNEL_TCGEN05, GMM_KERNEL_TCGEN05_PAIR)
GMM_FLAG_FORCE_GENERIC = 0x1
GMM_FLAG_FORCE_PAIR = 0x2
GMM_FLAG_NO_PAIR = 0x4
GMM_FLAG_ALLOW_TF32 = 0x8
GMM_ERR_DEVICE_WAIT = -7
GMM_ERR_NOT_FUSABLE = -8
GMM_STATUS_BAD_PEER_INDEX = 0x40000000

FORM_3D3D, FORM_2D3D, FORM_3D2D, FORM_2D2D = 0, 1, 2, 3

# Every symbol include/grouped_mm_b200.h declares.
EXPORTED_SYMBOLS = (
    "gmm_abi_version",
    "gmm_error_string",
    "gmm_last_cuda_error",
    "gmm_workspace_bytes",
    "gmm_group_maps_bytes",
    "grouped_mm_3d3d",
    "grouped_mm_2d2d",
    "grouped_mm_2d3d",
    "grouped_mm_3d2d",
    "grouped_mm_2d3d_swiglu",
    "grouped_mm_2d3d_static_scratch",
    "gmm_zero_past_offsets",
    "gmm_select_kernel",
    "gmm_check_status",
    "gmm_selftest_wait_timeout",
    "gmm_route_workspace_bytes",
    "gmm_route_build",
    "gmm_permute_rows",
    "gmm_combine_rows",
    "gmm_scatter_rows_to_peers",
    "gmm_combine_rows_from_peers",
)


class GmmTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("ndim", ctypes.c_int32),
        ("size", ctypes.c_int64 * 3),
        ("stride", ctypes.c_int64 * 3),
    ]


class GmmLaunch(ctypes.Structure):
    _fields_ = [
        ("stream", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("flags", ctypes.c_uint32),
        ("group_maps", ctypes.c_void_p),
        ("group_maps_bytes", ctypes.c_size_t),
    ]


_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Loads the shared library once and declares the argument types of its entry points."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA library has not been built. Run "
                "`python -m grouped_mm_bf16_b200.build` (needs nvcc). There is no CPU or PyTorch fallback."
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        tp, lp = ctypes.POINTER(GmmTensor), ctypes.POINTER(GmmLaunch)
        lib.gmm_abi_version.restype = ctypes.c_int
        lib.gmm_abi_version.argtypes = []
        lib.gmm_error_string.restype = ctypes.c_char_p
        lib.gmm_error_string.argtypes = [ctypes.c_int]
        lib.gmm_last_cuda_error.restype = ctypes.c_char_p
        lib.gmm_last_cuda_error.argtypes = []
        lib.gmm_workspace_bytes.restype = ctypes.c_size_t
        lib.gmm_workspace_bytes.argtypes = []
        lib.gmm_group_maps_bytes.restype = ctypes.c_size_t
        lib.gmm_group_maps_bytes.argtypes = [ctypes.c_int32]
        lib.grouped_mm_3d3d.restype = ctypes.c_int
        lib.grouped_mm_3d3d.argtypes = [tp, tp, tp, lp]
        for name in ("grouped_mm_2d2d", "grouped_mm_2d3d", "grouped_mm_3d2d", "grouped_mm_2d3d_swiglu"):
            fn = getattr(lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [tp, tp, ctypes.c_void_p, ctypes.c_int32, tp, lp]
        lib.grouped_mm_2d3d_static_scratch.restype = ctypes.c_int
        lib.grouped_mm_2d3d_static_scratch.argtypes = [tp, tp, ctypes.c_void_p, ctypes.c_int32, tp, ctypes.c_void_p,
                                                       ctypes.c_uint32, ctypes.POINTER(ctypes.c_void_p)]
        lib.gmm_zero_past_offsets.restype = ctypes.c_int
        lib.gmm_zero_past_offsets.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64,
                                              ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int32,
                                              ctypes.c_void_p]
        lib.gmm_select_kernel.restype = ctypes.c_int
        lib.gmm_select_kernel.argtypes = [ctypes.c_int32, tp, tp, tp, ctypes.c_uint32]
        lib.gmm_check_status.restype = ctypes.c_int
        lib.gmm_check_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
        lib.gmm_selftest_wait_timeout.restype = ctypes.c_int
        lib.gmm_selftest_wait_timeout.argtypes = [vp, vp, i64]
        lib.gmm_route_workspace_bytes.restype = ctypes.c_size_t
        lib.gmm_route_workspace_bytes.argtypes = [i64, i32]
        lib.gmm_route_build.restype = ctypes.c_int
        lib.gmm_route_build.argtypes = [vp, i64, i32, vp, vp, vp, vp, ctypes.c_size_t, vp]
        lib.gmm_permute_rows.restype = ctypes.c_int
        lib.gmm_permute_rows.argtypes = [vp, i64, i64, i64, vp, i32, vp, i64, i64, vp]
        lib.gmm_combine_rows.restype = ctypes.c_int
        lib.gmm_combine_rows.argtypes = [vp, i32, i64, vp, vp, i32, i64, i32, vp, i32, i64, vp]
        lib.gmm_scatter_rows_to_peers.restype = ctypes.c_int
        lib.gmm_scatter_rows_to_peers.argtypes = [vp, i64, i64, i64, vp, i32, vp, vp, vp, i32, i64, i64, i64, vp, vp]
        lib.gmm_combine_rows_from_peers.restype = ctypes.c_int
        lib.gmm_combine_rows_from_peers.argtypes = [vp, i32, i32, i64, i64, vp, vp, vp, i32, i64, i32, vp, i32, i64,
                                                    vp, vp]
        _lib = lib
        return lib


def error_message(lib: ctypes.CDLL, status: int) -> str:
    msg = lib.gmm_error_string(status).decode()
    detail = lib.gmm_last_cuda_error().decode()
    return f"grouped_mm_b200: {msg}" + (f" [{detail}]" if detail and status == -5 else "")
