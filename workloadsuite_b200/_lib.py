"""ctypes binding of ``lib/libssd_b200.so`` (the C ABI of ``include/ssd_b200.h``).

There is no CPU or PyTorch fallback: if the library is missing it is built with
nvcc, and if that is impossible the import of the compute functions fails.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from . import build as _build

ABI_VERSION = 3

SSD_OK = 0
ERRORS = {
    -1: "SSD_ERR_NULL_POINTER", -2: "SSD_ERR_BAD_SHAPE", -3: "SSD_ERR_BAD_CHUNK", -4: "SSD_ERR_UNSUPPORTED",
    -5: "SSD_ERR_WORKSPACE", -6: "SSD_ERR_CUDA", -7: "SSD_ERR_MISALIGNED", -8: "SSD_ERR_TOO_LARGE",
    -9: "SSD_ERR_DEVICE_WAIT",
}
DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
KERNEL_AUTO, KERNEL_SCAN_F32, KERNEL_TCGEN05 = 0, 1, 2
FLAG_STATE_ONLY = 1
FLAG_REUSE_SEGMENTS = 2
FLAG_SEPARATE_EPILOGUE = 4
FLAG_INJECT_LOST_HANDOVER = 8

# every symbol include/ssd_b200.h declares
EXPORTS = (
    "ssd_b200_abi_version", "ssd_b200_strerror", "ssd_b200_workspace_bytes", "ssd_b200_kernel_name",
    "ssd_b200_forward", "ssd_b200_fold_states", "ssd_b200_host_scratch_bytes", "ssd_b200_forward_host",
    "ssd_b200_static_scratch_capacity", "ssd_b200_forward_static_scratch", "ssd_b200_plan",
    "ssd_b200_conv1d_silu", "ssd_b200_dt_prologue",
    "ssd_b200_xchg_create", "ssd_b200_xchg_connect", "ssd_b200_xchg_buffer", "ssd_b200_xchg_all_gather",
    "ssd_b200_xchg_destroy", "ssd_b200_step",
)
XCHG_HANDLE_BYTES = 64


class SsdArgs(C.Structure):
    """Mirror of ``struct SsdArgs`` in ``include/ssd_b200.h``."""

    _fields_ = [
        ("X", C.c_void_p), ("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p), ("dt", C.c_void_p),
        ("initial_state", C.c_void_p), ("Y", C.c_void_p), ("final_state", C.c_void_p),
        ("final_logdecay", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
        ("batch", C.c_int32), ("seqlen", C.c_int32), ("nheads", C.c_int32), ("headdim", C.c_int32),
        ("dstate", C.c_int32), ("ngroups", C.c_int32), ("chunk", C.c_int32), ("dtype", C.c_int32),
        ("kernel", C.c_int32), ("flags", C.c_int32), ("nsegments", C.c_int32), ("wait_limit_ms", C.c_int32),
        ("x_stride", C.c_int64 * 3), ("a_stride", C.c_int64 * 3), ("b_stride", C.c_int64 * 3),
        ("c_stride", C.c_int64 * 3), ("dt_stride", C.c_int64 * 3), ("y_stride", C.c_int64 * 3),
        ("D", C.c_void_p), ("Z", C.c_void_p), ("z_stride", C.c_int64 * 3),
    ]


_LIB = None


def lib_path() -> Path:
    return _build.LIB


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load (building first if needed) the shared library and declare its prototypes."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not path.exists() or not _build.is_current() or os.environ.get("SSD_B200_REBUILD") == "1":
        # missing, or built from other sources than the ones beside it: never run a stale binary
        if not build_if_missing:
            raise RuntimeError(f"{path} is missing or stale; run `python -m workloadsuite_b200.build`")
        _build.build(force=os.environ.get("SSD_B200_REBUILD") == "1")
    lib = C.CDLL(str(path))
    lib.ssd_b200_abi_version.restype = C.c_int
    lib.ssd_b200_strerror.restype = C.c_char_p
    lib.ssd_b200_strerror.argtypes = [C.c_int]
    lib.ssd_b200_workspace_bytes.restype = C.c_size_t
    lib.ssd_b200_workspace_bytes.argtypes = [C.POINTER(SsdArgs)]
    lib.ssd_b200_kernel_name.restype = C.c_char_p
    lib.ssd_b200_kernel_name.argtypes = [C.POINTER(SsdArgs)]
    lib.ssd_b200_forward.restype = C.c_int
    lib.ssd_b200_forward.argtypes = [C.POINTER(SsdArgs), C.c_void_p]
    lib.ssd_b200_fold_states.restype = C.c_int
    lib.ssd_b200_fold_states.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                         C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_void_p]
    lib.ssd_b200_host_scratch_bytes.restype = C.c_size_t
    lib.ssd_b200_host_scratch_bytes.argtypes = [C.POINTER(SsdArgs)]
    lib.ssd_b200_forward_host.restype = C.c_int
    lib.ssd_b200_forward_host.argtypes = [C.POINTER(SsdArgs), C.c_void_p, C.c_size_t]
    lib.ssd_b200_static_scratch_capacity.restype = C.c_size_t
    lib.ssd_b200_static_scratch_capacity.argtypes = []
    lib.ssd_b200_forward_static_scratch.restype = C.c_int
    lib.ssd_b200_forward_static_scratch.argtypes = [C.POINTER(SsdArgs), C.c_void_p]
    lib.ssd_b200_plan.restype = C.c_int
    lib.ssd_b200_plan.argtypes = [C.POINTER(SsdArgs), C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.ssd_b200_conv1d_silu.restype = C.c_int
    lib.ssd_b200_conv1d_silu.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                         C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]
    lib.ssd_b200_dt_prologue.restype = C.c_int
    lib.ssd_b200_dt_prologue.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
    lib.ssd_b200_step.restype = C.c_int
    lib.ssd_b200_step.argtypes = [C.c_void_p] * 9 + [C.c_int32] * 6 + [C.c_void_p]
    lib.ssd_b200_xchg_create.restype = C.c_int
    lib.ssd_b200_xchg_create.argtypes = [C.c_size_t, C.c_int32, C.POINTER(C.c_void_p), C.c_void_p]
    lib.ssd_b200_xchg_connect.restype = C.c_int
    lib.ssd_b200_xchg_connect.argtypes = [C.c_void_p, C.c_void_p, C.c_int32]
    lib.ssd_b200_xchg_buffer.restype = C.c_void_p
    lib.ssd_b200_xchg_buffer.argtypes = [C.c_void_p]
    lib.ssd_b200_xchg_all_gather.restype = C.c_int
    lib.ssd_b200_xchg_all_gather.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_int32, C.c_void_p]
    lib.ssd_b200_xchg_destroy.restype = C.c_int
    lib.ssd_b200_xchg_destroy.argtypes = [C.c_void_p]
    got = lib.ssd_b200_abi_version()
    if got != ABI_VERSION:
        raise RuntimeError(f"libssd_b200 ABI version {got}, binding expects {ABI_VERSION}; rebuild the library")
    _LIB = lib
    return lib


def strerror(code: int) -> str:
    return load().ssd_b200_strerror(code).decode()
