"""The C-ABI library without a GPU: it builds, loads, exports every declared symbol and
rejects bad arguments with the documented codes before touching the device."""
import ctypes as C
import re
from pathlib import Path

import pytest

from workloadsuite_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    return _lib.load()


def test_header_symbols_all_exported(lib):
    header = (ROOT / "include" / "ssd_b200.h").read_text()
    declared = set(re.findall(r"\b(ssd_b200_\w+)\s*\(", header))
    assert declared, "no declarations found in the header"
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_struct_layout_matches_header():
    # 14 pointer/size_t fields, 12 int32, 7 x 3 int64
    assert C.sizeof(_lib.SsdArgs) == 14 * 8 + 12 * 4 + 21 * 8
    assert _lib.SsdArgs.batch.offset == 96
    assert _lib.SsdArgs.x_stride.offset == 144


def _args(**kw):
    a = _lib.SsdArgs()
    a.batch, a.seqlen, a.nheads, a.headdim, a.dstate, a.ngroups, a.chunk = 2, 128, 4, 64, 16, 2, 64
    a.dtype = _lib.DTYPE_F32
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_error_codes_for_bad_arguments(lib):
    assert lib.ssd_b200_forward(None, None) == -1
    assert lib.ssd_b200_forward(C.byref(_args(ngroups=3)), None) == -2          # heads % groups (model_ref.py:37-38)
    assert lib.ssd_b200_forward(C.byref(_args(seqlen=100)), None) == -3         # seq % chunk (model_ref.py:106)
    assert lib.ssd_b200_forward(C.byref(_args(dtype=7)), None) == -4
    assert lib.ssd_b200_forward(C.byref(_args()), None) == -1                   # pointers missing
    assert lib.ssd_b200_forward(C.byref(_args(batch=0)), None) == -2
    for code in range(-8, 1):
        assert lib.ssd_b200_strerror(code)


def test_kernel_choice_and_workspace_queries(lib):
    a = _args()
    assert lib.ssd_b200_kernel_name(C.byref(a)) == b"scan_f32"                 # fp32 -> CUDA-core scan
    assert lib.ssd_b200_kernel_name(C.byref(_args(seqlen=100))) == b"invalid"
    a = _args(nsegments=2, seqlen=256)
    units, np_ = 2 * 4, 16 * 64
    assert lib.ssd_b200_workspace_bytes(C.byref(a)) >= units * 2 * (np_ + 1) * 4
    assert lib.ssd_b200_workspace_bytes(C.byref(_args(nsegments=1))) == 0
    assert lib.ssd_b200_host_scratch_bytes(C.byref(_args())) > 0
    assert lib.ssd_b200_fold_states(None, 0, None, 0, None, None, 2, 1, 4, 4, None) == -1


def test_python_api_has_no_cpu_path():
    import torch

    from workloadsuite_b200 import ssd_forward

    X = torch.zeros(1, 64, 2, 64)
    A = torch.zeros(1, 64, 2)
    B = torch.zeros(1, 64, 1, 16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ssd_forward(X, A, B, B, 64)
