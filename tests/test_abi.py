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


def test_step_and_exchange_entry_points_reject_bad_arguments_on_the_host(lib):
    """No device is touched: every call returns before a launch (the pointers are made-up numbers)."""
    P = 0x10000
    step = lambda *a: lib.ssd_b200_step(*a)
    ok_shape = (2, 8, 64, 128, 2, _lib.DTYPE_BF16, None)
    assert step(None, P, P, P, None, None, None, P, P, *ok_shape) == -1                      # x missing
    assert step(P, P, P, P, None, None, None, P, P, 2, 8, 64, 128, 3, _lib.DTYPE_BF16, None) == -2    # heads % groups
    assert step(P, P, P, P, None, None, None, P, P, 2, 8, 32, 128, 2, _lib.DTYPE_BF16, None) == -4    # head dim
    assert step(P, P, P, P, None, None, None, P, P, 2, 8, 64, 100, 2, _lib.DTYPE_BF16, None) == -4    # state size
    assert step(P, P, P, P, None, None, None, P + 4, P, *ok_shape) == -7                     # state alignment
    ctx = C.c_void_p()
    handle = (C.c_ubyte * _lib.XCHG_HANDLE_BYTES)()
    assert lib.ssd_b200_xchg_create(1024, 2, None, handle) == -1
    assert lib.ssd_b200_xchg_create(1024, 0, C.byref(ctx), handle) == -2
    assert lib.ssd_b200_xchg_create(0, 2, C.byref(ctx), handle) == -2
    assert lib.ssd_b200_xchg_buffer(None) is None
    assert lib.ssd_b200_xchg_all_gather(None, P, 1024, None, 0, None) == -2


def test_python_wrappers_refuse_cpu_tensors():
    import torch
    import workloadsuite_b200 as W

    x = torch.zeros(1, 2, 64)
    with pytest.raises(RuntimeError):
        W.ssd_step(x, torch.zeros(1, 2), torch.zeros(1, 1, 16), torch.zeros(1, 1, 16), torch.zeros(1, 2, 16, 64))


def test_misaligned_states_and_bad_wait_limit_are_rejected_on_the_host(lib):
    """The tensor-core kernels move the fp32 states as 16-byte vectors: a state pointer that is only 4-byte aligned
    must come back as an error code (explicit kernel) or take the fp32 scan (automatic choice), never reach a
    kernel.  No device is touched: the pointers are made-up numbers."""
    a = _shape(2, 256, 4, 64, 128, 1, 128, _lib.DTYPE_BF16)
    a.X, a.A, a.B, a.C, a.Y = 0x10000, 0x20000, 0x30000, 0x40000, 0x50000
    assert lib.ssd_b200_kernel_name(C.byref(a)) == b"tcgen05"
    a.initial_state = 0x60004
    assert lib.ssd_b200_kernel_name(C.byref(a)) == b"scan_f32"             # automatic choice avoids the vector path
    a.kernel = _lib.KERNEL_TCGEN05
    assert lib.ssd_b200_forward(C.byref(a), None) == -7                     # SSD_ERR_MISALIGNED
    a.initial_state, a.final_state = 0x60000, 0x70008
    assert lib.ssd_b200_forward(C.byref(a), None) == -7
    b = _shape(2, 256, 4, 64, 128, 1, 128, _lib.DTYPE_BF16)
    b.wait_limit_ms = -1
    assert lib.ssd_b200_forward(C.byref(b), None) == -2
    assert b"wait" in lib.ssd_b200_strerror(-9)


def test_chained_scratch_is_sized_by_hand_over_slots(lib):
    """One launch with sequences handed from CTA to CTA needs one slot per CTA and head of the pair, whatever the
    number of sequences: config 2 fits the 16 MiB of the allocation-free entry point."""
    need = lib.ssd_b200_workspace_bytes(C.byref(_shape(4, 8192, 80, 64, 128, 1, 256, _lib.DTYPE_BF16)))
    assert 2 * 148 * 128 * 64 * 4 <= need < (16 << 20)
    assert need == lib.ssd_b200_workspace_bytes(C.byref(_shape(8, 8192, 80, 64, 128, 1, 256, _lib.DTYPE_BF16)))


def test_python_wrappers_validate_devices_and_out_before_any_pointer_is_used():
    import torch

    from workloadsuite_b200 import ssd

    x = torch.zeros(1, 64, 2, 64)
    other = torch.zeros(1, 64, 2, device="meta")
    with pytest.raises(ValueError, match="share one device"):
        ssd._same_device(x, A=other)
    ssd._same_device(x, A=torch.zeros(1, 64, 2), dt=None)
    with pytest.raises(ValueError, match="shape"):
        ssd._check_out(torch.zeros(1, 64, 2, 32), x)
    with pytest.raises(ValueError, match="shape"):
        ssd._check_out(torch.zeros(1, 64, 2, 64, dtype=torch.float16), x)
    with pytest.raises(ValueError, match="innermost"):
        ssd._check_out(torch.zeros(1, 64, 64, 2).transpose(2, 3), x)
    ssd._check_out(torch.zeros(1, 64, 4, 64)[:, :, ::2], x)                   # a strided view of rows is fine
    # the reference block's X: sequence-contiguous, channel-strided (model_ref.py:83-89) -> copied into rows once
    xt = torch.zeros(1, 2 * 64, 64).transpose(1, 2).unflatten(-1, (2, 64))
    assert xt.stride(-1) != 1 and ssd._rows_contiguous(xt).stride(-1) == 1
    assert ssd._rows_contiguous(x) is x
    with pytest.raises(ValueError, match="share one device"):
        ssd._check(x, other, torch.zeros(1, 64, 1, 16), torch.zeros(1, 64, 1, 16), None, None)


def test_python_api_has_no_cpu_path():
    import torch

    from workloadsuite_b200 import ssd_forward

    X = torch.zeros(1, 64, 2, 64)
    A = torch.zeros(1, 64, 2)
    B = torch.zeros(1, 64, 1, 16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ssd_forward(X, A, B, B, 64)


def _shape(b, s, h, p, n, g, chunk, dtype):
    a = _lib.SsdArgs()
    a.batch, a.seqlen, a.nheads, a.headdim, a.dstate, a.ngroups, a.chunk = b, s, h, p, n, g, chunk
    a.dtype = dtype
    a.x_stride = (C.c_int64 * 3)(s * h * p, h * p, p)
    a.y_stride = (C.c_int64 * 3)(s * h * p, h * p, p)
    a.a_stride = (C.c_int64 * 3)(s * h, h, 1)
    a.b_stride = (C.c_int64 * 3)(s * g * n, g * n, n)
    a.c_stride = (C.c_int64 * 3)(s * g * n, g * n, n)
    return a


def _plan(lib, a):
    k, nseg, launches = C.c_int32(), C.c_int32(), C.c_int32()
    assert lib.ssd_b200_plan(C.byref(a), C.byref(k), C.byref(nseg), C.byref(launches)) == 0
    return k.value, nseg.value, launches.value


def test_plan_of_the_benchmark_configurations(lib):
    """How the host logic schedules the baseline's configurations (no device involved): kernel family, cuts per
    sequence and kernel launches."""
    TC, SCAN = 2, 1
    # config 2: 160 head pairs for 148 SMs -> tiles dealt out evenly inside one launch, state handed on through scratch
    k, nseg, launches = _plan(lib, _shape(4, 8192, 80, 64, 128, 1, 256, _lib.DTYPE_BF16))
    assert (k, launches) == (TC, 1) and nseg == 2
    assert lib.ssd_b200_workspace_bytes(C.byref(_shape(4, 8192, 80, 64, 128, 1, 256, _lib.DTYPE_BF16))) > 0
    # its head shards at 2 and 8 GPUs (80 and 20 head pairs for 148 SMs): the same even deal in one launch, each CTA
    # first scanning the last piece of its range from zero so that the pieces after it need not wait ("look-back")
    for heads in (40, 10):
        k, nseg, launches = _plan(lib, _shape(4, 8192, heads, 64, 128, 1, 256, _lib.DTYPE_BF16))
        assert k == TC and nseg > 1 and launches == 1
    # config 3 (one long sequence, 16 pairs): look-back too; its state-only run and the run that reuses the segment
    # states (the two halves of a sequence-sharded forward) stay two passes and a fold
    k, nseg, launches = _plan(lib, _shape(1, 131072, 32, 64, 128, 1, 256, _lib.DTYPE_BF16))
    assert k == TC and nseg > 1 and launches == 1
    so = _shape(1, 131072, 32, 64, 128, 1, 256, _lib.DTYPE_BF16)
    so.flags = _lib.FLAG_STATE_ONLY
    k, nseg, launches = _plan(lib, so)
    assert k == TC and nseg > 4 and launches == 2
    so.flags = _lib.FLAG_REUSE_SEGMENTS
    assert _plan(lib, so) == (TC, nseg, 2)
    # 96 pairs of only 16 tiles (config 1): the state-only scans and the start-ups would eat the gain: whole sequences
    assert _plan(lib, _shape(8, 2048, 24, 64, 128, 1, 256, _lib.DTYPE_BF16))[1:] == (1, 1)
    assert _plan(lib, _shape(8, 8192, 24, 64, 128, 1, 256, _lib.DTYPE_BF16))[1:] == (2, 1)
    # config 4 (6144 short sequences): whole sequences, one launch
    assert _plan(lib, _shape(256, 512, 48, 64, 64, 8, 128, _lib.DTYPE_BF16)) == (TC, 1, 1)
    # config 0 is fp32: the CUDA-core recurrence
    assert _plan(lib, _shape(16, 128, 8, 64, 16, 8, 64, _lib.DTYPE_F32))[0] == SCAN
    # odd heads per group cannot pair up: still the tensor-core family (one head per CTA)
    assert _plan(lib, _shape(2, 512, 3, 64, 128, 3, 128, _lib.DTYPE_F16))[0] == TC


def test_host_pipeline_scratch_sizes(lib):
    """The host-buffer entry sizes its device scratch from the shape alone: chunks of at most 24 MiB of X, four slots."""
    big = lib.ssd_b200_host_scratch_bytes(C.byref(_shape(4, 8192, 80, 64, 128, 1, 256, _lib.DTYPE_BF16)))
    small = lib.ssd_b200_host_scratch_bytes(C.byref(_shape(2, 512, 8, 64, 64, 2, 128, _lib.DTYPE_BF16)))
    assert 0 < small < big < (1 << 30)
    assert big >= 4 * 2 * (24 << 20) * 0.9            # X and Y of four 24 MiB chunks
    assert lib.ssd_b200_host_scratch_bytes(C.byref(_shape(2, 500, 8, 64, 64, 2, 128, _lib.DTYPE_BF16))) == 0   # ragged
