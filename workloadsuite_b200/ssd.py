"""Functional SSD forward on B200: ``ssd_forward`` and its host-buffer variant.

Replaces ``SSDLayer._ssd_core`` of the reference (``workloads/mamba/model_ref.py:123-162``)
with hand-written sm_100a kernels reached through the C ABI of ``include/ssd_b200.h``.
PyTorch supplies device memory and the current stream only.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.DTYPE_F32, torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16}
_KERNELS = {None: _lib.KERNEL_AUTO, "auto": _lib.KERNEL_AUTO, "scan_f32": _lib.KERNEL_SCAN_F32,
            "tcgen05": _lib.KERNEL_TCGEN05}

_workspaces: dict = {}
_status: dict = {}


def _status_word(device) -> torch.Tensor:
    key = (device.type, device.index)
    st = _status.get(key)
    if st is None:
        st = torch.zeros(1024, dtype=torch.int32, device=device)
        _status[key] = st
    return st


def device_status(device="cuda:0", clear: bool = True) -> int:
    """Synchronises and returns the kernels' status word for ``device`` (0 = fine; 1/2/3 = a bounded
    wait on TMA / tensor-core / intra-CTA synchronisation ran out and the kernel gave up; 6 = the wait for
    the piece of a sequence handed over by another CTA ran out; 7 = the peer-memory exchange waited in vain for
    another rank)."""
    device = torch.device(device)
    st = _status_word(device)
    torch.cuda.synchronize(device)
    v = int(st[0].item())
    if clear and v:
        st.zero_()
    return v


class SsdError(RuntimeError):
    """An SSD_ERR_* code from the native library that has no closer Python exception."""


def _raise(code: int):
    msg = f"{_lib.ERRORS.get(code, code)}: {_lib.strerror(code)}"
    if code in (-2, -3):
        # the reference raises ValueError for bad head/group counts (model_ref.py:37-38) and an
        # einops error (a ValueError-like shape error) for seq_len % block_len != 0 (model_ref.py:106)
        raise ValueError(msg)
    if code == -4:
        raise NotImplementedError(msg)
    raise SsdError(msg)


def _strides3(t: torch.Tensor, name: str):
    """Element strides of the three outer axes; a size-1 axis gets its contiguous stride
    (its real stride is arbitrary and may break the 16-byte rule of TMA descriptors)."""
    if t.stride(-1) != 1 and t.shape[-1] != 1:
        raise ValueError(f"{name}: innermost axis must be contiguous")
    st = list(t.stride()[:3])
    inner = t.shape[3]
    for d in (2, 1, 0):
        if t.shape[d] == 1:
            st[d] = inner
        inner = max(inner, st[d] * t.shape[d])
    return (C.c_int64 * 3)(*st)


def _same_device(ref: torch.Tensor, **tensors):
    """Every tensor handed to the library must live where X lives: a pointer into host memory or into another
    GPU's memory would fault inside a kernel instead of raising here."""
    for name, t in tensors.items():
        if t is not None and t.device != ref.device:
            raise ValueError(f"{name} is on {t.device}, X is on {ref.device}: all tensors must share one device")


def _rows_contiguous(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """The kernels read rows of p (or n) contiguous elements.  A tensor whose innermost axis is strided -- the
    reference block hands ``_ssd_core`` an X that is sequence-contiguous and channel-strided, a permuted
    ``[b, d, l]`` buffer (``model_ref.py:83-89``) -- is copied once into the row layout (one read and one
    write of the tensor); anything else is passed through as the view it is."""
    if t is None or t.stride(-1) == 1 or t.shape[-1] == 1:
        return t
    return t.contiguous()


def _check_out(out: torch.Tensor, like: torch.Tensor, name: str = "out"):
    if out.shape != like.shape or out.dtype != like.dtype or out.device != like.device:
        raise ValueError(f"{name} must have the shape {tuple(like.shape)}, dtype {like.dtype} and device of X")
    if out.dim() and out.stride(-1) != 1 and out.shape[-1] != 1:
        raise ValueError(f"{name}: innermost axis must be contiguous")


def _check(X, A, B, Cm, dt, initial_states):
    if X.dim() != 4 or A.dim() != 3 or B.dim() != 4 or Cm.dim() != 4:
        raise ValueError("expected X[b,s,h,p], A[b,s,h], B[b,s,g,n], C[b,s,g,n]")
    _same_device(X, A=A, B=B, C=Cm, dt=dt, initial_states=initial_states)
    b, s, h, p = X.shape
    g, n = B.shape[2], B.shape[3]
    if A.shape != (b, s, h) or B.shape[:2] != (b, s) or Cm.shape != B.shape:
        raise ValueError("inconsistent shapes")
    if X.dtype not in _DTYPES or B.dtype != X.dtype or Cm.dtype != X.dtype:
        raise TypeError("X, B, C must share one dtype of float32/float16/bfloat16")
    if A.dtype != torch.float32:
        raise TypeError("A (per-token log-decay) must be float32")
    if dt is not None and (dt.shape != (b, s, h) or dt.dtype != X.dtype):
        raise ValueError("dt must be [b,s,h] in the dtype of X")
    if initial_states is not None and (initial_states.shape != (b, h, n, p) or initial_states.dtype != torch.float32):
        raise ValueError("initial_states must be float32 [b,h,n,p]")
    return b, s, h, p, g, n


def _fill(args, X, A, B, Cm, dt, initial_states, Y, final_state, final_ld, chunk, kernel, nsegments, state_only,
          reuse_segments=False):
    b, s, h, p = X.shape
    args.X, args.A, args.B, args.C = X.data_ptr(), A.data_ptr(), B.data_ptr(), Cm.data_ptr()
    args.dt = dt.data_ptr() if dt is not None else None
    args.initial_state = initial_states.data_ptr() if initial_states is not None else None
    args.Y = Y.data_ptr() if Y is not None else None
    args.final_state = final_state.data_ptr() if final_state is not None else None
    args.final_logdecay = final_ld.data_ptr() if final_ld is not None else None
    args.batch, args.seqlen, args.nheads, args.headdim = b, s, h, p
    args.dstate, args.ngroups = B.shape[3], B.shape[2]
    args.chunk = chunk
    args.dtype = _DTYPES[X.dtype]
    if kernel not in _KERNELS:
        raise ValueError(f"kernel must be one of {sorted(k for k in _KERNELS if k)}")
    args.kernel = _KERNELS[kernel]
    args.status = _status_word(X.device).data_ptr() if X.is_cuda else None
    args.flags = (_lib.FLAG_STATE_ONLY if state_only else 0) | (_lib.FLAG_REUSE_SEGMENTS if reuse_segments else 0)
    args.nsegments = int(nsegments or 0)
    args.x_stride = _strides3(X, "X")
    args.a_stride = (C.c_int64 * 3)(*A.stride())
    args.b_stride = _strides3(B, "B")
    args.c_stride = _strides3(Cm, "C")
    if dt is not None:
        args.dt_stride = (C.c_int64 * 3)(*dt.stride())
    if Y is not None:
        args.y_stride = _strides3(Y, "Y")


def _workspace(device, nbytes: int) -> Optional[torch.Tensor]:
    if nbytes == 0:
        return None
    key = (device.type, device.index)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def ssd_forward(
    X: torch.Tensor,
    A: torch.Tensor,
    B: torch.Tensor,
    C_: torch.Tensor,
    chunk: int,
    dt: Optional[torch.Tensor] = None,
    initial_states: Optional[torch.Tensor] = None,
    return_final_state: bool = False,
    return_logdecay: bool = False,
    state_only: bool = False,
    kernel: Optional[str] = None,
    nsegments: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    reuse_segments: bool = False,
    D: Optional[torch.Tensor] = None,
    z: Optional[torch.Tensor] = None,
    separate_epilogue: bool = False,
    wait_limit_ms: int = 0,
    inject_lost_handover: bool = False,
    out_final_state: Optional[torch.Tensor] = None,
    out_logdecay: Optional[torch.Tensor] = None,
):
    """Mamba-2 SSD forward ``Y = SSD(X, A, B, C)`` on the current CUDA stream.

    X [b,s,h,p]; A [b,s,h] float32 per-token log-decay (the reference's ``A_dt``,
    ``model_ref.py:103``); B, C [b,s,g,n] *ungrouped* (head j reads group
    ``j // (h//g)``, ``model_ref.py:97-99``); dt [b,s,h] or None for ``X`` already
    scaled (``model_ref.py:144``); initial_states float32 [b,h,n,p] (the layout of
    the carry at ``model_ref.py:153``) or None for zeros.  ``chunk`` is the
    reference's ``block_len``: it must divide ``s`` (as at ``model_ref.py:106``);
    the result does not otherwise depend on it.  Views with a contiguous innermost
    axis are accepted as they are; a tensor whose innermost axis is strided (the
    reference block's own X, ``model_ref.py:83-89``) is first copied into the row layout.
    All tensors must be on X's device.  No host synchronisation.

    ``nsegments``: None lets the library choose; 1 keeps sequences whole; more cuts them (see ``plan``):
    the tensor-core kernel deals the tiles of all sequences out evenly over the SMs inside one launch, the other
    kernels scan that many segments in two passes joined by a fold.

    A sequence that is cut into segments uses one scratch buffer per device, kept between
    calls and shared by all of them: calls that may overlap on the GPU (different streams)
    must be serialised by the caller, and ``reuse_segments`` relies on no other segmented
    call on that device coming between the two runs.

    ``D`` [h] and ``z`` [b,s,h,p] (dtype of X) add the layer's skip and gate to the kernel's epilogue:
    ``Y <- (Y + X * D[head]) * silu(z)`` (``model_ref.py:116-118``), evaluated in float32 and rounded once;
    either may be given alone.  Note that the skip term uses ``X`` as passed, i.e. before ``dt``.
    ``separate_epilogue`` runs them as a kernel of their own even where the main kernel could fuse them.

    Returns Y [b,s,h,p] in X's dtype, plus the float32 final state [b,h,n,p] and/or
    the summed log-decay [b,h] when asked.  With ``state_only`` no Y is produced.
    ``out_final_state`` / ``out_logdecay`` (contiguous float32 tensors of those shapes on X's device, the state
    16-byte aligned) receive them in place of fresh tensors, e.g. slices of an exchange buffer.
    ``reuse_segments`` tells a segmented two-pass scan that the previous call on this device was the
    ``state_only`` run over the same tensors, so its per-segment states need not be recomputed.

    Every wait inside the kernels is bounded (about a second; ``wait_limit_ms`` sets another bound): a kernel
    that runs into the bound writes a code to the device status word (``device_status``) and returns.
    ``inject_lost_handover`` exists to test that path: see ``SSD_FLAG_INJECT_LOST_HANDOVER``.
    """
    if not X.is_cuda:
        raise RuntimeError("ssd_forward needs CUDA tensors (there is no CPU path); see ssd_forward_host")
    b, s, h, p, g, n = _check(X, A, B, C_, dt, initial_states)
    if h % g != 0:
        raise ValueError("n_heads must be divisible by n_groups")
    X, B, C_, z = _rows_contiguous(X), _rows_contiguous(B), _rows_contiguous(C_), _rows_contiguous(z)
    if initial_states is not None:
        initial_states = initial_states.contiguous()
    if D is not None:
        if D.shape != (h,):
            raise ValueError("D must be [h]")
        D = D.to(device=X.device, dtype=torch.float32).contiguous()
    if z is not None and (z.shape != X.shape or z.dtype != X.dtype or z.device != X.device):
        raise ValueError("z must be a tensor [b,s,h,p] in the dtype and on the device of X")
    if state_only and (D is not None or z is not None):
        raise ValueError("D / z apply to Y; a state-only run produces none")
    if out is not None:
        if state_only:
            raise ValueError("a state-only run writes no Y: do not pass out")
        _check_out(out, X)
    lib = _lib.load()
    dev = X.device
    want_final = return_final_state or state_only
    Y = None
    if not state_only:
        Y = out if out is not None else torch.empty((b, s, h, p), dtype=X.dtype, device=dev)
    final_state = final_ld = None
    if want_final:
        final_state = out_final_state if out_final_state is not None else \
            torch.empty((b, h, n, p), dtype=torch.float32, device=dev)
    if return_logdecay:
        final_ld = out_logdecay if out_logdecay is not None else torch.empty((b, h), dtype=torch.float32, device=dev)
    for name, t, shape in (("out_final_state", out_final_state, (b, h, n, p)), ("out_logdecay", out_logdecay, (b, h))):
        if t is not None and (t.shape != shape or t.dtype != torch.float32 or t.device != dev or not t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous float32 tensor {list(shape)} on the device of X")
    args = _lib.SsdArgs()
    _fill(args, X, A, B, C_, dt, initial_states, Y, final_state, final_ld, chunk, kernel, nsegments, state_only,
          reuse_segments)
    if separate_epilogue:
        args.flags |= _lib.FLAG_SEPARATE_EPILOGUE
    if inject_lost_handover:
        args.flags |= _lib.FLAG_INJECT_LOST_HANDOVER
    args.wait_limit_ms = int(wait_limit_ms)
    if D is not None:
        args.D = D.data_ptr()
    if z is not None:
        args.Z = z.data_ptr()
        args.z_stride = _strides3(z, "z")
    with torch.cuda.device(dev):
        need = lib.ssd_b200_workspace_bytes(C.byref(args))
        ws = _workspace(dev, need)
        if ws is not None:
            args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        rc = lib.ssd_b200_forward(C.byref(args), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if rc != _lib.SSD_OK:
        _raise(rc)
    outs = [] if state_only else [Y]
    if want_final:
        outs.append(final_state)
    if return_logdecay:
        outs.append(final_ld)
    return outs[0] if len(outs) == 1 else tuple(outs)


def conv1d_silu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal depthwise conv1d + SiLU on the current CUDA stream: ``silu(conv1d(x^T)[..., :l])^T`` of
    ``model_ref.py:83-86`` without the transposes.

    x [b,l,d] with a contiguous channel axis (a column slice of the projection output is fine); weight the
    ``nn.Conv1d(d, d, k, groups=d)`` parameter [d,1,k] (or [d,k]); bias [d] or None.  Returns [b,l,d] contiguous
    in x's dtype (fp32 accumulation, one rounding).
    """
    if not x.is_cuda:
        raise RuntimeError("conv1d_silu needs CUDA tensors (there is no CPU path)")
    if x.dim() != 3 or x.stride(2) != 1 or x.dtype not in _DTYPES:
        raise ValueError("x must be [b,l,d] float32/float16/bfloat16 with a contiguous channel axis")
    b, l, d = x.shape
    _same_device(x, weight=weight, bias=bias, out=out)
    w = weight.reshape(d, -1).to(x.dtype).contiguous()
    taps = w.shape[1]
    if bias is not None:
        if bias.shape != (d,):
            raise ValueError("bias must be [d]")
        bias = bias.to(x.dtype).contiguous()
    if out is None:
        out = torch.empty((b, l, d), dtype=x.dtype, device=x.device)
    else:
        _check_out(out, x)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.ssd_b200_conv1d_silu(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
                                      out.data_ptr(), b, l, d, taps, _DTYPES[x.dtype], x.stride(0), x.stride(1),
                                      out.stride(0), out.stride(1),
                                      C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
    if rc != _lib.SSD_OK:
        _raise(rc)
    return out


def dt_prologue(dt_raw: torch.Tensor, dt_bias: Optional[torch.Tensor], A_log: torch.Tensor):
    """``dt = softplus(dt_raw + dt_bias)`` and ``A_dt = -exp(A_log) * dt.float()`` (``model_ref.py:94, 102-103``) in one
    pass on the current CUDA stream.  dt_raw [b,l,h] with a contiguous head axis (a column slice of the projection
    output is fine); dt_bias [h] or None; A_log [h] float32.  Returns (dt [b,l,h] in dt_raw's dtype, A_dt float32)."""
    if not dt_raw.is_cuda:
        raise RuntimeError("dt_prologue needs CUDA tensors (there is no CPU path)")
    if dt_raw.dim() != 3 or dt_raw.stride(2) != 1 or dt_raw.dtype not in _DTYPES:
        raise ValueError("dt_raw must be [b,l,h] float32/float16/bfloat16 with a contiguous head axis")
    b, l, h = dt_raw.shape
    _same_device(dt_raw, dt_bias=dt_bias, A_log=A_log)
    if A_log.shape != (h,) or (dt_bias is not None and dt_bias.shape != (h,)):
        raise ValueError("dt_bias and A_log must be [h]")
    if dt_bias is not None:
        dt_bias = dt_bias.to(dt_raw.dtype).contiguous()
    A_log = A_log.to(dtype=torch.float32).contiguous()
    dt = torch.empty((b, l, h), dtype=dt_raw.dtype, device=dt_raw.device)
    A_dt = torch.empty((b, l, h), dtype=torch.float32, device=dt_raw.device)
    lib = _lib.load()
    with torch.cuda.device(dt_raw.device):
        rc = lib.ssd_b200_dt_prologue(dt_raw.data_ptr(), dt_raw.stride(0), dt_raw.stride(1),
                                      dt_bias.data_ptr() if dt_bias is not None else None, A_log.data_ptr(),
                                      dt.data_ptr(), A_dt.data_ptr(), b, l, h, _DTYPES[dt_raw.dtype],
                                      C.c_void_p(torch.cuda.current_stream(dt_raw.device).cuda_stream))
    if rc != _lib.SSD_OK:
        _raise(rc)
    return dt, A_dt


def ssd_step(x: torch.Tensor, a: torch.Tensor, B: torch.Tensor, C_: torch.Tensor, state: torch.Tensor,
             dt: Optional[torch.Tensor] = None, D: Optional[torch.Tensor] = None, z: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token of the recurrence on the current CUDA stream, ``state`` updated in place (decode-style use of the carry
    of ``model_ref.py:152-157``): ``state <- exp(a) state + B (x) (dt x)``, ``y = C . state``, then the layer's skip and
    gate (``model_ref.py:116-118``) when ``D`` / ``z`` are given.

    x [b,h,p] (p = 64), a [b,h] float32 (the token's ``A_dt``), B and C [b,g,n], dt [b,h] or None, D [h], z [b,h,p],
    state float32 [b,h,n,p] (what ``ssd_forward(..., return_final_state=True)`` returns).  Returns y [b,h,p].
    Equal, within the kernels' tolerances, to ``ssd_forward`` over a one-token sequence with ``initial_states=state``.
    """
    if not x.is_cuda:
        raise RuntimeError("ssd_step needs CUDA tensors (there is no CPU path)")
    if x.dim() != 3 or B.dim() != 3 or state.dim() != 4 or x.dtype not in _DTYPES:
        raise ValueError("expected x [b,h,p], B/C [b,g,n], state [b,h,n,p]")
    b, h, p = x.shape
    g, n = B.shape[1], B.shape[2]
    _same_device(x, a=a, B=B, C=C_, state=state, dt=dt, D=D, z=z, out=out)
    if h % g != 0:
        raise ValueError("n_heads must be divisible by n_groups")
    if (a.shape != (b, h) or a.dtype != torch.float32 or B.shape != (b, g, n) or C_.shape != (b, g, n)
            or B.dtype != x.dtype or C_.dtype != x.dtype or state.shape != (b, h, n, p) or state.dtype != torch.float32
            or not state.is_contiguous()):
        raise ValueError("a must be float32 [b,h], B/C [b,g,n] in x's dtype, state contiguous float32 [b,h,n,p]")
    if dt is not None and (dt.shape != (b, h) or dt.dtype != x.dtype):
        raise ValueError("dt must be [b,h] in x's dtype")
    if z is not None and (z.shape != x.shape or z.dtype != x.dtype):
        raise ValueError("z must be [b,h,p] in x's dtype")
    if D is not None:
        if D.shape != (h,):
            raise ValueError("D must be [h]")
        D = D.to(dtype=torch.float32).contiguous()
    x, a, B, C_ = x.contiguous(), a.contiguous(), B.contiguous(), C_.contiguous()
    dt = None if dt is None else dt.contiguous()
    z = None if z is None else z.contiguous()
    if out is None:
        out = torch.empty((b, h, p), dtype=x.dtype, device=x.device)
    elif out.shape != (b, h, p) or out.dtype != x.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous [b,h,p] tensor in x's dtype")
    ptr = lambda t: None if t is None else t.data_ptr()
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.ssd_b200_step(ptr(x), ptr(a), ptr(B), ptr(C_), ptr(dt), ptr(D), ptr(z), ptr(state), ptr(out),
                               b, h, p, n, g, _DTYPES[x.dtype],
                               C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
    if rc != _lib.SSD_OK:
        _raise(rc)
    return out


def kernel_name(X, A, B, C_, chunk, kernel=None) -> str:
    """Which kernel family ``ssd_forward`` would run for these tensors."""
    _check(X, A, B, C_, None, None)
    args = _lib.SsdArgs()
    _fill(args, X, A, B, C_, None, None, None, None, None, chunk, kernel, 0, False)
    return _lib.load().ssd_b200_kernel_name(C.byref(args)).decode()


def plan(X, A, B, C_, chunk, kernel=None, nsegments=None, state_only=False, reuse_segments=False) -> dict:
    """Kernel family, segments per sequence, kernel launches and scratch bytes ``ssd_forward`` uses."""
    _check(X, A, B, C_, None, None)
    args = _lib.SsdArgs()
    _fill(args, X, A, B, C_, None, None, None, None, None, chunk, kernel, nsegments, state_only, reuse_segments)
    lib = _lib.load()
    k, nseg, launches = C.c_int32(), C.c_int32(), C.c_int32()
    rc = lib.ssd_b200_plan(C.byref(args), C.byref(k), C.byref(nseg), C.byref(launches))
    if rc != _lib.SSD_OK:
        _raise(rc)
    return {"kernel": lib.ssd_b200_kernel_name(C.byref(args)).decode(), "nsegments": nseg.value,
            "launches": launches.value, "workspace_bytes": int(lib.ssd_b200_workspace_bytes(C.byref(args)))}


def fold_states(states: torch.Tensor, logdecays: torch.Tensor, rank: int,
                initial: Optional[torch.Tensor] = None) -> torch.Tensor:
    """State entering shard ``rank`` of a sequence-sharded scan.

    states float32 [R,b,h,n,p] (each shard's final state when scanned from zero),
    logdecays float32 [R,b,h]; both may be strided along R (slices of one
    all-gather buffer).  ``H_in(r+1) = exp(D_r) H_in(r) + F_r``.
    """
    if not states.is_cuda:
        raise RuntimeError("fold_states needs CUDA tensors (there is no CPU path)")
    R, b, h, n, p = states.shape
    _same_device(states, logdecays=logdecays, initial=initial)
    if logdecays.shape != (R, b, h) or (initial is not None and initial.shape != (b, h, n, p)):
        raise ValueError("expected states [R,b,h,n,p], logdecays [R,b,h], initial [b,h,n,p]")
    if not states[0].is_contiguous() or not logdecays[0].is_contiguous():
        states, logdecays = states.contiguous(), logdecays.contiguous()
    if states.dtype != torch.float32 or logdecays.dtype != torch.float32:
        raise TypeError("states and logdecays must be float32")
    if initial is not None:
        if initial.dtype != torch.float32:
            raise TypeError("initial must be float32")
        initial = initial.contiguous()
    out = torch.empty((b, h, n, p), dtype=torch.float32, device=states.device)
    lib = _lib.load()
    with torch.cuda.device(states.device):
        rc = lib.ssd_b200_fold_states(states.data_ptr(), states.stride(0) if R > 1 else b * h * n * p,
                                      logdecays.data_ptr(), logdecays.stride(0) if R > 1 else b * h,
                                      initial.data_ptr() if initial is not None else None, out.data_ptr(), R, rank,
                                      b * h, n * p, C.c_void_p(torch.cuda.current_stream(states.device).cuda_stream))
    if rc != _lib.SSD_OK:
        _raise(rc)
    return out


class HostRunner:
    """Reusable host-buffer forward: owns the device scratch for one problem shape.

    ``run`` takes CPU tensors (pinned memory gives full PCIe rate), copies them to
    the GPU in slices, computes and copies Y back into ``out``; it returns after
    the result is in host memory.
    """

    def __init__(self, b, s, h, p, n, g, chunk, dtype, device="cuda:0", kernel=None, has_dt=False):
        self.shape = (b, s, h, p, n, g)
        self.chunk, self.dtype, self.kernel = chunk, dtype, kernel
        self.device = torch.device(device)
        self.lib = _lib.load()
        a = _lib.SsdArgs()
        a.batch, a.seqlen, a.nheads, a.headdim, a.dstate, a.ngroups = b, s, h, p, n, g
        a.chunk, a.dtype, a.kernel = chunk, _DTYPES[dtype], _KERNELS[kernel]
        a.dt = 1 if has_dt else None  # only NULL-ness matters for sizing
        with torch.cuda.device(self.device):
            nbytes = self.lib.ssd_b200_host_scratch_bytes(C.byref(a))
            if nbytes == 0:
                raise ValueError("invalid problem shape")
            self.scratch = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def run(self, X, A, B, C_, out, dt=None, initial_states=None, final_state=None):
        b, s, h, p, n, g = self.shape
        for t in (X, A, B, C_, out):
            if t.is_cuda or not t.is_contiguous():
                raise ValueError("HostRunner.run takes contiguous CPU tensors")
        a = _lib.SsdArgs()
        a.batch, a.seqlen, a.nheads, a.headdim, a.dstate, a.ngroups = b, s, h, p, n, g
        a.chunk, a.dtype, a.kernel = self.chunk, _DTYPES[self.dtype], _KERNELS[self.kernel]
        a.X, a.A, a.B, a.C, a.Y = X.data_ptr(), A.data_ptr(), B.data_ptr(), C_.data_ptr(), out.data_ptr()
        a.dt = dt.data_ptr() if dt is not None else None
        a.initial_state = initial_states.data_ptr() if initial_states is not None else None
        a.final_state = final_state.data_ptr() if final_state is not None else None
        with torch.cuda.device(self.device):
            rc = self.lib.ssd_b200_forward_host(C.byref(a), self.scratch.data_ptr(), self.scratch.numel())
        if rc != _lib.SSD_OK:
            _raise(rc)
        self.h2d_bytes = sum(t.numel() * t.element_size() for t in (X, A, B, C_, dt, initial_states) if t is not None)
        self.d2h_bytes = sum(t.numel() * t.element_size() for t in (out, final_state) if t is not None)
        return out


def ssd_forward_host(X, A, B, C_, chunk, dt=None, initial_states=None, kernel=None, device="cuda:0"):
    """One-shot host-buffer forward: CPU tensors in, CPU tensor out (computed on the GPU)."""
    b, s, h, p, g, n = _check(X, A, B, C_, dt, initial_states)
    if h % g != 0:
        raise ValueError("n_heads must be divisible by n_groups")
    if s % chunk != 0:
        raise ValueError("seq_len must be a multiple of chunk")
    r = HostRunner(b, s, h, p, n, g, chunk, X.dtype, device=device, kernel=kernel, has_dt=dt is not None)
    out = torch.empty_like(X).contiguous()
    return r.run(X.contiguous(), A.contiguous(), B.contiguous(), C_.contiguous(), out,
                 dt=None if dt is None else dt.contiguous(),
                 initial_states=None if initial_states is None else initial_states.contiguous())
