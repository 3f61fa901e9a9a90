"""CPU oracle for the Mamba-2 SSD chunked-scan forward.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the algorithm of the
reference hot path ``SSDLayer._ssd_core`` (reference file
``workloads/mamba/model_ref.py:123-162``).  It is the checker used by the test
suite, by the smoke test and by the CPU-baseline leg of the benchmark; the
product path (``workloadsuite_b200``) never imports it.

Three restatements are provided:

* ``ssd_chunked``  -- line-by-line restatement of ``model_ref.py:135-162`` with
  the reference's hard-wired ``.to(torch.float16)`` casts replaced by
  ``.to(dtype)``; run with ``dtype=torch.float16`` it is bit-identical to the
  unmodified reference (pinned by ``tests/test_oracle.py`` against the golden
  fixtures generated from the reference itself).  It additionally accepts
  ungrouped B/C (``[b,s,g,n]``, broadcast as at ``model_ref.py:97-99``), an
  initial state seeding the carry of ``model_ref.py:153`` and can return the
  final carry, which the reference computes and discards.
* ``ssd_recurrence`` -- the token-by-token definition the chunked form is
  algebraically equal to (``H_t = exp(a_t) H_{t-1} + B_t (x) x_t``,
  ``y_t = C_t . H_t``), evaluated in float64.  Ground truth for features the
  reference lacks (initial/final states, sequence sharding).
* ``ssd_layer_pre`` / ``ssd_layer_post`` -- the reference block's own code
  around the core (``model_ref.py:68-110`` and ``:115-119``), used to test the
  drop-in ``Model``.

Parity status: the reference's own tests hold no golden vector for this path
("parity unpinned" by the reference); the oracle is pinned instead against
outputs of the reference code itself, run in the build container and committed
under ``tests/golden/``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

# --------------------------------------------------------------------------
# Chunked form (model_ref.py:135-162), dtype-generic
# --------------------------------------------------------------------------


def _broadcast_groups(t: torch.Tensor, n_heads: int) -> torch.Tensor:
    """[b,s,g,n] -> [b,s,h,n]; head j uses group j // (h/g) (model_ref.py:97-99)."""
    g = t.shape[2]
    if g == n_heads:
        return t
    if n_heads % g != 0:
        raise ValueError("n_heads must be divisible by n_groups")
    return t.repeat_interleave(n_heads // g, dim=2)


def ssd_chunked(
    X: torch.Tensor,
    A: torch.Tensor,
    B: torch.Tensor,
    C: torch.Tensor,
    chunk: int,
    dt: Optional[torch.Tensor] = None,
    initial_states: Optional[torch.Tensor] = None,
    dtype: Optional[torch.dtype] = None,
    return_final_state: bool = False,
):
    """Chunked SSD forward, following ``model_ref.py:135-162`` statement by statement.

    X [b,s,h,p]; A [b,s,h] per-token log-decay (the reference's ``A_dt``), fp32
    in the reference; B, C [b,s,g,n]; dt [b,s,h] or None (== 1);
    initial_states [b,h,n,p] (the layout of the carry at ``model_ref.py:153``).
    ``dtype`` is the "half" type of the reference's casts (default: X.dtype).
    Returns Y [b,s,h,p] in ``dtype`` (and the fp32-like carry if asked).
    """
    b, s, h, p = X.shape
    if s % chunk != 0:
        raise ValueError("seq_len must be a multiple of chunk")
    dtype = dtype or X.dtype
    wide = torch.float64 if dtype == torch.float64 else torch.float32
    c = s // chunk
    Bh = _broadcast_groups(B, h)
    Ch = _broadcast_groups(C, h)
    n = Bh.shape[-1]
    X_b = X.reshape(b, c, chunk, h, p).to(dtype)
    B_b = Bh.reshape(b, c, chunk, h, n).to(dtype)
    C_b = Ch.reshape(b, c, chunk, h, n).to(dtype)
    A_dt_b = A.reshape(b, c, chunk, h).to(wide)

    A_cumsum = torch.cumsum(A_dt_b, dim=2)                      # :135
    A_cumsum = A_cumsum.permute(0, 1, 3, 2)                     # :136  b c h l

    L = torch.exp(A_cumsum[..., :, None] - A_cumsum[..., None, :])   # :139
    mask = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool))    # :140
    L = L.masked_fill(~mask, 0.0)                                    # :141

    M = torch.einsum("bclhn,bcshn->bchls", C_b, B_b)            # :143
    if dt is None:
        X_scaled = X_b
    else:
        X_scaled = X_b * dt.reshape(b, c, chunk, h).to(dtype).unsqueeze(-1)   # :144
    Y_diag = torch.einsum("bchls,bcshp->bclhp", (L * M).to(dtype), X_scaled)  # :145

    decay_to_end = torch.exp(A_cumsum[..., -1:] - A_cumsum).to(dtype)         # :148
    block_state = torch.einsum("bclhn,bchl,bclhp->bchnp", B_b, decay_to_end, X_scaled)  # :149
    chunk_decay = torch.exp(A_cumsum[..., -1])                                # :150

    states = []
    if initial_states is None:
        hcar = torch.zeros(b, h, n, p, dtype=wide)                            # :153
    else:
        hcar = initial_states.to(wide).clone()
    for i in range(c):                                                        # :154
        states.append(hcar.to(dtype))                                         # :155
        hcar = hcar * chunk_decay[:, i, :, None, None] + block_state[:, i].to(wide)  # :156
    states = torch.stack(states, dim=1)                                       # :157

    decay_from_start = torch.exp(A_cumsum).to(dtype)                          # :160
    Y_off = torch.einsum("bclhn,bchnp,bchl->bclhp", C_b, states, decay_from_start)  # :161
    Y = (Y_diag + Y_off).reshape(b, s, h, p)                                  # :162
    if return_final_state:
        return Y, hcar
    return Y


# --------------------------------------------------------------------------
# Token-by-token definition, float64
# --------------------------------------------------------------------------


def ssd_recurrence(
    X: torch.Tensor,
    A: torch.Tensor,
    B: torch.Tensor,
    C: torch.Tensor,
    dt: Optional[torch.Tensor] = None,
    initial_states: Optional[torch.Tensor] = None,
    return_final_state: bool = False,
):
    """float64 recurrence H_t = e^{a_t} H_{t-1} + B_t (x) x~_t ; y_t = C_t . H_t.

    Same argument layout as :func:`ssd_chunked`.  Returns float64 tensors.
    """
    b, s, h, p = X.shape
    X64 = X.double()
    if dt is not None:
        X64 = X64 * dt.double().unsqueeze(-1)
    A64 = A.double()
    B64 = _broadcast_groups(B, h).double()
    C64 = _broadcast_groups(C, h).double()
    n = B64.shape[-1]
    H = torch.zeros(b, h, n, p, dtype=torch.float64) if initial_states is None else initial_states.double().clone()
    Y = torch.empty(b, s, h, p, dtype=torch.float64)
    dec = torch.exp(A64)
    for t in range(s):
        H = H * dec[:, t, :, None, None] + B64[:, t, :, :, None] * X64[:, t, :, None, :]
        Y[:, t] = torch.einsum("bhn,bhnp->bhp", C64[:, t], H)
    if return_final_state:
        return Y, H
    return Y


def total_logdecay(A: torch.Tensor) -> torch.Tensor:
    """Sum of the per-token log-decay over the sequence, [b,h] float64."""
    return A.double().sum(dim=1)


# --------------------------------------------------------------------------
# Sequence sharding algebra (what the multi-GPU path computes), on CPU
# --------------------------------------------------------------------------


def fold_incoming_state(states: torch.Tensor, logdecays: torch.Tensor, rank: int,
                        initial: Optional[torch.Tensor] = None) -> torch.Tensor:
    """State entering shard ``rank`` given every shard's zero-start final state.

    states [R,b,h,n,p]: final carry of shard r when started from zero;
    logdecays [R,b,h]: sum of log-decay over shard r.  The recurrence is linear,
    so  H_in(r+1) = exp(D_r) H_in(r) + F_r  with H_in(0) = initial (or 0).
    """
    acc = torch.zeros_like(states[0], dtype=torch.float64) if initial is None else initial.double().clone()
    for q in range(rank):
        acc = acc * torch.exp(logdecays[q].double())[..., None, None] + states[q].double()
    return acc


# --------------------------------------------------------------------------
# The reference block around the core (for the drop-in Model tests)
# --------------------------------------------------------------------------


def ssd_layer_pre(layer, u: torch.Tensor):
    """``SSDLayer.forward`` up to the core call (``model_ref.py:69-103``).

    ``layer`` is any module with the reference's parameter names.  Returns
    (x[b,s,h,p], z, B[b,s,g,n], C[b,s,g,n], dt[b,s,h], A_dt[b,s,h] fp32) with
    B/C left *ungrouped* (the GQA repeat of ``:97-99`` is applied by the core).
    """
    import torch.nn.functional as F

    batch, seq_len, _ = u.shape
    u = layer.norm(u)                                                        # :72
    zxbcdt = layer.in_proj(u)                                                # :75
    gn = layer.n_groups * layer.d_state
    x, z, B, C, dt = torch.split(zxbcdt, [layer.d_inner, layer.d_inner, gn, gn, layer.n_heads], dim=-1)  # :76
    x = causal_conv1d_silu(x, layer.conv1d.weight, layer.conv1d.bias)        # :83-86
    x = x.reshape(batch, seq_len, layer.n_heads, layer.d_head)               # :89
    B = B.reshape(batch, seq_len, layer.n_groups, layer.d_state)             # :90
    C = C.reshape(batch, seq_len, layer.n_groups, layer.d_state)             # :91
    dt = F.softplus(dt + layer.dt_bias)                                      # :94
    A = -torch.exp(layer.A_log)                                              # :102
    A_dt = A * dt.float()                                                    # :103
    return x, z, B, C, dt, A_dt


def causal_conv1d_silu(x: torch.Tensor, weight: torch.Tensor, bias=None, dtype=None) -> torch.Tensor:
    """Causal depthwise conv + SiLU of ``SSDLayer.forward`` (``model_ref.py:83-86`` with the ``nn.Conv1d`` of
    ``:50-58``): x [b,l,d], weight [d,1,k], bias [d]; the same operator calls as the reference, in ``dtype``
    (default: x's dtype; ``torch.float64`` for an exact reference).  Returns [b,l,d]."""
    import torch.nn.functional as F

    dtype = dtype or x.dtype
    d, k = weight.shape[0], weight.shape[-1]
    xt = x.to(dtype).transpose(1, 2)                                          # :83
    y = F.conv1d(xt, weight.to(dtype).reshape(d, 1, k), None if bias is None else bias.to(dtype),
                 padding=k - 1, groups=d)[..., : x.shape[1]]                  # :84
    return F.silu(y).transpose(1, 2)                                          # :85-86


def ssd_epilogue(Y: torch.Tensor, x: torch.Tensor, D=None, z=None, dtype=None) -> torch.Tensor:
    """Skip and gate of ``SSDLayer.forward`` after the core (``model_ref.py:116-118``), without the projection:
    ``(Y + x * D[head]) * silu(z)`` on [b,s,h,p] tensors, each step cast to ``dtype`` as the reference does
    (default: the dtype of Y); pass ``torch.float64`` for an exact reference."""
    import torch.nn.functional as F

    dtype = dtype or Y.dtype
    out = Y.to(dtype)
    if D is not None:
        out = out + x.to(dtype) * D.to(dtype).view(1, 1, -1, 1)                # :116
    if z is not None:
        out = out * F.silu(z.to(dtype))                                      # :118
    return out


def ssd_layer_post(layer, Y: torch.Tensor, x: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
    """``SSDLayer.forward`` after the core call (``model_ref.py:116-119``)."""
    import torch.nn.functional as F

    b, s, h, p = Y.shape
    Y = Y + x * layer.D.view(1, 1, -1, 1)                                    # :116
    Y = Y.reshape(b, s, h * p)                                               # :117
    Y = Y * F.silu(z)                                                        # :118
    return layer.out_proj(Y)                                                 # :119


# --------------------------------------------------------------------------
# Error metrics and synthetic inputs
# --------------------------------------------------------------------------


def error_metrics(Y: torch.Tensor, Yref: torch.Tensor):
    """(worst per-(batch,head) max-abs error over max-abs reference, global relative Frobenius error).

    Magnitudes differ by many orders between (batch, head) pairs when the
    log-decay is positive, so the max-abs error is normalised per pair.
    Tensors are [b,s,h,p].
    """
    Y = Y.double()
    Yref = Yref.double()
    diff = (Y - Yref).abs()
    num = diff.amax(dim=(1, 3))
    den = Yref.abs().amax(dim=(1, 3)).clamp_min(1e-300)
    per_bh = (num / den).max().item()
    fro = (diff.pow(2).sum().sqrt() / Yref.pow(2).sum().sqrt().clamp_min(1e-300)).item()
    return per_bh, fro


# name -> (batch, seq, heads, d_head, d_state, groups, chunk, dtype, has_initial_states)
CONFIGS = {
    "cfg0": dict(b=16, s=128, h=8, p=64, n=16, g=8, chunk=64, dtype="f32", init=False, decay="normal"),
    "cfg1": dict(b=8, s=2048, h=24, p=64, n=128, g=1, chunk=256, dtype="bf16", init=False, decay="mamba"),
    "cfg2": dict(b=4, s=8192, h=80, p=64, n=128, g=1, chunk=256, dtype="bf16", init=False, decay="mamba"),
    "cfg3": dict(b=1, s=131072, h=32, p=64, n=128, g=1, chunk=256, dtype="bf16", init=False, decay="mamba"),
    "cfg4": dict(b=256, s=512, h=48, p=64, n=64, g=8, chunk=128, dtype="bf16", init=True, decay="mamba"),
}

_DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def make_inputs(b, s, h, p, n, g, dtype="bf16", init=False, decay="mamba", seed=0, decay_scale=1.0, **_):
    """Seeded synthetic inputs with the distributions of the benchmark configs.

    decay="normal": A ~ N(0,1) (config 0).  decay="mamba": A = -dt * exp(A_log),
    dt = softplus(N(-4,1)) per token and head, A_log ~ U(log 1, log 16) per head.
    ``decay_scale`` multiplies A (use 1e-2 for slow decays that make the
    inter-chunk and inter-shard state terms matter).  Generated on the CPU in
    fp32, then cast, so that a CPU oracle and a GPU kernel see identical values.
    """
    gen = torch.Generator().manual_seed(seed)
    td = _DTYPES[dtype] if isinstance(dtype, str) else dtype
    X = torch.randn(b, s, h, p, generator=gen).to(td)
    Bm = torch.randn(b, s, g, n, generator=gen).to(td)
    Cm = torch.randn(b, s, g, n, generator=gen).to(td)
    if decay == "normal":
        A = torch.randn(b, s, h, generator=gen)
    else:
        dt = torch.nn.functional.softplus(torch.randn(b, s, h, generator=gen) - 4.0)
        A_log = torch.empty(h).uniform_(math.log(1.0), math.log(16.0), generator=gen)
        A = -dt * torch.exp(A_log)
    A = (A * decay_scale).float()
    out = dict(X=X, A=A, B=Bm, C=Cm)
    if init:
        out["initial_states"] = (torch.randn(b, h, n, p, generator=gen) * 0.1).float()
    return out
