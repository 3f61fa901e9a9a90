"""Drop-in replacement of the reference ``workloads/mamba/model_ref.py`` module.

Exports the reference's workload contract -- ``Model``, ``get_init_inputs()``,
``get_inputs()`` (reference ``README.md:26-29``) -- with the same constructor
arguments, parameter names, shapes and dtypes (``model_ref.py:49-66,170-199``), so
a ``state_dict`` moves between the two unchanged.  The SSD core
(``SSDLayer._ssd_core``, ``model_ref.py:123-162``) runs in the sm_100a kernels of
this package; the projections, the causal conv, the norms and the gate around it
stay PyTorch host code, as in the reference (``model_ref.py:68-121``).

The file can be loaded by path (the reference harness does so,
``bench.py:104-115``): it locates its own package.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch
import torch.nn as nn
import torch.nn.functional as F

_PKG_PARENT = str(Path(__file__).resolve().parent.parent)
if _PKG_PARENT not in sys.path:
    sys.path.insert(0, _PKG_PARENT)

from workloadsuite_b200.ssd import conv1d_silu, dt_prologue, ssd_forward  # noqa: E402


@torch.compiler.disable
def _dt(dt_raw, dt_bias, A_log):
    return dt_prologue(dt_raw, dt_bias, A_log)


@torch.compiler.disable
def _conv(x, weight, bias):
    return conv1d_silu(x, weight, bias)


@torch.compiler.disable
def _core(x, A_dt, B, C, dt, block_len, D, z):
    """The SSD core with the layer's skip and gate (``model_ref.py:116-118``) applied in the kernel's epilogue."""
    return ssd_forward(x, A_dt, B, C, block_len, dt=dt, D=D, z=z)


def _tma_friendly(t: torch.Tensor) -> torch.Tensor:
    """A view is passed through when its rows start on 16-byte boundaries, else copied."""
    per16 = 16 // t.element_size()
    ok = t.stride(-1) == 1 and all(st % per16 == 0 for st in t.stride()[:-1]) and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


class SSDLayer(nn.Module):
    """Single Mamba-2 SSD block (reference ``model_ref.py:13-121``)."""

    def __init__(self, d_model: int, n_heads: int, d_state: int, d_head: int, n_groups: int,
                 block_len: int = 64, conv_kernel: int = 4):
        super().__init__()
        self.d_model = d_model
        self.n_heads = n_heads
        self.d_state = d_state
        self.d_head = d_head
        self.n_groups = n_groups
        self.block_len = block_len
        if self.n_heads % self.n_groups != 0:
            raise ValueError("n_heads must be divisible by n_groups")
        self.d_inner = self.n_heads * self.d_head
        self.d_proj = 2 * self.d_inner + 2 * self.n_groups * self.d_state + self.n_heads

        self.in_proj = nn.Linear(self.d_model, self.d_proj, bias=False, dtype=torch.float16)
        self.conv1d = nn.Conv1d(self.d_inner, self.d_inner, kernel_size=conv_kernel, padding=conv_kernel - 1,
                                groups=self.d_inner, bias=True, dtype=torch.float16)
        self.A_log = nn.Parameter(torch.log(torch.arange(1, self.n_heads + 1, dtype=torch.float32)))
        self.D = nn.Parameter(torch.ones(self.n_heads, dtype=torch.float16))
        self.dt_bias = nn.Parameter(torch.zeros(self.n_heads, dtype=torch.float16) - 4.0)
        self.out_proj = nn.Linear(self.d_inner, self.d_model, bias=False, dtype=torch.float16)
        self.norm = nn.RMSNorm(self.d_model, dtype=torch.float16)

    def forward(self, u: torch.Tensor) -> torch.Tensor:
        batch, seq_len, _ = u.shape
        if seq_len % self.block_len != 0:
            raise ValueError(f"seq_len {seq_len} is not a multiple of block_len {self.block_len}")
        u = self.norm(u)
        zxbcdt = self.in_proj(u)
        gn = self.n_groups * self.d_state
        x, z, B, C, dt = torch.split(zxbcdt, [self.d_inner, self.d_inner, gn, gn, self.n_heads], dim=-1)

        # causal depthwise conv + SiLU (model_ref.py:83-86) straight from the projection's columns, no transposes
        x = _conv(x, self.conv1d.weight, self.conv1d.bias).view(batch, seq_len, self.n_heads, self.d_head)
        B = _tma_friendly(B.unflatten(-1, (self.n_groups, self.d_state)))   # ungrouped: no GQA repeat
        C = _tma_friendly(C.unflatten(-1, (self.n_groups, self.d_state)))

        dt, A_dt = _dt(dt, self.dt_bias, self.A_log)      # softplus(dt + bias), -exp(A_log) dt   (model_ref.py:94, 102-103)

        z = _tma_friendly(z.unflatten(-1, (self.n_heads, self.d_head)))     # a view of the projection output
        Y = _core(x, A_dt, B, C, dt, self.block_len, self.D, z)             # (Y + x D) silu(z), model_ref.py:116-118
        return self.out_proj(Y.view(batch, seq_len, self.d_inner))


class Model(nn.Module):
    """Stack of SSD blocks with residuals and a final RMSNorm (reference ``model_ref.py:165-204``)."""

    def __init__(self, d_model: int, n_layers: int, n_heads: int, d_state: int, d_head: int, n_groups: int,
                 block_len: int = 64, conv_kernel: int = 4):
        super().__init__()
        self.d_model = d_model
        self.n_layers = n_layers
        self.layers = nn.ModuleList(
            [SSDLayer(d_model, n_heads, d_state, d_head, n_groups, block_len, conv_kernel) for _ in range(n_layers)]
        )
        self.final_norm = nn.RMSNorm(d_model, dtype=torch.float16)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for layer in self.layers:
            x = x + layer(x)
        return self.final_norm(x)


# production configuration of the reference (model_ref.py:211-221)
d_model = 2048
n_layers = 24
n_heads = 128
d_state = 128
d_head = 64
n_groups = 8
block_len = 64
conv_kernel = 4

batch_size = 8
seq_length = 2048


def get_inputs():
    return [torch.randn(batch_size, seq_length, d_model, dtype=torch.float16)]


def get_init_inputs():
    return [d_model, n_layers, n_heads, d_state, d_head, n_groups, block_len, conv_kernel]
