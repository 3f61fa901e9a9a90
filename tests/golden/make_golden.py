"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Run in a container that has the reference checkout:

    python tests/golden/make_golden.py --reference /path/to/WorkloadSuite

It loads ``workloads/mamba/model_ref.py`` by file path (the way the reference's
own ``bench.py:104-115`` does), calls ``SSDLayer._ssd_core``
(``model_ref.py:123-162``) and the whole ``Model`` on small seeded inputs in the
reference's native fp16 on the CPU, and stores inputs and outputs as ``.npz``;
``layer_tiny`` also holds the intermediates of one ``SSDLayer.forward``.
The fixtures pin the CPU oracle (``oracle/ssd_oracle.py``) and, through it, the
CUDA kernels; nothing at test time needs the reference checkout.
"""
from __future__ import annotations

import argparse
import importlib.util
import math
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_reference(root: Path):
    path = root / "workloads" / "mamba" / "model_ref.py"
    spec = importlib.util.spec_from_file_location("ws_mamba_model_ref", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ws_mamba_model_ref"] = mod
    spec.loader.exec_module(mod)
    return mod


def core_case(mod, name, *, b, s, h, p, n, g, chunk, seed, decay_scale=1.0, with_dt=False):
    gen = torch.Generator().manual_seed(seed)
    X = torch.randn(b, s, h, p, generator=gen).half()
    Bm = torch.randn(b, s, g, n, generator=gen).half()
    Cm = torch.randn(b, s, g, n, generator=gen).half()
    dtv = torch.nn.functional.softplus(torch.randn(b, s, h, generator=gen) - 4.0)
    A_log = torch.empty(h).uniform_(math.log(1.0), math.log(16.0), generator=gen)
    A = (-dtv * torch.exp(A_log) * decay_scale).float()
    dt = (dtv.half() * 8.0) if with_dt else torch.ones(b, s, h, dtype=torch.float16)

    layer = mod.SSDLayer(d_model=64, n_heads=h, d_state=n, d_head=p, n_groups=g, block_len=chunk)
    r = h // g
    Bh = Bm.repeat_interleave(r, dim=2)
    Ch = Cm.repeat_interleave(r, dim=2)
    c = s // chunk
    with torch.inference_mode():
        Y = layer._ssd_core(
            X.reshape(b, c, chunk, h, p), Bh.reshape(b, c, chunk, h, n), Ch.reshape(b, c, chunk, h, n),
            dt.reshape(b, c, chunk, h), A.reshape(b, c, chunk, h), b,
        )
    Y = Y.reshape(b, s, h, p)
    assert torch.isfinite(Y).all()
    out = dict(X=X.numpy(), A=A.numpy(), B=Bm.numpy(), C=Cm.numpy(), Y=Y.numpy(), chunk=np.int64(chunk))
    if with_dt:
        out["dt"] = dt.numpy()
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, tuple(Y.shape), "max|Y| =", float(Y.abs().max()))


def model_case(mod, name, *, d_model, n_layers, n_heads, d_state, d_head, n_groups, block_len, b, s, seed):
    torch.manual_seed(seed)
    model = mod.Model(d_model, n_layers, n_heads, d_state, d_head, n_groups, block_len, 4).eval()
    with torch.no_grad():
        for layer in model.layers:
            # the default A_log/dt_bias give decays of exp(-0.018*k); keep them
            layer.D.copy_(torch.randn(n_heads).half())
    gen = torch.Generator().manual_seed(seed + 1)
    u = torch.randn(b, s, d_model, generator=gen).half()
    with torch.inference_mode():
        y = model(u)
    assert torch.isfinite(y).all()
    out = {"__input": u.numpy(), "__output": y.numpy(),
           "__init": np.array([d_model, n_layers, n_heads, d_state, d_head, n_groups, block_len, 4], dtype=np.int64)}
    for k, v in model.state_dict().items():
        out[k] = v.numpy()
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, tuple(y.shape), "max|y| =", float(y.abs().max()))


def layer_case(mod, name, *, d_model, n_heads, d_state, d_head, n_groups, block_len, b, s, seed):
    """Intermediates of ONE unmodified ``SSDLayer.forward`` (``model_ref.py:68-121``), captured with hooks and by
    wrapping the bound ``_ssd_core`` of the instance (the source is not touched): the projection output, what the
    core receives (x after conv+SiLU, dt after softplus, A_dt) and returns, and what ``out_proj`` receives (the
    core output after skip and gate)."""
    torch.manual_seed(seed)
    layer = mod.SSDLayer(d_model=d_model, n_heads=n_heads, d_state=d_state, d_head=d_head, n_groups=n_groups,
                         block_len=block_len).eval()
    with torch.no_grad():
        layer.D.copy_(torch.randn(n_heads).half())
        layer.dt_bias.copy_((torch.randn(n_heads) - 3.0).half())
    cap = {}
    layer.in_proj.register_forward_hook(lambda m, i, o: cap.__setitem__("zxbcdt", o.detach().clone()))
    layer.out_proj.register_forward_pre_hook(lambda m, i: cap.__setitem__("y_gated", i[0].detach().clone()))
    inner = layer._ssd_core

    def spy(X_b, B_b, C_b, dt_b, A_dt_b, batch):
        Y = inner(X_b, B_b, C_b, dt_b, A_dt_b, batch)
        cap.update(x=X_b.detach().clone(), dt=dt_b.detach().clone(), A_dt=A_dt_b.detach().clone(),
                   y_core=Y.detach().clone())
        return Y

    layer._ssd_core = spy
    gen = torch.Generator().manual_seed(seed + 1)
    u = torch.randn(b, s, d_model, generator=gen).half()
    with torch.inference_mode():
        out = layer(u)
    assert torch.isfinite(out).all()
    h, p = n_heads, d_head
    res = {
        "__shape": np.array([d_model, n_heads, d_state, d_head, n_groups, block_len, b, s], dtype=np.int64),
        "u": u.numpy(), "out": out.numpy(), "zxbcdt": cap["zxbcdt"].numpy(),
        "x": cap["x"].reshape(b, s, h, p).numpy(), "dt": cap["dt"].reshape(b, s, h).numpy(),
        "A_dt": cap["A_dt"].reshape(b, s, h).numpy(), "y_core": cap["y_core"].reshape(b, s, h, p).numpy(),
        "y_gated": cap["y_gated"].reshape(b, s, h, p).numpy(),
    }
    for k, v in layer.state_dict().items():
        res["w." + k] = v.numpy()
    np.savez_compressed(HERE / f"{name}.npz", **res)
    print(name, "max|y_gated| =", float(cap["y_gated"].abs().max()))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, required=True)
    args = ap.parse_args()
    mod = load_reference(args.reference)
    torch.set_num_threads(4)
    core_case(mod, "core_n16_q64", b=1, s=256, h=4, p=64, n=16, g=4, chunk=64, seed=11)
    core_case(mod, "core_n128_q64_slow", b=1, s=256, h=2, p=64, n=128, g=2, chunk=64, seed=12, decay_scale=0.05)
    core_case(mod, "core_n64_grouped_q32", b=2, s=128, h=4, p=64, n=64, g=2, chunk=32, seed=13, decay_scale=0.2)
    core_case(mod, "core_n128_q128_dt", b=1, s=256, h=2, p=64, n=128, g=1, chunk=128, seed=14, with_dt=True)
    model_case(mod, "model_tiny", d_model=64, n_layers=2, n_heads=2, d_state=128, d_head=64, n_groups=1,
               block_len=64, b=2, s=128, seed=21)
    layer_case(mod, "layer_tiny", d_model=64, n_heads=4, d_state=64, d_head=64, n_groups=2, block_len=64, b=2, s=256,
               seed=31)


if __name__ == "__main__":
    main()
