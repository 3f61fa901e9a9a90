"""The CPU oracle against the reference's own outputs and against the fp64 definition.

Golden ``.npz`` files were produced by ``tests/golden/make_golden.py`` from the
unmodified reference ``SSDLayer._ssd_core`` (``workloads/mamba/model_ref.py:123-162``).
"""
import numpy as np
import pytest
import torch

from oracle import ssd_oracle as O

CORE_CASES = ["core_n16_q64", "core_n128_q64_slow", "core_n64_grouped_q32", "core_n128_q128_dt"]


def _load(golden_dir, name):
    z = np.load(golden_dir / f"{name}.npz")
    d = {k: torch.from_numpy(z[k]) for k in z.files if k != "chunk"}
    d["chunk"] = int(z["chunk"])
    return d


@pytest.mark.parametrize("name", CORE_CASES)
def test_chunked_oracle_is_bit_identical_to_reference_fp16(golden_dir, name):
    d = _load(golden_dir, name)
    Y = O.ssd_chunked(d["X"], d["A"], d["B"], d["C"], d["chunk"], dt=d.get("dt"), dtype=torch.float16)
    assert Y.dtype == torch.float16
    assert torch.equal(Y, d["Y"])


@pytest.mark.parametrize("name", CORE_CASES)
def test_recurrence_agrees_with_reference_within_fp16_rounding(golden_dir, name):
    d = _load(golden_dir, name)
    Y = O.ssd_recurrence(d["X"], d["A"], d["B"], d["C"], dt=d.get("dt"))
    per_bh, fro = O.error_metrics(d["Y"], Y)
    assert per_bh < 5e-3 and fro < 2e-3, (per_bh, fro)


def test_chunked_fp64_equals_recurrence():
    inp = O.make_inputs(b=2, s=96, h=4, p=8, n=12, g=2, dtype=torch.float64, init=True, seed=3, decay_scale=0.3)
    Yc, Hc = O.ssd_chunked(inp["X"], inp["A"], inp["B"], inp["C"], 32, initial_states=inp["initial_states"],
                           dtype=torch.float64, return_final_state=True)
    Yr, Hr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], initial_states=inp["initial_states"],
                              return_final_state=True)
    assert O.error_metrics(Yc, Yr)[0] < 1e-12
    assert (Hc - Hr).abs().max() / Hr.abs().max() < 1e-12


def test_chunk_length_independence_fp64():
    inp = O.make_inputs(b=1, s=128, h=2, p=4, n=6, g=1, dtype=torch.float64, seed=4, decay_scale=0.1)
    Y16 = O.ssd_chunked(inp["X"], inp["A"], inp["B"], inp["C"], 16, dtype=torch.float64)
    Y64 = O.ssd_chunked(inp["X"], inp["A"], inp["B"], inp["C"], 64, dtype=torch.float64)
    assert O.error_metrics(Y16, Y64)[0] < 1e-12


def test_config0_fp32_within_1e4_of_definition():
    cfg = dict(O.CONFIGS["cfg0"])
    inp = O.make_inputs(seed=0, **cfg)
    Y = O.ssd_chunked(inp["X"], inp["A"], inp["B"], inp["C"], cfg["chunk"], dtype=torch.float32)
    Yr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"])
    per_bh, fro = O.error_metrics(Y, Yr)
    assert per_bh < 1e-4 and fro < 1e-4, (per_bh, fro)


def test_rejects_ragged_sequence_and_bad_groups():
    inp = O.make_inputs(b=1, s=48, h=4, p=4, n=4, g=2, dtype=torch.float32, seed=1)
    with pytest.raises(ValueError):
        O.ssd_chunked(inp["X"], inp["A"], inp["B"], inp["C"], 32)
    bad = O.make_inputs(b=1, s=32, h=4, p=4, n=4, g=3, dtype=torch.float32, seed=1)
    with pytest.raises(ValueError):
        O.ssd_chunked(bad["X"], bad["A"], bad["B"], bad["C"], 32)


def test_sequence_shard_fold_reproduces_unsharded_state():
    R = 4
    inp = O.make_inputs(b=2, s=64 * R, h=3, p=4, n=5, g=1, dtype=torch.float64, init=True, seed=5, decay_scale=0.02)
    _, Hfull = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], initial_states=inp["initial_states"],
                                return_final_state=True)
    Yfull = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], initial_states=inp["initial_states"])
    finals, lds = [], []
    for r in range(R):
        sl = slice(64 * r, 64 * (r + 1))
        _, F = O.ssd_recurrence(inp["X"][:, sl], inp["A"][:, sl], inp["B"][:, sl], inp["C"][:, sl],
                                return_final_state=True)
        finals.append(F)
        lds.append(O.total_logdecay(inp["A"][:, sl]))
    finals, lds = torch.stack(finals), torch.stack(lds)
    for r in range(R):
        sl = slice(64 * r, 64 * (r + 1))
        Hin = O.fold_incoming_state(finals, lds, r, initial=inp["initial_states"])
        Yr = O.ssd_recurrence(inp["X"][:, sl], inp["A"][:, sl], inp["B"][:, sl], inp["C"][:, sl], initial_states=Hin)
        assert O.error_metrics(Yr, Yfull[:, sl])[0] < 1e-12
    Hend = O.fold_incoming_state(finals, lds, R, initial=inp["initial_states"])
    assert (Hend - Hfull).abs().max() / Hfull.abs().max() < 1e-12


def test_layer_oracle_reproduces_reference_model_output(golden_dir):
    """``ssd_layer_pre`` -> ``ssd_chunked`` -> ``ssd_epilogue`` -> ``out_proj`` (the oracle's restatement of
    ``SSDLayer.forward``, ``model_ref.py:68-121``) against the output the unmodified reference model produced
    for the same weights and input (fixture written by tests/golden/make_golden.py)."""
    from workloadsuite_b200 import mamba_model as M

    z = np.load(golden_dir / "model_tiny.npz")
    model = M.Model(*[int(v) for v in z["__init"]]).eval()
    model.load_state_dict({k: torch.from_numpy(z[k]) for k in z.files if not k.startswith("__")}, strict=True)
    u = torch.from_numpy(z["__input"])
    with torch.inference_mode():
        for layer in model.layers:
            x, zz, B, C, dt, A_dt = O.ssd_layer_pre(layer, u)
            Y = O.ssd_chunked(x, A_dt, B, C, layer.block_len, dt=dt)
            Y = O.ssd_epilogue(Y, x, layer.D, zz.reshape(Y.shape))
            u = u + layer.out_proj(Y.reshape(u.shape[0], u.shape[1], -1))
        out = model.final_norm(u)
    ref = torch.from_numpy(z["__output"])
    assert out.dtype == ref.dtype
    err = (out.double() - ref.double()).abs().max().item() / ref.double().abs().max().item()
    assert err < 2e-3, err   # same operations in the same precision; only kernel-level summation order may differ


def _layer_fixture(golden_dir):
    z = np.load(golden_dir / "layer_tiny.npz")
    d_model, h, n, p, g, block_len, b, s = [int(v) for v in z["__shape"]]
    t = {k: torch.from_numpy(z[k]) for k in z.files if k != "__shape"}
    d_inner, gn = h * p, g * n
    x_raw, zz, B, C, dt_raw = torch.split(t["zxbcdt"], [d_inner, d_inner, gn, gn, h], dim=-1)
    t.update(x_raw=x_raw, z=zz.reshape(b, s, h, p), B=B.reshape(b, s, g, n), C=C.reshape(b, s, g, n), dt_raw=dt_raw)
    return t, block_len


def test_oracle_pieces_equal_the_reference_layer_intermediates(golden_dir):
    """Conv+SiLU, dt discretisation, core and skip/gate of the oracle against what the unmodified reference layer
    computed at the same points (fixture ``layer_tiny.npz``, captured with hooks): bit-identical in fp16."""
    import torch.nn.functional as F

    t, block_len = _layer_fixture(golden_dir)
    x = O.causal_conv1d_silu(t["x_raw"], t["w.conv1d.weight"], t["w.conv1d.bias"])
    assert torch.equal(x.reshape(t["x"].shape), t["x"])                                    # model_ref.py:83-89
    dt = F.softplus(t["dt_raw"] + t["w.dt_bias"])                                            # :94
    assert torch.equal(dt, t["dt"])
    A_dt = -torch.exp(t["w.A_log"]) * dt.float()                                             # :102-103
    assert torch.equal(A_dt, t["A_dt"])
    Y = O.ssd_chunked(t["x"], t["A_dt"], t["B"], t["C"], block_len, dt=t["dt"])               # :123-162
    assert torch.equal(Y, t["y_core"])
    assert torch.equal(O.ssd_epilogue(Y, t["x"], t["w.D"], t["z"]), t["y_gated"])             # :116-118


def test_reference_bytecode_reproduces_the_golden_outputs(golden_dir):
    """``oracle/_ref`` (the unmodified reference, byte-compiled by ``oracle/build_ref.py`` where the checkout is
    present) is what the benchmark's CPU arm times: it must give the golden outputs bit for bit."""
    import numpy as np

    from oracle import build_ref as R

    mod = R.load_model_ref()
    if mod is None:
        pytest.skip("oracle/_ref was not built on this machine")
    assert R.load_ref_bench() is not None
    for name in ("core_n16_q64", "core_n64_grouped_q32", "core_n128_q128_dt"):
        z = np.load(golden_dir / f"{name}.npz")
        d = {k: torch.from_numpy(z[k]) for k in z.files if k != "chunk"}
        h, g = d["X"].shape[2], d["B"].shape[2]
        Bh, Ch = d["B"].repeat_interleave(h // g, 2), d["C"].repeat_interleave(h // g, 2)
        with torch.inference_mode():
            Y = R.reference_core(mod, d["X"], d["A"], Bh, Ch, int(z["chunk"]), dt=d.get("dt"))
        assert torch.equal(Y, d["Y"]), name
