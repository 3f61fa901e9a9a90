"""Parity of the CUDA SSD forward (called through the C ABI) with the CPU oracle.

Tolerances (worst per-(batch, head) max-abs error over max-abs reference, and global
relative Frobenius error): 1e-4 for float32, 2e-2 for bfloat16/float16 -- the figures
the task states per dtype.  The oracle is the float64 token recurrence unless a golden
output of the reference itself is available."""
import numpy as np
import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-4, torch.float16: 2e-2, torch.bfloat16: 2e-2}
DEV = "cuda:0"


def _ssd():
    import workloadsuite_b200 as W

    return W


@pytest.fixture(autouse=True)
def _no_device_side_timeouts():
    """Every kernel wait is bounded; a wait that ran out leaves a code in the status word."""
    yield
    if torch.cuda.is_available():
        assert _ssd().device_status(DEV) == 0


def _kernels_for(dtype, p, n):
    ks = ["scan_f32"]
    if dtype in (torch.float16, torch.bfloat16) and p == 64 and n in (64, 128):
        ks.append("tcgen05")
    return ks


def _tc_available():
    W = _ssd()
    X = torch.zeros(1, 128, 1, 64, dtype=torch.bfloat16, device=DEV)
    A = torch.zeros(1, 128, 1, device=DEV)
    B = torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16, device=DEV)
    return W.kernel_name(X, A, B, B, 128) == "tcgen05"


def _to_dev(inp):
    return {k: v.to(DEV) for k, v in inp.items()}


def _run_and_check(inp, chunk, kernel=None, tol=None, dt=None, **kw):
    W = _ssd()
    d = _to_dev(inp)
    init = d.get("initial_states")
    dtd = dt.to(DEV) if dt is not None else None
    out = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], chunk, dt=dtd, initial_states=init, return_final_state=True,
                        kernel=kernel, **kw)
    Y, H = out
    torch.cuda.synchronize()
    Yr, Hr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], dt=dt, initial_states=inp.get("initial_states"),
                              return_final_state=True)
    per_bh, fro = O.error_metrics(Y.cpu(), Yr)
    tol = tol or TOL[inp["X"].dtype]
    assert per_bh < tol and fro < tol, (kernel, per_bh, fro)
    herr = ((H.cpu().double() - Hr).abs().amax(dim=(2, 3)) / Hr.abs().amax(dim=(2, 3)).clamp_min(1e-30)).max().item()
    assert herr < tol, ("final state", kernel, herr)
    return Y, H


# ---------------------------------------------------------------- golden fixtures (reference outputs)

@pytest.mark.parametrize("name", ["core_n16_q64", "core_n128_q64_slow", "core_n64_grouped_q32", "core_n128_q128_dt"])
def test_matches_reference_golden_fp16(golden_dir, name):
    W = _ssd()
    z = np.load(golden_dir / f"{name}.npz")
    d = {k: torch.from_numpy(z[k]).to(DEV) for k in z.files if k != "chunk"}
    chunk = int(z["chunk"])
    n = d["B"].shape[-1]
    for kernel in _kernels_for(torch.float16, 64, n):
        if kernel == "tcgen05" and not _tc_available():
            continue
        Y = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], chunk, dt=d.get("dt"), kernel=kernel)
        per_bh, fro = O.error_metrics(Y.cpu(), d["Y"].cpu())
        assert per_bh < 2e-2 and fro < 2e-2, (name, kernel, per_bh, fro)


# ---------------------------------------------------------------- the benchmark configurations

def test_config0_fp32_full_size():
    cfg = dict(O.CONFIGS["cfg0"])
    inp = O.make_inputs(seed=0, **cfg)
    _run_and_check(inp, cfg["chunk"])


SHRUNK = {
    # same head/state geometry and distributions as the named config, fewer tokens/heads
    "cfg1": dict(b=2, s=512, h=3, p=64, n=128, g=1, chunk=256, dtype="bf16", decay="mamba"),
    "cfg2": dict(b=1, s=1024, h=4, p=64, n=128, g=1, chunk=256, dtype="bf16", decay="mamba"),
    "cfg3": dict(b=1, s=2048, h=2, p=64, n=128, g=1, chunk=256, dtype="bf16", decay="mamba"),
    "cfg4": dict(b=3, s=512, h=12, p=64, n=64, g=2, chunk=128, dtype="bf16", init=True, decay="mamba"),
}


@pytest.mark.parametrize("name", sorted(SHRUNK))
@pytest.mark.parametrize("decay_scale", [1.0, 0.02])
def test_shrunken_configs_bf16(name, decay_scale):
    cfg = dict(SHRUNK[name])
    inp = O.make_inputs(seed=1, decay_scale=decay_scale, **cfg)
    for kernel in _kernels_for(torch.bfloat16, cfg["p"], cfg["n"]):
        if kernel == "tcgen05" and not _tc_available():
            continue
        _run_and_check(inp, cfg["chunk"], kernel=kernel)


# ---------------------------------------------------------------- edge cases

@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_single_chunk_and_many_chunks(dtype):
    for s, chunk in [(64, 64), (128, 128), (1024, 32)]:
        inp = O.make_inputs(b=1, s=s, h=2, p=64, n=64, g=2, dtype=dtype, seed=2, decay_scale=0.1)
        for kernel in _kernels_for(dtype, 64, 64):
            if kernel == "tcgen05" and (not _tc_available() or s % 128):
                continue
            _run_and_check(inp, chunk, kernel=kernel)


@pytest.mark.parametrize("g", [1, 2, 8])
def test_group_counts(g):
    inp = O.make_inputs(b=2, s=256, h=8, p=64, n=64, g=g, dtype=torch.bfloat16, seed=3, decay_scale=0.05)
    for kernel in _kernels_for(torch.bfloat16, 64, 64):
        if kernel == "tcgen05" and not _tc_available():
            continue
        _run_and_check(inp, 128, kernel=kernel)


def test_initial_state_axis_order_with_p_not_equal_n():
    # state layout is [b,h,n,p] (the carry of model_ref.py:153); p=32, n=64 tells the axes apart
    inp = O.make_inputs(b=2, s=128, h=4, p=32, n=64, g=1, dtype=torch.float32, init=True, seed=4, decay_scale=0.05)
    _run_and_check(inp, 64)
    inp = O.make_inputs(b=1, s=128, h=2, p=128, n=32, g=2, dtype=torch.float32, init=True, seed=4, decay_scale=0.05)
    _run_and_check(inp, 64)


def test_fast_decay_underflows_cleanly():
    inp = O.make_inputs(b=1, s=256, h=2, p=64, n=128, g=1, dtype=torch.bfloat16, seed=5, decay_scale=40.0)
    for kernel in _kernels_for(torch.bfloat16, 64, 128):
        if kernel == "tcgen05" and not _tc_available():
            continue
        Y, H = _run_and_check(inp, 128, kernel=kernel)
        assert torch.isfinite(Y).all() and torch.isfinite(H).all()


def test_dt_scaling():
    inp = O.make_inputs(b=1, s=256, h=2, p=64, n=64, g=1, dtype=torch.float16, seed=6, decay_scale=0.1)
    dt = (torch.rand(1, 256, 2) + 0.5).half()
    for kernel in _kernels_for(torch.float16, 64, 64):
        if kernel == "tcgen05" and not _tc_available():
            continue
        _run_and_check(inp, 64, kernel=kernel, dt=dt)


def test_strided_views_are_accepted():
    W = _ssd()
    inp = O.make_inputs(b=2, s=256, h=4, p=64, n=64, g=2, dtype=torch.bfloat16, seed=7, decay_scale=0.1)
    d = _to_dev(inp)
    # X, B, C as slices of one wide projection output, the way the block produces them (model_ref.py:76)
    wide = torch.zeros(2, 256, 4 * 64 + 2 * 2 * 64 + 8, dtype=torch.bfloat16, device=DEV)
    wide[..., : 256] = d["X"].flatten(2)
    wide[..., 256: 384] = d["B"].flatten(2)
    wide[..., 384: 512] = d["C"].flatten(2)
    Xv = wide[..., :256].unflatten(-1, (4, 64))
    Bv = wide[..., 256:384].unflatten(-1, (2, 64))
    Cv = wide[..., 384:512].unflatten(-1, (2, 64))
    assert not Xv.is_contiguous()
    for kernel in _kernels_for(torch.bfloat16, 64, 64):
        if kernel == "tcgen05" and not _tc_available():
            continue
        Y1 = W.ssd_forward(Xv, d["A"], Bv, Cv, 128, kernel=kernel)
        Y2 = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 128, kernel=kernel)
        assert torch.equal(Y1, Y2)


def test_ragged_and_invalid_arguments_raise():
    W = _ssd()
    inp = _to_dev(O.make_inputs(b=1, s=192, h=4, p=64, n=64, g=2, dtype=torch.float32, seed=8))
    with pytest.raises(ValueError):
        W.ssd_forward(inp["X"], inp["A"], inp["B"], inp["C"], 128)          # 192 % 128 (model_ref.py:106)
    bad = _to_dev(O.make_inputs(b=1, s=128, h=4, p=64, n=64, g=3, dtype=torch.float32, seed=8))
    with pytest.raises(ValueError):
        W.ssd_forward(bad["X"], bad["A"], bad["B"], bad["C"], 64)           # 4 % 3 (model_ref.py:37-38)
    odd = _to_dev(O.make_inputs(b=1, s=64, h=2, p=48, n=16, g=1, dtype=torch.float32, seed=8))
    with pytest.raises(NotImplementedError):
        W.ssd_forward(odd["X"], odd["A"], odd["B"], odd["C"], 64)           # head dim outside the kernels


# ---------------------------------------------------------------- segmentation (scratch-memory path)

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_segmented_scan_equals_unsegmented(dtype):
    inp = O.make_inputs(b=1, s=1024, h=2, p=64, n=64, g=1, dtype=dtype, init=True, seed=9, decay_scale=0.02)
    for kernel in _kernels_for(dtype, 64, 64):
        if kernel == "tcgen05" and not _tc_available():
            continue
        Y1, H1 = _run_and_check(inp, 128, kernel=kernel, nsegments=1)
        Y4, H4 = _run_and_check(inp, 128, kernel=kernel, nsegments=4)
        assert O.error_metrics(Y4.cpu(), Y1.cpu())[0] < TOL[dtype]
        Y3, _ = _run_and_check(inp, 128, kernel=kernel, nsegments=3)   # last segment shorter
        assert O.error_metrics(Y3.cpu(), Y1.cpu())[0] < TOL[dtype]


def test_chained_segments_tensor_core():
    """At least one (batch, head-pair) sequence per SM: the tiles of all sequences are dealt out evenly over the
    CTAs of one launch, and a sequence cut that way hands its state from CTA to CTA through scratch."""
    if not _tc_available():
        pytest.skip("tensor-core kernel not available")
    W = _ssd()
    inp = O.make_inputs(b=40, s=1024, h=8, p=64, n=128, g=2, dtype=torch.bfloat16, init=True, seed=21,
                        decay_scale=0.02)
    d = _to_dev(inp)
    assert W.plan(d["X"], d["A"], d["B"], d["C"], 256, nsegments=4)["launches"] == 1
    Y1, H1 = _run_and_check(inp, 256, kernel="tcgen05", nsegments=1)
    Y4, H4 = _run_and_check(inp, 256, kernel="tcgen05", nsegments=4)
    assert O.error_metrics(Y4.cpu(), Y1.cpu())[0] < 2e-2
    H, D = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 256, state_only=True, return_logdecay=True,
                         kernel="tcgen05", nsegments=2, initial_states=d["initial_states"])
    assert ((H - H1).abs().max() / H1.abs().max()) < 1e-3
    assert torch.allclose(D.cpu().double(), O.total_logdecay(inp["A"]), rtol=1e-5, atol=1e-5)


def test_one_head_per_cta_variant_when_groups_are_single_heads():
    """Heads that do not pair up inside a B/C group (one head per group) take the single-head kernel."""
    if not _tc_available():
        pytest.skip("tensor-core kernel not available")
    inp = O.make_inputs(b=2, s=512, h=3, p=64, n=128, g=3, dtype=torch.float16, init=True, seed=22, decay_scale=0.05)
    _run_and_check(inp, 128, kernel="tcgen05")
    _run_and_check(inp, 128, kernel="tcgen05", nsegments=2)


def test_reuse_of_segment_states_after_a_state_only_run():
    """The sequence-sharded forward runs state-only, exchanges states, then runs again seeded: the second
    run may reuse the per-segment states of the first (two-pass segmented scan)."""
    W = _ssd()
    inp = O.make_inputs(b=1, s=2048, h=4, p=64, n=128, g=1, dtype=torch.bfloat16, init=True, seed=23,
                        decay_scale=0.01)
    d = _to_dev(inp)
    for kernel in _kernels_for(torch.bfloat16, 64, 128):
        if kernel == "tcgen05" and not _tc_available():
            continue
        want = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 256, initial_states=d["initial_states"], kernel=kernel,
                             nsegments=4)
        W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 256, state_only=True, kernel=kernel, nsegments=4)
        got = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 256, initial_states=d["initial_states"], kernel=kernel,
                            nsegments=4, reuse_segments=True)
        # (the plain tensor-core run joins its pieces in another order of operations: look-back in one launch)
        assert max(O.error_metrics(got.cpu(), want.cpu())) < 5e-3
        again = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 256, initial_states=d["initial_states"], kernel=kernel,
                              nsegments=4, reuse_segments=True)
        assert torch.equal(got, again)


def test_state_only_and_logdecay_outputs():
    W = _ssd()
    inp = O.make_inputs(b=2, s=512, h=3, p=64, n=64, g=1, dtype=torch.bfloat16, seed=10, decay_scale=0.05)
    d = _to_dev(inp)
    for nseg in (1, 4):
        H, D = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 128, state_only=True, return_logdecay=True,
                             kernel="scan_f32", nsegments=nseg)
        _, Hr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], return_final_state=True)
        assert ((H.cpu().double() - Hr).abs().max() / Hr.abs().max()) < 1e-4
        assert torch.allclose(D.cpu().double(), O.total_logdecay(inp["A"]), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_token_by_token_steps_with_a_carried_state_equal_one_forward(dtype):
    """Decode-style use of the same entry point: one token per call (``chunk`` 1), the state carried from call to
    call through ``initial_states`` / ``return_final_state`` (the carry of ``model_ref.py:152-157``), against the
    unsharded float64 recurrence over the whole run of tokens and against one forward over all of them."""
    W = _ssd()
    steps = 6
    inp = O.make_inputs(b=3, s=steps, h=8, p=64, n=128, g=2, dtype=dtype, init=True, seed=23)
    d = {k: v.to(DEV) for k, v in inp.items()}
    H = d["initial_states"]
    ys = []
    for t in range(steps):
        sl = slice(t, t + 1)
        y, H = W.ssd_forward(d["X"][:, sl], d["A"][:, sl], d["B"][:, sl], d["C"][:, sl], 1, initial_states=H,
                             return_final_state=True)
        ys.append(y)
    Y = torch.cat(ys, dim=1).cpu()
    Yr, Hr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], initial_states=inp["initial_states"],
                              return_final_state=True)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert O.error_metrics(Y, Yr)[0] < tol
    assert float((H.cpu() - Hr.float()).abs().max() / Hr.abs().max()) < 1e-5
    Y1, H1 = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 1, initial_states=d["initial_states"], return_final_state=True)
    assert O.error_metrics(Y1.cpu(), Yr)[0] < tol
    assert float((H1.cpu() - H.cpu()).abs().max() / Hr.abs().max()) < 1e-5
    assert W.device_status(DEV) == 0


@pytest.mark.parametrize("dtype,n,g,epi", [(torch.bfloat16, 128, 2, True), (torch.float16, 64, 1, False),
                                           (torch.float32, 16, 4, True), (torch.bfloat16, 256, 8, False),
                                           (torch.float16, 32, 2, True)])
def test_step_kernel_equals_the_recurrence_and_the_forward(dtype, n, g, epi):
    """``ssd_step`` token by token (state carried in place) against the float64 recurrence over the whole run of
    tokens, and against ``ssd_forward`` over the same tokens; with the layer's skip and gate in one of the cases."""
    W = _ssd()
    steps, b, h = 5, 3, 8
    inp = O.make_inputs(b=b, s=steps, h=h, p=64, n=n, g=g, dtype=dtype, init=True, seed=31, decay_scale=0.3)
    gen = torch.Generator().manual_seed(32)
    dt = (0.05 + torch.rand(b, steps, h, generator=gen)).to(dtype)
    D = torch.randn(h, generator=gen) if epi else None
    z = torch.randn(b, steps, h, 64, generator=gen).to(dtype) if epi else None
    d = _to_dev(inp)
    state = d["initial_states"].clone()
    ys = []
    for t in range(steps):
        ys.append(W.ssd_step(d["X"][:, t], d["A"][:, t], d["B"][:, t], d["C"][:, t], state, dt=dt[:, t].to(DEV),
                             D=None if D is None else D.to(DEV), z=None if z is None else z[:, t].to(DEV)))
    Y = torch.stack(ys, dim=1).cpu()
    Yr, Hr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], dt=dt, initial_states=inp["initial_states"],
                              return_final_state=True)
    if epi:
        Yr = O.ssd_epilogue(Yr, inp["X"].double(), D.double(), z.double(), dtype=torch.float64)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert max(O.error_metrics(Y, Yr)) < tol
    assert float((state.cpu().double() - Hr).abs().max() / Hr.abs().max()) < (1e-5 if dtype == torch.float32 else 5e-3)
    try:
        Yf, Hf = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 1, dt=dt.to(DEV), initial_states=d["initial_states"],
                               return_final_state=True, D=None if D is None else D.to(DEV),
                               z=None if z is None else z.to(DEV))
    except NotImplementedError:      # (a state size only the step kernel covers)
        return
    assert max(O.error_metrics(Y, Yf.cpu().double())) < tol
    assert float((state - Hf).abs().max() / Hf.abs().max()) < 5e-3


def test_fold_states_matches_oracle():
    W = _ssd()
    gen = torch.Generator().manual_seed(11)
    states = torch.randn(4, 2, 3, 16, 8, generator=gen)
    lds = -torch.rand(4, 2, 3, generator=gen)
    init = torch.randn(2, 3, 16, 8, generator=gen)
    for r in range(5):
        got = W.fold_states(states.to(DEV), lds.to(DEV), r, init.to(DEV)).cpu()
        want = O.fold_incoming_state(states, lds, r, init)
        assert torch.allclose(got.double(), want, rtol=1e-5, atol=1e-6)


def test_run_to_run_determinism():
    W = _ssd()
    inp = _to_dev(O.make_inputs(b=2, s=512, h=4, p=64, n=128, g=1, dtype=torch.bfloat16, seed=12))
    for kernel in _kernels_for(torch.bfloat16, 64, 128):
        if kernel == "tcgen05" and not _tc_available():
            continue
        Y1 = W.ssd_forward(inp["X"], inp["A"], inp["B"], inp["C"], 256, kernel=kernel)
        Y2 = W.ssd_forward(inp["X"], inp["A"], inp["B"], inp["C"], 256, kernel=kernel)
        assert torch.equal(Y1, Y2)


# ---------------------------------------------------------------- full-size configurations: properties

def _full(name, seed=0):
    cfg = dict(O.CONFIGS[name])
    return cfg, O.make_inputs(seed=seed, **cfg)


@pytest.mark.parametrize("name", ["cfg1", "cfg2"])
def test_full_size_properties(name):
    """At full size the oracle is too slow for every unit, so check (i) a sample of
    (batch, head) units against it, (ii) exact homogeneity Y(2X) == 2 Y(X) (scaling by two
    is exact in binary floating point) and (iii) splitting the sequence in two with the
    carried state reproduces the one-pass result."""
    W = _ssd()
    cfg, inp = _full(name)
    d = _to_dev(inp)
    chunk = cfg["chunk"]
    Y = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], chunk)
    assert torch.isfinite(Y).all()
    # (i) sampled units
    for (bi, hi) in [(0, 0), (cfg["b"] - 1, cfg["h"] - 1), (cfg["b"] // 2, cfg["h"] // 3)]:
        Yr = O.ssd_recurrence(inp["X"][bi:bi + 1, :, hi:hi + 1], inp["A"][bi:bi + 1, :, hi:hi + 1],
                              inp["B"][bi:bi + 1], inp["C"][bi:bi + 1])
        per_bh, fro = O.error_metrics(Y[bi:bi + 1, :, hi:hi + 1].cpu(), Yr)
        assert per_bh < 2e-2 and fro < 2e-2, (bi, hi, per_bh, fro)
    # (ii) homogeneity, bitwise
    Y2 = W.ssd_forward(d["X"] * 2, d["A"], d["B"], d["C"], chunk)
    assert torch.equal(Y2, Y * 2)
    # (iii) split + carry
    half = cfg["s"] // 2
    Ya, Ha = W.ssd_forward(d["X"][:, :half], d["A"][:, :half], d["B"][:, :half], d["C"][:, :half], chunk,
                           return_final_state=True)
    Yb = W.ssd_forward(d["X"][:, half:], d["A"][:, half:], d["B"][:, half:], d["C"][:, half:], chunk,
                       initial_states=Ha)
    per_bh, fro = O.error_metrics(torch.cat([Ya, Yb], 1).cpu(), Y.cpu())
    assert per_bh < 2e-2 and fro < 5e-3, (per_bh, fro)


def _check_sampled_units(Y, inp, units, H=None, tol=2e-2):
    """Sampled (batch, head) units of a full-size run against the float64 recurrence (one oracle call per batch
    entry, all its sampled heads at once)."""
    h, g = inp["X"].shape[2], inp["B"].shape[2]
    by_batch = {}
    for bi, hi in units:
        by_batch.setdefault(bi, []).append(hi)
    for bi, heads in by_batch.items():
        hs = torch.tensor(heads)
        gs = hs // (h // g)
        init = inp["initial_states"][bi:bi + 1, hs] if "initial_states" in inp else None
        # one oracle head per sampled head, each with the B/C of its own group (model_ref.py:97-99)
        Yr, Hr = O.ssd_recurrence(inp["X"][bi:bi + 1, :, hs], inp["A"][bi:bi + 1, :, hs], inp["B"][bi:bi + 1, :, gs],
                                  inp["C"][bi:bi + 1, :, gs], initial_states=init, return_final_state=True)
        per_bh, fro = O.error_metrics(Y[bi:bi + 1, :, hs.to(Y.device)].cpu(), Yr)
        assert per_bh < tol and fro < tol, (bi, heads, per_bh, fro)
        if H is not None:
            Hg = H[bi:bi + 1, hs.to(H.device)].cpu().double()
            herr = ((Hg - Hr).abs().amax(dim=(2, 3)) / Hr.abs().amax(dim=(2, 3)).clamp_min(1e-30)).max().item()
            assert herr < tol, ("final state", bi, heads, herr)


@pytest.mark.parametrize("decay_scale", [1.0, 0.02])
def test_full_size_config3_long_sequence(decay_scale):
    """Config 3 at its stated size (one sequence of 131 072 tokens, 32 heads: 16 head pairs of 1 024 tiles, dealt out
    over 148 CTAs in pieces of 110-111 tiles that fold up to nine predecessors): first, last and two middle heads
    against the float64 recurrence over all tokens, with the configuration's own decays and with slow decays (so
    that what crosses the cuts matters), plus the final state; and the two-pass path (state-only run, then the run
    that reuses its segment states) against the same."""
    W = _ssd()
    cfg, inp = _full("cfg3", seed=3)
    if decay_scale != 1.0:
        inp["A"] = inp["A"] * decay_scale
    d = _to_dev(inp)
    plan = W.plan(d["X"], d["A"], d["B"], d["C"], cfg["chunk"])
    assert plan["nsegments"] > 1 and plan["launches"] == 1 and plan["kernel"] == "tcgen05"     # look-back, 148 pieces
    Y, H = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], cfg["chunk"], return_final_state=True)
    torch.cuda.synchronize()
    assert torch.isfinite(Y).all() and torch.isfinite(H).all()
    _check_sampled_units(Y, inp, [(0, 0), (0, 13), (0, 18), (0, cfg["h"] - 1)], H=H)
    if decay_scale != 1.0:
        H2 = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], cfg["chunk"], state_only=True)
        Y2 = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], cfg["chunk"], reuse_segments=True)
        torch.cuda.synchronize()
        _check_sampled_units(Y2, inp, [(0, 0), (0, cfg["h"] - 1)], H=H2)


def test_full_size_config4_many_short_sequences_with_initial_states():
    """Config 4 at its stated size (256 x 48 units of 512 tokens, 8 B/C groups of 6 heads, d_state 64, fp32 initial
    states [256,48,64,64]): first, last and middle units, heads of different groups, Y and final state."""
    W = _ssd()
    cfg, inp = _full("cfg4", seed=4)
    assert inp["initial_states"].shape == (256, 48, 64, 64) and inp["B"].shape[2] == 8
    d = _to_dev(inp)
    Y, H = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], cfg["chunk"], initial_states=d["initial_states"],
                         return_final_state=True)
    torch.cuda.synchronize()
    assert torch.isfinite(Y).all() and torch.isfinite(H).all()
    units = [(0, 0), (0, 5), (0, 6), (255, 47), (255, 41), (128, 20), (77, 7), (3, 30)]   # groups 0, 1, 3, 5, 6, 7
    _check_sampled_units(Y, inp, units, H=H)
    # the same with slow decays: the initial state then reaches every token of the 512
    inp2 = dict(inp)
    inp2["A"] = inp["A"] * 0.02
    Y2, H2 = W.ssd_forward(d["X"], inp2["A"].to(DEV), d["B"], d["C"], cfg["chunk"], initial_states=d["initial_states"],
                           return_final_state=True)
    _check_sampled_units(Y2, inp2, [(0, 0), (255, 47), (100, 11)], H=H2)


# ---------------------------------------------------------------- the reference-side binding and the give-up path

def _integration_snippet():
    """The replacement body of ``SSDLayer._ssd_core`` exactly as INTEGRATION.md prints it."""
    import re
    from pathlib import Path

    text = (Path(__file__).resolve().parent.parent / "INTEGRATION.md").read_text()
    m = re.search(r"```python\n(from workloadsuite_b200 import ssd_forward\n.*?)```", text, re.S)
    assert m, "the binding snippet is missing from INTEGRATION.md"
    ns = {}
    exec(m.group(1), ns)
    return ns["_ssd_core"]


def test_reference_binding_accepts_the_reference_layers_own_layout():
    """``SSDLayer.forward`` hands ``_ssd_core`` an X that is sequence-contiguous and channel-strided (a permuted
    [b, d, l] tensor, model_ref.py:83-89,106) and B/C repeated to heads (:97-99).  The binding of INTEGRATION.md,
    run verbatim on tensors laid out that way, must equal the call on contiguous tensors."""
    W = _ssd()
    core = _integration_snippet()
    b, s, h, p, n, l = 2, 512, 4, 64, 128, 64
    inp = O.make_inputs(b=b, s=s, h=h, p=p, n=n, g=h, dtype=torch.float16, seed=51, decay_scale=0.1)
    d = _to_dev(inp)
    x_bdl = d["X"].reshape(b, s, h * p).transpose(1, 2).contiguous()            # [b, d, l], what the conv produces
    X = x_bdl.transpose(1, 2).view(b, s, h, p)                                   # rearrange "b d l -> b l d", :86-89
    assert X.stride() == (h * p * s, 1, p * s, s) and torch.equal(X, d["X"])
    dt = (0.5 + torch.rand(b, s, h, device=DEV)).half()
    c = s // l
    Y = core(None, X.reshape(b, c, l, h, p), d["B"].reshape(b, c, l, h, n), d["C"].reshape(b, c, l, h, n),
             dt.reshape(b, c, l, h), d["A"].reshape(b, c, l, h), b)
    want = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], l, dt=dt)
    assert Y.shape == (b, c, l, h, p) and torch.equal(Y.reshape(b, s, h, p), want)
    Yr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], dt=dt.cpu())
    assert max(O.error_metrics(want.cpu(), Yr)) < 2e-2


def test_reference_layer_with_the_binding_patched_in():
    """The unmodified reference ``SSDLayer`` (bytecode under oracle/_ref, when it was built) with only ``_ssd_core``
    replaced by the binding of INTEGRATION.md, against the same layer untouched, both on the GPU in fp16."""
    from oracle import build_ref as R

    mod = R.load_model_ref()
    if mod is None:
        pytest.skip("oracle/_ref was not built on this machine")
    core = _integration_snippet()
    torch.manual_seed(7)
    layer = mod.SSDLayer(d_model=256, n_heads=8, d_state=128, d_head=64, n_groups=2, block_len=64).to(DEV).eval()
    u = torch.randn(2, 512, 256, dtype=torch.float16, device=DEV)
    with torch.inference_mode():
        ref = layer(u)
        layer._ssd_core = core.__get__(layer)
        got = layer(u)
    err = ((got.double() - ref.double()).abs().max() / ref.double().abs().max()).item()
    assert err < 2e-2, err


def test_torch_compile_contract_of_the_dropin_model():
    """The reference harness compiles the very model instance it timed (bench.py:185: fullgraph=False) and the
    reference's tests check compiled == eager with the eager backend (tests/test_diverse_workloads.py:74-83)."""
    from workloadsuite_b200 import mamba_model as M

    torch.manual_seed(3)
    model = M.Model(128, 2, 4, 128, 64, 2, 64, 4).to(DEV).eval()
    x = torch.randn(2, 256, 128, dtype=torch.float16, device=DEV)
    try:
        with torch.inference_mode():
            want = model(x)
            compiled = torch.compile(model, backend="eager", fullgraph=False)
            got = compiled(x)
            got2 = compiled(x)
        assert torch.equal(got, want) and torch.equal(got2, want)
    finally:
        torch._dynamo.reset()


def test_gate_whose_rows_are_not_16_byte_aligned_takes_the_standalone_epilogue():
    W = _ssd()
    inp = O.make_inputs(b=1, s=256, h=4, p=64, n=128, g=1, dtype=torch.bfloat16, seed=52, decay_scale=0.05)
    d = _to_dev(inp)
    gen = torch.Generator().manual_seed(53)
    z = torch.randn(1, 256, 4, 64, generator=gen).bfloat16()
    D = torch.randn(4, generator=gen)
    buf = torch.zeros(z.numel() + 1, dtype=torch.bfloat16, device=DEV)
    zv = buf[1:].view(1, 256, 4, 64)                # same strides, address off by one element
    zv.copy_(z)
    assert zv.data_ptr() % 16 != 0
    Y = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 128, D=D.to(DEV), z=zv)
    Y2 = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 128, D=D.to(DEV), z=z.to(DEV), separate_epilogue=True)
    assert torch.equal(Y, Y2)


def test_a_wait_that_runs_out_is_reported_and_the_next_forward_is_fine():
    """Every device-side wait is bounded.  Here one is made to run out: in a launch whose sequences are handed from
    CTA to CTA, the first CTA leaves without publishing (``inject_lost_handover``), so the CTA that continues its
    sequence waits -- for 3 ms instead of the default second -- gives up, every role of that CTA leaves, tensor
    memory is freed, the kernel returns by itself and the status word reads 6.  The context stays usable: the same
    forward without the injection is then correct."""
    import time

    if not _tc_available():
        pytest.skip("tensor-core kernel not available")
    W = _ssd()
    # 200 head pairs x 4 tiles over 148 CTAs: the first CTA gets tiles 0..4, i.e. one whole sequence and the first
    # tile of the next, whose remaining tiles wait on the second CTA for a state that never comes
    inp = O.make_inputs(b=50, s=512, h=8, p=64, n=128, g=2, dtype=torch.bfloat16, seed=54, decay_scale=0.05)
    d = _to_dev(inp)
    assert W.plan(d["X"], d["A"], d["B"], d["C"], 256, nsegments=2)["launches"] == 1      # chained
    W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 256, nsegments=2)                       # warm
    assert W.device_status(DEV) == 0
    t0 = time.perf_counter()
    W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 256, nsegments=2, wait_limit_ms=3, inject_lost_handover=True)
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    assert W.device_status(DEV) == 6                 # STATUS_WAIT_TIMEOUT_CHAIN; the call above cleared the word
    assert took < 0.5, took                          # it gave up after milliseconds, not after the default second
    Y = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 256, nsegments=2)
    torch.cuda.synchronize()
    assert W.device_status(DEV) == 0
    Yr = O.ssd_recurrence(inp["X"][:2], inp["A"][:2], inp["B"][:2], inp["C"][:2])
    assert max(O.error_metrics(Y[:2].cpu(), Yr)) < 2e-2
    Yl = O.ssd_recurrence(inp["X"][-1:], inp["A"][-1:], inp["B"][-1:], inp["C"][-1:])
    assert max(O.error_metrics(Y[-1:].cpu(), Yl)) < 2e-2


# ---------------------------------------------------------------- host-buffer entry point and the drop-in Model

@pytest.mark.parametrize("case", ["pairs_bf16", "pairs_fp16_dt_segmented", "chained_bf16_dt", "single_heads_fp16", "fp32_simt",
                                  "skip_only", "gate_only"])
def test_skip_and_gate_epilogue(case):
    """``Y <- (Y + X * D) * silu(z)`` (``model_ref.py:116-118``) applied by the kernels: fused in the two-head
    tensor-core kernel, a kernel of its own behind the others.  Reference: fp64 recurrence + fp64 epilogue."""
    W = _ssd()
    kw = dict(p=64, n=128, g=1, init=False, decay_scale=0.05)
    nseg, kernel, use_dt, use_D, use_z = None, None, False, True, True
    if case == "pairs_bf16":
        shape = dict(b=2, s=512, h=4, dtype=torch.bfloat16, seed=41)
    elif case == "pairs_fp16_dt_segmented":
        shape, nseg, use_dt = dict(b=1, s=1024, h=4, dtype=torch.float16, seed=42), 4, True
    elif case == "chained_bf16_dt":
        shape, nseg, use_dt = dict(b=40, s=512, h=8, dtype=torch.bfloat16, seed=43), 2, True
        kw["g"] = 2
    elif case == "single_heads_fp16":
        shape = dict(b=2, s=256, h=3, dtype=torch.float16, seed=44)
        kw["g"] = 3
    elif case == "fp32_simt":
        shape, kernel = dict(b=2, s=256, h=4, dtype=torch.float32, seed=45), "scan_f32"
        kw["n"] = 16
    elif case == "skip_only":
        shape, use_z = dict(b=1, s=256, h=2, dtype=torch.bfloat16, seed=46), False
    else:
        shape, use_D = dict(b=1, s=256, h=2, dtype=torch.bfloat16, seed=47), False
    dtype = shape["dtype"]
    if dtype != torch.float32 and kernel is None and not _tc_available():
        pytest.skip("tensor-core kernel not available")
    inp = O.make_inputs(**shape, **kw)
    gen = torch.Generator().manual_seed(shape["seed"] + 100)
    b, s, h, p = inp["X"].shape
    D = torch.randn(h, generator=gen) if use_D else None
    z = torch.randn(b, s, h, p, generator=gen).to(dtype) if use_z else None
    dt = (0.05 + torch.rand(b, s, h, generator=gen)).to(dtype) if use_dt else None
    d = _to_dev(inp)
    Y = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 128, dt=None if dt is None else dt.to(DEV), kernel=kernel,
                      nsegments=nseg, D=None if D is None else D.to(DEV), z=None if z is None else z.to(DEV))
    torch.cuda.synchronize()
    Yr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], dt=dt)
    Yr = O.ssd_epilogue(Yr.double(), inp["X"].double(), None if D is None else D.double(),
                        None if z is None else z.double(), dtype=torch.float64)
    per_bh, fro = O.error_metrics(Y.cpu(), Yr)
    assert per_bh < TOL[dtype] and fro < TOL[dtype], (case, per_bh, fro)


@pytest.mark.parametrize("dtype,taps,sliced", [(torch.float16, 4, True), (torch.bfloat16, 4, False), (torch.float32, 3, True),
                                               (torch.float16, 2, False)])
def test_causal_conv1d_silu(dtype, taps, sliced):
    """The X producer (``model_ref.py:83-86``): CUDA kernel against the reference's operator calls in fp64; the input
    may be a column slice of a wider projection output, ragged last token chunk included."""
    W = _ssd()
    gen = torch.Generator().manual_seed(300 + taps)
    b, l, d = 3, 200, 192
    wide = torch.randn(b, l, d + 72, generator=gen).to(dtype)
    x = wide[..., 8:8 + d] if sliced else wide[..., :d].contiguous()
    weight = (torch.randn(d, 1, taps, generator=gen) * 0.5).to(dtype)
    bias = torch.randn(d, generator=gen).to(dtype)
    y = W.conv1d_silu(x.to(DEV) if not sliced else wide.to(DEV)[..., 8:8 + d], weight.to(DEV), bias.to(DEV))
    torch.cuda.synchronize()
    ref = O.causal_conv1d_silu(x, weight, bias, dtype=torch.float64)
    err = (y.cpu().double() - ref).abs().max().item() / ref.abs().max().item()
    assert y.shape == (b, l, d) and y.is_contiguous()
    assert err < (1e-5 if dtype == torch.float32 else 5e-3), err
    y2 = W.conv1d_silu(x.to(DEV).contiguous(), weight.to(DEV), None)
    ref2 = O.causal_conv1d_silu(x, weight, None, dtype=torch.float64)
    assert (y2.cpu().double() - ref2).abs().max().item() / ref2.abs().max().item() < (1e-5 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_dt_prologue(dtype):
    """``softplus(dt + dt_bias)`` and ``A_dt = -exp(A_log) dt.float()`` (``model_ref.py:94, 102-103``) against the same
    PyTorch operator calls on the CPU, from a column slice of a wider tensor."""
    import torch.nn.functional as F

    W = _ssd()
    gen = torch.Generator().manual_seed(77)
    b, l, h = 2, 300, 24
    wide = (torch.randn(b, l, h + 40, generator=gen) * 3 - 2).to(dtype)
    wide[0, 0, 8] = 30.0                                   # beyond softplus' linear threshold
    bias = (torch.randn(h, generator=gen) - 2).to(dtype)
    A_log = torch.log(torch.arange(1, h + 1, dtype=torch.float32))
    dt, A_dt = W.dt_prologue(wide.to(DEV)[..., 8:8 + h], bias.to(DEV), A_log.to(DEV))
    torch.cuda.synchronize()
    dt_ref = F.softplus(wide[..., 8:8 + h].float() + bias.float()) if dtype == torch.float32 else \
        F.softplus((wide[..., 8:8 + h] + bias).float()).to(dtype)
    A_ref = -torch.exp(A_log) * dt_ref.float()
    tol = 5e-6 if dtype == torch.float32 else 2 ** (-7 if dtype == torch.bfloat16 else -10)
    assert dt.dtype == dtype and A_dt.dtype == torch.float32
    assert ((dt.cpu().float() - dt_ref.float()).abs() / dt_ref.float().abs().clamp_min(1e-6)).max().item() < tol
    assert ((A_dt.cpu() - A_ref).abs() / A_ref.abs().clamp_min(1e-6)).max().item() < tol
    # A_dt is formed from the ROUNDED dt, as the reference does
    assert torch.allclose(A_dt.cpu(), -torch.exp(A_log) * dt.cpu().float(), rtol=1e-6, atol=0)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_randomised_shapes_modes_and_epilogues(seed):
    """Seeded random draws over group layout, state size, dtype, tiles per sequence, chunk, dt, initial state,
    segment count, state-only mode and the skip/gate epilogue (a few with enough sequences for the chained mode),
    against the fp64 recurrence; the device status word must stay clean."""
    import random

    if not _tc_available():
        pytest.skip("tensor-core kernel not available")
    W = _ssd()
    from workloadsuite_b200 import ssd as S

    rnd = random.Random(seed)
    for it in range(12):
        n, dtype = rnd.choice([64, 128]), rnd.choice([torch.bfloat16, torch.float16])
        g, hpg = rnd.choice([1, 2, 4]), rnd.choice([2, 4, 6])
        h = g * hpg
        tiles = rnd.choice([1, 2, 3, 5, 8])
        b = rnd.choice([1, 2, 3, 5]) if it % 4 else -(-300 // h)      # every fourth draw: >= 150 head pairs
        s = 128 * tiles
        chunk = rnd.choice([c for c in (32, 64, 128, 256) if s % c == 0])
        init, use_dt, epi = rnd.random() < 0.5, rnd.random() < 0.5, rnd.random() < 0.4
        nseg = rnd.choice([None, None, 2, 3])
        state_only = (not epi) and rnd.random() < 0.15
        inp = O.make_inputs(b=b, s=s, h=h, p=64, n=n, g=g, dtype=dtype, init=init, seed=100 * seed + it,
                            decay_scale=rnd.choice([1.0, 0.1, 0.02]))
        gen = torch.Generator().manual_seed(1000 * seed + it)
        dt = (0.02 + torch.rand(b, s, h, generator=gen)).to(dtype) if use_dt else None
        D = torch.randn(h, generator=gen) if epi else None
        z = torch.randn(b, s, h, 64, generator=gen).to(dtype) if epi else None
        d = _to_dev(inp)
        kw = dict(dt=None if dt is None else dt.to(DEV), initial_states=d.get("initial_states"), nsegments=nseg)
        if state_only:
            Y, H = None, W.ssd_forward(d["X"], d["A"], d["B"], d["C"], chunk, state_only=True, **kw)
        else:
            Y, H = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], chunk, return_final_state=True,
                                 D=None if D is None else D.to(DEV), z=None if z is None else z.to(DEV), **kw)
        torch.cuda.synchronize()
        assert S.device_status(DEV) == 0
        Yr, Hr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], dt=dt,
                                  initial_states=inp.get("initial_states"), return_final_state=True)
        herr = ((H.cpu().double() - Hr).abs().amax(dim=(2, 3)) / Hr.abs().amax(dim=(2, 3)).clamp_min(1e-30)).max().item()
        case = dict(it=it, b=b, s=s, h=h, g=g, n=n, dtype=dtype, chunk=chunk, nseg=nseg, dt=use_dt, init=init, epi=epi)
        assert herr < 2e-2, (case, herr)
        if Y is not None:
            if epi:
                Yr = O.ssd_epilogue(Yr, inp["X"].double(), D.double(), z.double(), dtype=torch.float64)
            assert max(O.error_metrics(Y.cpu(), Yr)) < 2e-2, case


def test_host_buffer_forward_equals_device_forward():
    W = _ssd()
    inp = O.make_inputs(b=3, s=512, h=8, p=64, n=64, g=2, dtype=torch.bfloat16, init=True, seed=13, decay_scale=0.1)
    d = _to_dev(inp)
    Yd = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], 128, initial_states=d["initial_states"])
    Yh = W.ssd_forward_host(inp["X"].pin_memory(), inp["A"].pin_memory(), inp["B"].pin_memory(),
                            inp["C"].pin_memory(), 128, initial_states=inp["initial_states"])
    assert not Yh.is_cuda
    assert torch.equal(Yh, Yd.cpu())


def test_host_buffer_forward_carries_the_state_across_sequence_chunks():
    """A batch entry longer than one host chunk: the scan continues from chunk to chunk through the device-resident
    state; initial and final states and the summed log-decay come through."""
    W = _ssd()
    inp = O.make_inputs(b=2, s=4096, h=16, p=64, n=128, g=2, dtype=torch.bfloat16, init=True, seed=14, decay_scale=0.02)
    r = W.HostRunner(2, 4096, 16, 64, 128, 2, 256, torch.bfloat16, device=str(DEV))
    out = torch.empty_like(inp["X"]).pin_memory()
    fin = torch.empty(2, 16, 128, 64).pin_memory()
    r.run(inp["X"].pin_memory(), inp["A"].pin_memory(), inp["B"].pin_memory(), inp["C"].pin_memory(), out,
          initial_states=inp["initial_states"].pin_memory(), final_state=fin)
    Yr, Hr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], initial_states=inp["initial_states"],
                              return_final_state=True)
    per_bh, fro = O.error_metrics(out, Yr)
    assert per_bh < 2e-2 and fro < 2e-2, (per_bh, fro)
    assert ((fin.double() - Hr).abs().max() / Hr.abs().max()).item() < 2e-2


def test_host_buffer_forward_groups_short_batch_entries():
    """Many short sequences: several whole batch entries travel and run as one chunk (the last group is smaller);
    per-entry initial and final states come through."""
    W = _ssd()
    inp = O.make_inputs(b=37, s=256, h=8, p=64, n=64, g=2, dtype=torch.bfloat16, init=True, seed=15, decay_scale=0.05)
    r = W.HostRunner(37, 256, 8, 64, 64, 2, 128, torch.bfloat16, device=str(DEV))
    out = torch.empty_like(inp["X"]).pin_memory()
    fin = torch.empty(37, 8, 64, 64).pin_memory()
    r.run(inp["X"].pin_memory(), inp["A"].pin_memory(), inp["B"].pin_memory(), inp["C"].pin_memory(), out,
          initial_states=inp["initial_states"].pin_memory(), final_state=fin)
    Yr, Hr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"], initial_states=inp["initial_states"],
                              return_final_state=True)
    per_bh, fro = O.error_metrics(out, Yr)
    assert per_bh < 2e-2 and fro < 2e-2, (per_bh, fro)
    herr = ((fin.double() - Hr).abs().amax(dim=(2, 3)) / Hr.abs().amax(dim=(2, 3)).clamp_min(1e-30)).max().item()
    assert herr < 2e-2, herr


def test_layer_kernels_match_reference_layer_intermediates(golden_dir):
    """Conv+SiLU, dt discretisation and core + fused skip/gate on the GPU against what the unmodified reference layer
    computed at the same points (``layer_tiny.npz``: captured with hooks inside ``SSDLayer.forward``)."""
    W = _ssd()
    z = np.load(golden_dir / "layer_tiny.npz")
    d_model, h, n, p, g, block_len, b, s = [int(v) for v in z["__shape"]]
    t = {k: torch.from_numpy(z[k]).to(DEV) for k in z.files if k != "__shape"}
    d_inner, gn = h * p, g * n
    proj = t["zxbcdt"]
    x = W.conv1d_silu(proj[..., :d_inner], t["w.conv1d.weight"], t["w.conv1d.bias"])             # model_ref.py:83-86
    ref_x = t["x"].reshape(b, s, d_inner).double()
    assert ((x.double() - ref_x).abs().max() / ref_x.abs().max()).item() < 5e-3
    dt, A_dt = W.dt_prologue(proj[..., 2 * d_inner + 2 * gn:], t["w.dt_bias"], t["w.A_log"])      # :94, 102-103
    assert ((dt.float() - t["dt"].float()).abs() / t["dt"].float().abs().clamp_min(1e-6)).max().item() < 2e-3
    assert ((A_dt - t["A_dt"]).abs() / t["A_dt"].abs().clamp_min(1e-6)).max().item() < 2e-3
    # core with the reference's own inputs, skip and gate fused (:123-162, 116-118)
    B = proj[..., 2 * d_inner:2 * d_inner + gn].reshape(b, s, g, n).contiguous()
    C_ = proj[..., 2 * d_inner + gn:2 * d_inner + 2 * gn].reshape(b, s, g, n).contiguous()
    zz = proj[..., d_inner:2 * d_inner].reshape(b, s, h, p).contiguous()
    for sep in (False, True):
        Y = W.ssd_forward(t["x"], t["A_dt"], B, C_, block_len, dt=t["dt"], D=t["w.D"].float(), z=zz,
                          separate_epilogue=sep)
        per_bh, fro = O.error_metrics(Y.cpu(), t["y_gated"].cpu())
        assert per_bh < 2e-2 and fro < 2e-2, (sep, per_bh, fro)
    Yc = W.ssd_forward(t["x"], t["A_dt"], B, C_, block_len, dt=t["dt"])
    per_bh, fro = O.error_metrics(Yc.cpu(), t["y_core"].cpu())
    assert per_bh < 2e-2 and fro < 2e-2, (per_bh, fro)


def test_dropin_model_matches_reference_golden(golden_dir):
    from workloadsuite_b200 import mamba_model as M

    z = np.load(golden_dir / "model_tiny.npz")
    init = [int(v) for v in z["__init"]]
    model = M.Model(*init).eval()
    sd = {k: torch.from_numpy(z[k]) for k in z.files if not k.startswith("__")}
    missing = model.load_state_dict(sd, strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    model = model.to(DEV)
    u = torch.from_numpy(z["__input"]).to(DEV)
    with torch.inference_mode():
        y = model(u)
    assert y.dtype == torch.float16 and y.shape == u.shape
    ref = torch.from_numpy(z["__output"]).double()
    err = (y.cpu().double() - ref).abs().max().item() / ref.abs().max().item()
    assert err < 2e-2, err


def test_dropin_module_contract():
    """Same checks the reference applies to its workloads (tests/test_diverse_workloads.py:61-72)."""
    import importlib.util
    from pathlib import Path

    path = Path(__file__).resolve().parent.parent / "workloadsuite_b200" / "mamba_model.py"
    spec = importlib.util.spec_from_file_location("ws_mamba_model", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert callable(mod.get_inputs) and callable(mod.get_init_inputs)
    assert mod.get_init_inputs() == [2048, 24, 128, 128, 64, 8, 64, 4]
    model = mod.Model(128, 1, 4, 128, 64, 2, 64, 4).to(DEV).eval()
    x = torch.randn(2, 256, 128, dtype=torch.float16, device=DEV)
    with torch.inference_mode():
        y = model(x)
        y2 = model(x)
    assert isinstance(y, torch.Tensor) and torch.isfinite(y).all() and torch.equal(y, y2)
    with pytest.raises(ValueError):
        mod.SSDLayer(64, 6, 16, 64, 4)
