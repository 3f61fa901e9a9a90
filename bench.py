#!/usr/bin/env python
"""Benchmark of the SSD forward: tokens/s, fraction of the HBM roofline, CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

One "step" is one SSD forward over the whole workload.  Default workload: the
Mamba-2-2.7B layer shape (batch 4, seq 8192, 80 heads, d_head 64, d_state 128, chunk
256, one B/C group, bf16 with fp32 log-decay), head-sharded over N GPUs with no
collective (total work fixed: strong scaling).  ``--workload cfg3`` runs the 128K-token
sequence-parallel configuration (one exchange of states per step); with more than one
GPU it is also timed after the default workload and reported under
``other_configs["cfg3:seqN"]``.  Inputs are seeded synthetic tensors with the
distributions of the configuration.  Prints ONE JSON line on rank 0.

Before anything is timed, at every N, a small slow-decay case (cross-chunk and cross-shard
terms matter) is cut the way the timed workload is sharded, run through the same code path,
gathered on rank 0 and compared with the float64 recurrence of ``oracle/``; the result is the
``parity`` object of the line and a failure ends the run with a non-zero exit code.

The ``--steps`` block is repeated until at least half a second of GPU time has been measured;
``ms_per_step`` is the median block (each block: barrier + synchronize on both sides, CUDA
events, max over ranks).

On one GPU the line also carries ``other_configs``: the other configurations kernel-only, the
default workload with the layer's skip/gate fused into the kernel's epilogue (next to the same
steps as PyTorch passes), the conv1d+SiLU kernel on the workload's shape, and the drop-in
``Model`` next to the reference ``Model`` timed by the reference's own harness functions.

``--impl reference`` times the reference's own ``SSDLayer._ssd_core`` (``model_ref.py:123-162``:
the bytecode that ``oracle/build_ref.py`` compiles from the unmodified reference into
``oracle/_ref/``; the oracle's bit-identical restatement when that directory was never built, and
for the fp32 configuration, which the fp16-only reference cannot run) on all host cores, on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIGS = {
    "cfg0": dict(b=16, s=128, h=8, p=64, n=16, g=8, chunk=64, dtype="f32", init=False, decay="normal"),
    "cfg1": dict(b=8, s=2048, h=24, p=64, n=128, g=1, chunk=256, dtype="bf16", init=False, decay="mamba"),
    "cfg2": dict(b=4, s=8192, h=80, p=64, n=128, g=1, chunk=256, dtype="bf16", init=False, decay="mamba"),
    "cfg3": dict(b=1, s=131072, h=32, p=64, n=128, g=1, chunk=256, dtype="bf16", init=False, decay="mamba"),
    "cfg4": dict(b=256, s=512, h=48, p=64, n=64, g=8, chunk=128, dtype="bf16", init=True, decay="mamba"),
}
WORKLOAD_NAMES = {
    "cfg0": "reference-style fp32 b16 s128 h8 p64 n16",
    "cfg1": "mamba2-130m-layer b8 s2048 h24 p64 n128 chunk256 bf16",
    "cfg2": "mamba2-2.7b-layer b4 s8192 h80 p64 n128 chunk256 g1 bf16",
    "cfg3": "long-context b1 s131072 h32 p64 n128 chunk256 g1 bf16",
    "cfg4": "short-seqs b256 s512 h48 p64 n64 g8 chunk128 bf16 + initial states",
}
SEQ_EXCHANGE = "auto"
TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
L2_BYTES = 126e6
MIN_TIMED_SECONDS = 0.5
PARITY_TOL = {"f32": 1e-4, "bf16": 2e-2, "f16": 2e-2}


def line_config(name, world, seq_parallel):
    """The ``config`` object: the same keys and values in both arms (``--impl reference`` included)."""
    return {"workload": WORKLOAD_NAMES[name], "name": name,
            "parallelism": ("seq%d+state-exchange" % world) if seq_parallel else ("heads%d" % world),
            "l2": "rotating input sets larger than L2 between timed iterations"}


def algorithmic_bytes(cfg, h=None, s=None):
    """X read + Y write + B + C + fp32 log-decay (+ fp32 initial states), per step."""
    e = 4 if cfg["dtype"] == "f32" else 2
    h = h or cfg["h"]
    s = s or cfg["s"]
    g = cfg["g"] if h == cfg["h"] else max(1, cfg["g"] * h // cfg["h"])
    per_token = 2 * h * cfg["p"] * e + 2 * g * cfg["n"] * e + 4 * h
    total = cfg["b"] * s * per_token
    if cfg.get("init"):
        total += cfg["b"] * h * cfg["n"] * cfg["p"] * 4
    return total


def gen_inputs(cfg, device, seed, h=None, s=None):
    """Seeded synthetic inputs on ``device`` (distributions of the configuration)."""
    b, p, n = cfg["b"], cfg["p"], cfg["n"]
    h = h or cfg["h"]
    s = s or cfg["s"]
    g = cfg["g"] if h == cfg["h"] else max(1, cfg["g"] * h // cfg["h"])
    td = TDT[cfg["dtype"]]
    gen = torch.Generator(device=device).manual_seed(seed)
    X = torch.randn(b, s, h, p, generator=gen, device=device, dtype=torch.float32).to(td)
    B = torch.randn(b, s, g, n, generator=gen, device=device, dtype=torch.float32).to(td)
    C = torch.randn(b, s, g, n, generator=gen, device=device, dtype=torch.float32).to(td)
    if cfg["decay"] == "normal":
        A = torch.randn(b, s, h, generator=gen, device=device)
    else:
        dt = torch.nn.functional.softplus(torch.randn(b, s, h, generator=gen, device=device) - 4.0)
        A_log = torch.empty(h, device=device).uniform_(0.0, math.log(16.0), generator=gen)
        A = -dt * torch.exp(A_log)
    out = dict(X=X, A=A.float().contiguous(), B=B, C=C)
    if cfg.get("init"):
        out["initial_states"] = torch.randn(b, h, n, p, generator=gen, device=device) * 0.1
    return out


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs (read-only)."""

    def __init__(self, index):
        self.samples = []
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            try:  # CUDA ordinals follow CUDA_VISIBLE_DEVICES, NVML's do not
                uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            self._stop.wait(0.01)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr:
            self._thr.join(timeout=1)

    def summary(self, t0, t1):
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        nv = self.nv
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples[-20:]
        names = {}
        for attr, nm in (("nvmlClocksThrottleReasonSwPowerCap", "sw_power_cap"),
                         ("nvmlClocksThrottleReasonHwSlowdown", "hw_slowdown"),
                         ("nvmlClocksThrottleReasonSwThermalSlowdown", "sw_thermal_slowdown"),
                         ("nvmlClocksThrottleReasonHwThermalSlowdown", "hw_thermal_slowdown"),
                         ("nvmlClocksThrottleReasonHwPowerBrakeSlowdown", "hw_power_brake"),
                         ("nvmlClocksThrottleReasonApplicationsClocksSetting", "applications_clocks_setting")):
            if hasattr(nv, attr):
                names[getattr(nv, attr)] = nm
        seen = set()
        for _, _, r in inside:
            for bit, nm in names.items():
                if r & bit:
                    seen.add(nm)
        try:
            mx = nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM)
        except Exception:
            mx = None
        med = statistics.median([m for _, m, _ in inside]) if inside else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(seen), "samples": len(inside)}


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            d = json.loads(f.read_text())
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def captured_traffic(workload, world):
    """DRAM bytes (read + write) of one launch of the dominant kernel from the ncu summary under ``profiles/``,
    or None.  A summary counts only if it names this workload at one GPU and was captured from the kernels
    that run now: its ``kernel sources`` line must equal the fingerprint of the package's CUDA sources."""
    if world != 1:
        return None
    try:
        from workloadsuite_b200 import build as B

        stamp = B.source_fingerprint()
        for f in sorted((ROOT / "profiles").glob("*.md")):
            m = re.search(r"^traffic_bytes_per_launch:\s*([0-9.eE+]+)\s+workload:\s*(\w+)\s+kernel sources:\s*(\w+)",
                          f.read_text(), re.M)
            if m and m.group(2) == workload and stamp.startswith(m.group(3)):
                return float(m.group(1))
    except Exception:
        pass
    return None


# ----------------------------------------------------------------------------- reference (CPU) arm

def reference_callable(cfg):
    """(fn(inp, Bh, Ch) -> Y, kind): the unmodified reference core when ``oracle/_ref`` is built and the
    configuration is half precision (the reference is hard-wired to fp16, model_ref.py:145), else the port."""
    from oracle import build_ref as R
    from oracle import ssd_oracle as O

    mod = None
    if cfg["dtype"] != "f32":
        try:
            mod = R.load_model_ref()
        except Exception:
            mod = None
    if mod is not None:
        return (lambda inp, Bh, Ch: R.reference_core(mod, inp["X"], inp["A"], Bh, Ch, cfg["chunk"])), "reference"
    dtype = torch.float32 if cfg["dtype"] == "f32" else torch.float16
    return (lambda inp, Bh, Ch: O.ssd_chunked(inp["X"], inp["A"], Bh, Ch, cfg["chunk"], dtype=dtype)), "port"


def cpu_reference_sample(cfg, steps, warmup):
    """Times the reference core (fp16 as in the reference) on all host cores.

    Sample: one batch entry of the workload with all heads and the full sequence (for the
    128K configuration a 16K-token prefix), B/C broadcast to heads outside the timed
    region as the reference's caller does (model_ref.py:97-99)."""
    from oracle import ssd_oracle as O

    # a launcher such as torchrun exports OMP_NUM_THREADS=1 to its workers: use the host's cores anyway
    torch.set_num_threads(os.cpu_count() or 1)
    b, s, h = 1, min(cfg["s"], 16384), cfg["h"]
    c = dict(cfg)
    c.update(b=b, s=s)
    dtype = torch.float32 if cfg["dtype"] == "f32" else torch.float16
    inp = O.make_inputs(seed=0, **{**c, "dtype": dtype})
    Bh = inp["B"].repeat_interleave(h // c["g"], dim=2).contiguous()
    Ch = inp["C"].repeat_interleave(h // c["g"], dim=2).contiguous()
    fn, kind = reference_callable(cfg)
    times = []
    with torch.inference_mode():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            fn(inp, Bh, Ch)
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt)
    med = statistics.median(times)
    sample = f"batch 1 of {cfg['b']}, seq {s} of {cfg['s']}, all {h} heads, {dtype}".replace("torch.", "")
    return b * s / med, med, sample, kind


def run_reference(args, cfg, rank, world):
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    tps, med, sample, kind = cpu_reference_sample(cfg, steps, warmup)
    seq_parallel = args.workload == "cfg3" and world > 1
    line = {
        "impl": "reference", "metric": "ssd_forward_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": med * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16" if cfg["dtype"] != "f32" else "f32", "data": "synthetic",
        "config": line_config(args.workload, world, seq_parallel),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": sample, "host_cpus": os.cpu_count()},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our arm

def time_blocks(fn, nsets, steps, warmup, dist_on, min_seconds=MIN_TIMED_SECONDS, max_blocks=500):
    """Warm up, then time blocks of exactly ``steps`` steps -- each bracketed by barrier + synchronize, CUDA
    events on the current stream, max over ranks -- until ``min_seconds`` of GPU time have been measured.
    Returns (median block ms / steps, wall t0, wall t1, list of block ms)."""
    import torch.distributed as dist

    for i in range(warmup):
        fn(i % nsets)
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)

    def one_block():
        torch.cuda.synchronize()
        if dist_on:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for i in range(steps):
            fn(i % nsets)
        e1.record()
        torch.cuda.synchronize()
        if dist_on:
            dist.barrier()
        ms = e0.elapsed_time(e1)
        if dist_on:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    t0 = time.perf_counter()
    blocks = [one_block()]
    # (the first block's time is already the max over ranks, so every rank derives the same count)
    nblocks = min(max_blocks, max(1, int(math.ceil(min_seconds * 1e3 / max(blocks[0], 1e-3)))))
    for _ in range(nblocks - 1):
        blocks.append(one_block())
    t1 = time.perf_counter()
    return statistics.median(blocks) / steps, t0, t1, blocks


def parity_leg(mode, rank, world, dev, kw):
    """A small slow-decay case cut the way the timed workload is sharded, run through the same code path,
    gathered on rank 0 and compared with the float64 recurrence (oracle).  Returns the ``parity`` object
    (on every rank: the verdict is broadcast)."""
    import torch.distributed as dist

    import workloadsuite_b200 as W
    from oracle import ssd_oracle as O
    from workloadsuite_b200 import sharded

    if mode == "seq":
        case = dict(b=1, s=1024 * max(world, 2), h=4, p=64, n=128, g=1, dtype="bf16", decay="mamba", chunk=256)
    else:
        case = dict(b=2, s=1024, h=16, p=64, n=128, g=1, dtype="bf16", decay="mamba", chunk=256)
    inp = O.make_inputs(seed=4242, decay_scale=0.02, **case)       # the same tensors on every rank
    chunk = case["chunk"]
    if mode == "seq" and world > 1:
        s_loc = case["s"] // world
        sl = slice(rank * s_loc, (rank + 1) * s_loc)
        d = {k: v[:, sl].contiguous().to(dev) for k, v in inp.items()}
        eng = sharded.SequenceShardedSSD(exchange=SEQ_EXCHANGE)
        Yl = eng.forward(d["X"], d["A"], d["B"], d["C"], chunk, **kw)
        cat_dim = 1
    else:
        full = {k: v.to(dev) for k, v in inp.items()}
        d = sharded.shard_heads(full["X"], full["A"], full["B"], full["C"], rank, world) if world > 1 else full
        Yl = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], chunk, **kw)
        cat_dim = 2
    torch.cuda.synchronize()
    status = W.device_status(dev)
    if world > 1:
        parts = [torch.empty_like(Yl) for _ in range(world)] if rank == 0 else None
        dist.gather(Yl.contiguous(), parts, dst=0)
        Y = torch.cat(parts, dim=cat_dim) if rank == 0 else None
    else:
        Y = Yl
    verdict = torch.zeros(4, dtype=torch.float64, device=dev)
    if rank == 0:
        Yr = O.ssd_recurrence(inp["X"], inp["A"], inp["B"], inp["C"])
        per_bh, fro = O.error_metrics(Y.cpu(), Yr)
        tol = PARITY_TOL[case["dtype"]]
        ok = per_bh < tol and fro < tol and bool(torch.isfinite(Y).all())
        verdict = torch.tensor([per_bh, fro, tol, 1.0 if ok else 0.0], dtype=torch.float64, device=dev)
    st = torch.tensor([float(status)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.broadcast(verdict, src=0)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
    per_bh, fro, tol, ok = [float(v) for v in verdict.tolist()]
    return {"per_bh": per_bh, "fro": fro, "tol": tol, "ok": bool(ok) and st.item() == 0, "device_status": int(st.item()),
            "against": "float64 token recurrence (oracle)",
            "case": ("sequence-sharded " if mode == "seq" else "head-sharded ") +
                    f"b{case['b']} s{case['s']} h{case['h']} p64 n128 bf16, log-decay x0.02, {world} rank(s)"}


def build_step(W, sharded, cfg, rank, world, dev, kw, no_graphs, seq_parallel):
    """Inputs, step function (CUDA-graph replay where possible) and launch accounting for one workload."""
    if seq_parallel:
        s_loc, h_loc = cfg["s"] // world, cfg["h"]
    else:
        h0, h1, _, _ = sharded.head_shard_bounds(cfg["h"], cfg["g"], rank, world)
        s_loc, h_loc = cfg["s"], h1 - h0
    set_bytes = algorithmic_bytes(cfg, h=h_loc, s=s_loc)
    nsets = min(16, max(2, int(math.ceil(2.5 * L2_BYTES / set_bytes))))
    sets = [gen_inputs(cfg, dev, seed=1000 * rank + i, h=h_loc, s=s_loc) for i in range(nsets)]
    outs = [torch.empty_like(sets[i]["X"]) for i in range(nsets)]
    chunk = cfg["chunk"]
    plan = W.plan(sets[0]["X"], sets[0]["A"], sets[0]["B"], sets[0]["C"], chunk, **kw)
    info = dict(set_bytes=set_bytes, nsets=nsets, plan=plan, s_loc=s_loc, h_loc=h_loc,
                kernel=W.kernel_name(sets[0]["X"], sets[0]["A"], sets[0]["B"], sets[0]["C"], chunk,
                                     kernel=kw.get("kernel")))
    if seq_parallel:
        eng = sharded.SequenceShardedSSD(cuda_graphs=not no_graphs, exchange=SEQ_EXCHANGE)
        info["launches"] = eng.launches_per_step(sets[0]["X"], sets[0]["A"], sets[0]["B"], sets[0]["C"], chunk, **kw)
        info["launch_mode"] = eng.launch_mode()

        def step(i):
            d = sets[i]
            eng.forward(d["X"], d["A"], d["B"], d["C"], chunk, out=outs[i], **kw)

        info["engine"] = eng
        return sets, outs, step, info

    info["launches"] = plan["launches"]

    def step(i):
        d = sets[i]
        W.ssd_forward(d["X"], d["A"], d["B"], d["C"], chunk, initial_states=d.get("initial_states"), out=outs[i], **kw)

    # A step is a fixed sequence of launches: capture it once per input set and replay, so that the
    # timed region measures the GPU and not the Python/driver launch path (which dominates at N=8).
    info["launch_mode"] = "eager"
    run_step = step
    if not no_graphs:
        try:
            for i in range(nsets):
                step(i)                      # allocates the workspace outside capture
            torch.cuda.synchronize()
            cap = torch.cuda.Stream()
            graphs = []
            with torch.cuda.stream(cap):
                for i in range(nsets):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=cap):
                        step(i)
                    graphs.append(g)
            torch.cuda.synchronize()

            def run_step(i, graphs=graphs):
                graphs[i].replay()

            info["launch_mode"] = "cuda_graph"
        except Exception as exc:  # fall back to plain launches
            sys.stderr.write(f"[bench] CUDA graph capture failed ({type(exc).__name__}: {exc}); timing eager launches\n")
            run_step = step
    return sets, outs, run_step, info


def model_through_reference_harness(dev, steps, with_compile=True):
    """The drop-in ``Model`` and the reference ``Model`` (``model_ref.py:165-229``, production configuration: 24
    layers, b8 s2048 d_model 2048, fp16) timed on this GPU by the reference's own ``_benchmark``
    (``bench.py:138-170``) under ``torch.inference_mode()`` as ``_bench_workload`` does (``bench.py:230-233``), with
    shared weights, plus the output parity of the two on sampled rows; and the reference under ``torch.compile``
    through the reference's ``_compile_and_bench`` (about a minute of compilation)."""
    from oracle import build_ref as R
    from workloadsuite_b200 import mamba_model as MM

    out = {"shape": "24 layers, b8 s2048 d_model2048 h128 p64 n128 g8 block64 fp16"}
    rb, rm = R.load_ref_bench(), R.load_model_ref()
    init = MM.get_init_inputs()
    torch.manual_seed(0)
    ours = MM.Model(*init).to(dev).eval()
    x = torch.randn(MM.batch_size, MM.seq_length, MM.d_model, dtype=torch.float16, device=dev)
    runs = max(3, min(10, steps // 5))
    if rb is None or rm is None:
        out["reference"] = "oracle/_ref was not built on this machine: drop-in Model only"
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.inference_mode():
            for _ in range(2):
                ours(x)
            e0.record()
            for _ in range(runs):
                ours(x)
            e1.record()
        torch.cuda.synchronize()
        out["dropin"] = {"median_ms": e0.elapsed_time(e1) / runs}
        return out
    common = dict(device_type="cuda", warmup=2, runs=runs)
    with torch.inference_mode():
        out["dropin"] = rb._benchmark(ours, [x], **common)
        yo = ours(x)
    ref = rm.Model(*init).to(dev).eval()
    ref.load_state_dict(ours.state_dict(), strict=True)
    with torch.inference_mode():
        out["reference_eager"] = rb._benchmark(ref, [x], **common)
        yr = ref(x)
        if with_compile:
            # the reference harness's second variant: the very instance it timed, under torch.compile
            # (bench.py:172-201, 241-253; mode "default", dynamic False, fullgraph False)
            out["reference_torch_compile"] = rb._compile_and_bench(ref, [x], compile_mode="default", dynamic=False,
                                                                   **common)
    rows = torch.linspace(0, MM.seq_length - 1, 64, device=dev).long()
    a, b_ = yo[:, rows].double(), yr[:, rows].double()
    out["parity_sampled_rows"] = {"max_abs_err_over_max_abs_ref": float((a - b_).abs().max() / b_.abs().max()),
                                  "tol": 2e-2, "finite": bool(torch.isfinite(yo).all())}
    out["speedup_vs_reference_eager"] = out["reference_eager"]["median_ms"] / out["dropin"]["median_ms"]
    if "median_ms" in out.get("reference_torch_compile", {}):
        out["speedup_vs_reference_torch_compile"] = (out["reference_torch_compile"]["median_ms"] /
                                                     out["dropin"]["median_ms"])
    out["tokens_per_s"] = MM.batch_size * MM.seq_length / (out["dropin"]["median_ms"] * 1e-3)
    del ref, ours
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(CONFIGS))
    ap.add_argument("--kernel", default=None, choices=[None, "auto", "scan_f32", "tcgen05"])
    ap.add_argument("--nsegments", type=int, default=0)
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-others", action="store_true")
    ap.add_argument("--others", default="configs,skip_gate,conv,step,model",
                    help="which single-GPU extras to time: configs, skip_gate, conv, step, model (comma-separated)")
    ap.add_argument("--seq-exchange", default="auto", choices=["auto", "peer", "collective"],
                    help="state exchange of the sequence-sharded forward: this library's peer-memory kernel, "
                         "torch.distributed's all-gather, or the first when the ranks can map each other's memory")
    ap.add_argument("--no-parity", action="store_true", help="skip the parity leg (profiling runs only)")
    ap.add_argument("--no-model-compile", action="store_true",
                    help="skip the torch.compile variant of the reference Model (about a minute of compilation)")
    ap.add_argument("--min-seconds", type=float, default=MIN_TIMED_SECONDS,
                    help="repeat the --steps block until this much GPU time has been measured")
    ap.add_argument("--no-graphs", action="store_true",
                    help="launch every step from Python instead of replaying one CUDA graph per input set")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = CONFIGS[args.workload]
    global SEQ_EXCHANGE
    SEQ_EXCHANGE = args.seq_exchange

    if args.impl == "reference":
        run_reference(args, cfg, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the SSD kernels have no CPU fallback")
    import torch.distributed as dist

    import workloadsuite_b200 as W
    from workloadsuite_b200 import sharded

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist_on = world > 1
    if dist_on:
        dist.init_process_group("nccl", device_id=dev)
    n_gpus = world
    kw = dict(kernel=args.kernel, nsegments=args.nsegments or None)
    seq_parallel = args.workload == "cfg3" and world > 1

    # ---- parity before timing, through the code path that is timed
    parity = None
    if not args.no_parity:
        parity = parity_leg("seq" if seq_parallel else "heads", rank, world, dev, kw)
        if not parity["ok"]:
            if rank == 0:
                print(json.dumps({"metric": "ssd_forward_tokens_per_s", "value": None, "n_gpus": n_gpus,
                                  "parity": parity, "error": "parity leg failed; nothing was timed"}), flush=True)
            if dist_on:
                dist.destroy_process_group()
            raise SystemExit(3)

    sets, outs, run_step, info = build_step(W, sharded, cfg, rank, world, dev, kw, args.no_graphs, seq_parallel)
    set_bytes, nsets, plan = info["set_bytes"], info["nsets"], info["plan"]

    sampler = ClockSampler(local)
    sampler.start()
    ms_step, t0, t1, blocks = time_blocks(run_step, nsets, args.steps, args.warmup, dist_on, args.min_seconds)
    sampler.stop()
    clocks = sampler.summary(t0, t1)
    phases = None
    if "engine" in info:     # (how the step was launched is known once it has run)
        info["launch_mode"] = info["engine"].launch_mode()
        phases = info["engine"].phase_times_ms()

    tokens = cfg["b"] * cfg["s"]
    value = tokens / (ms_step * 1e-3)
    peak, peak_kind = measured_peaks()
    total_bytes = algorithmic_bytes(cfg)          # whole job
    achieved = set_bytes / (ms_step * 1e-3) / 1e9  # this GPU's share over the step time
    kname = info["kernel"]

    # ---- end to end through the host-buffer entry point (pinned host tensors, copies timed)
    e2e = None
    try:
        if args.e2e_steps <= 0:
            raise RuntimeError("skipped (--e2e-steps 0)")
        hs = {k: v.cpu().pin_memory() for k, v in sets[0].items()}
        hout = torch.empty_like(hs["X"]).pin_memory()
        runner = W.HostRunner(cfg["b"], info["s_loc"], info["h_loc"], cfg["p"], cfg["n"], sets[0]["B"].shape[2],
                              cfg["chunk"], TDT[cfg["dtype"]], device=dev, kernel=args.kernel)
        runner.run(hs["X"], hs["A"], hs["B"], hs["C"], hout, initial_states=hs.get("initial_states"))
        if dist_on:
            dist.barrier()
        torch.cuda.synchronize()
        tt0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            runner.run(hs["X"], hs["A"], hs["B"], hs["C"], hout, initial_states=hs.get("initial_states"))
        torch.cuda.synchronize()
        el = (time.perf_counter() - tt0) / args.e2e_steps
        if dist_on:
            t = torch.tensor([el], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            el = float(t.item())
        # What the link alone allows: the same byte counts as two plain pinned copies, one per direction, started
        # together on two streams with no dependence between them (the pipeline's Y can only leave after its X arrived).
        copies_ms = None
        try:
            nin, nout = int(runner.h2d_bytes), int(runner.d2h_bytes)
            hin = torch.empty(nin, dtype=torch.uint8).pin_memory()
            hback = torch.empty(nout, dtype=torch.uint8).pin_memory()
            din = torch.empty(nin, dtype=torch.uint8, device=dev)
            dback = torch.empty(nout, dtype=torch.uint8, device=dev)
            s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

            def copies():
                with torch.cuda.stream(s_in):
                    din.copy_(hin, non_blocking=True)
                with torch.cuda.stream(s_out):
                    hback.copy_(dback, non_blocking=True)

            copies()
            torch.cuda.synchronize()
            tc0 = time.perf_counter()
            for _ in range(args.e2e_steps):
                copies()
            torch.cuda.synchronize()
            copies_ms = (time.perf_counter() - tc0) / args.e2e_steps * 1e3
            del hin, hback, din, dback
        except Exception:
            copies_ms = None
        e2e = {"value": tokens / el, "unit": "tokens/s", "ms_per_step": el * 1e3,
               "h2d_bytes_per_step": runner.h2d_bytes, "d2h_bytes_per_step": runner.d2h_bytes,
               "copies_alone_ms": copies_ms,
               "frac_of_copies_alone": (copies_ms / (el * 1e3)) if copies_ms else None,
               "note": "ssd_b200_forward_host: pinned host tensors in, Y back to host, copies inside the timed region"
               + (" (sequence shards run independently: no state exchange on this path)" if seq_parallel else "")}
        del hs, hout, runner
    except Exception as exc:  # report rather than lose the device-side numbers
        e2e = {"value": None, "unit": "tokens/s", "error": f"{type(exc).__name__}: {exc}"}

    others = {}
    del sets, outs, run_step
    info.pop("engine", None)
    torch.cuda.empty_cache()

    # ---- more than one GPU: the 128K sequence-parallel configuration too, with its own parity leg
    if world > 1 and args.workload != "cfg3" and not args.no_others:
        key = "cfg3:seq%d" % world
        try:
            c3 = CONFIGS["cfg3"]
            p3 = None if args.no_parity else parity_leg("seq", rank, world, dev, kw)
            s3, o3, step3, info3 = build_step(W, sharded, c3, rank, world, dev, kw, args.no_graphs, True)
            ms3, _, _, blocks3 = time_blocks(step3, info3["nsets"], max(5, args.steps // 2), 3, dist_on, args.min_seconds)
            others[key] = {"tokens_per_s": c3["b"] * c3["s"] / (ms3 * 1e-3), "ms_per_step": ms3, "blocks": len(blocks3),
                           "hbm_frac_of_measured": info3["set_bytes"] / (ms3 * 1e-3) / 1e9 / peak,
                           "launch": info3["engine"].launch_mode(), "exchange": info3["engine"].exchange_mode(),
                           "kernel_launches_per_step": info3["launches"],
                           "segments_per_sequence": info3["plan"]["nsegments"], "parity": p3,
                           "phases_ms": info3["engine"].phase_times_ms()}
            del s3, o3, step3, info3
            torch.cuda.empty_cache()
        except Exception as exc:
            others[key] = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- other configurations, kernel-only, single GPU
    extras = set() if args.no_others else {e.strip() for e in args.others.split(",") if e.strip()}
    if world == 1 and extras:
        for name in ("cfg0", "cfg1", "cfg3", "cfg4"):
            if name == args.workload or "configs" not in extras:
                continue
            try:
                c = CONFIGS[name]
                ss, oo, st, inf = build_step(W, sharded, c, 0, 1, dev, dict(kernel=args.kernel, nsegments=None),
                                             args.no_graphs, False)
                ms, _, _, bl = time_blocks(st, inf["nsets"], max(5, args.steps // 2), 3, False, args.min_seconds / 2)
                others[name] = {"tokens_per_s": c["b"] * c["s"] / (ms * 1e-3), "ms_per_step": ms,
                                "hbm_frac_of_measured": inf["set_bytes"] / (ms * 1e-3) / 1e9 / peak,
                                "kernel": inf["kernel"], "launch": inf["launch_mode"],
                                "segments_per_sequence": inf["plan"]["nsegments"],
                                "kernel_launches_per_step": inf["launches"]}
                del ss, oo, st
                torch.cuda.empty_cache()
            except Exception as exc:
                others[name] = {"error": f"{type(exc).__name__}: {exc}"}

        # The same workload with the layer's skip and gate, (Y + x D) silu(z) of model_ref.py:116-118, fused into the
        # kernel's epilogue, next to the same three steps done as separate PyTorch passes over Y.
        try:
            if "skip_gate" not in extras:
                raise KeyError("skipped")
            c = CONFIGS[args.workload]
            sb = algorithmic_bytes(c) + c["b"] * c["s"] * c["h"] * c["p"] * 2   # + one read of z
            ns = min(16, max(2, int(math.ceil(2.5 * L2_BYTES / sb))))
            ss = [gen_inputs(c, dev, seed=177 + i) for i in range(ns)]
            oo = [torch.empty_like(x["X"]) for x in ss]
            zz = [torch.randn_like(x["X"]) for x in ss]
            Dv = torch.randn(c["h"], device=dev)

            def st_fused(i):
                d = ss[i]
                W.ssd_forward(d["X"], d["A"], d["B"], d["C"], c["chunk"], initial_states=d.get("initial_states"),
                              out=oo[i], kernel=args.kernel, D=Dv, z=zz[i])

            def st_unfused(i):
                d = ss[i]
                Y = W.ssd_forward(d["X"], d["A"], d["B"], d["C"], c["chunk"], initial_states=d.get("initial_states"),
                                  out=oo[i], kernel=args.kernel)
                Y = Y + d["X"] * Dv.to(Y.dtype).view(1, 1, -1, 1)
                Y = Y * torch.nn.functional.silu(zz[i])

            def st_separate(i):
                d = ss[i]
                W.ssd_forward(d["X"], d["A"], d["B"], d["C"], c["chunk"], initial_states=d.get("initial_states"),
                              out=oo[i], kernel=args.kernel, D=Dv, z=zz[i], separate_epilogue=True)

            ms_f, _, _, _ = time_blocks(st_fused, ns, max(5, args.steps // 2), 3, False, args.min_seconds / 2)
            ms_s, _, _, _ = time_blocks(st_separate, ns, max(5, args.steps // 2), 3, False, args.min_seconds / 4)
            ms_u, _, _, _ = time_blocks(st_unfused, ns, max(5, args.steps // 2), 3, False, args.min_seconds / 4)
            others[args.workload + "+skip_gate"] = {
                "tokens_per_s": c["b"] * c["s"] / (ms_f * 1e-3), "ms_per_step": ms_f,
                "hbm_frac_of_measured": sb / (ms_f * 1e-3) / 1e9 / peak,
                "ms_per_step_with_standalone_epilogue_kernel": ms_s,
                "ms_per_step_with_pytorch_epilogue": ms_u}
            del ss, oo, zz
            torch.cuda.empty_cache()
        except KeyError:
            pass
        except Exception as exc:
            others[args.workload + "+skip_gate"] = {"error": f"{type(exc).__name__}: {exc}"}

        # The X producer of the same workload: causal depthwise conv1d(k=4) + SiLU (model_ref.py:83-86) over
        # [b, s, h*p], read as a column slice of a projection-sized buffer; bytes = one read + one write.
        try:
            if "conv" not in extras:
                raise KeyError("skipped")
            c = CONFIGS[args.workload]
            dch = c["h"] * c["p"]
            wdt = TDT[c["dtype"]]
            wide = [torch.randn(c["b"], c["s"], 2 * dch + 64, device=dev, dtype=wdt) for _ in range(2)]
            yo = [torch.empty(c["b"], c["s"], dch, device=dev, dtype=wdt) for _ in range(2)]
            cw = torch.randn(dch, 1, 4, device=dev, dtype=wdt)
            cb = torch.randn(dch, device=dev, dtype=wdt)

            def st_conv(i):
                W.conv1d_silu(wide[i][..., :dch], cw, cb, out=yo[i])

            ms_c, _, _, _ = time_blocks(st_conv, 2, max(5, args.steps // 2), 3, False, args.min_seconds / 4)
            cbytes = 2 * c["b"] * c["s"] * dch * wide[0].element_size()
            others[args.workload + ":conv1d_silu"] = {"ms_per_step": ms_c, "GBps": cbytes / (ms_c * 1e-3) / 1e9,
                                                      "hbm_frac_of_measured": cbytes / (ms_c * 1e-3) / 1e9 / peak}
            del wide, yo
            torch.cuda.empty_cache()
        except KeyError:
            pass
        except Exception as exc:
            others[args.workload + ":conv1d_silu"] = {"error": f"{type(exc).__name__}: {exc}"}

        # Decode-style use: one token per call with the state carried in place (the carry of model_ref.py:152-157), at
        # the reference's production layer shape.  Bytes = the fp32 state read and written once (+ x, y, z, B, C).
        try:
            if "step" not in extras:
                raise KeyError("skipped")
            sb_, sh_, sn_, sg_, sdt = 8, 128, 128, 8, torch.float16
            nst = 6                                  # 6 x 67 MB of state: more than L2 between repeats
            stt = [torch.randn(sb_, sh_, sn_, 64, device=dev) for _ in range(nst)]
            xs_ = torch.randn(sb_, sh_, 64, device=dev, dtype=sdt)
            zs_ = torch.randn(sb_, sh_, 64, device=dev, dtype=sdt)
            Bs_ = torch.randn(sb_, sg_, sn_, device=dev, dtype=sdt)
            Cs_ = torch.randn(sb_, sg_, sn_, device=dev, dtype=sdt)
            dts_ = (0.01 + 0.1 * torch.rand(sb_, sh_, device=dev)).to(sdt)
            as_ = -torch.rand(sb_, sh_, device=dev)
            Ds_ = torch.ones(sh_, device=dev)
            ys_ = torch.empty_like(xs_)

            def st_step(i):
                W.ssd_step(xs_, as_, Bs_, Cs_, stt[i], dt=dts_, D=Ds_, z=zs_, out=ys_)

            ms_t, _, _, _ = time_blocks(st_step, nst, max(5, args.steps // 2), 3, False, args.min_seconds / 4)
            tbytes = 2 * stt[0].numel() * 4 + 3 * xs_.numel() * 2 + 2 * Bs_.numel() * 2
            others["decode_step_b8_h128_n128"] = {"ms_per_step": ms_t, "GBps": tbytes / (ms_t * 1e-3) / 1e9,
                                                   "hbm_frac_of_measured": tbytes / (ms_t * 1e-3) / 1e9 / peak,
                                                   "note": "ssd_step: one token, fp32 state [8,128,128,64] updated in place"}
            del stt
            torch.cuda.empty_cache()
        except KeyError:
            pass
        except Exception as exc:
            others["decode_step_b8_h128_n128"] = {"error": f"{type(exc).__name__}: {exc}"}

        # The whole Model (reference contract: Model / get_init_inputs / get_inputs, model_ref.py:165-229) at the
        # reference's production configuration, drop-in next to the reference, timed by the reference's harness.
        try:
            if "model" in extras:
                others["mamba_model_24_layers"] = model_through_reference_harness(
                    dev, args.steps, with_compile=not args.no_model_compile)
        except Exception as exc:
            others["mamba_model_24_layers"] = {"error": f"{type(exc).__name__}: {exc}"}
            torch.cuda.empty_cache()

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            tps, med, sample, kind = cpu_reference_sample(cfg, 3, 1)
            cpu_baseline = {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": kind,
                            "sample": sample, "host_cpus": os.cpu_count(), "s_per_sample": med}
        except Exception as exc:
            cpu_baseline = {"value": None, "unit": "tokens/s", "error": f"{type(exc).__name__}: {exc}"}

    if rank == 0:
        line = {
            "metric": "ssd_forward_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": n_gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
            "config": line_config(args.workload, world, seq_parallel),
            "run": {"l2": f"{nsets} rotating input sets of {set_bytes / 1e6:.0f} MB per GPU (> L2)",
                    "kernel": kname, "launch": info["launch_mode"], "segments_per_sequence": plan["nsegments"],
                    "kernel_launches_per_step": info["launches"], "timed_blocks": len(blocks),
                    "block_ms_min_median_max": [min(blocks), statistics.median(blocks), max(blocks)],
                    "timed_gpu_seconds": sum(blocks) * 1e-3, "phases_ms": phases},
            "parity": parity,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "frac_of_8TBs": achieved / 8000.0,
                         "traffic": captured_traffic(args.workload, world),
                         "algorithmic_bytes_per_step_per_gpu": set_bytes, "algorithmic_bytes_whole_job": total_bytes},
            "cpu_baseline": cpu_baseline,
            "e2e": e2e,
            "gpu_launches": args.steps * info["launches"],
            "clocks": clocks,
        }
        if others:
            line["other_configs"] = others
        print(json.dumps(line), flush=True)
    if dist_on:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
