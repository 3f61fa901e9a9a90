#!/usr/bin/env python
"""Benchmark of the SSD forward: tokens/s, fraction of the HBM roofline, CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl reference]

One "step" is one SSD forward over the whole workload.  Default workload: the
Mamba-2-2.7B layer shape (batch 4, seq 8192, 80 heads, d_head 64, d_state 128, chunk
256, one B/C group, bf16 with fp32 log-decay), head-sharded over N GPUs with no
collective (total work fixed: strong scaling).  ``--workload cfg3`` runs the 128K-token
sequence-parallel configuration (one all-gather of states per step).  Inputs are seeded
synthetic tensors with the distributions of the configuration.  Prints ONE JSON line
on rank 0.

On one GPU the line also carries ``other_configs``: the other configurations kernel-only, the default workload with
the layer's skip/gate fused into the kernel's epilogue (next to the same steps as PyTorch passes), the conv1d+SiLU
kernel on the workload's shape and the drop-in ``Model`` (two layers of the reference's production shape).

``--impl reference`` times the reference algorithm (the CPU restatement of
``SSDLayer._ssd_core`` in ``oracle/``, bit-identical to the reference in fp16) on the
host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
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
TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
L2_BYTES = 126e6

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu capture summarised
# in profiles/ssd_tc2_kernel_cfg2.md (same command line as this bench, --steps 2 --warmup 3); None where no capture
# of that (workload, kernel, world size) exists.
NCU_TRAFFIC_BYTES = {("cfg2", "tcgen05", 1): 666.1e6}


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


# ----------------------------------------------------------------------------- reference (CPU) arm

def cpu_reference_sample(cfg, steps, warmup):
    """Times the reference algorithm (oracle port, fp16 as in the reference) on host cores.

    Sample: one batch entry of the workload with all heads and the full sequence (for the
    128K configuration a 16K-token prefix), B/C broadcast to heads outside the timed
    region as the reference's caller does (model_ref.py:97-99)."""
    from oracle import ssd_oracle as O

    b, s, h = 1, min(cfg["s"], 16384), cfg["h"]
    c = dict(cfg)
    c.update(b=b, s=s)
    dtype = torch.float32 if cfg["dtype"] == "f32" else torch.float16
    inp = O.make_inputs(seed=0, **{**c, "dtype": dtype})
    Bh = inp["B"].repeat_interleave(h // c["g"], dim=2).contiguous()
    Ch = inp["C"].repeat_interleave(h // c["g"], dim=2).contiguous()
    times = []
    with torch.inference_mode():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            O.ssd_chunked(inp["X"], inp["A"], Bh, Ch, c["chunk"], dtype=dtype)
            dt = time.perf_counter() - t0
            if i >= warmup:
                times.append(dt)
    med = statistics.median(times)
    sample = f"batch 1 of {cfg['b']}, seq {s} of {cfg['s']}, all {h} heads, {dtype}".replace("torch.", "")
    return b * s / med, med, sample


def run_reference(args, cfg, rank):
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    steps, warmup = min(steps, 5), min(warmup, 2)
    tps, med, sample = cpu_reference_sample(cfg, steps, warmup)
    line = {
        "impl": "reference", "metric": "ssd_forward_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": med * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16" if cfg["dtype"] != "f32" else "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_NAMES[args.workload], "name": args.workload},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample, "host_cpus": os.cpu_count()},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our arm

def time_steps(fn, nsets, steps, warmup, dist_on):
    import torch.distributed as dist

    for i in range(warmup):
        fn(i % nsets)
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(steps):
        fn(i % nsets)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    if dist_on:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if dist_on:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps, t0, t1


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
    ap.add_argument("--no-graphs", action="store_true",
                    help="launch every step from Python instead of replaying one CUDA graph per input set")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = CONFIGS[args.workload]

    if args.impl == "reference":
        run_reference(args, cfg, rank)
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

    seq_parallel = args.workload == "cfg3" and world > 1
    if seq_parallel:
        s_loc, h_loc = cfg["s"] // world, cfg["h"]
    else:
        h0, h1, _, _ = sharded.head_shard_bounds(cfg["h"], cfg["g"], rank, world)
        s_loc, h_loc = cfg["s"], h1 - h0
    set_bytes = algorithmic_bytes(cfg, h=h_loc, s=s_loc)
    nsets = max(2, int(math.ceil(2.5 * L2_BYTES / set_bytes)))
    nsets = min(nsets, 16)
    sets = [gen_inputs(cfg, dev, seed=1000 * rank + i, h=h_loc, s=s_loc) for i in range(nsets)]
    outs = [torch.empty_like(sets[i]["X"]) for i in range(nsets)]
    chunk = cfg["chunk"]
    kw = dict(kernel=args.kernel, nsegments=args.nsegments or None)

    plan = W.plan(sets[0]["X"], sets[0]["A"], sets[0]["B"], sets[0]["C"], chunk, **kw)
    if seq_parallel:
        # state-only run + cross-rank fold + seeded run that reuses the per-segment states (NCCL's own
        # all-gather kernel and two small copies into the send buffer are not counted)
        p_state = W.plan(sets[0]["X"], sets[0]["A"], sets[0]["B"], sets[0]["C"], chunk, state_only=True, **kw)
        seeded = plan["launches"] - 1 if plan["nsegments"] > 1 and plan["launches"] == 3 else plan["launches"]
        launches_per_step = [p_state["launches"] + 1 + seeded]
    else:
        launches_per_step = [plan["launches"]]
    if seq_parallel:
        # the local phases replay CUDA graphs; the all-gather is launched normally
        eng = sharded.SequenceShardedSSD(cuda_graphs=not args.no_graphs)

        def step(i):
            d = sets[i]
            eng.forward(d["X"], d["A"], d["B"], d["C"], chunk, out=outs[i], **kw)
    else:
        def step(i):
            d = sets[i]
            W.ssd_forward(d["X"], d["A"], d["B"], d["C"], chunk, initial_states=d.get("initial_states"),
                          out=outs[i], **kw)

    # A step is a fixed sequence of launches: capture it once per input set and replay, so that the
    # timed region measures the GPU and not the Python/driver launch path (which dominates at N=8).
    launch_mode = "eager"
    run_step = step
    if seq_parallel:
        launch_mode = "eager" if args.no_graphs else "cuda_graph (local phases) + eager all-gather"
    elif not args.no_graphs:
        try:
            for i in range(nsets):
                step(i)                      # allocates the workspace and warms NCCL outside capture
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

            launch_mode = "cuda_graph"
        except Exception as exc:  # fall back to plain launches
            sys.stderr.write(f"[bench] CUDA graph capture failed ({type(exc).__name__}: {exc}); timing eager launches\n")
            run_step = step
            launch_mode = "eager"

    sampler = ClockSampler(local)
    sampler.start()
    ms_step, t0, t1 = time_steps(run_step, nsets, args.steps, args.warmup, dist_on)
    sampler.stop()
    clocks = sampler.summary(t0, t1)

    tokens = cfg["b"] * cfg["s"]
    value = tokens / (ms_step * 1e-3)
    peak, peak_kind = measured_peaks()
    total_bytes = algorithmic_bytes(cfg)          # whole job
    achieved = set_bytes / (ms_step * 1e-3) / 1e9  # this GPU's share over the step time
    kname = W.kernel_name(sets[0]["X"], sets[0]["A"], sets[0]["B"], sets[0]["C"], chunk, kernel=args.kernel)

    # ---- end to end through the host-buffer entry point (pinned host tensors, copies timed)
    e2e = None
    try:
        if args.e2e_steps <= 0:
            raise RuntimeError("skipped (--e2e-steps 0)")
        hs = {k: v.cpu().pin_memory() for k, v in sets[0].items()}
        hout = torch.empty_like(hs["X"]).pin_memory()
        runner = W.HostRunner(cfg["b"], s_loc, h_loc, cfg["p"], cfg["n"], sets[0]["B"].shape[2], chunk,
                              TDT[cfg["dtype"]], device=dev, kernel=args.kernel)
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
        e2e = {"value": tokens / el, "unit": "tokens/s", "ms_per_step": el * 1e3,
               "h2d_bytes_per_step": runner.h2d_bytes, "d2h_bytes_per_step": runner.d2h_bytes,
               "note": "ssd_b200_forward_host: pinned host tensors in, Y back to host, copies inside the timed region"
               + (" (sequence shards run independently: no state exchange on this path)" if seq_parallel else "")}
        del hs, hout, runner
    except Exception as exc:  # report rather than lose the device-side numbers
        e2e = {"value": None, "unit": "tokens/s", "error": f"{type(exc).__name__}: {exc}"}

    # ---- other configurations, kernel-only, single GPU
    others = {}
    if world == 1 and not args.no_others:
        del sets, outs
        torch.cuda.empty_cache()
        for name in ("cfg0", "cfg1", "cfg3", "cfg4"):
            if name == args.workload:
                continue
            try:
                c = CONFIGS[name]
                sb = algorithmic_bytes(c)
                ns = min(16, max(2, int(math.ceil(2.5 * L2_BYTES / sb))))
                ss = [gen_inputs(c, dev, seed=77 + i) for i in range(ns)]
                oo = [torch.empty_like(x["X"]) for x in ss]

                def st(i, ss=ss, oo=oo, c=c):
                    d = ss[i]
                    W.ssd_forward(d["X"], d["A"], d["B"], d["C"], c["chunk"],
                                  initial_states=d.get("initial_states"), out=oo[i], kernel=args.kernel)

                ms, _, _ = time_steps(st, ns, max(5, args.steps // 2), 3, False)
                others[name] = {"tokens_per_s": c["b"] * c["s"] / (ms * 1e-3), "ms_per_step": ms,
                                "hbm_frac_of_measured": sb / (ms * 1e-3) / 1e9 / peak,
                                "kernel": W.kernel_name(ss[0]["X"], ss[0]["A"], ss[0]["B"], ss[0]["C"], c["chunk"],
                                                        kernel=args.kernel)}
                del ss, oo
                torch.cuda.empty_cache()
            except Exception as exc:
                others[name] = {"error": f"{type(exc).__name__}: {exc}"}

        # The same workload with the layer's skip and gate, (Y + x D) silu(z) of model_ref.py:116-118, fused into the
        # kernel's epilogue, next to the same three steps done as separate PyTorch passes over Y.
        try:
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

            ms_f, _, _ = time_steps(st_fused, ns, max(5, args.steps // 2), 3, False)
            ms_u, _, _ = time_steps(st_unfused, ns, max(5, args.steps // 2), 3, False)
            others[args.workload + "+skip_gate"] = {
                "tokens_per_s": c["b"] * c["s"] / (ms_f * 1e-3), "ms_per_step": ms_f,
                "hbm_frac_of_measured": sb / (ms_f * 1e-3) / 1e9 / peak,
                "ms_per_step_with_pytorch_epilogue": ms_u}
            del ss, oo, zz
            torch.cuda.empty_cache()
        except Exception as exc:
            others[args.workload + "+skip_gate"] = {"error": f"{type(exc).__name__}: {exc}"}

        # The X producer of the same workload: causal depthwise conv1d(k=4) + SiLU (model_ref.py:83-86) over
        # [b, s, h*p], read as a column slice of a projection-sized buffer; bytes = one read + one write.
        try:
            c = CONFIGS[args.workload]
            dch = c["h"] * c["p"]
            wdt = torch.bfloat16 if c["dtype"] == "bf16" else (torch.float16 if c["dtype"] == "f16" else torch.float32)
            wide = [torch.randn(c["b"], c["s"], 2 * dch + 64, device=dev, dtype=wdt) for _ in range(2)]
            yo = [torch.empty(c["b"], c["s"], dch, device=dev, dtype=wdt) for _ in range(2)]
            cw = torch.randn(dch, 1, 4, device=dev, dtype=wdt)
            cb = torch.randn(dch, device=dev, dtype=wdt)

            def st_conv(i):
                W.conv1d_silu(wide[i][..., :dch], cw, cb, out=yo[i])

            ms_c, _, _ = time_steps(st_conv, 2, max(5, args.steps // 2), 3, False)
            cbytes = 2 * c["b"] * c["s"] * dch * wide[0].element_size()
            others[args.workload + ":conv1d_silu"] = {"ms_per_step": ms_c, "GBps": cbytes / (ms_c * 1e-3) / 1e9,
                                                      "hbm_frac_of_measured": cbytes / (ms_c * 1e-3) / 1e9 / peak}
            del wide, yo
            torch.cuda.empty_cache()
        except Exception as exc:
            others[args.workload + ":conv1d_silu"] = {"error": f"{type(exc).__name__}: {exc}"}

        # The drop-in Model (reference contract: Model / get_init_inputs / get_inputs, model_ref.py:165-229) at the
        # reference's production layer shape, two layers instead of 24: projections on cuBLAS, conv, core, skip and gate
        # on this library's kernels.
        try:
            from workloadsuite_b200 import mamba_model as MM
            init = MM.get_init_inputs()
            init[1] = 2
            model = MM.Model(*init).to(dev).eval()
            xin = [torch.randn(MM.batch_size, MM.seq_length, MM.d_model, device=dev, dtype=torch.float16) for _ in range(2)]

            def st_model(i):
                with torch.inference_mode():
                    model(xin[i])

            ms_m, _, _ = time_steps(st_model, 2, max(5, args.steps // 5), 3, False)
            others["mamba_model_2_layers"] = {"ms_per_step": ms_m, "ms_per_layer": ms_m / 2,
                                              "tokens_per_s": MM.batch_size * MM.seq_length / (ms_m * 1e-3),
                                              "shape": "b8 s2048 d_model2048 h128 p64 n128 g8 block64 fp16"}
            del model, xin
            torch.cuda.empty_cache()
        except Exception as exc:
            others["mamba_model_2_layers"] = {"error": f"{type(exc).__name__}: {exc}"}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            tps, med, sample = cpu_reference_sample(cfg, 3, 1)
            cpu_baseline = {"value": tps, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                            "sample": sample, "host_cpus": os.cpu_count(), "s_per_sample": med}
        except Exception as exc:
            cpu_baseline = {"value": None, "unit": "tokens/s", "error": f"{type(exc).__name__}: {exc}"}

    if rank == 0:
        line = {
            "metric": "ssd_forward_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": n_gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
            "config": {"workload": WORKLOAD_NAMES[args.workload], "name": args.workload,
                       "parallelism": ("seq%d+allgather" % world) if seq_parallel else ("heads%d" % world),
                       "l2": f"{nsets} rotating input sets of {set_bytes / 1e6:.0f} MB per GPU (> L2)",
                       "kernel": kname, "launch": launch_mode, "segments_per_sequence": plan["nsegments"],
                       "kernel_launches_per_step": launches_per_step[0]},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind, "frac_of_8TBs": achieved / 8000.0,
                         "traffic": NCU_TRAFFIC_BYTES.get((args.workload, kname, world)),
                         "algorithmic_bytes_per_step_per_gpu": set_bytes, "algorithmic_bytes_whole_job": total_bytes},
            "cpu_baseline": cpu_baseline,
            "e2e": e2e,
            "gpu_launches": args.steps * launches_per_step[0],
            "clocks": clocks,
        }
        if others:
            line["other_configs"] = others
        print(json.dumps(line), flush=True)
    if dist_on:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
