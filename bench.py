"""Benchmark of the fused block-INT8 MoE layer (tokens/s) on 1..N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = routing (softmax top-k) + the fused expert layer over one batch of synthetic
tokens.  N = 1 runs the DeepSeek-V3-shape prefill configuration (E=256, top_k=8, M=4096,
H=7168, I=2048) as the headline line and adds a `sweep` over the decode sizes (M = 1..256 of the
same shape) and the Zipf-routed Qwen3-shape configuration, each timed as the median of CUDA-graph
replays; N > 1 runs the same layer with the experts sharded over the ranks (expert parallelism,
M tokens per rank; dispatch records and result rows stored straight into the peer GPUs' memory by the
library's kernels, NCCL for the counts and two barriers; the all-to-all transport is timed beside it)
after checking the sharded result of both transports against the single-GPU layer on a small case.
Prints ONE JSON line.

`value` is timed with every input resident in HBM; `e2e` is the same step called with
pinned HOST buffers (x and router logits copied in, y copied back, inside the timed
region).  Every configuration streams more weight bytes than L2 holds, so consecutive steps
cannot reuse cached operands.  `--impl reference` times the reference's own pure-torch
implementation of the path on the host cores on a bounded sample of the same workload (the
reference's functions themselves when a checkout is found, else their restatement).
"""
from __future__ import annotations

import argparse
import ctypes
import importlib.util
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fused_moe_w8a8_block_int8_tokens_per_s"
UNIT = "tokens/s"
DECODE_SWEEP = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def load_synthetic():
    """The input generators, loaded by path: importing the package would load the CUDA library, which the
    reference arm must not do."""
    spec = importlib.util.spec_from_file_location("_lo_synthetic", os.path.join(ROOT, "lightop_b200", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def make_config(name: str, cfg: dict, world: int) -> dict:
    """The workload description both arms print, key for key."""
    return {"workload": name, "E": cfg["E"], "top_k": cfg["topk"], "M": cfg["M"], "hidden": cfg["H"],
            "intermediate": cfg["I"], "parallelism": "single" if world == 1 else f"ep{world}",
            "l2": "every step streams more weight bytes than L2 holds; no flush needed"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def int8_peak():
    """INT8 tensor ceiling from the MMA-only loop (bench_mma_peak, built next to this file): POPS at N=128 / N=256."""
    exe = os.path.join(ROOT, "bench_mma_peak")
    if not os.path.exists(exe):
        return None
    try:
        out = subprocess.run([exe], capture_output=True, text=True, timeout=120).stdout.strip().splitlines()
        d = json.loads(out[-1])
        return {"n128_pops": d["int8_pops_n128"], "n256_pops": d["int8_pops_n256"],
                "how": "kind::i8 MMA-only loop on every SM, M=128, K=32, CUDA events"}
    except Exception as e:  # the number is context, not a gate
        return {"error": repr(e)}


def profile_traffic():
    """DRAM bytes per expert hit of the dominant kernel, from the committed ncu summaries (profiles/dram_traffic.md)."""
    table = {}
    path = os.path.join(ROOT, "profiles", "dram_traffic.md")
    if os.path.exists(path):
        for line in open(path):
            m = re.match(r"\|\s*`([a-z_0-9]+)`\s*\|\s*([0-9.eE+]+)\s*\|\s*([0-9.eE+]+)\s*\|", line)
            if m:
                table[m.group(1)] = (float(m.group(2)), float(m.group(3)))
    return table


class ClockSampler:
    """Samples SM clocks and throttle reasons (NVML, read-only) in a thread while the timed region runs."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int, period_s: float = 0.004):
        self.index = index
        self.period = period_s
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._first = threading.Event()
        self.thread = None
        self.error = None

    def _run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            # NVML enumerates physical devices: honour CUDA_VISIBLE_DEVICES when it lists plain indices
            idx = self.index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                parts = [v.strip() for v in vis.split(",") if v.strip()]
                if idx < len(parts) and parts[idx].isdigit():
                    idx = int(parts[idx])
            h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            while not self._stop.is_set():
                self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                try:
                    mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    mask = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for name, bit in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
                self._first.set()
                time.sleep(self.period)
        except Exception as e:  # NVML missing or refused: report it, do not fail the benchmark
            self.error = repr(e)
            self._first.set()

    def start(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        self._first.wait(timeout=5.0)      # NVML start-up can take a while: the first sample lands before the timed region

    def stop(self):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "samples": 0, "reasons": [self.error or "no samples"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "samples": len(self.samples),
                "reasons": sorted(self.reasons)}


def cuda_time_ms(fn, steps: int, stream) -> float:
    """Device time of `steps` calls of fn on `stream`, synchronised on both sides."""
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    for _ in range(steps):
        fn()
    end.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(end)


def graph_median_ms(step, replays: int = 50, warmup: int = 10):
    """Median device time of one CUDA-graph replay of `step` (the reference's harness times graph replays too,
    test/moe_w8a8/benchmark_moe_int8.py:532-557): at decode sizes the host's launch overhead would otherwise be
    part of the number."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(warmup):
        graph.replay()
    times = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(replays):
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times), min(times)


class E2ERunner:
    """The step with pinned host buffers in and out.  Every step copies its own inputs in and its own result out;
    steps are independent, so the copies of neighbouring steps overlap the compute of the current one (two device
    buffer sets, one stream each for H2D and D2H)."""

    def __init__(self, dev, x, logits, compute):
        self.dev = dev
        self.compute = compute          # compute(x_dev, logits_dev, buffer_index) -> y on the current stream
        self.x_h, self.l_h = x.cpu().pin_memory(), logits.cpu().pin_memory()
        self.y_h = [torch.empty(x.shape, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        self.x_d = [torch.empty_like(x) for _ in range(2)]
        self.l_d = [torch.empty_like(logits) for _ in range(2)]
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.h2d_bytes = self.x_h.numel() * 2 + self.l_h.numel() * 4
        self.d2h_bytes = self.y_h[0].numel() * 2

    def run(self, steps: int) -> float:
        """Device milliseconds from the first H2D copy to the last D2H copy of `steps` steps."""
        stream = torch.cuda.current_stream(self.dev)
        in_done = [torch.cuda.Event() for _ in range(steps)]
        comp_done = [torch.cuda.Event() for _ in range(steps)]
        out_done = [torch.cuda.Event() for _ in range(steps)]
        # y of step i stays referenced until step i+2 is enqueued, i.e. until the compute stream has been told to wait
        # for its copy-out: its memory then goes back to the allocator's cache in stream order, and a steady-state step
        # allocates nothing new from the driver
        keep = [None, None]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record(stream)
        self.s_in.wait_event(t0)
        for i in range(steps):
            b = i & 1
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(comp_done[i - 2])       # the buffers of step i-2 are free again
                self.x_d[b].copy_(self.x_h, non_blocking=True)
                self.l_d[b].copy_(self.l_h, non_blocking=True)
                in_done[i].record(self.s_in)
            stream.wait_event(in_done[i])
            if i >= 2:
                stream.wait_event(out_done[i - 2])               # y of step i-2 has left the device
            y = self.compute(self.x_d[b], self.l_d[b], b)
            keep[b] = y
            comp_done[i].record(stream)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(comp_done[i])
                self.y_h[b].copy_(y, non_blocking=True)
                out_done[i].record(self.s_out)
        stream.wait_event(out_done[steps - 1])
        t1.record(stream)
        torch.cuda.synchronize()
        return t0.elapsed_time(t1)

    def copy_only_ms(self, reps: int = 5):
        """H2D and D2H copy time of one step's buffers by themselves (median)."""
        h2d, d2h = [], []
        y = torch.empty(self.y_h[0].shape, dtype=torch.bfloat16, device=self.dev)
        for _ in range(reps):
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            torch.cuda.synchronize()
            e[0].record()
            self.x_d[0].copy_(self.x_h, non_blocking=True)
            self.l_d[0].copy_(self.l_h, non_blocking=True)
            e[1].record()
            self.y_h[0].copy_(y, non_blocking=True)
            e[2].record()
            torch.cuda.synchronize()
            h2d.append(e[0].elapsed_time(e[1]))
            d2h.append(e[1].elapsed_time(e[2]))
        return statistics.median(h2d), statistics.median(d2h)


# --------------------------------------------------------------------------- CPU arms

def reference_functions():
    """(route, fused layer, kind).  With a reference checkout ($LIGHTOP_REF or baseline/_ref) the layer's two heavy
    functions are the reference's own (test/moe_w8a8/benchmark_moe_int8.py:60-139, loaded without importing its
    package) inside the expert loop of its per-channel sibling (:163-201); without one, their restatement."""
    from oracle import moe_block_int8 as O
    from oracle import ref_extract
    if ref_extract.reference_root() is not None:
        try:
            quant, mm = ref_extract.reference_block_functions()

            def layer_ref(x, w1, w2, w1_s, w2_s, w, ids):
                return O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids, quant_fn=quant, matmul_fn=mm)
            return O.route_topk_softmax, layer_ref, "reference"
        except Exception:
            pass
    return O.route_topk_softmax, O.fused_moe_block_int8, "port"


def cpu_sample(cfg, syn, n_experts_sample: int, weights=None, x=None, logits=None):
    """Routed rows of the first `n_experts_sample` experts of one batch: (callable step, rows, kind)."""
    route, layer, kind = reference_functions()
    E, k, M, H, I = cfg["E"], cfg["topk"], cfg["M"], cfg["H"], cfg["I"]
    n = min(n_experts_sample, E)
    if weights is None:
        w1, w2, w1_s, w2_s = syn.make_weights(n, H, I, seed=0)
    else:
        w1, w2, w1_s, w2_s = (t[:n].cpu() for t in weights)
    if x is None:
        x, logits = syn.make_activations(M, H, E, seed=1, zipf=cfg.get("zipf"))
    x, logits = x.cpu(), logits.cpu()
    w, ids = route(logits, k, renormalize=True)
    keep = ids < n
    rows = int(keep.sum())
    # slots routed elsewhere get weight 0 and an id outside the sample: the expert loop skips them
    ids_s = torch.where(keep, ids, torch.full_like(ids, n))
    w_s = w * keep

    def step():
        route(logits, k, renormalize=True)
        layer(x, w1, w2, w1_s, w2_s, w_s, ids_s)
    return step, rows, kind, n


def cpu_baseline(cfg, syn, weights, x, logits, n_experts_sample: int, threads: int):
    torch.set_num_threads(threads)
    step, rows, kind, n = cpu_sample(cfg, syn, n_experts_sample, weights, x, logits)
    t0 = time.perf_counter()
    step()
    dt = time.perf_counter() - t0
    return {"value": (rows / cfg["topk"]) / dt, "unit": UNIT, "cores": threads, "kind": kind,
            "sample": f"the reference's pure-torch path ({'its own functions' if kind == 'reference' else 'restatement'}) over the "
                      f"{rows} routed rows of the first {n} of {cfg['E']} experts of the same batch, {dt:.1f} s; tokens = rows / top_k"}


def run_reference(args, rank: int, world: int):
    """The reference's CPU implementation of the path on the host cores, a bounded sample per step."""
    if rank != 0:
        return None
    syn = load_synthetic()
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    name = args.workload or ("c1_dsv3_prefill" if world == 1 else "c3_dsv3_ep_rank")
    cfg = dict(syn.CONFIGS[name])
    if args.tokens:
        cfg["M"] = args.tokens
    if args.experts:
        cfg["E"] = args.experts
    step, rows, kind, n = cpu_sample(cfg, syn, args.cpu_sample_experts)
    for _ in range(min(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = (rows / cfg["topk"]) / dt
    sample = (f"the reference's pure-torch path ({'its own functions' if kind == 'reference' else 'restatement'}) over the {rows} "
              f"routed rows of the first {n} of {cfg['E']} experts of one batch per step ({dt:.1f} s/step); tokens = rows / top_k")
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32 torch on int8 codes", "data": "synthetic",
        "config": make_config(name, cfg, world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# --------------------------------------------------------------------------- GPU arm, one GPU

def gate_up_alg_bytes(M, k, H, I, experts_hit, channel=False):
    """Algorithmic bytes of one gate_up launch: int8 weights + block scales of the experts hit (2I x H each), the
    int8 activations + scales read once, the int8 act + scales written once."""
    rows = M * k
    if channel:
        return experts_hit * (2.0 * I * H + 4.0 * 2 * I) + M * (H + 4.0) + rows * (2.0 * 2 * I * 2 + I + 4.0)
    return (experts_hit * (2.0 * I * H + 4.0 * (2 * I // 128) * (H // 128)) + M * (H + 4.0 * H / 128)
            + rows * (I + 4.0 * I / 128))


def stage_times(lightop_b200, _lib, step, reps: int):
    """Per-kernel durations of the fused call (separate pass, events between its kernels)."""
    lib = _lib.load()
    lib.lo_profile_enable(1)
    stage = [0.0] * 5
    buf = (ctypes.c_float * 5)()
    for _ in range(reps):
        step()
        _lib.check(lib.lo_profile_read(buf), "profile read")
        for i in range(5):
            stage[i] += buf[i] / reps
    lib.lo_profile_enable(0)
    return {"align": stage[0], "group_quant_scatter": stage[1], "gemm_gate_up": stage[2], "gemm_down": stage[3],
            "moe_sum": stage[4]}


def run_ours(args, rank: int, world: int, local_rank: int):
    import lightop_b200
    from lightop_b200 import _lib, synthetic

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        return run_ep(args, rank, world, dev)

    name = args.workload or "c1_dsv3_prefill"
    cfg = dict(synthetic.CONFIGS[name])
    custom = bool(args.tokens or args.experts or args.workload or args.quant != "block")
    if args.tokens:
        cfg["M"] = args.tokens
    if args.experts:
        cfg["E"] = args.experts
    E, k, M, H, I = cfg["E"], cfg["topk"], cfg["M"], cfg["H"], cfg["I"]
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=0, device=dev)
    channel = args.quant == "channel"
    if channel:
        # per-channel W8A8 mode of the same layer: same int8 weights, one scale per output channel
        w1_s, w2_s = synthetic.make_channel_scales(E, H, I, seed=0, device=dev)
        quant_kw = dict(use_int8_w8a8=True, per_channel_quant=True, block_shape=None)
    else:
        quant_kw = dict(use_int8_w8a8=True, block_shape=[128, 128])
    lib = _lib.load()
    stream = torch.cuda.current_stream(dev)
    hbm_peak, peak_kind = measured_peaks()
    traffic_table = profile_traffic()

    def make_step(x, logits, w1, w2, w1_s, w2_s, kw):
        Mx = x.shape[0]
        tw = torch.empty(Mx, k, dtype=torch.float32, device=dev)
        ti = torch.empty(Mx, k, dtype=torch.int32, device=dev)
        cache13 = torch.empty(Mx * k * x.shape[1], dtype=torch.bfloat16, device=dev)
        holder = {}

        def step():
            lightop_b200.moe.topk_softmax(tw, ti, None, logits, True)
            holder["y"] = lightop_b200.moe.fused_experts_impl_int8(x, w1, w2, tw, ti, cache13, w1_scale=w1_s, w2_scale=w2_s, **kw)
        return step, ti, holder

    x, logits = synthetic.make_activations(M, H, E, seed=1, device=dev, zipf=cfg.get("zipf"))
    step, ti, _ = make_step(x, logits, w1, w2, w1_s, w2_s, quant_kw)

    # end-to-end arm: pinned host buffers in, pinned host buffer out
    tw2 = [torch.empty(M, k, dtype=torch.float32, device=dev) for _ in range(2)]
    ti2 = [torch.empty(M, k, dtype=torch.int32, device=dev) for _ in range(2)]
    c13 = [torch.empty(M * k * H, dtype=torch.bfloat16, device=dev) for _ in range(2)]

    def compute(xd, ld, b):
        lightop_b200.moe.topk_softmax(tw2[b], ti2[b], None, ld, True)
        return lightop_b200.moe.fused_experts_impl_int8(xd, w1, w2, tw2[b], ti2[b], c13[b], w1_scale=w1_s, w2_scale=w2_s, **quant_kw)
    e2e = E2ERunner(dev, x, logits, compute)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    lightop_b200.check_device_status(dev)

    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = lib.lo_launch_count()
    total_ms = cuda_time_ms(step, args.steps, stream)
    launches = lib.lo_launch_count() - launches0
    clocks = sampler.stop()
    ms_per_step = total_ms / args.steps

    e2e.run(3)
    # three runs of K steps each; the line reports the fastest and lists all three (a run on these shared hosts
    # occasionally contains a stall of tens of milliseconds that is not the step's)
    e2e_runs = [e2e.run(args.steps) / args.steps for _ in range(3)]
    e2e_ms = min(e2e_runs)
    h2d_ms, d2h_ms = e2e.copy_only_ms()

    stage = stage_times(lightop_b200, _lib, step, args.steps)
    lightop_b200.check_device_status(dev)

    experts_hit = int(torch.unique(ti).numel())
    rows_routed = M * k

    def roofline_of(Mx, hit, stage_ms, chan=False):
        g1_bytes = gate_up_alg_bytes(Mx, k, H, I, hit, chan)
        g1_s = stage_ms["gemm_gate_up"] * 1e-3
        key = "gate_up_channel" if chan else ("gate_up_prefill" if Mx * k / max(hit, 1) > 64 else "gate_up_decode")
        per_expert = traffic_table.get(key)
        traffic = None if per_expert is None else hit * per_expert[0] + Mx * k * per_expert[1]
        return {"bound": "hbm", "kernel": "grouped_gemm_kernel<channel> + silu_mul_token_quant_kernel" if chan
                else "grouped_gemm_kernel<gate_up>", "achieved": g1_bytes / g1_s / 1e9, "peak": hbm_peak,
                "peak_kind": peak_kind, "unit": "GB/s", "frac": g1_bytes / g1_s / 1e9 / hbm_peak, "traffic": traffic,
                "traffic_source": f"profiles/dram_traffic.md row `{key}` (ncu dram bytes per expert hit and per routed row)",
                "ms_per_launch": stage_ms["gemm_gate_up"], "stage_ms": stage_ms}

    roofline = roofline_of(M, experts_hit, stage, channel)
    layer_bytes = synthetic.alg_bytes(M, E, H, I, experts_hit)
    flops = synthetic.alg_flops(M, k, H, I)

    # ------------------------------------------------------------------ sweep: decode sizes and the Zipf configuration
    sweep = None
    if not custom and not args.no_sweep:
        sweep = []
        sampler = ClockSampler(local_rank)
        sampler.start()
        x256, l256 = synthetic.make_activations(256, H, E, seed=1, device=dev)

        def entry(wname, Mx, xs, ls, weights, Ex, Hx, Ix):
            st, ti_s, _ = make_step(xs, ls, *weights, dict(use_int8_w8a8=True, block_shape=[128, 128]))
            own = ClockSampler(local_rank, period_s=0.001)       # clocks seen during this entry's replays
            own.start()
            med, best = graph_median_ms(st, replays=max(50, args.graph_replays))
            own_clocks = own.stop()
            hit = int(torch.unique(ti_s).numel())
            sm = stage_times(lightop_b200, _lib, st, 5)
            lb = synthetic.alg_bytes(Mx, Ex, Hx, Ix, hit)
            g1 = gate_up_alg_bytes(Mx, k, Hx, Ix, hit) / (sm["gemm_gate_up"] * 1e-3) / 1e9
            return {"workload": wname, "M": Mx, "ms_per_step": med, "ms_best": best, "tokens_per_s": Mx / (med * 1e-3),
                    "experts_hit": hit, "layer_alg_gbs": lb / (med * 1e-3) / 1e9, "layer_frac": lb / (med * 1e-3) / 1e9 / hbm_peak,
                    "gate_up_frac": g1 / hbm_peak, "stage_ms": sm, "clocks": own_clocks,
                    "timing": f"median of {max(50, args.graph_replays)} CUDA-graph replays"}

        for Mx in DECODE_SWEEP:
            sweep.append(entry("c2_dsv3_decode", Mx, x256[:Mx].contiguous(), l256[:Mx].contiguous(), (w1, w2, w1_s, w2_s), E, H, I))
        c4 = dict(synthetic.CONFIGS["c4_qwen3_zipf"])
        w4 = synthetic.make_weights(c4["E"], c4["H"], c4["I"], seed=0, device=dev)
        x4, l4 = synthetic.make_activations(c4["M"], c4["H"], c4["E"], seed=1, device=dev, zipf=c4.get("zipf"))
        sweep.append(entry("c4_qwen3_zipf", c4["M"], x4, l4, w4, c4["E"], c4["H"], c4["I"]))
        del w4, x4, l4
        sweep_clocks = sampler.stop()
        lightop_b200.check_device_status(dev)
    else:
        sweep_clocks = None

    cpu = None
    if not args.no_cpu_baseline and not channel:
        cpu = cpu_baseline(cfg, synthetic, (w1, w2, w1_s, w2_s), x, logits, args.cpu_sample_experts, os.cpu_count() or 1)

    line = {
        "metric": METRIC, "value": M / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int8 -> int32, fp32 %s scaling, bf16 in/out" % ("per-channel" if channel else "block"),
        "data": "synthetic",
        "config": make_config(name + ("+per_channel_quant" if channel else ""), cfg, 1),
        "experts_hit": experts_hit,
        "tflops": flops / (ms_per_step * 1e-3) / 1e12,
        "layer_alg_gbs": layer_bytes / (ms_per_step * 1e-3) / 1e9,
        "layer_frac_of_hbm_roofline": layer_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak,
        "e2e": {"value": M / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms, "ms_per_step_runs": e2e_runs,
                "h2d_bytes_per_step": e2e.h2d_bytes, "d2h_bytes_per_step": e2e.d2h_bytes,
                "h2d_copy_only_ms": h2d_ms, "d2h_copy_only_ms": d2h_ms,
                "overlap": "copies of neighbouring steps overlap compute (double-buffered, 3 streams)"},
        "gpu_launches": int(launches),
        "gpu_launches_how": "counted by the library (lo_launch_count) over the timed region",
        "clocks": clocks, "roofline": roofline, "int8_peak": int8_peak(), "cpu_baseline": cpu,
    }
    if sweep is not None:
        line["sweep"] = sweep
        line["sweep_clocks"] = sweep_clocks
    return line


# --------------------------------------------------------------------------- GPU arm, expert parallelism

def ep_parity_check(lightop_b200, synthetic, ExpertParallelMoE, dist, rank, world, dev):
    """A small sharded case against the single-GPU layer on the rank's own tokens: every rank builds ALL the weights
    from one seed, runs the expert-parallel step over NCCL with the CUDA kernels, and compares bit for bit."""
    E, k, M, H, I = 8 * world, 4, 96, 512, 256
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=7, device=dev)
    x, logits = synthetic.make_activations(M, H, E, seed=50 + rank, device=dev)
    tw = torch.empty(M, k, dtype=torch.float32, device=dev)
    ti = torch.empty(M, k, dtype=torch.int32, device=dev)
    lightop_b200.moe.topk_softmax(tw, ti, None, logits, True)
    c13 = torch.empty(M * k * H, dtype=torch.bfloat16, device=dev)
    local = lightop_b200.moe.fused_experts_impl_int8(x, w1, w2, tw, ti, c13, use_int8_w8a8=True, block_shape=[128, 128],
                                                     w1_scale=w1_s, w2_scale=w2_s)
    El = E // world
    sl = slice(rank * El, (rank + 1) * El)
    ok, worst, send = True, 0.0, None
    per_transport = {}
    for transport in ("peer", "collective"):
        layer = ExpertParallelMoE(w1[sl].contiguous(), w2[sl].contiguous(), w1_s[sl].contiguous(), w2_s[sl].contiguous(), E,
                                  transport=transport)
        y = layer.forward(x, tw, ti)
        y = layer.forward(x, tw, ti)         # a second step reuses the landing zones
        torch.cuda.synchronize()
        lightop_b200.check_device_status(dev)
        equal = torch.tensor([1 if torch.equal(y, local) else 0], dtype=torch.int32, device=dev)
        maxdiff = (y.float() - local.float()).abs().max().reshape(1)
        dist.all_reduce(equal, op=dist.ReduceOp.MIN)
        dist.all_reduce(maxdiff, op=dist.ReduceOp.MAX)
        per_transport[transport] = bool(equal.item() == 1)
        ok = ok and per_transport[transport]
        worst = max(worst, float(maxdiff.item()))
        send, recv = layer.last_counts
        layer.close()
    return {"bit_equal": ok, "ranks": world, "max_abs_diff": worst, "per_transport": per_transport,
            "case": {"E": E, "top_k": k, "M_per_rank": M, "hidden": H, "intermediate": I},
            "rows_sent_to_peers_rank0": sum(send) - send[rank],
            "against": "fused_experts_impl_int8 with all experts on the rank's own GPU, same tokens"}


def run_ep(args, rank: int, world: int, dev: torch.device):
    """The N>1 leg: DeepSeek-V3 shape, experts split over the ranks, M tokens per rank."""
    import torch.distributed as dist
    import lightop_b200
    from lightop_b200 import _lib, synthetic
    from lightop_b200.ep import ExpertParallelMoE

    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    name = args.workload or "c3_dsv3_ep_rank"
    cfg = dict(synthetic.CONFIGS[name])
    if args.tokens:
        cfg["M"] = args.tokens
    if args.experts:
        cfg["E"] = args.experts
    E, k, M, H, I = cfg["E"], cfg["topk"], cfg["M"], cfg["H"], cfg["I"]
    if E % world:
        raise ValueError(f"{E} experts do not split over {world} ranks")
    parity = ep_parity_check(lightop_b200, synthetic, ExpertParallelMoE, dist, rank, world, dev)

    E_local = E // world
    w1, w2, w1_s, w2_s = synthetic.make_weights(E_local, H, I, seed=100 + rank, device=dev)
    x, logits = synthetic.make_activations(M, H, E, seed=1 + rank, device=dev, zipf=cfg.get("zipf"))
    layer = ExpertParallelMoE(w1, w2, w1_s, w2_s, E)
    tw = [torch.empty(M, k, dtype=torch.float32, device=dev) for _ in range(2)]
    ti = [torch.empty(M, k, dtype=torch.int32, device=dev) for _ in range(2)]
    stream = torch.cuda.current_stream(dev)
    holder = {}

    def step():
        lightop_b200.moe.topk_softmax(tw[0], ti[0], None, logits, True)
        holder["y"] = layer.forward(x, tw[0], ti[0])

    def compute(xd, ld, b):
        lightop_b200.moe.topk_softmax(tw[b], ti[b], None, ld, True)
        return layer.forward(xd, tw[b], ti[b])
    e2e = E2ERunner(dev, x, logits, compute)

    def timed(fn, steps):
        dist.barrier()
        ms = fn(steps)
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        return float(t.item())

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    lightop_b200.check_device_status(dev)
    sampler = ClockSampler(dev.index)
    sampler.start()
    launches0 = lib.lo_launch_count()
    ms_per_step = timed(lambda n: cuda_time_ms(step, n, stream), args.steps) / args.steps
    launches = lib.lo_launch_count() - launches0
    clocks = sampler.stop()
    e2e.run(2)
    e2e_runs = [timed(e2e.run, args.steps) / args.steps for _ in range(3)]
    e2e_ms = min(e2e_runs)
    h2d_ms, d2h_ms = e2e.copy_only_ms()
    # stage breakdown of the step on rank 0 (a separate pass: events after every stage)
    layer.profile = True
    acc = {}
    for _ in range(3):
        dist.barrier()
        step()
        for kname, v in layer.stage_ms().items():
            acc[kname] = acc.get(kname, 0.0) + v / 3
    layer.profile = False
    lightop_b200.check_device_status(dev)
    # the same step with the exchange as NCCL all-to-all collectives, for comparison
    other = ExpertParallelMoE(w1, w2, w1_s, w2_s, E, transport="collective" if layer.transport == "peer" else "peer")

    def step_other():
        lightop_b200.moe.topk_softmax(tw[0], ti[0], None, logits, True)
        holder["y2"] = other.forward(x, tw[0], ti[0])
    for _ in range(3):
        step_other()
    other_ms = timed(lambda n: cuda_time_ms(step_other, n, stream), 5) / 5
    same_bits = torch.tensor([1 if torch.equal(holder["y"], holder["y2"]) else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(same_bits, op=dist.ReduceOp.MIN)
    other.close()

    send_counts, recv_counts = layer.last_counts
    rows_recv = sum(recv_counts)
    remote_rows = sum(send_counts) - send_counts[rank]
    total_tokens = M * world
    flops = synthetic.alg_flops(M, k, H, I) * world
    hbm_peak, peak_kind = measured_peaks()
    peak8 = int8_peak() if rank == 0 else None
    tensor_frac = None
    if peak8 and "n256_pops" in peak8 and acc.get("experts"):
        # the experts stage of one rank against the INT8 tensor ceiling (chunks of up to 160 tokens: between the N=128
        # and the N=256 rate; the N=256 figure is the stricter denominator)
        tensor_frac = synthetic.alg_flops(rows_recv / k, k, H, I) / (acc["experts"] * 1e-3) / 1e15 / peak8["n256_pops"]
    comm_glue = sum(v for kname, v in acc.items() if kname != "experts")
    line = {
        "metric": METRIC, "value": total_tokens / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x int8 -> int32, fp32 block scaling, bf16 in/out", "data": "synthetic",
        "config": make_config(name, cfg, world),
        "ep": {"experts_per_rank": E_local, "rows_received_rank0": rows_recv, "rows_sent_to_peers_rank0": remote_rows,
               "dispatch_bytes_per_row": int(lib.lo_ep_dispatch_row_bytes(H)), "combine_bytes_per_row": 2 * H,
               "transport": layer.transport,
               "transport_how": ("records and result rows are stored into the destination rank's device memory by the "
                                 "dispatch kernel and by the down GEMM's epilogue (plain stores over NVLink); per step one "
                                 "all-gather of the counts and two one-word all-reduces as barriers")
               if layer.transport == "peer" else "three all-to-all collectives per step (counts, records, result rows)",
               "other_transport": {"name": other.transport, "ms_per_step": other_ms, "same_bits": bool(same_bits.item() == 1)},
               "collectives_per_step": 3},
        "ep_parity": parity,
        "stage_ms": acc, "comm_and_glue_frac_of_step": comm_glue / max(sum(acc.values()), 1e-9),
        "tflops": flops / (ms_per_step * 1e-3) / 1e12,
        "e2e": {"value": total_tokens / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms, "ms_per_step_runs": e2e_runs,
                "h2d_bytes_per_step": e2e.h2d_bytes * world, "d2h_bytes_per_step": e2e.d2h_bytes * world,
                "h2d_copy_only_ms": h2d_ms, "d2h_copy_only_ms": d2h_ms,
                "overlap": "copies of neighbouring steps overlap compute (double-buffered, 3 streams)"},
        "gpu_launches": int(launches),
        "gpu_launches_how": "counted by the library (lo_launch_count) on rank 0 over the timed region; NCCL's kernels are not ours",
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (experts stage: align, permute, gate_up, down)",
                     "achieved": None if not acc.get("experts") else synthetic.alg_flops(rows_recv / k, k, H, I) / (acc["experts"] * 1e-3) / 1e12,
                     "peak": None if not peak8 or "n256_pops" not in peak8 else peak8["n256_pops"] * 1e3,
                     "peak_kind": "kind::i8 MMA-only loop at N=256, this run", "unit": "TFLOP/s", "frac": tensor_frac,
                     "traffic": None, "hbm_peak_gbs": hbm_peak, "hbm_peak_kind": peak_kind},
        "int8_peak": peak8, "cpu_baseline": None,
    }
    dist.barrier()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--tokens", type=int, default=0, help="override the token count M of the workload")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count E (small profiling cases)")
    ap.add_argument("--quant", default="block", choices=["block", "channel"],
                    help="block = the 128x128 block-INT8 path (the headline metric); channel = the per-channel W8A8 mode "
                         "of the same layer (1 GPU, no CPU baseline)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the decode / Zipf sweep of the 1-GPU run")
    ap.add_argument("--graph-replays", type=int, default=50)
    ap.add_argument("--cpu-sample-experts", type=int, default=256)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    # stdout carries the one JSON line only: anything a library prints to file descriptor 1 (NCCL's
    # version banner, for one) goes to stderr; the line itself is written to the saved descriptor.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(line):
        os.write(json_fd, (json.dumps(line) + "\n").encode())

    if args.impl == "reference":
        if args.steps > 3:
            args.steps = 3          # each step is seconds of CPU work
        line = run_reference(args, rank, world)
        if line is not None:
            emit(line)
        return
    line = run_ours(args, rank, world, local_rank)
    if line is not None and rank == 0:
        emit(line)
    if world > 1:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
