"""Benchmark of the fused block-INT8 MoE layer (tokens/s) on 1..N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = routing (softmax top-k) + the fused expert layer over one batch of synthetic
tokens.  N = 1 runs the DeepSeek-V3-shape prefill configuration (E=256, top_k=8, M=4096,
H=7168, I=2048); N > 1 runs the same layer with the experts sharded over the ranks
(expert parallelism, M tokens per rank, dispatch/combine over NCCL).  Prints ONE JSON line.

`value` is timed with every input resident in HBM; `e2e` is the same step called with
pinned HOST buffers (x and router logits copied in, y copied back, inside the timed
region).  The weights (11.3 GB) are larger than L2, so consecutive steps cannot reuse
cached operands.  `--impl reference` times the reference's own pure-torch implementation
of the path (the oracle) on the host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
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


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


def cpu_baseline(cfg, w1, w2, w1_s, w2_s, x, logits, n_experts_sample: int, threads: int):
    """The oracle on the host cores over the tokens routed to the first `n_experts_sample` experts."""
    from oracle import moe_block_int8 as O
    torch.set_num_threads(threads)
    E, k = cfg["E"], cfg["topk"]
    xc, lc = x.cpu(), logits.cpu()
    w, ids = O.route_topk_softmax(lc, k, renormalize=True)
    sel = list(range(min(n_experts_sample, E)))
    w1c = w1[sel].cpu()
    w2c = w2[sel].cpu()
    w1sc, w2sc = w1_s[sel].cpu(), w2_s[sel].cpu()
    keep = ids < len(sel)
    rows = int(keep.sum())
    t0 = time.perf_counter()
    # slots routed elsewhere get weight 0 and an id outside the sample: the oracle's expert loop skips them
    O.fused_moe_block_int8(xc, w1c, w2c, w1sc, w2sc, w * keep, torch.where(keep, ids, torch.full_like(ids, len(sel))))
    dt = time.perf_counter() - t0
    tokens_equiv = rows / k
    return tokens_equiv / dt, dt, rows


def run_ours(args, rank: int, world: int, local_rank: int):
    import lightop_b200
    from lightop_b200 import _lib, synthetic

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        from lightop_b200 import ep
        return ep.bench_step_setup(args, rank, world, dev)

    name = args.workload or "c1_dsv3_prefill"
    cfg = dict(synthetic.CONFIGS[name])
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
    x, logits = synthetic.make_activations(M, H, E, seed=1, device=dev, zipf=cfg.get("zipf"))
    tw = torch.empty(M, k, dtype=torch.float32, device=dev)
    ti = torch.empty(M, k, dtype=torch.int32, device=dev)
    cache13 = torch.empty(M * k * H, dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream(dev)
    out_holder = {}

    def step():
        lightop_b200.moe.topk_softmax(tw, ti, None, logits, True)
        out_holder["y"] = lightop_b200.moe.fused_experts_impl_int8(
            x, w1, w2, tw, ti, cache13, w1_scale=w1_s, w2_scale=w2_s, **quant_kw)

    # end-to-end arm: pinned host buffers in, pinned host buffer out.  Every step copies its own x and
    # logits in and its own y out; steps are independent, so the copies of neighbouring steps overlap
    # the compute of the current one (two device buffer sets, one stream each for H2D and D2H).
    x_h = x.cpu().pin_memory()
    l_h = logits.cpu().pin_memory()
    y_h = [torch.empty(M, H, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    x_d = [torch.empty_like(x) for _ in range(2)]
    l_d = [torch.empty_like(logits) for _ in range(2)]
    tw2 = [torch.empty_like(tw) for _ in range(2)]
    ti2 = [torch.empty_like(ti) for _ in range(2)]
    c13 = [cache13, torch.empty_like(cache13)]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def run_e2e(steps):
        """Returns device milliseconds from the first H2D copy to the last D2H copy of `steps` steps."""
        in_done = [torch.cuda.Event() for _ in range(steps)]
        comp_done = [torch.cuda.Event() for _ in range(steps)]
        out_done = [torch.cuda.Event() for _ in range(steps)]
        keep = []
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record(stream)
        s_in.wait_event(t0)
        for i in range(steps):
            b = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(comp_done[i - 2])       # the buffers of step i-2 are free again
                x_d[b].copy_(x_h, non_blocking=True)
                l_d[b].copy_(l_h, non_blocking=True)
                in_done[i].record(s_in)
            stream.wait_event(in_done[i])
            if i >= 2:
                stream.wait_event(out_done[i - 2])          # y of step i-2 has left the device
            lightop_b200.moe.topk_softmax(tw2[b], ti2[b], None, l_d[b], True)
            y = lightop_b200.moe.fused_experts_impl_int8(
                x_d[b], w1, w2, tw2[b], ti2[b], c13[b], w1_scale=w1_s, w2_scale=w2_s, **quant_kw)
            keep.append(y)
            comp_done[i].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[i])
                y_h[b].copy_(y, non_blocking=True)
                out_done[i].record(s_out)
        stream.wait_event(out_done[steps - 1])
        t1.record(stream)
        torch.cuda.synchronize()
        return t0.elapsed_time(t1)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    lightop_b200.check_device_status(dev)

    sampler = ClockSampler(local_rank)
    sampler.start()
    total_ms = cuda_time_ms(step, args.steps, stream)
    clocks = sampler.stop()
    ms_per_step = total_ms / args.steps

    run_e2e(3)
    e2e_ms = run_e2e(args.steps) / args.steps

    # per-kernel durations of the fused call (separate pass, events between its kernels)
    lib = _lib.load()
    lib.lo_profile_enable(1)
    stage = [0.0] * 5
    buf = (ctypes.c_float * 5)()
    for _ in range(args.steps):
        step()
        _lib.check(lib.lo_profile_read(buf), "profile read")
        for i in range(5):
            stage[i] += buf[i] / args.steps
    lib.lo_profile_enable(0)
    lightop_b200.check_device_status(dev)

    experts_hit = int(torch.unique(ti).numel())
    rows_routed = M * k
    hbm_peak, peak_kind = measured_peaks()
    # dominant kernel: the gate_up grouped GEMM.  Algorithmic bytes per launch: int8 weights + block scales of
    # the experts hit (2I x H each), the int8 activations + scales read once, the int8 act + scales written once.
    g1_bytes = (experts_hit * (2.0 * I * H + 4.0 * (2 * I // 128) * (H // 128)) + M * (H + 4.0 * H / 128)
                + rows_routed * (I + 4.0 * I / 128))
    if channel:
        # per-channel: int8 weights + one scale per channel, int8 activations + one scale per row read,
        # bf16 gate_up rows written, read again by the SiLU*mul+quant kernel (same stage), int8 act written
        g1_bytes = (experts_hit * (2.0 * I * H + 4.0 * 2 * I) + M * (H + 4.0)
                    + rows_routed * (2.0 * 2 * I * 2 + I + 4.0))
    g1_s = stage[2] * 1e-3
    # DRAM traffic of the dominant kernel from the committed ncu captures (profiles/), scaled by the experts hit:
    # 128 rows per expert -> 1.316 GB read + 10.4 MB written per 32 experts; decode-size chunks -> no re-reads.
    if rows_routed / max(experts_hit, 1) > 64:
        traffic = experts_hit / 32.0 * (1.316404e9 + 10.436608e6)
        traffic_src = "profiles/grouped_gemm_prefill_e32_m512.md (ncu dram bytes of the E=32, M=512 case) x experts_hit/32"
    else:
        traffic = experts_hit / 32.0 * (0.945233e9 + 4.008e6)
        traffic_src = "profiles/grouped_gemm_decode_e32_m64.md (ncu dram bytes of the E=32, M=64 case) x experts_hit/32"
    if channel:
        # gate_up launch of the committed capture: 973.8 MB read + 10.6 MB written per 32 experts at 128 rows each
        # (bf16 output rows scale with the routed rows, not with the experts)
        traffic = experts_hit / 32.0 * 973.80864e6 + rows_routed / 4096.0 * 10.649856e6
        traffic_src = ("profiles/grouped_gemm_channel_prefill_e32_m512.md (ncu dram bytes of the E=32, M=512 case): reads x "
                       "experts_hit/32, writes x routed rows/4096; GEMM launch only")
    roofline = {"bound": "hbm", "kernel": "grouped_gemm_kernel<channel> + silu_mul_token_quant_kernel" if channel
                else "grouped_gemm_kernel<gate_up>", "achieved": g1_bytes / g1_s / 1e9,
                "peak": hbm_peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": g1_bytes / g1_s / 1e9 / hbm_peak,
                "traffic": traffic, "traffic_source": traffic_src, "ms_per_launch": stage[2],
                "stage_ms": {"align": stage[0], "group_quant_scatter": stage[1], "gemm_gate_up": stage[2],
                             "gemm_down": stage[3], "moe_sum": stage[4]}}
    layer_bytes = synthetic.alg_bytes(M, E, H, I, experts_hit)
    flops = synthetic.alg_flops(M, k, H, I)

    cpu = None
    if not args.no_cpu_baseline and not channel:
        threads = os.cpu_count() or 1
        n_sample = args.cpu_sample_experts
        v, dt, rows = cpu_baseline(cfg, w1, w2, w1_s, w2_s, x, logits, n_sample, threads)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"oracle (pure-torch restatement of the reference path) over the {rows} routed rows of the first "
                         f"{n_sample} of {E} experts of the same batch, {dt:.1f} s; tokens = rows / top_k"}

    line = {
        "metric": METRIC, "value": M / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int8 -> int32, fp32 %s scaling, bf16 in/out" % ("per-channel" if channel else "block"),
        "data": "synthetic",
        "config": {"workload": name + ("+per_channel_quant" if channel else ""), "E": E, "top_k": k, "M": M,
                   "hidden": H, "intermediate": I,
                   "experts_hit": experts_hit, "l2": "weights (11.3 GB) exceed L2; no flush needed"},
        "tflops": flops / (ms_per_step * 1e-3) / 1e12,
        "layer_alg_gbs": layer_bytes / (ms_per_step * 1e-3) / 1e9,
        "layer_frac_of_hbm_roofline": layer_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak,
        "e2e": {"value": M / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": x_h.numel() * 2 + l_h.numel() * 4, "d2h_bytes_per_step": y_h[0].numel() * 2,
                "overlap": "copies of neighbouring steps overlap compute (double-buffered, 3 streams)"},
        # router, align, [wide chunk table of the down GEMM from 64 rows per expert on], quantise, two GEMMs
        # [+ SiLU/quant kernel in the per-channel mode], top-k sum
        "gpu_launches": (7 if channel else (7 if M * k // E >= 64 else 6)) * args.steps,
        "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
    }
    return line


def run_reference(args, rank: int, world: int):
    """The reference's CPU implementation of the path (oracle port) on the host cores, bounded sample per step."""
    if rank != 0:
        return None
    from lightop_b200 import synthetic
    from oracle import moe_block_int8 as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    name = args.workload or ("c1_dsv3_prefill" if world == 1 else "c3_dsv3_ep_rank")
    cfg = dict(synthetic.CONFIGS[name])
    E, k, M, H, I = cfg["E"], cfg["topk"], cfg["M"], cfg["H"], cfg["I"]
    n_sample = args.cpu_sample_experts
    w1, w2, w1_s, w2_s = synthetic.make_weights(n_sample, H, I, seed=0)
    x, logits = synthetic.make_activations(M, H, E, seed=1, zipf=cfg.get("zipf"))
    w, ids = O.route_topk_softmax(logits, k, renormalize=True)
    keep = ids < n_sample
    rows = int(keep.sum())
    ids_s = torch.where(keep, ids, torch.full_like(ids, n_sample))
    w_s = w * keep

    def step():
        O.route_topk_softmax(logits, k, renormalize=True)
        O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w_s, ids_s)

    for _ in range(min(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    value = (rows / k) / dt
    sample = (f"oracle over the {rows} routed rows of the first {n_sample} of {E} experts of one batch per step "
              f"({dt:.1f} s/step); tokens = rows / top_k")
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32 torch on int8 codes", "data": "synthetic",
        "config": {"workload": name, "E": E, "top_k": k, "M": M, "hidden": H, "intermediate": I},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


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
