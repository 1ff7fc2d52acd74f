"""Expert parallelism for the block-INT8 MoE layer: experts sharded over the ranks of one node.

One process per GPU.  Rank r owns experts [r*E/R, (r+1)*E/R).  A step on every rank:

  1. group-quantise the rank's own tokens once (int8 row + H/128 fp32 scales: 7392 B per row at
     H=7168 instead of 14336 B of bf16);
  2. pack one row per routed (token, slot) by destination rank (ep_scatter with the rank as the
     "expert", stable order) and exchange the per-pair row counts;
  3. dispatch all-to-all-v: int8 rows, scales, and per row (local expert id, routed weight);
  4. expert side: lo_expert_rows_block_int8 on the received rows (grouped GEMMs, fused epilogues,
     weight applied as in the single-GPU layer);
  5. combine all-to-all-v: bf16 rows back to their source rank, in the order they were sent;
  6. top-k sum per token in slot order with fp32 accumulation (ep_gather with unit weights), so the
     result has the same bits as the single-GPU layer.
Optionally (micro_batches > 1) a step is cut into micro-batches: the dispatch of one and the combine of
another travel over NVLink while the experts compute (asynchronous collectives on the communication stream).

The reference contains only the local halves of 2 and 6 (csrc/kernels/deepgemm_moe_permute.cu;
sequence in test/test_ep_gather_scatter_moe.py:205-296) and simulates EP on one device with an
expert_map (test/moe_w8a8/test_kernel_moe_ep8.py:98-153); the exchange is left to the serving stack.
Here it is torch.distributed all_to_all_single (NCCL over NVLink on GPUs, gloo on CPU for the tests of
the bookkeeping).  The pack / expert / combine steps are hooks so that the CPU tests can run the same
driver with torch stand-ins; the defaults are the CUDA kernels.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch
import torch.distributed as dist


# --------------------------------------------------------------------------- CUDA hooks

def _cuda_pack(xq, xs, topk_ids, rank_of_expert, world, rows):
    from .moe import ep_scatter
    counts = None
    T, k = topk_ids.shape
    out_q = torch.empty(rows, xq.shape[1], dtype=torch.int8, device=xq.device)
    out_s = torch.empty(rows, xs.shape[1], dtype=torch.float32, device=xq.device)
    m_idx = torch.empty(rows, dtype=torch.int32, device=xq.device)
    inv = torch.empty(T, k, dtype=torch.int32, device=xq.device)
    ep_scatter(xq, xs, topk_ids, rank_of_expert, counts, out_q, out_s, m_idx, inv, world, 1)
    return out_q, out_s, inv


def _cuda_quant(x):
    from .quant import per_token_group_quant_int8
    return per_token_group_quant_int8(x, 128)


def _cuda_combine(rows_back, topk_ids, inv):
    from .moe import ep_gather
    T, k = topk_ids.shape
    out = torch.empty(T, rows_back.shape[1], dtype=rows_back.dtype, device=rows_back.device)
    ones = torch.ones(T, k, dtype=torch.float32, device=rows_back.device)
    ep_gather(rows_back, topk_ids, ones, inv, None, out)
    return out


class _CudaExperts:
    """Expert-side compute on the local shard through the C ABI."""

    def __init__(self, w1, w2, w1_s, w2_s):
        self.w1, self.w2 = w1.contiguous(), w2.contiguous()
        self.w1_s, self.w2_s = w1_s.float().contiguous(), w2_s.float().contiguous()
        self._ws = None

    def __call__(self, rq, rs, r_expert, r_weight):
        from . import _lib, device_status_word
        lib = _lib.load()
        T, H = rq.shape
        E, N, _ = self.w1.shape
        I = N // 2
        out = torch.empty(T, H, dtype=torch.bfloat16, device=rq.device)
        if T == 0:
            return out
        nbytes = lib.lo_fused_moe_workspace_bytes(T, E, E, 1, H, I)
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = torch.empty(nbytes, dtype=torch.uint8, device=rq.device)
        with torch.cuda.device(rq.device):
            st = lib.lo_expert_rows_block_int8(
                _lib.ptr(rq), _lib.ptr(rs), _lib.ptr(r_expert), _lib.ptr(r_weight), _lib.ptr(self.w1),
                _lib.ptr(self.w2), _lib.ptr(self.w1_s), _lib.ptr(self.w2_s), T, E, H, I, _lib.ptr(out),
                _lib.ptr(self._ws), self._ws.numel(), _lib.ptr(device_status_word(rq.device)),
                _lib.current_stream(rq.device))
        _lib.check(st, "lo_expert_rows_block_int8")
        return out


# --------------------------------------------------------------------------- driver

class ExpertParallelMoE:
    """Block-INT8 MoE layer with the experts of this rank; ``forward`` is collective over ``group``."""

    def __init__(self, w1_local: torch.Tensor, w2_local: torch.Tensor, w1_scale: torch.Tensor,
                 w2_scale: torch.Tensor, num_experts_global: int, group=None,
                 quant_fn: Optional[Callable] = None, pack_fn: Optional[Callable] = None,
                 expert_fn: Optional[Callable] = None, combine_fn: Optional[Callable] = None,
                 micro_batches: int = 1, micro_batch_min_tokens: int = 512):
        self.group = group
        # With micro_batches > 1 a step of at least micro_batches * micro_batch_min_tokens tokens is cut into
        # micro-batches whose exchanges overlap the expert compute of their neighbours (see forward).  Off by
        # default: on 2 and on 8 B200s the pipelined step measured 2-8 % slower than the plain one -- the
        # exchange is a small part of the step, every micro-batch streams the rank's expert weights again,
        # and the collectives' kernels compete for SMs with the persistent GEMM.
        self.micro_batches = max(1, int(micro_batches))
        self.micro_batch_min_tokens = int(micro_batch_min_tokens)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E_local = w1_local.shape[0]
        if self.E_local * self.world != num_experts_global:
            raise ValueError(f"{num_experts_global} experts do not split into {self.world} shards of {self.E_local}")
        self.E = num_experts_global
        dev = w1_local.device
        self.rank_of_expert = (torch.arange(self.E, device=dev) // self.E_local).to(torch.int32)
        self.quant_fn = quant_fn or _cuda_quant
        self.pack_fn = pack_fn or _cuda_pack
        self.expert_fn = expert_fn or _CudaExperts(w1_local, w2_local, w1_scale, w2_scale)
        self.combine_fn = combine_fn or _cuda_combine
        self.last_counts = None   # (send_counts, recv_counts) of the last step, for inspection

    def _all_to_all(self, send: torch.Tensor, send_counts: List[int], recv_counts: List[int]) -> torch.Tensor:
        recv = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        dist.all_to_all_single(recv, send, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=self.group)
        return recv

    def _all_to_all_async(self, send: torch.Tensor, send_counts: List[int], recv_counts: List[int]):
        recv = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        work = dist.all_to_all_single(recv, send, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                                      group=self.group, async_op=True)
        return recv, work

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        """Collective over the group.  With micro_batches > 1 (and enough tokens) the tokens are cut into
        micro-batches; the dispatch of micro-batch i + 1 and the combine of micro-batch i - 1 travel while the
        experts work on micro-batch i.  Tokens are independent of one another, so the result has the same bits
        either way."""
        T, k = topk_ids.shape
        dev = x.device
        nmb = self.micro_batches if T >= self.micro_batches * self.micro_batch_min_tokens else 1
        bounds = [T * i // nmb for i in range(nmb + 1)]
        ids_all = topk_ids.to(torch.int64)
        # 1. rows per destination rank and micro-batch, exchanged in ONE small collective (and one host read) so
        #    that every rank knows what it receives
        dest_all = self.rank_of_expert.to(torch.int64)[ids_all]                          # [T, k]
        send_counts_t = torch.stack([torch.bincount(dest_all[bounds[i]:bounds[i + 1]].reshape(-1), minlength=self.world)
                                     for i in range(nmb)], dim=1).contiguous()             # [world, nmb]
        recv_counts_t = torch.empty_like(send_counts_t)
        dist.all_to_all_single(recv_counts_t, send_counts_t, group=self.group)
        send_all = send_counts_t.tolist()
        recv_all = recv_counts_t.tolist()
        # 2. per micro-batch: quantise once, pack one row per routed (token, slot) by destination rank
        mbs = []
        for i in range(nmb):
            lo_t, hi_t = bounds[i], bounds[i + 1]
            ids = ids_all[lo_t:hi_t]
            tk_ids = topk_ids[lo_t:hi_t]
            send_counts = [int(send_all[r][i]) for r in range(self.world)]
            recv_counts = [int(recv_all[r][i]) for r in range(self.world)]
            rows = (hi_t - lo_t) * k
            if sum(send_counts) != rows:
                raise RuntimeError("dispatch bookkeeping lost rows")
            xq, xs = self.quant_fn(x[lo_t:hi_t])
            pq, ps, inv = self.pack_fn(xq, xs, tk_ids, self.rank_of_expert, self.world, rows)
            # per packed row: local expert id on the destination rank and the routed weight
            flat_inv = inv.reshape(-1).to(torch.int64)
            meta_e = torch.empty(rows, dtype=torch.int32, device=dev)
            meta_w = torch.empty(rows, dtype=torch.float32, device=dev)
            meta_e[flat_inv] = (ids % self.E_local).reshape(-1).to(torch.int32)
            meta_w[flat_inv] = topk_weights[lo_t:hi_t].reshape(-1).to(torch.float32)
            mbs.append(dict(send=send_counts, recv=recv_counts, payload=(pq, ps, meta_e, meta_w), ids=tk_ids, inv=inv))
        self.last_counts = ([sum(m["send"][r] for m in mbs) for r in range(self.world)],
                            [sum(m["recv"][r] for m in mbs) for r in range(self.world)])

        def dispatch(m):
            m["in_flight"] = [self._all_to_all_async(t, m["send"], m["recv"]) for t in m["payload"]]

        # 3.-5. software pipeline: dispatch(i + 1) and combine(i - 1) are in flight during expert(i)
        dispatch(mbs[0])
        for i, m in enumerate(mbs):
            received = []
            for recv, work in m["in_flight"]:
                work.wait()
                received.append(recv)
            if i + 1 < nmb:
                dispatch(mbs[i + 1])
            out_rows = self.expert_fn(*received)
            m["out_rows"] = out_rows                     # kept alive until the combine has completed
            m["back"] = self._all_to_all_async(out_rows, m["recv"], m["send"])
        # 6. top-k sum in slot order
        outs = []
        for m in mbs:
            back, work = m["back"]
            work.wait()
            outs.append(self.combine_fn(back, m["ids"], m["inv"]))
        return outs[0] if nmb == 1 else torch.cat(outs, dim=0)


# --------------------------------------------------------------------------- benchmark leg (N > 1)

def bench_step_setup(args, rank: int, world: int, dev: torch.device):
    """The N>1 leg of bench.py: DeepSeek-V3 shape, experts split over the ranks, M tokens per rank."""
    import json  # noqa: F401
    import lightop_b200
    from . import synthetic
    import bench as B   # bench.py is the caller; reuse its timing helpers

    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    name = args.workload or "c3_dsv3_ep_rank"
    cfg = dict(synthetic.CONFIGS[name])
    if args.tokens:
        cfg["M"] = args.tokens
    if args.experts:
        cfg["E"] = args.experts
    E, k, M, H, I = cfg["E"], cfg["topk"], cfg["M"], cfg["H"], cfg["I"]
    if E % world:
        raise ValueError(f"{E} experts do not split over {world} ranks")
    E_local = E // world
    w1, w2, w1_s, w2_s = synthetic.make_weights(E_local, H, I, seed=100 + rank, device=dev)
    x, logits = synthetic.make_activations(M, H, E, seed=1 + rank, device=dev, zipf=cfg.get("zipf"))
    import os
    nmb_env = os.environ.get("LIGHTOP_EP_MICRO_BATCHES")
    layer = ExpertParallelMoE(w1, w2, w1_s, w2_s, E, **({"micro_batches": int(nmb_env)} if nmb_env else {}))
    tw = torch.empty(M, k, dtype=torch.float32, device=dev)
    ti = torch.empty(M, k, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev)
    holder = {}

    def step():
        lightop_b200.moe.topk_softmax(tw, ti, None, logits, True)
        holder["y"] = layer.forward(x, tw, ti)

    x_h, l_h = x.cpu().pin_memory(), logits.cpu().pin_memory()
    y_h = torch.empty(M, H, dtype=torch.bfloat16).pin_memory()
    x_d, l_d = torch.empty_like(x), torch.empty_like(logits)

    def step_e2e():
        x_d.copy_(x_h, non_blocking=True)
        l_d.copy_(l_h, non_blocking=True)
        lightop_b200.moe.topk_softmax(tw, ti, None, l_d, True)
        y_h.copy_(layer.forward(x_d, tw, ti), non_blocking=True)

    def timed(fn, steps):
        dist.barrier()
        ms = B.cuda_time_ms(fn, steps, stream)
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        return float(t.item())

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    lightop_b200.check_device_status(dev)
    sampler = B.ClockSampler(dev.index)
    sampler.start()
    ms_per_step = timed(step, args.steps) / args.steps
    clocks = sampler.stop()
    for _ in range(2):
        step_e2e()
    e2e_ms = timed(step_e2e, args.steps) / args.steps
    lightop_b200.check_device_status(dev)

    send_counts, recv_counts = layer.last_counts
    rows_recv = sum(recv_counts)
    remote_rows = sum(send_counts) - send_counts[rank]
    total_tokens = M * world
    flops = synthetic.alg_flops(M, k, H, I) * world
    hbm_peak, peak_kind = B.measured_peaks()
    line = {
        "metric": B.METRIC, "value": total_tokens / (ms_per_step * 1e-3), "unit": B.UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x int8 -> int32, fp32 block scaling, bf16 in/out", "data": "synthetic",
        "config": {"workload": name, "E": E, "top_k": k, "M_per_rank": M, "hidden": H, "intermediate": I,
                   "parallelism": f"ep{world}", "experts_per_rank": E_local,
                   "micro_batches": layer.micro_batches if M >= layer.micro_batches * layer.micro_batch_min_tokens else 1,
                   "rows_received_rank0": rows_recv, "rows_sent_to_peers_rank0": remote_rows,
                   "dispatch_bytes_per_row": H + 4 * (H // 128) + 8, "combine_bytes_per_row": 2 * H,
                   "l2": "per-rank weights (>=1.4 GB) exceed L2; no flush needed"},
        "tflops": flops / (ms_per_step * 1e-3) / 1e12,
        "e2e": {"value": total_tokens / (e2e_ms * 1e-3), "unit": B.UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": (x_h.numel() * 2 + l_h.numel() * 4) * world,
                "d2h_bytes_per_step": y_h.numel() * 2 * world},
        # own kernels per step: the router, then per micro-batch quantise, pack (2), align, permute, two GEMMs, gather ...
        # (+ the wide chunk table of the down GEMM when a rank receives 64 rows per local expert or more)
        "gpu_launches": (1 + (10 + (1 if rows_recv // max(E_local, 1) >= 64 else 0))
                         * (layer.micro_batches if M >= layer.micro_batches * layer.micro_batch_min_tokens else 1))
        * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "grouped_gemm_kernel<gate_up>", "achieved": None, "peak": hbm_peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": None, "traffic": None,
                     "note": "per-kernel roofline is reported by the N=1 run; the N>1 step adds NCCL all-to-all-v"},
        "cpu_baseline": None,
    }
    dist.barrier()
    return line
