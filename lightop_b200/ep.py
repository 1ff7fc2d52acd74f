"""Expert parallelism for the block-INT8 MoE layer: experts sharded over the ranks of one node.

One process per GPU.  Rank r owns experts [r*E/R, (r+1)*E/R).  A step on every rank:

  1. group-quantise the rank's own tokens once (int8 row + H/128 fp32 scales: 7392 B per row at
     H=7168 instead of 14336 B of bf16);
  2. pack ONE record per routed (token, slot), grouped by destination rank in stable order: the int8 row, its
     scales, the slot's expert id on the destination rank and its routed weight (lo_ep_dispatch_pack; 7408 B at
     H=7168); the records per destination are counted on the device;
  3. exchange the per-pair record counts (one small all-to-all, one host read per step: all-to-all-v wants
     its split sizes on the host);
  4. dispatch: one all-to-all-v of the records;
  5. expert side: lo_expert_rows_block_int8_packed on the received records (grouped GEMMs, fused epilogues,
     weight applied as in the single-GPU layer);
  6. combine: one all-to-all-v of bf16 rows back to their source rank, in the order they were sent;
  7. top-k sum per token in slot order with fp32 accumulation (ep_gather with unit weights), so the
     result has the same bits as the single-GPU layer.

The reference contains only the local halves of 2 and 7 (csrc/kernels/deepgemm_moe_permute.cu;
sequence in test/test_ep_gather_scatter_moe.py:205-296) and simulates EP on one device with an
expert_map (test/moe_w8a8/test_kernel_moe_ep8.py:98-153); the exchange is left to the serving stack.
Here it is torch.distributed all_to_all_single (NCCL over NVLink on GPUs, gloo on CPU for the tests of
the bookkeeping).  The quantise / pack / expert / combine steps are hooks so that the CPU tests can run the
same driver with torch stand-ins; the defaults are the CUDA kernels.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist


def record_layout(H: int):
    """(record bytes, offset of the scales, offset of (expert id, weight)) of a dispatch record."""
    groups = H // 128
    stride = (H + 4 * groups + 8 + 15) // 16 * 16
    return stride, H, H + 4 * groups


# --------------------------------------------------------------------------- CUDA hooks

def _cuda_quant(x):
    from .quant import per_token_group_quant_int8
    return per_token_group_quant_int8(x, 128)


def _cuda_pack(xq, xs, topk_ids, topk_weights, rank_of_expert, experts_per_rank, world):
    from . import _lib
    lib = _lib.load()
    T, k = topk_ids.shape
    H = xq.shape[1]
    dev = xq.device
    stride = int(lib.lo_ep_dispatch_row_bytes(H))
    packed = torch.empty(T * k, stride, dtype=torch.uint8, device=dev)
    dest = torch.empty(T * k, dtype=torch.int32, device=dev)
    inv = torch.empty(T, k, dtype=torch.int32, device=dev)
    counts = torch.empty(world, dtype=torch.int32, device=dev)
    ids = topk_ids.contiguous()
    w = topk_weights.to(torch.float32).contiguous()
    with torch.cuda.device(dev):
        st = lib.lo_ep_dispatch_pack(_lib.ptr(xq), _lib.ptr(xs), _lib.ptr(ids), _lib.dtype_code(ids.dtype), _lib.ptr(w),
                                     _lib.ptr(rank_of_expert), T, k, H, experts_per_rank, world, _lib.ptr(packed),
                                     _lib.ptr(dest), _lib.ptr(inv), _lib.ptr(counts), _lib.current_stream(dev))
    _lib.check(st, "lo_ep_dispatch_pack")
    return packed, inv, counts


def _cuda_combine(rows_back, topk_ids, inv):
    from .moe import ep_gather
    T, k = topk_ids.shape
    out = torch.empty(T, rows_back.shape[1], dtype=rows_back.dtype, device=rows_back.device)
    ones = torch.ones(T, k, dtype=torch.float32, device=rows_back.device)
    ep_gather(rows_back, topk_ids, ones, inv, None, out)
    return out


class _CudaExperts:
    """Expert-side compute on the local shard through the C ABI, on dispatch records."""

    def __init__(self, w1, w2, w1_s, w2_s):
        self.w1, self.w2 = w1.contiguous(), w2.contiguous()
        self.w1_s, self.w2_s = w1_s.float().contiguous(), w2_s.float().contiguous()
        self._ws = None

    def __call__(self, packed):
        from . import _lib, device_status_word
        lib = _lib.load()
        T = packed.shape[0]
        E, N, H = self.w1.shape
        I = N // 2
        out = torch.empty(T, H, dtype=torch.bfloat16, device=packed.device)
        if T == 0:
            return out
        nbytes = lib.lo_expert_rows_packed_workspace_bytes(T, E, H, I)
        if self._ws is None or self._ws.numel() < nbytes:
            self._ws = torch.empty(nbytes, dtype=torch.uint8, device=packed.device)
        with torch.cuda.device(packed.device):
            st = lib.lo_expert_rows_block_int8_packed(
                _lib.ptr(packed), T, _lib.ptr(self.w1), _lib.ptr(self.w2), _lib.ptr(self.w1_s), _lib.ptr(self.w2_s),
                E, H, I, _lib.ptr(out), _lib.ptr(self._ws), self._ws.numel(),
                _lib.ptr(device_status_word(packed.device)), _lib.current_stream(packed.device))
        _lib.check(st, "lo_expert_rows_block_int8_packed")
        return out


# --------------------------------------------------------------------------- driver

STAGES = ("quantise", "pack", "counts", "dispatch", "experts", "combine", "gather")


class ExpertParallelMoE:
    """Block-INT8 MoE layer with the experts of this rank; ``forward`` is collective over ``group``."""

    def __init__(self, w1_local: torch.Tensor, w2_local: torch.Tensor, w1_scale: torch.Tensor,
                 w2_scale: torch.Tensor, num_experts_global: int, group=None,
                 quant_fn: Optional[Callable] = None, pack_fn: Optional[Callable] = None,
                 expert_fn: Optional[Callable] = None, combine_fn: Optional[Callable] = None):
        self.group = group
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
        self.last_counts = None            # (send_counts, recv_counts) of the last step, for inspection
        self.profile = False               # record a CUDA event after every stage of forward()
        self._events: List[torch.cuda.Event] = []

    def _all_to_all(self, send: torch.Tensor, send_counts: List[int], recv_counts: List[int]) -> torch.Tensor:
        recv = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        dist.all_to_all_single(recv, send, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=self.group)
        return recv

    def _mark(self):
        if self.profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._events.append(ev)

    def stage_ms(self) -> Dict[str, float]:
        """Device milliseconds per stage of the last profiled forward() (the collectives include waiting for peers)."""
        torch.cuda.synchronize()
        ev = self._events
        return {name: ev[i].elapsed_time(ev[i + 1]) for i, name in enumerate(STAGES)} if len(ev) == len(STAGES) + 1 else {}

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        """Collective over the group: every rank calls it with its own tokens."""
        T, k = topk_ids.shape
        self._events = []
        self._mark()
        xq, xs = self.quant_fn(x)
        self._mark()
        packed, inv, counts = self.pack_fn(xq, xs, topk_ids, topk_weights, self.rank_of_expert, self.E_local, self.world)
        self._mark()
        # records per (source, destination) pair: every rank learns what it receives; all-to-all-v wants the split
        # sizes on the host, which is the step's one host read (the pack kernels are already queued behind it)
        recv_counts_t = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts_t, counts, group=self.group)
        both = torch.stack([counts, recv_counts_t]).tolist()
        send_counts, recv_counts = [int(v) for v in both[0]], [int(v) for v in both[1]]
        if sum(send_counts) != T * k:
            raise RuntimeError("dispatch bookkeeping lost rows")
        self.last_counts = (send_counts, recv_counts)
        self._mark()
        received = self._all_to_all(packed, send_counts, recv_counts)
        self._mark()
        out_rows = self.expert_fn(received)
        self._mark()
        back = self._all_to_all(out_rows, recv_counts, send_counts)
        self._mark()
        y = self.combine_fn(back, topk_ids, inv)
        self._mark()
        return y
