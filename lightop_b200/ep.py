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
Two transports carry steps 4 and 6:

  * "peer" (the default on GPUs): every rank owns two landing zones in device memory that the other ranks have
    mapped (lo_peer_alloc / lo_peer_export / lo_peer_open).  The dispatch kernel stores each record straight into
    the destination rank's receive buffer (lo_ep_dispatch_put) and the down GEMM's epilogue stores each result row
    straight into the source rank's return buffer (lo_expert_rows_block_int8_packed_put), both with plain stores
    over NVLink, so the transfers ride inside the kernels that produce the data; a small all-reduce after each of
    the two kernels tells every rank that its zone is complete.  Step 3 becomes an all-gather of the counts, from
    which every rank derives where its runs of records begin in the other ranks' zones.
  * "collective": torch.distributed all_to_all_single (NCCL on GPUs, gloo on CPU for the tests of the
    bookkeeping).

Both give the same bits.  The quantise / pack / expert / combine steps are hooks so that the CPU tests can run the
collective driver with torch stand-ins; the defaults are the CUDA kernels.
"""
from __future__ import annotations

import os
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


def peer_routes(mat, me: int, record_bytes: int, row_bytes: int, peer_recv, peer_ret):
    """Where rank ``me`` writes, from the R x R matrix of record counts (``mat[s][d]`` = records rank s sends to rank d).

    Returns ``(first_out, seg_dst, first_in, seg_ret)``:
    ``first_out[d]``  packed position of this rank's first record for rank d (its records are grouped by destination);
    ``seg_dst[d]``    address of that record in rank d's receive zone: the runs of the lower ranks come first;
    ``first_in[s]``   index of the first record received from rank s (R + 1 entries, the last one the total);
    ``seg_ret[s]``    address, in rank s's return zone, of the result row of that record: rank s keeps its rows in the
                      order it packed them, so the rows for the ranks below ``me`` come first.
    An address of 0 stands for an empty run.  ``peer_recv`` / ``peer_ret`` are the zones' base addresses as this rank
    sees them."""
    R = len(mat)
    first_out, seg_dst, first_in, seg_ret = [], [], [], []
    run = 0
    for d in range(R):
        first_out.append(run)
        run += mat[me][d]
        before = sum(mat[s][d] for s in range(me))
        seg_dst.append(peer_recv[d] + before * record_bytes if mat[me][d] else 0)
    run = 0
    for s in range(R):
        first_in.append(run)
        run += mat[s][me]
        before = sum(mat[s][d] for d in range(me))
        seg_ret.append(peer_ret[s] + before * row_bytes if mat[s][me] else 0)
    first_in.append(run)
    return first_out, seg_dst, first_in, seg_ret


# --------------------------------------------------------------------------- peer landing zones

class PeerUnavailable(RuntimeError):
    """The landing zones of the peer transport could not be set up on some rank (raised on every rank)."""


class _PeerZones:
    """This rank's receive and return buffers and the mappings of every other rank's.  All methods that change the
    buffers are collective over the group and take arguments that are equal on every rank."""

    def __init__(self, group, dev, rank, world):
        from . import _lib
        self.lib = _lib.load()
        self.group, self.dev, self.rank, self.world = group, dev, rank, world
        self.recv_bytes = 0
        self.ret_bytes = 0
        self.own = [0, 0]                                   # receive zone, return zone
        self.peer_recv = [0] * world
        self.peer_ret = [0] * world
        self._opened: List[int] = []
        self._held = False          # set while a (possibly partial) set-up is in place, so that release() is collective

    def ensure(self, recv_bytes: int, ret_bytes: int) -> None:
        """Grow the zones to at least these sizes (the same numbers on every rank).  Collective; raises
        PeerUnavailable on EVERY rank when any rank could not allocate, export or map a zone (the ranks agree on the
        outcome before anybody leaves, so no rank is left waiting in a collective)."""
        if recv_bytes <= self.recv_bytes and ret_bytes <= self.ret_bytes:
            return
        import ctypes
        recv_bytes = max(self.recv_bytes, (recv_bytes * 5 // 4 + 4095) // 4096 * 4096)
        ret_bytes = max(self.ret_bytes, (ret_bytes * 5 // 4 + 4095) // 4096 * 4096)
        # nobody may still be writing into a zone that is about to go away
        torch.cuda.synchronize(self.dev)
        dist.barrier(group=self.group)
        self.release()
        hb = int(self.lib.lo_peer_handle_bytes())
        mine = torch.zeros(2, hb, dtype=torch.uint8)
        ok, why = True, ""
        self._held = True
        with torch.cuda.device(self.dev):
            for i, nbytes in enumerate((recv_bytes, ret_bytes)):
                p = ctypes.c_void_p()
                if ok and self.lib.lo_peer_alloc(nbytes, ctypes.byref(p)) == 0:
                    self.own[i] = int(p.value)
                    buf = (ctypes.c_uint8 * hb)()
                    if self.lib.lo_peer_export(self.own[i], buf) == 0:
                        mine[i] = torch.frombuffer(bytearray(buf), dtype=torch.uint8)
                        continue
                if ok:
                    ok, why = False, (self.lib.lo_last_error() or b"").decode()
            everyone = torch.empty(self.world, 2, hb, dtype=torch.uint8, device=self.dev)
            dist.all_gather_into_tensor(everyone, mine.to(self.dev), group=self.group)
            everyone = everyone.cpu()
            for r in range(self.world):
                if r == self.rank:
                    self.peer_recv[r], self.peer_ret[r] = self.own
                    continue
                got = [0, 0]
                for i in range(2):
                    raw = bytes(everyone[r, i].tolist())
                    p = ctypes.c_void_p()
                    if ok and any(raw) and self.lib.lo_peer_open(raw, ctypes.byref(p)) == 0:
                        got[i] = int(p.value)
                        self._opened.append(int(p.value))
                    elif ok:
                        ok, why = False, (self.lib.lo_last_error() or b"").decode() or f"rank {r} exported no zone"
                self.peer_recv[r], self.peer_ret[r] = got
            verdict = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.dev)
            dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=self.group)
        if int(verdict.item()) != 1:
            self.release()
            raise PeerUnavailable(why or "another rank could not set up its landing zones")
        self.recv_bytes, self.ret_bytes = recv_bytes, ret_bytes
        dist.barrier(group=self.group)

    def release(self) -> None:
        """Unmap the peers' zones, then (after everyone has) free this rank's.  Collective."""
        if not any(self.own) and not self._opened and not self._held:
            return
        self._held = False
        with torch.cuda.device(self.dev):
            for p in self._opened:
                self.lib.lo_peer_close(p)
            self._opened = []
            dist.barrier(group=self.group)
            for i in range(2):
                if self.own[i]:
                    self.lib.lo_peer_free(self.own[i])
                    self.own[i] = 0
        self.peer_recv = [0] * self.world
        self.peer_ret = [0] * self.world
        self.recv_bytes = self.ret_bytes = 0


# --------------------------------------------------------------------------- driver

STAGES = ("quantise", "pack", "counts", "dispatch", "experts", "combine", "gather")


class ExpertParallelMoE:
    """Block-INT8 MoE layer with the experts of this rank; ``forward`` is collective over ``group``.

    transport: "peer", "collective" or None = peer on CUDA with the built-in hooks (LIGHTOP_B200_EP_TRANSPORT overrides
    the default), collective otherwise."""

    def __init__(self, w1_local: torch.Tensor, w2_local: torch.Tensor, w1_scale: torch.Tensor,
                 w2_scale: torch.Tensor, num_experts_global: int, group=None,
                 quant_fn: Optional[Callable] = None, pack_fn: Optional[Callable] = None,
                 expert_fn: Optional[Callable] = None, combine_fn: Optional[Callable] = None,
                 transport: Optional[str] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E_local = w1_local.shape[0]
        if self.E_local * self.world != num_experts_global:
            raise ValueError(f"{num_experts_global} experts do not split into {self.world} shards of {self.E_local}")
        self.E = num_experts_global
        dev = w1_local.device
        self.dev = dev
        self.rank_of_expert = (torch.arange(self.E, device=dev) // self.E_local).to(torch.int32)
        builtin = pack_fn is None and expert_fn is None and combine_fn is None and quant_fn is None
        if transport is None:
            transport = os.environ.get("LIGHTOP_B200_EP_TRANSPORT") or ("peer" if builtin and dev.type == "cuda" else "collective")
        if transport not in ("peer", "collective"):
            raise ValueError(f"unknown transport {transport!r}")
        if transport == "peer" and not (builtin and dev.type == "cuda"):
            raise ValueError("the peer transport runs the built-in CUDA kernels only")
        self.transport = transport
        self.transport_note = ""           # why the peer transport was given up, if it was
        self.quant_fn = quant_fn or _cuda_quant
        self.pack_fn = pack_fn or _cuda_pack
        self.expert_fn = expert_fn or _CudaExperts(w1_local, w2_local, w1_scale, w2_scale)
        self.combine_fn = combine_fn or _cuda_combine
        self.last_counts = None            # (send_counts, recv_counts) of the last step, for inspection
        self.profile = False               # record a CUDA event after every stage of forward()
        self._events: List[torch.cuda.Event] = []
        self._zones = _PeerZones(group, dev, self.rank, self.world) if transport == "peer" else None
        self._flag = torch.zeros(1, dtype=torch.int32, device=dev) if transport == "peer" else None
        self._mat_host = None

    def close(self) -> None:
        """Give the landing zones back (collective; only the peer transport holds any)."""
        if self._zones is not None:
            torch.cuda.synchronize(self.dev)
            self._zones.release()

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
        if self.transport == "peer":
            return self._forward_peer(x, topk_weights, topk_ids)
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

    def _everyone_done(self):
        """Every rank's kernels queued so far have completed (their stores to this rank's zones have landed) before
        anything queued after this call runs: a one-word all-reduce in stream order."""
        dist.all_reduce(self._flag, group=self.group)

    def _forward_peer(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        from . import _lib, device_status_word
        lib = _lib.load()
        T, k = topk_ids.shape
        H = x.shape[1]
        dev, R, me = self.dev, self.world, self.rank
        ex = self.expert_fn
        stride = int(lib.lo_ep_dispatch_row_bytes(H))
        self._events = []
        self._mark()
        if T:
            xq, xs = self.quant_fn(x)
        else:               # a rank without tokens still takes part in the step
            xq = torch.empty(0, H, dtype=torch.int8, device=dev)
            xs = torch.empty(0, H // 128, dtype=torch.float32, device=dev)
        self._mark()
        ids = topk_ids.contiguous()
        w = topk_weights.to(torch.float32).contiguous()
        dest = torch.empty(T * k, dtype=torch.int32, device=dev)
        inv = torch.empty(T, k, dtype=torch.int32, device=dev)
        counts = torch.empty(R, dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.lo_ep_dispatch_plan(_lib.ptr(ids), _lib.dtype_code(ids.dtype), _lib.ptr(self.rank_of_expert), T, k, R,
                                               _lib.ptr(dest), _lib.ptr(inv), _lib.ptr(counts), _lib.current_stream(dev)),
                       "lo_ep_dispatch_plan")
        self._mark()
        # the whole R x R matrix of record counts on every rank (the step's one host read): it fixes where every
        # run of records begins in every zone
        mat_t = torch.empty(R, R, dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(mat_t, counts, group=self.group)
        # read through page-locked memory that a kernel writes, not through a copy engine: the engine may be busy
        # with a caller's large device-to-host transfer, behind which a small copy would wait
        if self._mat_host is None:
            self._mat_host = torch.empty(R * R, dtype=torch.int32).pin_memory()
        with torch.cuda.device(dev):
            _lib.check(lib.lo_words_to_host(_lib.ptr(mat_t), self._mat_host.data_ptr(), R * R, _lib.current_stream(dev)),
                       "lo_words_to_host")
        seen = torch.cuda.Event()
        seen.record()
        seen.synchronize()
        mat = self._mat_host.view(R, R).tolist()               # mat[s][d]: records rank s sends to rank d
        send_counts = [int(v) for v in mat[me]]
        recv_counts = [int(mat[s][me]) for s in range(R)]
        if sum(send_counts) != T * k:
            raise RuntimeError("dispatch bookkeeping lost rows")
        self.last_counts = (send_counts, recv_counts)
        rows_recv = sum(recv_counts)
        need_recv = max(sum(mat[s][d] for s in range(R)) for d in range(R))
        need_ret = max(sum(mat[s]) for s in range(R))
        try:
            self._zones.ensure(max(need_recv, 1) * stride, max(need_ret, 1) * 2 * H)
        except PeerUnavailable as e:
            # every rank got the same exception: all of them switch to the all-to-all transport, for good
            if self.rank == 0:
                import sys
                print(f"lightop_b200.ep: peer transport unavailable ({e}); using all-to-all collectives", file=sys.stderr)
            self.transport, self._zones, self.transport_note = "collective", None, str(e)
            return self.forward(x, topk_weights, topk_ids)
        z = self._zones
        first_out, seg_dst, first_in, seg_ret = peer_routes(mat, me, stride, 2 * H, z.peer_recv, z.peer_ret)
        i32 = torch.tensor(first_out + first_in, dtype=torch.int32, device=dev)
        i64 = torch.tensor(seg_dst + seg_ret, dtype=torch.int64, device=dev)
        self._mark()
        with torch.cuda.device(dev):
            _lib.check(lib.lo_ep_dispatch_put(_lib.ptr(xq), _lib.ptr(xs), _lib.ptr(ids), _lib.dtype_code(ids.dtype), _lib.ptr(w),
                                              _lib.ptr(self.rank_of_expert), _lib.ptr(inv), T, k, H, self.E_local, R,
                                              i32.data_ptr(), i64.data_ptr(), _lib.current_stream(dev)), "lo_ep_dispatch_put")
        self._everyone_done()
        self._mark()
        if rows_recv:
            E, N, _ = ex.w1.shape
            I = N // 2
            nbytes = lib.lo_expert_rows_packed_workspace_bytes(rows_recv, E, H, I)
            if ex._ws is None or ex._ws.numel() < nbytes:
                ex._ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            with torch.cuda.device(dev):
                _lib.check(lib.lo_expert_rows_block_int8_packed_put(
                    z.own[0], rows_recv, _lib.ptr(ex.w1), _lib.ptr(ex.w2), _lib.ptr(ex.w1_s), _lib.ptr(ex.w2_s), E, H, I,
                    i32.data_ptr() + 4 * R, i64.data_ptr() + 8 * R, R, _lib.ptr(ex._ws), ex._ws.numel(),
                    _lib.ptr(device_status_word(dev)), _lib.current_stream(dev)), "lo_expert_rows_block_int8_packed_put")
        self._mark()
        self._everyone_done()
        self._mark()
        y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        if T:
            ones = torch.ones(T, k, dtype=torch.float32, device=dev)
            with torch.cuda.device(dev):
                _lib.check(lib.lo_ep_gather(z.own[1], _lib.ptr(ids), _lib.dtype_code(ids.dtype), _lib.ptr(ones), _lib.ptr(inv), 0,
                                            _lib.ptr(y), T, k, H, _lib.current_stream(dev)), "lo_ep_gather")
        self._mark()
        # keep the small tables alive until the kernels that read them have run
        self._keep = (i32, i64, ones if T else None, dest)
        return y
