"""CPU test (gloo, world_size 2) of the expert-parallel driver's bookkeeping.

The driver (lightop_b200/ep.py) is run with torch stand-ins for its CUDA hooks and the oracle as the
expert-side compute; every rank's output must equal the single-process oracle on that rank's tokens
bit for bit.  A second case makes the ranks disagree on the expert count and expects the error on the
host, before any collective.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lightop_b200 import synthetic
from oracle import moe_block_int8 as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _pack_torch(xq, xs, topk_ids, topk_weights, rank_of_expert, experts_per_rank, world):
    """Torch model of lo_ep_dispatch_pack: one record per routed (token, slot), grouped by destination rank."""
    from lightop_b200.ep import record_layout
    T, k = topk_ids.shape
    H = xq.shape[1]
    stride, off_s, off_m = record_layout(H)
    dest = rank_of_expert.long()[topk_ids.long()].reshape(-1)
    order = torch.sort(dest, stable=True)[1]               # record -> flat (token, slot)
    inv = torch.empty(T * k, dtype=torch.int32)
    inv[order] = torch.arange(T * k, dtype=torch.int32)
    tok = order // k
    packed = torch.zeros(T * k, stride, dtype=torch.uint8)
    packed[:, :H] = xq[tok].view(torch.uint8)
    packed[:, off_s:off_m] = xs[tok].contiguous().view(torch.uint8).reshape(T * k, -1)
    e_local = (topk_ids.reshape(-1)[order].long() % experts_per_rank).to(torch.int32)
    packed[:, off_m:off_m + 4] = e_local.view(torch.uint8).reshape(-1, 4)
    packed[:, off_m + 4:off_m + 8] = topk_weights.reshape(-1)[order].float().contiguous().view(torch.uint8).reshape(-1, 4)
    counts = torch.bincount(dest, minlength=world).to(torch.int32)
    return packed, inv.view(T, k), counts


def _combine_torch(rows_back, topk_ids, inv):
    T, k = topk_ids.shape
    return rows_back[inv.long()].float().sum(dim=1).to(rows_back.dtype)


def _make_expert_fn(w1, w2, w1_s, w2_s):
    def fn(packed):
        from lightop_b200.ep import record_layout
        H = w2.shape[1]
        stride, off_s, off_m = record_layout(H)
        rq = packed[:, :H].contiguous().view(torch.int8)
        rs = packed[:, off_s:off_m].contiguous().view(torch.float32)
        r_expert = packed[:, off_m:off_m + 4].contiguous().view(torch.int32).reshape(-1)
        r_weight = packed[:, off_m + 4:off_m + 8].contiguous().view(torch.float32).reshape(-1)
        out = torch.zeros(rq.shape[0], H, dtype=torch.bfloat16)
        for e in range(w1.shape[0]):
            m = r_expert == e
            if m.any():
                h = O.block_int8_matmul(rq[m], w1[e], rs[m], w1_s[e], (128, 128), torch.bfloat16)
                d = h.shape[-1] // 2
                act = torch.nn.functional.silu(h[:, :d]) * h[:, d:]
                q2, s2 = O.group_quant_int8(act.contiguous(), 128)
                o = O.block_int8_matmul(q2, w2[e], s2, w2_s[e], (128, 128), torch.bfloat16)
                out[m] = o * r_weight[m].view(-1, 1).to(torch.bfloat16)
        return out
    return fn


def _worker(rank, world, port, q, mode):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from lightop_b200.ep import ExpertParallelMoE
        E, k, M, H, I = 8, 3, 21 + 5 * rank, 256, 256
        w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=0)
        x, logits = synthetic.make_activations(M, H, E, seed=10 + rank)
        w, ids = O.route_topk_softmax(logits, k)
        El = E // world
        sl = slice(rank * El, (rank + 1) * El)
        if mode == "mismatch":
            try:
                ExpertParallelMoE(w1[sl], w2[sl], w1_s[sl], w2_s[sl], E + 1,
                                  quant_fn=lambda t: O.group_quant_int8(t, 128), pack_fn=_pack_torch,
                                  expert_fn=lambda *a: None, combine_fn=_combine_torch)
                q.put((rank, "no error"))
            except ValueError as e:
                q.put((rank, "ValueError"))
            return
        layer = ExpertParallelMoE(w1[sl], w2[sl], w1_s[sl], w2_s[sl], E,
                                  quant_fn=lambda t: O.group_quant_int8(t.contiguous(), 128), pack_fn=_pack_torch,
                                  expert_fn=_make_expert_fn(w1[sl], w2[sl], w1_s[sl], w2_s[sl]),
                                  combine_fn=_combine_torch)
        y = layer.forward(x, w, ids)
        y_ref = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids)
        send, recv = layer.last_counts
        q.put((rank, bool(torch.equal(y, y_ref)), sum(send) == M * k, send, recv))
    finally:
        dist.destroy_process_group()


def _run(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, mode)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(res)


def test_ep_two_ranks_match_single_process_oracle():
    res = _run("forward")
    assert [r[1] for r in res] == [True, True], res
    assert all(r[2] for r in res)
    # what rank 0 sends to rank 1 is what rank 1 receives from rank 0
    assert res[0][3][1] == res[1][4][0] and res[1][3][0] == res[0][4][1]


def test_ep_rejects_inconsistent_sharding_on_the_host():
    res = _run("mismatch")
    assert [r[1] for r in res] == ["ValueError", "ValueError"]


def test_peer_routes_tile_the_zones_exactly():
    """Host bookkeeping of the peer transport: over all ranks, the runs written into a receive zone tile it without gap
    or overlap in source-rank order, and the return routes send every result row back to the packed position it came
    from."""
    from lightop_b200.ep import peer_routes
    import random
    rnd = random.Random(3)
    for R in (1, 2, 3, 8):
        mat = [[rnd.choice([0, 0, 1, 5, 17, 200]) for _ in range(R)] for _ in range(R)]
        rec, row = 7408, 14336
        recv_base = [1_000_000_000 * (r + 1) for r in range(R)]
        ret_base = [50_000_000_000 + 1_000_000_000 * r for r in range(R)]
        routes = [peer_routes(mat, me, rec, row, recv_base, ret_base) for me in range(R)]
        for d in range(R):
            # receive zone of rank d: runs of rank 0, 1, ... back to back
            at = recv_base[d]
            for s in range(R):
                first_out, seg_dst, first_in, seg_ret = routes[s]
                if mat[s][d]:
                    assert seg_dst[d] == at
                    at += mat[s][d] * rec
                else:
                    assert seg_dst[d] == 0
            # ... which is exactly how rank d indexes what it received
            assert routes[d][2] == [sum(mat[s][d] for s in range(i)) for i in range(R + 1)]
        for s in range(R):
            # the rows rank d returns to rank s land where s packed its records for d
            first_out = routes[s][0]
            assert first_out == [sum(mat[s][:d]) for d in range(R)]
            for d in range(R):
                seg_ret = routes[d][3]
                assert seg_ret[s] == (ret_base[s] + first_out[d] * row if mat[s][d] else 0)
