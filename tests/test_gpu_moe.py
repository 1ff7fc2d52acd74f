"""GPU parity tests of the grouped GEMM and of the fused layer against the oracle and the goldens."""
import ctypes
import os

import pytest
import torch

from lightop_b200 import synthetic
from oracle import moe_block_int8 as O
from util import assert_gemm_close, assert_out_close, out_errors

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def lo():
    import lightop_b200
    return lightop_b200


def _route(logits, k):
    w, ids = O.route_topk_softmax(logits, k, renormalize=True)
    return w, ids


def _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids, **kw):
    M, H = x.shape
    k = ids.shape[1]
    cache13 = torch.empty(M * k * max(w1.shape[1], H), dtype=torch.bfloat16, device=DEV)
    y = lo.moe.fused_experts_impl_int8(x.to(DEV), w1.to(DEV), w2.to(DEV), w.to(DEV), ids.to(DEV), cache13,
                                       use_int8_w8a8=True, block_shape=[128, 128],
                                       w1_scale=w1_s.to(DEV), w2_scale=w2_s.to(DEV), **kw)
    torch.cuda.synchronize()
    lo.check_device_status()
    return y


# ------------------------------ unfused grouped GEMM ---------------------------------

@pytest.mark.parametrize("M,E,k,N,K,bs", [(40, 4, 2, 256, 256, 16), (40, 4, 2, 256, 256, 128), (129, 8, 2, 384, 512, 64),
                                         (7, 8, 3, 128, 1024, 16), (300, 2, 1, 256, 128, 128)])
@pytest.mark.parametrize("with_weight", [False, True])
def test_moe_gemm_w8a8_block(lo, M, E, k, N, K, bs, with_weight):
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    aq, a_s = O.group_quant_int8(x, 128)
    B = torch.randint(-127, 128, (E, N, K), generator=g, dtype=torch.int8)
    b_s = torch.rand(E, N // 128, K // 128, generator=g) * 9e-3 + 1e-3
    w, ids = _route(torch.randn(M, E, generator=g), k)
    sorted_ids, expert_ids, npost = lo.moe.moe_align_block_size(ids.to(DEV), bs, E)
    out = torch.full((M, k, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    lo.moe.moe_gemm_w8a8(aq.to(DEV), B.to(DEV), out, a_s.to(DEV), b_s.to(DEV), w.to(DEV) if with_weight else None,
                         sorted_ids, expert_ids, npost, k, {"BLOCK_SIZE_M": bs})
    torch.cuda.synchronize()
    ref = torch.empty(M * k, N, dtype=torch.float32)
    flat = ids.reshape(-1)
    for e in range(E):
        m = flat == e
        if m.any():
            rows = torch.nonzero(m).reshape(-1) // k
            ref[m] = O.block_int8_matmul(aq[rows], B[e], a_s[rows], b_s[e], (128, 128), torch.float32)
    if with_weight:
        ref = ref * w.reshape(-1, 1)        # fp32 product before the cast, as the reference kernel (int8.py:521-530)
    ref = ref.to(torch.bfloat16)
    got = out.cpu().view(M * k, N)
    assert not torch.isnan(got.float()).any()
    if not with_weight:
        assert_gemm_close(got, ref, "grouped gemm")
    else:
        torch.testing.assert_close(got.float(), ref.float(), rtol=1e-2, atol=1e-2)


def test_moe_gemm_non_local_blocks_are_zero(lo):
    g = torch.Generator().manual_seed(0)
    M, E, k, N, K, bs = 64, 8, 2, 128, 256, 16
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    aq, a_s = O.group_quant_int8(x, 128)
    B = torch.randint(-127, 128, (4, N, K), generator=g, dtype=torch.int8)     # 4 local experts
    b_s = torch.rand(4, 1, K // 128, generator=g) * 9e-3 + 1e-3
    _, ids = _route(torch.randn(M, E, generator=g), k)
    emap = torch.tensor([-1, -1, -1, -1, 0, 1, 2, 3], dtype=torch.int32)
    sorted_ids, expert_ids, npost = lo.moe.moe_align_block_size(ids.to(DEV), bs, E, emap.to(DEV))
    out = torch.full((M, k, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    lo.moe.moe_gemm_w8a8(aq.to(DEV), B.to(DEV), out, a_s.to(DEV), b_s.to(DEV), None, sorted_ids, expert_ids, npost, k,
                         {"BLOCK_SIZE_M": bs})
    got = out.cpu().view(M * k, N)
    flat = ids.reshape(-1)
    for e in range(E):
        m = flat == e
        if not m.any():
            continue
        if e < 4:
            assert bool((got[m] == 0).all())        # reference: expert_id == -1 blocks write zeros (int8.py:441-449)
        else:
            rows = torch.nonzero(m).reshape(-1) // k
            assert_gemm_close(got[m], O.block_int8_matmul(aq[rows], B[e - 4], a_s[rows], b_s[e - 4], (128, 128), torch.bfloat16))


# ------------------------------ fused layer ---------------------------------------

def test_fused_c0_against_golden(lo, golden_dir):
    cfg = synthetic.CONFIGS["c0_tiny"]
    gold = torch.load(os.path.join(golden_dir, "c0_tiny.pt"))
    w1, w2, w1_s, w2_s = synthetic.make_weights(cfg["E"], cfg["H"], cfg["I"], seed=0)
    x, _ = synthetic.make_activations(cfg["M"], cfg["H"], cfg["E"], seed=1)
    y = _run_fused(lo, x, w1, w2, w1_s, w2_s, gold["topk_weights"], gold["topk_ids"])
    max_norm, mean_rel = assert_out_close(y, gold["y"], "c0")
    # this path reproduces the oracle's rounding sequence; it is expected to be far inside the bars
    assert mean_rel < 1e-3


def _stage2_from_workspace(lo, M, E, k, H, I, x, w1, w2, w1_s, w2_s, w, ids):
    """Run the C-ABI entry point directly with a test-owned workspace and return the intermediates."""
    from lightop_b200 import _lib
    lib = _lib.load()
    ws_bytes = lib.lo_fused_moe_workspace_bytes(M, E, E, k, H, I)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    off = (ctypes.c_int64 * 8)()
    assert lib.lo_fused_moe_workspace_layout(M, E, E, k, H, I, off) == 0
    cache3 = torch.empty(M * k * H, dtype=torch.bfloat16, device=DEV)
    out = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    t = [a.to(DEV).contiguous() for a in (x, w1, w2, w1_s, w2_s, w.float(), ids.to(torch.int32))]
    st = lib.lo_fused_moe_block_int8(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), t[4].data_ptr(),
                                     t[5].data_ptr(), t[6].data_ptr(), _lib.LO_I32, 0, E, M, E, k, H, I,
                                     cache3.data_ptr(), 0, out.data_ptr(), 0, 1.0, ws.data_ptr(), ws_bytes,
                                     status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    _lib.check(st, "fused")
    torch.cuda.synchronize()
    assert status.item() == 0
    cap = off[7]
    wsc = ws.cpu()
    header = wsc[off[0]:off[0] + 8].view(torch.int32)
    xq = wsc[off[1]:off[1] + cap * H].view(torch.int8).view(cap, H)
    xs = wsc[off[2]:off[2] + cap * (H // 128) * 4].view(torch.float32).view(cap, H // 128)
    sorted_ids = wsc[off[3]:off[3] + cap * 4].view(torch.int32)
    act_q = wsc[off[5]:off[5] + cap * I].view(torch.int8).view(cap, I)
    act_s = wsc[off[6]:off[6] + cap * (I // 128) * 4].view(torch.float32).view(cap, I // 128)
    return out.cpu(), header, xq, xs, sorted_ids, act_q, act_s


@pytest.mark.parametrize("name,shape", [("c0", (8, 2, 32, 256, 512)), ("ragged", (16, 4, 77, 512, 256)), ("big_chunk", (2, 1, 300, 256, 256)),
                                        ("wide_pair", (2, 1, 620, 256, 256)), ("wide_many", (8, 2, 580, 384, 256))])
def test_fused_intermediates_bit_exact(lo, name, shape):
    E, k, M, H, I = shape
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=0)
    x, logits = synthetic.make_activations(M, H, E, seed=1)
    w, ids = _route(logits, k)
    y_ref, inter = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids, return_intermediates=True)
    y, header, xq, xs, sorted_ids, act_q, act_s = _stage2_from_workspace(lo, M, E, k, H, I, x, w1, w2, w1_s, w2_s, w, ids)
    # the sort: bit-exact
    s_ref, _, n_ref = O.align_block_size(ids, E, 16)
    assert header[0].item() == n_ref.item()
    assert torch.equal(sorted_ids[: n_ref.item()], s_ref)
    pos = torch.nonzero(s_ref < M * k).reshape(-1)
    sid = s_ref[pos].long()
    # stage 1 quantisation (stored once per routed slot, in sorted order): bit-exact
    assert torch.equal(xq[pos], inter["a_q"][sid // k]) and torch.equal(xs[pos], inter["a_s"][sid // k])
    # stage 2 quantisation (after gate_up GEMM, SiLU*mul in bf16): compared row by row through the sort
    dq = (act_q[pos].int() - inter["act_q"][sid].int()).abs()
    frac_exact = float((dq == 0).float().mean())
    assert int(dq.max()) <= 1, f"stage-2 codes differ by {int(dq.max())}"
    assert frac_exact >= 0.999, f"only {frac_exact:.5f} of the stage-2 codes are identical"
    torch.testing.assert_close(act_s[pos], inter["act_s"][sid], rtol=1e-6, atol=0)
    assert_out_close(y, y_ref, name)


@pytest.mark.parametrize("E,k,M,H,I", [(8, 2, 1, 256, 512), (8, 2, 7, 256, 512), (16, 4, 33, 384, 256), (4, 1, 200, 256, 128), (32, 8, 129, 1024, 384)])
def test_fused_edge_shapes(lo, E, k, M, H, I):
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=3)
    x, logits = synthetic.make_activations(M, H, E, seed=4)
    w, ids = _route(logits, k)
    y_ref = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids)
    y = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    assert_out_close(y, y_ref, f"E{E}k{k}M{M}")


def test_fused_many_chunks(lo):
    # more than 1024 entries in the 128-row chunk table: the wide table of the down GEMM is derived in several rounds
    E, k, M, H, I = 8, 4, 36000, 256, 128
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=5)
    x, logits = synthetic.make_activations(M, H, E, seed=6)
    w, ids = _route(logits, k)
    y_ref = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids)
    y = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    assert_out_close(y, y_ref, "many chunks")


@pytest.mark.parametrize("M", [192, 196, 256, 476, 480, 700])
def test_fused_chunk_size_rule(lo, M):
    # rows per expert on average 48 / 49 / 64 / 119 / 120 / 175: the chunk table is cut at 64, 128, 128, 128, 160 and 160
    # rows, with experts on both sides of every cut (the routing is not uniform), so every instantiation meets split experts
    E, k, H, I = 8, 2, 256, 256
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=15)
    x, logits = synthetic.make_activations(M, H, E, seed=16)
    w, ids = _route(logits, k)
    y_ref = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids)
    y = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    assert_out_close(y, y_ref, f"chunk rule M={M}")


def test_fused_options(lo, monkeypatch):
    E, k, M, H, I = 8, 2, 50, 256, 256
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=5)
    x, logits = synthetic.make_activations(M, H, E, seed=6)
    w, ids = _route(logits, k)
    y_ref = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids)
    base = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    # int64 ids, scaling factor and shared output
    shared = torch.randn(M, H).to(torch.bfloat16)
    y = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids.long(), routed_scaling_factor=2.5, shared_output=shared.to(DEV))
    ref = (y_ref.float() * 2.5 + shared.float()).to(torch.bfloat16)
    assert_out_close(y, ref, "scaled+shared")
    # chunked execution gives the same bits as one chunk (tokens are independent)
    monkeypatch.setenv("LMSLIM_FUSED_MOE_CHUNK_SIZE", "16")
    chunked = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    assert torch.equal(chunked, base)
    monkeypatch.delenv("LMSLIM_FUSED_MOE_CHUNK_SIZE")
    # inplace
    xd = x.to(DEV).clone()
    cache13 = torch.empty(M * k * H, dtype=torch.bfloat16, device=DEV)
    out = lo.moe.fused_experts_impl_int8(xd, w1.to(DEV), w2.to(DEV), w.to(DEV), ids.to(DEV), cache13, inplace=True,
                                         use_int8_w8a8=True, block_shape=[128, 128], w1_scale=w1_s.to(DEV), w2_scale=w2_s.to(DEV))
    assert out.data_ptr() == xd.data_ptr() and torch.equal(out, base)


@pytest.mark.parametrize("E,M", [(4, 40), (2, 300)])     # 10 and 150 rows per expert (narrow and wide chunks)
def test_fused_router_weight_on_input(lo, E, M):
    H, I = 256, 256
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=7)
    x, logits = synthetic.make_activations(M, H, E, seed=8)
    w, ids = O.route_topk_softmax(logits, 1, renormalize=False)
    # torch model of the reference kernel's order: weight multiplies the gate_up sum before the cast (int8.py:521-530)
    aq, a_s = O.group_quant_int8(x, 128)
    ref = torch.zeros(M, H, dtype=torch.bfloat16)
    for e in range(E):
        m = ids.reshape(-1) == e
        if m.any():
            h = O.block_int8_matmul(aq[m], w1[e], a_s[m], w1_s[e], (128, 128), torch.float32)
            h = (h * w[m]).to(torch.bfloat16)
            act = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
            q2, s2 = O.group_quant_int8(act.contiguous(), 128)
            ref[m] = O.block_int8_matmul(q2, w2[e], s2, w2_s[e], (128, 128), torch.bfloat16)
    y = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids, apply_router_weight_on_input=True)
    assert_out_close(y, ref, "router weight on input")


def test_fused_expert_parallel_mask(lo):
    # EP simulated on one device the way the reference does (test/moe_w8a8/test_kernel_moe_ep8.py:98-153):
    # rank r of R owns a contiguous block of experts, the other experts map to -1.
    E, k, M, H, I, R = 16, 4, 60, 256, 256, 4
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=9)
    x, logits = synthetic.make_activations(M, H, E, seed=10)
    w, ids = _route(logits, k)
    y_full = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids).float()
    total = torch.zeros(M, H)
    per = E // R
    for r in range(R):
        emap = torch.full((E,), -1, dtype=torch.int32)
        emap[r * per:(r + 1) * per] = torch.arange(per, dtype=torch.int32)
        sl = slice(r * per, (r + 1) * per)
        y_r = _run_fused(lo, x, w1[sl], w2[sl], w1_s[sl], w2_s[sl], w, ids, expert_map=emap.to(DEV), global_num_experts=E)
        # oracle of the rank: weights of non-local slots zeroed
        local = (ids >= r * per) & (ids < (r + 1) * per)
        ref_r = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w * local, ids)
        assert_out_close(y_r, ref_r, f"rank {r}")
        total += y_r.float().cpu()
    max_norm, mean_rel = out_errors(total, y_full)
    assert max_norm < 2e-2 and mean_rel < 1e-2


def test_fused_is_deterministic_and_token_independent(lo):
    # size-independent properties: same bits run to run; permuting tokens permutes the output rows bit-for-bit
    E, k, M, H, I = 32, 8, 512, 1024, 512
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=11)
    x, logits = synthetic.make_activations(M, H, E, seed=12)
    w, ids = _route(logits, k)
    a = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    b = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    assert torch.equal(a, b)
    perm = torch.randperm(M, generator=torch.Generator().manual_seed(0))
    c = _run_fused(lo, x[perm], w1, w2, w1_s, w2_s, w[perm], ids[perm])
    assert torch.equal(c.cpu(), a.cpu()[perm])


def test_fused_zipf_imbalance(lo):
    # Qwen3-like geometry scaled down, Zipf(1.2) expert popularity: a few experts get many 128-row chunks
    E, k, M, H, I = 32, 4, 1500, 512, 384
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=13)
    x, logits = synthetic.make_activations(M, H, E, seed=14, zipf=1.2)
    w, ids = _route(logits, k)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=E)
    assert int(counts.max()) > 4 * 128
    y_ref = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids)
    y = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    assert_out_close(y, y_ref, "zipf")


# ------------------------------ expert parallelism on one device -----------------------

@pytest.mark.parametrize("transport", ["peer", "collective"])
def test_expert_rows_entry_point_and_ep_driver_world1(lo, transport):
    """The EP driver with a single rank (NCCL, world size 1) must give the bits of the fused layer, with the records
    and result rows carried by stores into landing zones ("peer") and by all-to-all ("collective")."""
    import socket
    import torch.distributed as dist
    from lightop_b200.ep import ExpertParallelMoE
    E, k, M, H, I = 16, 4, 70, 512, 256
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=21)
    x, logits = synthetic.make_activations(M, H, E, seed=22)
    w, ids = _route(logits, k)
    base = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    try:
        layer = ExpertParallelMoE(w1.to(DEV), w2.to(DEV), w1_s.to(DEV), w2_s.to(DEV), E, transport=transport)
        assert layer.transport == transport
        y = layer.forward(x.to(DEV), w.to(DEV), ids.to(DEV))
        layer.profile = True
        y3 = layer.forward(x.to(DEV), w.to(DEV), ids.to(DEV))
        stages = layer.stage_ms()
        layer.profile = False
        # a larger batch makes the peer transport grow its landing zones
        x2, logits2 = synthetic.make_activations(3 * M, H, E, seed=23)
        w_2, ids_2 = _route(logits2, k)
        y4 = layer.forward(x2.to(DEV), w_2.to(DEV), ids_2.to(DEV))
        torch.cuda.synchronize()
        lo.check_device_status()
        layer.close()
    finally:
        dist.destroy_process_group()
    assert torch.equal(y, base)
    assert torch.equal(y3, base)
    assert torch.equal(y4, _run_fused(lo, x2, w1, w2, w1_s, w2_s, w_2, ids_2))
    assert set(stages) == {"quantise", "pack", "counts", "dispatch", "experts", "combine", "gather"}
    assert_out_close(y, O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids), "ep world 1")


def test_ep_driver_falls_back_when_no_landing_zone_can_be_had(lo):
    """A rank that cannot allocate its landing zones makes every rank switch to the all-to-all transport; the failure
    is made on the host (a stand-in for the allocation call that reports an error)."""
    import socket
    import torch.distributed as dist
    from lightop_b200.ep import ExpertParallelMoE
    E, k, M, H, I = 8, 2, 40, 256, 256
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=24)
    x, logits = synthetic.make_activations(M, H, E, seed=25)
    w, ids = _route(logits, k)
    base = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)

    class NoAlloc:
        def __init__(self, lib):
            self._lib = lib

        def __getattr__(self, name):
            return getattr(self._lib, name)

        def lo_peer_alloc(self, nbytes, out):
            return 3

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    try:
        layer = ExpertParallelMoE(w1.to(DEV), w2.to(DEV), w1_s.to(DEV), w2_s.to(DEV), E, transport="peer")
        layer._zones.lib = NoAlloc(layer._zones.lib)
        y = layer.forward(x.to(DEV), w.to(DEV), ids.to(DEV))
        torch.cuda.synchronize()
        assert layer.transport == "collective" and layer.transport_note
        y2 = layer.forward(x.to(DEV), w.to(DEV), ids.to(DEV))
        torch.cuda.synchronize()
        layer.close()
    finally:
        dist.destroy_process_group()
    assert torch.equal(y, base) and torch.equal(y2, base)


# ------------------------------ dense block-INT8 linear -------------------------------

@pytest.mark.parametrize("m,n,k", [(1, 576, 7168), (7, 2048, 512), (48, 256, 1024), (128, 7168, 128), (300, 1536, 1536), (1024, 2304, 1152 + 128)])
def test_dense_block_int8_linear(lo, m, n, k):
    # shapes from the reference's dense block GEMM test (test/w8a8/test_w8a8_block.py:205-215); N = 576 and 2304
    # are not multiples of 128
    g = torch.Generator().manual_seed(m + n)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    aq, a_s = O.group_quant_int8(x, 128)
    B = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    b_s = torch.rand((n + 127) // 128, k // 128, generator=g) * 9e-3 + 1e-3
    ref = O.block_int8_matmul(aq, B, a_s, b_s, (128, 128), torch.bfloat16)
    out = lo.gemm_ops.matmul_block_int8(aq.to(DEV), B.to(DEV), a_s.to(DEV), b_s.to(DEV), [128, 128], torch.bfloat16)
    torch.cuda.synchronize()
    lo.check_device_status()
    assert_gemm_close(out, ref, "dense linear")
    # the assembly kernel's convention: activation scales transposed; the reference's own bar is allclose(1e-2, 5e-2)
    out2 = lo.gemm_ops.gemm_w8a8_asm(aq.to(DEV), B.to(DEV), a_s.t().contiguous().to(DEV), b_s.to(DEV), [128, 128], torch.bfloat16)
    assert torch.equal(out2, out)
    y = lo.gemm_ops.apply_w8a8_block_int8_linear(x.to(DEV), B.to(DEV), [128, 128], b_s.to(DEV))
    assert torch.equal(y, out)
