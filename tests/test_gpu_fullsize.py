"""GPU tests at the benchmark's full size (DeepSeek-V3 shape: E=256, top_k=8, M=4096, H=7168, I=2048).

The oracle cannot run the whole layer at this size in seconds, so parity is shown by
 * the oracle on the rows of a few experts (the layer restricted to them through an expert map),
 * bit-exact checks of the integer stages (routing ids, alignment, stage-1 quantisation) against the oracle,
 * size-independent properties: additivity over a partition of the experts, equivariance under a
   permutation of the tokens, run-to-run determinism, chunked execution.
"""
import pytest
import torch

from lightop_b200 import synthetic
from oracle import moe_block_int8 as O
from oracle import moe_channel_int8 as OC
from util import assert_out_close, topk_ids_match

pytestmark = pytest.mark.gpu
DEV = "cuda"
CFG = synthetic.CONFIGS["c1_dsv3_prefill"]


@pytest.fixture(scope="module")
def lo():
    import lightop_b200
    return lightop_b200


@pytest.fixture(scope="module")
def world(lo):
    E, k, M, H, I = CFG["E"], CFG["topk"], CFG["M"], CFG["H"], CFG["I"]
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=0, device=DEV)          # 11.3 GB of int8 on the device
    c1_s, c2_s = synthetic.make_channel_scales(E, H, I, seed=0, device=DEV)
    x, logits = synthetic.make_activations(M, H, E, seed=1, device=DEV)
    tw = torch.empty(M, k, dtype=torch.float32, device=DEV)
    ti = torch.empty(M, k, dtype=torch.int32, device=DEV)
    lo.moe.topk_softmax(tw, ti, None, logits, True)
    torch.cuda.synchronize()
    yield dict(w1=w1, w2=w2, w1_s=w1_s, w2_s=w2_s, c1_s=c1_s, c2_s=c2_s, x=x, logits=logits, tw=tw, ti=ti)
    del w1, w2
    torch.cuda.empty_cache()


def _block(lo, W, x, tw, ti, **kw):
    y = lo.moe.fused_experts_impl_int8(x, W["w1"], W["w2"], tw, ti, None, use_int8_w8a8=True, block_shape=[128, 128],
                                       w1_scale=W["w1_s"], w2_scale=W["w2_s"], **kw)
    torch.cuda.synchronize()
    lo.check_device_status()
    return y


def _channel(lo, W, x, tw, ti, **kw):
    y = lo.moe.fused_experts_impl_int8(x, W["w1"], W["w2"], tw, ti, None, use_int8_w8a8=True, per_channel_quant=True,
                                       w1_scale=W["c1_s"], w2_scale=W["c2_s"], **kw)
    torch.cuda.synchronize()
    lo.check_device_status()
    return y


def test_integer_stages_bit_exact(lo, world):
    E, k, M, H = CFG["E"], CFG["topk"], CFG["M"], CFG["H"]
    logits_c = world["logits"].cpu()
    w_ref, ids_ref = O.route_topk_softmax(logits_c, k, renormalize=True)
    assert topk_ids_match(world["ti"].cpu(), ids_ref, logits_c)
    torch.testing.assert_close(world["tw"].cpu(), w_ref, rtol=2e-5, atol=2e-6)
    # alignment of the 32768 routed slots: same sorted order, expert table and padded length as the oracle
    sorted_ids, expert_ids, npost = lo.moe.moe_align_block_size(world["ti"], 16, E)
    s_ref, e_ref, n_ref = O.align_block_size(world["ti"].cpu().reshape(-1), E, 16)
    n = int(n_ref)
    assert int(npost.item()) == n
    assert torch.equal(sorted_ids.cpu()[:n], s_ref[:n]) and torch.equal(expert_ids.cpu()[: n // 16], e_ref[: n // 16])
    # stage-1 quantisation of the whole activation matrix, both formats
    xc = world["x"].cpu()
    q, s = lo.quant.per_token_group_quant_int8(world["x"], 128)
    q_ref, s_ref2 = O.group_quant_int8(xc, 128)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref2)
    q, s = lo.quant.per_token_quant_int8(world["x"])
    q_ref, s_ref2 = OC.per_token_quant_int8(xc)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref2)


@pytest.mark.parametrize("mode", ["block", "channel"])
def test_layer_restricted_to_sampled_experts_matches_oracle(lo, world, mode):
    # four experts spread over the table; every other expert is mapped to -1 (not on this rank)
    E, k = CFG["E"], CFG["topk"]
    sel = [3, 77, 130, 255]
    emap = torch.full((E,), -1, dtype=torch.int32)
    emap[sel] = torch.arange(len(sel), dtype=torch.int32)
    sub = dict(world)
    for name in ("w1", "w2", "w1_s", "w2_s", "c1_s", "c2_s"):
        sub[name] = world[name][sel].contiguous()
    run = _block if mode == "block" else _channel
    y = run(lo, sub, world["x"], world["tw"], world["ti"], expert_map=emap.to(DEV), global_num_experts=E)
    xc, twc, tic = world["x"].cpu(), world["tw"].cpu(), world["ti"].cpu()
    keep = emap[tic.long()] >= 0
    rows = int(keep.sum())
    assert rows > 300          # about 4096 * 8 * 4 / 256 = 512 routed rows hit the sample
    if mode == "block":
        local = torch.where(keep, emap[tic.long()], torch.full_like(tic, len(sel)))
        y_ref = O.fused_moe_block_int8(xc, sub["w1"].cpu(), sub["w2"].cpu(), sub["w1_s"].cpu(), sub["w2_s"].cpu(),
                                       twc * keep, local)
    else:
        y_ref = OC.fused_moe_channel_int8(xc, sub["w1"].cpu(), sub["w2"].cpu(), sub["c1_s"].cpu(), sub["c2_s"].cpu(),
                                          twc, tic, expert_map=emap)
    touched = keep.any(dim=1)
    _, mean_rel = assert_out_close(y.cpu()[touched], y_ref[touched], f"{mode}: tokens routed to the sampled experts")
    assert mean_rel < 2e-3
    assert bool((y.cpu()[~touched] == 0).all())


@pytest.mark.parametrize("mode", ["block", "channel"])
def test_full_layer_properties(lo, world, mode, monkeypatch):
    E, M = CFG["E"], CFG["M"]
    run = _block if mode == "block" else _channel
    y = run(lo, world, world["x"], world["tw"], world["ti"])
    assert bool(torch.isfinite(y.float()).all())
    # determinism
    assert torch.equal(run(lo, world, world["x"], world["tw"], world["ti"]), y)
    # chunked execution (4 chunks of 1024 tokens) gives the same rows
    monkeypatch.setenv("LMSLIM_FUSED_MOE_CHUNK_SIZE", "1024")
    assert torch.equal(run(lo, world, world["x"], world["tw"], world["ti"]), y)
    monkeypatch.delenv("LMSLIM_FUSED_MOE_CHUNK_SIZE")
    # equivariance under a permutation of the tokens
    perm = torch.randperm(M, generator=torch.Generator().manual_seed(7)).to(DEV)
    yp = run(lo, world, world["x"][perm].contiguous(), world["tw"][perm].contiguous(), world["ti"][perm].contiguous())
    assert torch.equal(yp, y[perm])
    # additivity over a partition of the experts: two expert-parallel halves add up to the whole
    parts = []
    for lo_e, hi_e in ((0, E // 2), (E // 2, E)):
        emap = torch.full((E,), -1, dtype=torch.int32)
        emap[lo_e:hi_e] = torch.arange(hi_e - lo_e, dtype=torch.int32)
        sub = dict(world)
        for name in ("w1", "w2", "w1_s", "w2_s", "c1_s", "c2_s"):
            sub[name] = world[name][lo_e:hi_e]
        parts.append(run(lo, sub, world["x"], world["tw"], world["ti"], expert_map=emap.to(DEV),
                         global_num_experts=E).float())
    assert_out_close(parts[0] + parts[1], y, f"{mode}: expert halves add up")


# ------------------------------ the other benchmark configurations at their full shapes ------------------------------

def _check_sampled_experts(lo, W, x, tw, ti, E, sel, what, min_rows=1):
    """The block layer restricted to the experts `sel` (every other expert mapped to -1) against the oracle on the
    rows routed to them; tokens that touch none of them must come out zero."""
    emap = torch.full((E,), -1, dtype=torch.int32)
    emap[sel] = torch.arange(len(sel), dtype=torch.int32)
    sub = dict(W)
    for name in ("w1", "w2", "w1_s", "w2_s"):
        sub[name] = W[name][sel].contiguous()
    y = _block(lo, sub, x, tw, ti, expert_map=emap.to(DEV), global_num_experts=E)
    xc, twc, tic = x.cpu(), tw.cpu(), ti.cpu()
    keep = emap[tic.long()] >= 0
    assert int(keep.sum()) >= min_rows
    local = torch.where(keep, emap[tic.long()], torch.full_like(tic, len(sel)))
    y_ref = O.fused_moe_block_int8(xc, sub["w1"].cpu(), sub["w2"].cpu(), sub["w1_s"].cpu(), sub["w2_s"].cpu(), twc * keep, local)
    touched = keep.any(dim=1)
    assert_out_close(y.cpu()[touched], y_ref[touched], what)
    assert bool((y.cpu()[~touched] == 0).all())
    return int(keep.sum())


@pytest.mark.parametrize("M", [1, 8, 64, 256])
def test_decode_sizes_of_the_same_shape(lo, world, M):
    """Configuration c2: the first M rows of one fixed 256-row batch on the DeepSeek-V3 weights."""
    E, k, H = CFG["E"], CFG["topk"], CFG["H"]
    x256, l256 = synthetic.make_activations(256, H, E, seed=1, device=DEV)
    x, logits = x256[:M].contiguous(), l256[:M].contiguous()
    tw = torch.empty(M, k, dtype=torch.float32, device=DEV)
    ti = torch.empty(M, k, dtype=torch.int32, device=DEV)
    lo.moe.topk_softmax(tw, ti, None, logits, True)
    torch.cuda.synchronize()
    # integer stages: bit-exact
    w_ref, ids_ref = O.route_topk_softmax(logits.cpu(), k, renormalize=True)
    assert topk_ids_match(ti.cpu(), ids_ref, logits.cpu())
    torch.testing.assert_close(tw.cpu(), w_ref, rtol=2e-5, atol=2e-6)
    sorted_ids, expert_ids, npost = lo.moe.moe_align_block_size(ti, 16, E)
    s_ref, e_ref, n_ref = O.align_block_size(ti.cpu().reshape(-1), E, 16)
    n = int(n_ref)
    assert int(npost.item()) == n and torch.equal(sorted_ids.cpu()[:n], s_ref[:n])
    q, s = lo.quant.per_token_group_quant_int8(x, 128)
    q_ref, s_ref2 = O.group_quant_int8(x.cpu(), 128)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref2)
    # the layer on the (up to) eight experts with the most rows, against the oracle
    counts = torch.bincount(ti.cpu().reshape(-1).long(), minlength=E)
    sel = torch.argsort(counts, descending=True, stable=True)[:8]
    sel = sorted(int(e) for e in sel if counts[e] > 0)
    _check_sampled_experts(lo, world, x, tw, ti, E, sel, f"c2 M={M}")
    # whole layer: finite, deterministic
    y = _block(lo, world, x, tw, ti)
    assert bool(torch.isfinite(y.float()).all())
    assert torch.equal(_block(lo, world, x, tw, ti), y)


def test_zipf_routed_qwen3_shape(lo):
    """Configuration c4: E=128, top_k=8, M=2048, H=4096, I=1536, expert popularity ~ Zipf(1.2): the hottest expert
    gets an order of magnitude more rows than a chunk holds, most get a handful."""
    cfg = synthetic.CONFIGS["c4_qwen3_zipf"]
    E, k, M, H, I = cfg["E"], cfg["topk"], cfg["M"], cfg["H"], cfg["I"]
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=0, device=DEV)
    W = dict(w1=w1, w2=w2, w1_s=w1_s, w2_s=w2_s)
    x, logits = synthetic.make_activations(M, H, E, seed=1, device=DEV, zipf=cfg["zipf"])
    tw = torch.empty(M, k, dtype=torch.float32, device=DEV)
    ti = torch.empty(M, k, dtype=torch.int32, device=DEV)
    lo.moe.topk_softmax(tw, ti, None, logits, True)
    torch.cuda.synchronize()
    w_ref, ids_ref = O.route_topk_softmax(logits.cpu(), k, renormalize=True)
    assert topk_ids_match(ti.cpu(), ids_ref, logits.cpu())
    sorted_ids, expert_ids, npost = lo.moe.moe_align_block_size(ti, 16, E)
    s_ref, e_ref, n_ref = O.align_block_size(ti.cpu().reshape(-1), E, 16)
    n = int(n_ref)
    assert int(npost.item()) == n and torch.equal(sorted_ids.cpu()[:n], s_ref[:n])
    counts = torch.bincount(ti.cpu().reshape(-1).long(), minlength=E)
    order = torch.argsort(counts, descending=True, stable=True)
    hottest = int(order[0])
    assert int(counts[hottest]) > 8 * 128          # many chunks of one expert
    # the hottest expert, one from the middle of the ranking and the coldest one that is hit
    hit = [int(e) for e in order if counts[e] > 0]
    sel = sorted({hottest, hit[len(hit) // 2], hit[-1]})
    _check_sampled_experts(lo, W, x, tw, ti, E, sel, "c4 sampled experts", min_rows=int(counts[hottest]))
    y = _block(lo, W, x, tw, ti)
    assert bool(torch.isfinite(y.float()).all())
    assert torch.equal(_block(lo, W, x, tw, ti), y)
    del w1, w2, W
    torch.cuda.empty_cache()
