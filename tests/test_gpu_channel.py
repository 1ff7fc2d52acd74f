"""GPU parity tests of the per-channel W8A8 mode (per-token activation scales, per-output-channel
weight scales) against the oracle and the fixture made from the reference's torch functions."""
import os

import pytest
import torch

from lightop_b200 import synthetic
from oracle import moe_block_int8 as O
from oracle import moe_channel_int8 as OC
from util import assert_out_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def lo():
    import lightop_b200
    return lightop_b200


def _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids, **kw):
    y = lo.moe.fused_experts_impl_int8(x.to(DEV), w1.to(DEV), w2.to(DEV), w.to(DEV), ids.to(DEV), None,
                                       use_int8_w8a8=True, per_channel_quant=True, block_shape=None,
                                       w1_scale=w1_s.to(DEV), w2_scale=w2_s.to(DEV), **kw)
    torch.cuda.synchronize()
    lo.check_device_status()
    return y


# ------------------------------ the two quantisers ---------------------------------

@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(3, 257), (1, 7168), (64, 2048), (5, 8), (2, 3, 512)])
def test_per_token_quant_bit_exact(lo, dtype, shape):
    # (3, 257) bf16 with seed 5 is the reference's own case (test/test_quant_per_token_quant_int8.py:28-39)
    torch.manual_seed(5)
    x = torch.randn(shape).to(dtype)
    x.reshape(-1, shape[-1])[0, :] *= 0.0 if shape[0] > 2 else 1.0      # a row of zeros where there is room
    q, s = lo.quant.per_token_quant_int8(x.to(DEV))
    q_ref, s_ref = OC.per_token_quant_int8(x)
    assert q.shape == x.shape and s.shape == x.shape[:-1] + (1,)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)


def test_per_token_quant_empty(lo):
    q, s = lo.quant.per_token_quant_int8(torch.empty(0, 128, dtype=torch.bfloat16, device=DEV))
    assert q.shape == (0, 128) and s.shape == (0, 1)


@pytest.mark.parametrize("rows,d", [(1, 2048), (37, 256), (8, 4096), (130, 128)])
def test_silu_mul_quant(lo, rows, d):
    g = torch.Generator().manual_seed(rows + d)
    inter = (torch.randn(rows, 2 * d, generator=g) * 4).to(torch.bfloat16)
    if rows > 2:
        inter[1] = 0          # a row of zeros: scale 0, codes 0
    q, s = lo.activation.fuse_silu_mul_quant(inter.to(DEV))
    q_ref, s_ref = OC.silu_mul_quant_int8(inter)
    assert q.shape == (rows, d) and s.shape == (rows, 1)
    # expf on the device and in torch may differ in the last bit, which a bf16 rounding can expose: a
    # row's maximum (and with it the whole row's codes) may then move by one bf16 step
    torch.testing.assert_close(s.cpu(), s_ref, rtol=1e-2, atol=0)
    same_scale = (s.cpu() == s_ref).reshape(-1)
    assert float(same_scale.float().mean()) >= 0.95
    dq = (q.cpu().int() - q_ref.int()).abs()[same_scale]
    assert int(dq.max()) <= 1 and float((dq == 0).float().mean()) >= 0.9999


# ------------------------------ unfused grouped GEMM ---------------------------------

@pytest.mark.parametrize("M,E,k,N,K,bs", [(40, 4, 2, 256, 256, 16), (40, 4, 2, 256, 256, 128), (129, 8, 2, 384, 512, 64),
                                         (7, 8, 3, 128, 1024, 16), (300, 2, 1, 256, 128, 128), (64, 4, 2, 128, 7168, 32)])
@pytest.mark.parametrize("with_weight", [False, True])
def test_moe_gemm_w8a8_channel(lo, M, E, k, N, K, bs, with_weight):
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    aq, a_s = OC.per_token_quant_int8(x)
    B = torch.randint(-127, 128, (E, N, K), generator=g, dtype=torch.int8)
    b_s = torch.rand(E, N, 1, generator=g) * 9e-4 + 1e-4
    w, ids = O.route_topk_softmax(torch.randn(M, E, generator=g), k, renormalize=True)
    sorted_ids, expert_ids, npost = lo.moe.moe_align_block_size(ids.to(DEV), bs, E)
    out = torch.full((M, k, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    lo.moe.moe_gemm_w8a8(aq.to(DEV), B.to(DEV), out, a_s.to(DEV), b_s.to(DEV), w.to(DEV) if with_weight else None,
                         sorted_ids, expert_ids, npost, k, {"BLOCK_SIZE_M": bs})
    torch.cuda.synchronize()
    ref = torch.empty(M * k, N, dtype=torch.bfloat16)
    flat = ids.reshape(-1)
    wflat = w.reshape(-1)
    for e in range(E):
        m = flat == e
        if m.any():
            rows = torch.nonzero(m).reshape(-1) // k
            ref[m] = OC.per_token_matmul(aq[rows], B[e], a_s[rows], b_s[e], torch.bfloat16,
                                         row_weight=wflat[m] if with_weight else None)
    got = out.cpu().view(M * k, N)
    assert not torch.isnan(got.float()).any()
    assert torch.equal(got, ref)        # integer sums are exact and the fp32 scaling sequence is the oracle's


def test_moe_gemm_channel_non_local_blocks_are_zero(lo):
    g = torch.Generator().manual_seed(0)
    M, E, k, N, K, bs = 64, 8, 2, 128, 256, 16
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    aq, a_s = OC.per_token_quant_int8(x)
    B = torch.randint(-127, 128, (4, N, K), generator=g, dtype=torch.int8)
    b_s = torch.rand(4, N, 1, generator=g) * 9e-4 + 1e-4
    _, ids = O.route_topk_softmax(torch.randn(M, E, generator=g), k, renormalize=True)
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
            assert bool((got[m] == 0).all())
        else:
            rows = torch.nonzero(m).reshape(-1) // k
            assert torch.equal(got[m], OC.per_token_matmul(aq[rows], B[e - 4], a_s[rows], b_s[e - 4], torch.bfloat16))


# ------------------------------ fused layer ---------------------------------------

def test_fused_channel_c0_against_golden(lo, golden_dir):
    cfg = synthetic.CONFIGS["c0_tiny"]
    gold = torch.load(os.path.join(golden_dir, "channel_cases.pt"))
    w1, w2, _, _ = synthetic.make_weights(cfg["E"], cfg["H"], cfg["I"], seed=0)
    w1_s, w2_s = synthetic.make_channel_scales(cfg["E"], cfg["H"], cfg["I"], seed=0)
    x, _ = synthetic.make_activations(cfg["M"], cfg["H"], cfg["E"], seed=1)
    y = _run_fused(lo, x, w1, w2, w1_s.unsqueeze(-1), w2_s.unsqueeze(-1), gold["topk_weights"], gold["topk_ids"])
    assert_out_close(y, gold["y"], "c0 per-channel vs the reference's torch model")
    y_or = OC.fused_moe_channel_int8(x, w1, w2, w1_s, w2_s, gold["topk_weights"], gold["topk_ids"])
    _, mean_rel = assert_out_close(y, y_or, "c0 per-channel vs oracle")
    assert mean_rel < 1e-3


@pytest.mark.parametrize("E,k,M,H,I", [(8, 2, 1, 256, 128), (8, 2, 33, 512, 256), (16, 4, 200, 1024, 384),
                                       (4, 1, 300, 256, 128), (32, 8, 64, 7168, 256), (8, 8, 16, 256, 2048),
                                       # experts with 129..256 rows (one chunk, two activation boxes) and more (split)
                                       (4, 2, 320, 512, 256), (2, 1, 700, 256, 128), (8, 2, 1000, 384, 128)])
def test_fused_channel_shapes(lo, E, k, M, H, I):
    w1, w2, _, _ = synthetic.make_weights(E, H, I, seed=2)
    w1_s, w2_s = synthetic.make_channel_scales(E, H, I, seed=2)
    x, logits = synthetic.make_activations(M, H, E, seed=3)
    w, ids = O.route_topk_softmax(logits, k, renormalize=True)
    y = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    y_or = OC.fused_moe_channel_int8(x, w1, w2, w1_s, w2_s, w, ids)
    _, mean_rel = assert_out_close(y, y_or, f"per-channel E{E} k{k} M{M}")
    assert mean_rel < 2e-3


def test_fused_channel_options(lo, monkeypatch):
    E, k, M, H, I = 8, 2, 96, 512, 256
    w1, w2, _, _ = synthetic.make_weights(E, H, I, seed=4)
    w1_s, w2_s = synthetic.make_channel_scales(E, H, I, seed=4)
    x, logits = synthetic.make_activations(M, H, E, seed=5)
    w, ids = O.route_topk_softmax(logits, k, renormalize=True)
    base = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids)
    # chunked execution gives the same rows
    monkeypatch.setenv("LMSLIM_FUSED_MOE_CHUNK_SIZE", "40")
    assert torch.equal(_run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids), base)
    monkeypatch.delenv("LMSLIM_FUSED_MOE_CHUNK_SIZE")
    # int64 ids, scaling factor and shared output
    shared = torch.randn(M, H).to(torch.bfloat16)
    y = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids.to(torch.int64), routed_scaling_factor=2.5,
                   shared_output=shared.to(DEV))
    y_or = OC.fused_moe_channel_int8(x, w1, w2, w1_s, w2_s, w, ids, routed_scaling_factor=2.5, shared_output=shared)
    assert_out_close(y, y_or, "scaling factor + shared output")
    # expert-parallel mask: the two halves add up to the whole
    half = E // 2
    parts = []
    for lo_e, hi_e in ((0, half), (half, E)):
        emap = torch.full((E,), -1, dtype=torch.int32)
        emap[lo_e:hi_e] = torch.arange(hi_e - lo_e, dtype=torch.int32)
        parts.append(_run_fused(lo, x, w1[lo_e:hi_e], w2[lo_e:hi_e], w1_s[lo_e:hi_e], w2_s[lo_e:hi_e], w, ids,
                                expert_map=emap.to(DEV), global_num_experts=E).float())
    assert_out_close(parts[0] + parts[1], base, "expert halves")
    # the sibling entry point of the reference (no cache argument)
    y2 = lo.moe.fused_experts_impl_int8_marlin(x.to(DEV), w1.to(DEV), w2.to(DEV), w.to(DEV), ids.to(DEV),
                                               use_int8_w8a8=True, per_channel_quant=True,
                                               w1_scale=w1_s.to(DEV), w2_scale=w2_s.to(DEV))
    assert torch.equal(y2, base)
    # determinism
    assert torch.equal(_run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids), base)


def test_fused_channel_router_weight_on_input(lo):
    E, k, M, H, I = 8, 1, 70, 256, 128
    w1, w2, _, _ = synthetic.make_weights(E, H, I, seed=6)
    w1_s, w2_s = synthetic.make_channel_scales(E, H, I, seed=6)
    x, logits = synthetic.make_activations(M, H, E, seed=7)
    w, ids = O.route_topk_softmax(logits, k, renormalize=False)
    y = _run_fused(lo, x, w1, w2, w1_s, w2_s, w, ids, apply_router_weight_on_input=True)
    # oracle: weight multiplies the integer sum of the first GEMM (before its scales), none afterwards
    xq, xs = OC.per_token_quant_int8(x)
    ref = torch.zeros(M, H, dtype=torch.bfloat16)
    for e in range(E):
        rows = torch.nonzero(ids.reshape(-1) == e).reshape(-1)
        if rows.numel():
            h = OC.per_token_matmul(xq[rows], w1[e], xs[rows], w1_s[e], torch.bfloat16, row_weight=w.reshape(-1)[rows])
            aq, a_s = OC.silu_mul_quant_int8(h)
            ref[rows] = OC.per_token_matmul(aq, w2[e], a_s, w2_s[e], torch.bfloat16)
    assert_out_close(y, ref, "router weight on input")


def test_fused_channel_rejects_bad_arguments(lo):
    E, k, M, H, I = 4, 2, 8, 256, 128
    w1, w2, w1_b, w2_b = synthetic.make_weights(E, H, I, seed=0)
    w1_s, w2_s = synthetic.make_channel_scales(E, H, I, seed=0)
    x, logits = synthetic.make_activations(M, H, E, seed=1)
    w, ids = O.route_topk_softmax(logits, k, renormalize=True)
    with pytest.raises(RuntimeError):        # block scales handed to the per-channel mode
        _run_fused(lo, x, w1, w2, w1_b, w2_b, w, ids)
    with pytest.raises(AssertionError):      # neither block nor channel-wise (reference: int8.py:289-290)
        lo.moe.fused_experts_impl_int8(x.to(DEV), w1.to(DEV), w2.to(DEV), w.to(DEV), ids.to(DEV), None,
                                       use_int8_w8a8=True, per_channel_quant=False, block_shape=None,
                                       w1_scale=w1_s.to(DEV), w2_scale=w2_s.to(DEV))
