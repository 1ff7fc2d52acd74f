"""GPU parity tests of the grouped sigmoid gate and the id post-processing against the oracle
and the fixture made from the reference's torch model."""
import importlib.util
import os

import pytest
import torch

from oracle import moe_gate as OG

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def lo():
    import lightop_b200
    return lightop_b200


def canon(w, i):
    order = torch.argsort(i, dim=-1)
    return torch.gather(w, 1, order), torch.gather(i, 1, order)


def _ids_match(ids, ref_ids, x, bias):
    """Exact, except that a row may differ where the oracle's own selection scores are within an ulp or two
    of each other (device expf vs torch exp)."""
    if torch.equal(ids, ref_ids):
        return True
    s = torch.sigmoid(x.float()) + bias.float().unsqueeze(0)
    E = s.shape[1]
    for r in (ids != ref_ids).any(dim=1).nonzero().reshape(-1).tolist():
        a = set(ids[r].tolist()) - set(ref_ids[r].tolist())
        b = set(ref_ids[r].tolist()) - set(ids[r].tolist())
        if any(e >= E for e in a | b) or len(a) != len(b):
            return False
        sa = sorted(float(s[r, e]) for e in a)
        sb = sorted(float(s[r, e]) for e in b)
        if any(abs(u - v) > 4e-7 * max(1.0, abs(v)) for u, v in zip(sa, sb)):
            return False
    return True


def test_gate_against_golden(lo, golden_dir):
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(golden_dir, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    for entry in torch.load(os.path.join(golden_dir, "gate_cases.pt")):
        case = entry["case"]
        x, b = mg.gate_inputs(case)
        w, i = lo.moe.moe_fused_gate(x.to(DEV), b.to(DEV), *case[2:7])
        assert w.dtype == torch.float32 and i.dtype == torch.int32
        wc, ic = canon(w.cpu(), i.cpu())
        assert torch.equal(ic, entry["ids"]), case
        torch.testing.assert_close(wc, entry["weights"], rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("M,E,G,tg,k,sh,rsf", [
    (4096, 256, 8, 4, 8, 0, 2.5), (1, 256, 8, 4, 8, 0, 2.5), (300, 256, 8, 4, 9, 1, 2.5), (77, 128, 4, 2, 8, 0, 1.0),
    (65, 384, 16, 4, 8, 0, 1.0), (129, 512, 1, 1, 22, 0, 2.827), (40, 254, 2, 2, 14, 2, 1.5), (33, 896, 1, 1, 16, 0, 1.0),
    (10, 64, 2, 1, 6, 0, 0.0), (12, 1024, 32, 8, 32, 0, 1.0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_vs_oracle(lo, M, E, G, tg, k, sh, rsf, dtype):
    g = torch.Generator().manual_seed(M + E)
    x = torch.randn(M, E, generator=g).to(dtype)
    b = torch.randn(E, generator=g)
    w, i = lo.moe.moe_fused_gate(x.to(DEV), b.to(DEV), G, tg, k, sh, rsf)
    w_ref, i_ref = OG.fused_gate(x, b, G, tg, k, sh, rsf)
    w, i = w.cpu(), i.cpu()
    assert _ids_match(i, i_ref, x, b)
    same = (i == i_ref).all(dim=1)
    assert float(same.float().mean()) >= 0.99
    torch.testing.assert_close(w[same], w_ref[same], rtol=2e-5, atol=2e-6)
    # descending selection order within the routed slots is part of the contract
    assert torch.equal(i[same], i_ref[same])


def test_gate_options_and_ties(lo):
    # saturated logits and equal biases: all scores equal, the lower ids win, in order
    x = torch.full((3, 256), 40.0, device=DEV)
    b = torch.zeros(256, device=DEV)
    w, i = lo.moe.moe_fused_gate(x, b, 8, 4, 8, 0, 2.5)
    assert i.cpu().tolist() == [list(range(8))] * 3
    torch.testing.assert_close(w.cpu(), torch.full((3, 8), 2.5 / 8))
    # scale not applied on the output; int64 indices; bf16 bias
    g = torch.Generator().manual_seed(3)
    x = torch.randn(50, 256, generator=g)
    b = torch.randn(256, generator=g)
    w1, i1 = lo.moe.moe_fused_gate(x.to(DEV), b.to(DEV), 8, 4, 8, 0, 2.5, False, True)
    w_ref, i_ref = OG.fused_gate(x, b, 8, 4, 8, 0, 2.5, apply_routed_scaling_factor_on_output=False)
    assert i1.dtype == torch.int64 and torch.equal(i1.cpu().to(torch.int32), i_ref)
    torch.testing.assert_close(w1.cpu(), w_ref, rtol=2e-5, atol=2e-6)
    w2, i2 = lo.moe.moe_fused_gate(x.to(DEV), b.to(torch.bfloat16).to(DEV), 8, 4, 8, 0, 2.5)
    _, i2_ref = OG.fused_gate(x, b.to(torch.bfloat16), 8, 4, 8, 0, 2.5)
    assert _ids_match(i2.cpu(), i2_ref, x, b.to(torch.bfloat16))
    # empty batch
    w0, i0 = lo.moe.moe_fused_gate(torch.empty(0, 256, device=DEV), b.to(DEV), 8, 4, 8, 0, 2.5)
    assert w0.shape == (0, 8) and i0.shape == (0, 8)


def test_gate_rejects_bad_configurations(lo):
    from lightop_b200._lib import LightopError
    x = torch.zeros(4, 256, device=DEV)
    b = torch.zeros(256, device=DEV)
    for args in [(7, 4, 8, 0, 1.0),        # 256 is not divisible by 7 groups
                 (8, 9, 8, 0, 1.0),        # more groups kept than exist
                 (8, 1, 40, 0, 1.0),       # more experts than one group holds
                 (8, 4, 8, 8, 1.0)]:       # only shared slots
        with pytest.raises(LightopError):
            lo.moe.moe_fused_gate(x, b, *args)
    with pytest.raises(RuntimeError):
        lo.moe.moe_fused_gate(x, b[:100], 8, 4, 8, 0, 1.0)


def test_gate_feeds_the_expert_layer(lo):
    # the gate's ids and weights are what the fused layer consumes (ids int32, weights fp32)
    from lightop_b200 import synthetic
    from oracle import moe_block_int8 as O
    from util import assert_out_close
    E, k, M, H, I = 16, 4, 40, 256, 128
    w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=8)
    x, logits = synthetic.make_activations(M, H, E, seed=9)
    bias = torch.randn(E, generator=torch.Generator().manual_seed(1)) * 0.1
    w, ids = lo.moe.moe_fused_gate(logits.to(DEV), bias.to(DEV), 4, 2, k, 0, 1.0)
    y = lo.moe.fused_experts_impl_int8(x.to(DEV), w1.to(DEV), w2.to(DEV), w, ids, None, use_int8_w8a8=True,
                                       block_shape=[128, 128], w1_scale=w1_s.to(DEV), w2_scale=w2_s.to(DEV))
    w_ref, ids_ref = OG.fused_gate(logits, bias, 4, 2, k, 0, 1.0)
    assert torch.equal(ids.cpu(), ids_ref)
    assert_out_close(y, O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w_ref, ids_ref), "gate -> block-INT8 layer")


def test_topk_ids_postprocess(lo):
    # known answer of the reference (test/test_native_categorized_moe_api.py:147-169)
    ids = torch.tensor([[0, 2], [1, 3], [2, 0]], device=DEV, dtype=torch.int64)
    lo.moe.topk_ids_postprocess(ids, torch.tensor([10, 11, 12, 13], device=DEV, dtype=torch.int32),
                                torch.tensor([2], device=DEV, dtype=torch.int32))
    assert ids.cpu().tolist() == [[10, 12], [11, 13], [-1, -1]]
    # random case, int32 ids, int64 map, ids outside the map, either step alone
    g = torch.Generator().manual_seed(0)
    base = torch.randint(-2, 40, (100, 8), generator=g, dtype=torch.int32)
    lmap = torch.randperm(32, generator=g)
    for m, n in ((lmap, None), (None, torch.tensor([37])), (lmap, torch.tensor([0])), (lmap.to(torch.int32), torch.tensor([100]))):
        t = base.clone().to(DEV)
        lo.moe.topk_ids_postprocess(t, m.to(DEV) if m is not None else None, n.to(DEV) if n is not None else None)
        assert torch.equal(t.cpu(), OG.topk_ids_postprocess(base, m, n))
    lo.moe.topk_ids_postprocess(torch.empty(0, 8, dtype=torch.int32, device=DEV))


def _variant_ids_match(ids, ref_ids, score, bias):
    """Exact, except rows where the oracle's own selection scores tie within a few ulps (device vs torch math)."""
    if torch.equal(ids, ref_ids):
        return True
    s = score + bias.float().unsqueeze(0)
    E = s.shape[1]
    for r in (ids != ref_ids).any(dim=1).nonzero().reshape(-1).tolist():
        a = set(ids[r].tolist()) - set(ref_ids[r].tolist())
        b = set(ref_ids[r].tolist()) - set(ids[r].tolist())
        if any(e >= E for e in a | b) or len(a) != len(b):
            return False
        sa = sorted(float(s[r, e]) for e in a)
        sb = sorted(float(s[r, e]) for e in b)
        if any(abs(u - v) > 4e-7 * max(1.0, abs(v)) for u, v in zip(sa, sb)):
            return False
        if not a:                   # same set in another order: only neighbours with tied scores may swap
            sr = s[r, ref_ids[r].long().clamp(max=E - 1)]
            so = s[r, ids[r].long().clamp(max=E - 1)]
            if float((sr - so).abs().max()) > 4e-7 * max(1.0, float(sr.abs().max())):
                return False
    return True


def test_gate_variants_against_golden(lo, golden_dir):
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(golden_dir, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    fx = torch.load(os.path.join(golden_dir, "gate_variant_cases.pt"))
    for entry in fx["kimi"]:
        M, E, k, renorm, rsf, apply, seed = entry["case"]
        x, b = mg.variant_inputs(M, E, seed)
        w, i = lo.moe.kimi_k2_moe_fused_gate(x.to(DEV), b.to(DEV), k, renorm, rsf, apply)
        assert w.dtype == torch.float32 and i.dtype == torch.int32
        wc, ic = canon(w.cpu(), i.cpu())
        assert torch.equal(ic, entry["ids"]), entry["case"]
        torch.testing.assert_close(wc, entry["weights"], rtol=1e-5, atol=1e-6)
    for entry in fx["ssp"]:
        M, E, k, sh, renorm, rsf, apply, seed = entry["case"]
        x, b = mg.variant_inputs(M, E, seed)
        for fn in (lo.moe.moe_fused_gate_sqrtsoftplus, lo.moe.moe_fused_gate_sqrtsoftplus_v41_hcu):
            w, i = fn(x.to(DEV), b.to(DEV), k, sh, renorm, rsf, apply)
            assert torch.equal(i.cpu(), entry["ids"]), entry["case"]        # order included
            torch.testing.assert_close(w.cpu(), entry["weights"], rtol=1e-5, atol=1e-5)   # the reference test's bars


@pytest.mark.parametrize("M", [1, 16, 256, 513, 4096])
@pytest.mark.parametrize("E,k", [(384, 8), (256, 6)])
@pytest.mark.parametrize("renorm,apply", [(True, True), (True, False), (False, True)])
def test_kimi_gate_vs_oracle(lo, M, E, k, renorm, apply):
    g = torch.Generator().manual_seed(M * 3 + E + k)
    x, b = torch.randn(M, E, generator=g), torch.randn(E, generator=g)
    w, i = lo.moe.kimi_k2_moe_fused_gate(x.to(DEV), b.to(DEV), k, renorm, 2.5, apply)
    w_ref, i_ref = OG.kimi_k2_gate(x, b, k, renorm, 2.5, apply)
    w, i = w.cpu(), i.cpu()
    assert _variant_ids_match(i, i_ref, torch.sigmoid(x), b)
    same = (i == i_ref).all(dim=1)
    assert float(same.float().mean()) >= 0.99
    torch.testing.assert_close(w[same], w_ref[same], rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("M", [1, 16, 256, 513, 4096])
@pytest.mark.parametrize("k,sh", [(6, 0), (6, 1), (8, 0), (9, 2)])
@pytest.mark.parametrize("renorm,apply", [(True, False), (True, True), (False, False)])
def test_sqrtsoftplus_gate_vs_oracle(lo, M, k, sh, renorm, apply):
    # shapes and options of test/ci_tests/test_moe_fused_gate_sqrtsoftplus.py:89-99 and more
    g = torch.Generator().manual_seed(M * 5 + k + sh)
    x, b = torch.randn(M, 256, generator=g), torch.randn(256, generator=g)
    w, i = lo.moe.moe_fused_gate_sqrtsoftplus(x.to(DEV), b.to(DEV), k, sh, renorm, 2.5, apply)
    w_ref, i_ref = OG.sqrtsoftplus_gate(x, b, k, sh, renorm, 2.5, apply)
    w, i = w.cpu(), i.cpu()
    assert _variant_ids_match(i, i_ref, torch.sqrt(torch.log1p(torch.exp(x))), b)
    same = (i == i_ref).all(dim=1)
    assert float(same.float().mean()) >= 0.99
    torch.testing.assert_close(w[same], w_ref[same], rtol=1e-5, atol=1e-5)


def test_sqrtsoftplus_gate_padded_forms(lo):
    g = torch.Generator().manual_seed(77)
    x, b = torch.randn(40, 256, generator=g), torch.randn(256, generator=g)
    w_ref, i_ref = OG.sqrtsoftplus_gate(x, b, 7, 1, True, 2.5, True)
    for fn, pad in ((lo.moe.moe_fused_gate_sqrtsoftplus_v41_hcu_fused, 0), (lo.moe.moe_fused_gate_sqrtsoftplus_v41_hcu_deepep, -1)):
        for count in (torch.tensor([25], dtype=torch.int32), torch.tensor([0], dtype=torch.int64),
                      torch.tensor([40], dtype=torch.int64), torch.tensor([1000], dtype=torch.int32), None):
            w, i = fn(x.to(DEV), b.to(DEV), 7, 1, True, 2.5, True, count.to(DEV) if count is not None else None)
            assert i.dtype == torch.int64
            wr, ir = OG.mask_padded_rows(w_ref, i_ref, int(count) if count is not None else 40, pad)
            assert torch.equal(i.cpu(), ir)
            torch.testing.assert_close(w.cpu(), wr, rtol=1e-5, atol=1e-5)
    # the count lives on the device: a captured graph follows its changes
    count = torch.tensor([10], dtype=torch.int64, device=DEV)
    xd, bd = x.to(DEV), b.to(DEV)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        lo.moe.moe_fused_gate_sqrtsoftplus_v41_hcu_deepep(xd, bd, 7, 1, True, 2.5, True, count)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            w, i = lo.moe.moe_fused_gate_sqrtsoftplus_v41_hcu_deepep(xd, bd, 7, 1, True, 2.5, True, count)
    for n in (10, 33):
        count.fill_(n)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(i.cpu(), OG.mask_padded_rows(w_ref, i_ref, n, -1)[1])


def test_sqrtsoftplus_gate_per_token_bias_and_large_logits(lo):
    g = torch.Generator().manual_seed(78)
    x, b2 = torch.randn(37, 256, generator=g), torch.randn(37, 256, generator=g)
    for fn, safe in ((lo.moe.moe_fused_gate_sqrtsoftplus, False), (lo.moe.moe_fused_gate_sqrtsoftplus_v41_hcu, True)):
        w, i = fn(x.to(DEV), b2.to(DEV), 8, 1, True, 2.5, False)
        w_ref, i_ref = OG.sqrtsoftplus_gate(x, b2, 8, 1, True, 2.5, False, softplus_linear_above_20=safe)
        assert torch.equal(i.cpu(), i_ref)
        torch.testing.assert_close(w.cpu(), w_ref, rtol=1e-5, atol=1e-5)
    # logits beyond the overflow of exp: the second form keeps finite scores sqrt(x)
    xl = torch.randn(9, 256, generator=g) * 60
    w, i = lo.moe.moe_fused_gate_sqrtsoftplus_v41_hcu(xl.to(DEV), b2[0].contiguous().to(DEV), 6, 0, True, 1.0, False)
    w_ref, i_ref = OG.sqrtsoftplus_gate(xl, b2[0], 6, 0, True, 1.0, False, softplus_linear_above_20=True)
    assert torch.isfinite(w).all() and torch.equal(i.cpu(), i_ref)
    torch.testing.assert_close(w.cpu(), w_ref, rtol=1e-5, atol=1e-5)
    with pytest.raises(RuntimeError):
        lo.moe.moe_fused_gate_sqrtsoftplus(x.to(DEV), b2[:5].contiguous().to(DEV), 8)          # 2D bias of the wrong height
    with pytest.raises(RuntimeError):
        lo.moe.moe_fused_gate_sqrtsoftplus(x.to(DEV), b2[0].contiguous().to(DEV), 8, 0, True, 0.0)   # factor must be > 0


def test_gate_variants_edge_cases(lo):
    from lightop_b200._lib import LightopError
    b = torch.zeros(256, device=DEV)
    # logits so negative that every sqrt-softplus score is 0: no division by the zero sum
    w, i = lo.moe.moe_fused_gate_sqrtsoftplus(torch.full((2, 256), -200.0, device=DEV), b, 6, 0, True, 2.5, False)
    assert torch.equal(w.cpu(), torch.zeros(2, 6)) and i.cpu().tolist() == [list(range(6))] * 2
    # Kimi-K2 with every sigmoid 0: the 1e-20 keeps the quotient finite
    w, _ = lo.moe.kimi_k2_moe_fused_gate(torch.full((2, 384), -200.0, device=DEV), torch.zeros(384, device=DEV), 8)
    assert torch.equal(w.cpu(), torch.zeros(2, 8))
    w0, i0 = lo.moe.kimi_k2_moe_fused_gate(torch.empty(0, 384, device=DEV), torch.zeros(384, device=DEV), 8)
    assert w0.shape == (0, 8) and i0.shape == (0, 8)
    with pytest.raises(LightopError):
        lo.moe.moe_fused_gate_sqrtsoftplus(torch.zeros(2, 256, device=DEV), b, 6, 6)       # only shared slots
    with pytest.raises(LightopError):
        lo.moe.kimi_k2_moe_fused_gate(torch.zeros(2, 384, device=DEV), torch.zeros(384, device=DEV), 40)
    with pytest.raises(RuntimeError):
        lo.moe.moe_fused_gate_sqrtsoftplus_v41_hcu_fused(torch.zeros(2, 256, device=DEV), b, 6, 0, True, 1.0, False,
                                                         torch.zeros(1, device=DEV))      # a float count
