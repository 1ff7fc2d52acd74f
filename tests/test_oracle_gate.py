"""CPU tests of the grouped sigmoid gate oracle and of the id post-processing restatement."""
import importlib.util
import math
import os

import pytest
import torch

from oracle import moe_gate as OG
from oracle import ref_extract


def _golden_module(golden_dir):
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(golden_dir, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def canon(w, i):
    order = torch.argsort(i, dim=-1)
    return torch.gather(w, 1, order), torch.gather(i, 1, order)


def test_gate_matches_golden(golden_dir):
    mg = _golden_module(golden_dir)
    for entry in torch.load(os.path.join(golden_dir, "gate_cases.pt")):
        case = entry["case"]
        x, b = mg.gate_inputs(case)
        w, i = OG.fused_gate(x, b, *case[2:7])
        wc, ic = canon(w, i)
        assert torch.equal(ic, entry["ids"]), case
        torch.testing.assert_close(wc, entry["weights"], rtol=1e-6, atol=1e-6)   # the reference test's bars


def test_gate_order_and_ties():
    # equal biases with saturated logits: every sigmoid is exactly 1, the lower ids win
    x = torch.full((2, 32), 40.0)
    b = torch.zeros(32)
    w, i = OG.fused_gate(x, b, 4, 2, 4, 0, 1.0)
    assert i.tolist() == [[0, 1, 2, 3]] * 2
    torch.testing.assert_close(w, torch.full((2, 4), 0.25))
    # descending order of the selection score, weights from the unbiased probabilities
    x = torch.zeros(1, 8)
    b = torch.tensor([0.0, 0.3, 0.1, 0.0, 0.0, 0.2, 0.0, 0.0])
    w, i = OG.fused_gate(x, b, 1, 1, 3, 0, 2.0)
    assert i.tolist() == [[1, 5, 2]]
    torch.testing.assert_close(w, torch.full((1, 3), 2.0 / 3))
    w2, _ = OG.fused_gate(x, b, 1, 1, 3, 0, 2.0, apply_routed_scaling_factor_on_output=False)
    torch.testing.assert_close(w2, torch.full((1, 3), 1.0 / 3))
    # a shared expert takes the last slot with id E and weight 1 / factor * factor
    w3, i3 = OG.fused_gate(x, b, 1, 1, 3, 1, 2.0)
    assert i3.tolist() == [[1, 5, 8]]
    torch.testing.assert_close(w3, torch.tensor([[1.0, 1.0, 1.0]]))


def test_group_limit():
    # two groups of 4; group 1 has the two best experts, group 0 the single best: top-2 sum picks group 1
    x = torch.zeros(1, 8)
    b = torch.tensor([0.9, 0.0, 0.0, 0.0, 0.6, 0.6, 0.0, 0.0])
    _, i = OG.fused_gate(x, b, 2, 1, 2, 0, 1.0)
    assert sorted(i.tolist()[0]) == [4, 5]


def test_ids_postprocess_known_answer():
    # test/test_native_categorized_moe_api.py:147-169
    ids = torch.tensor([[0, 2], [1, 3], [2, 0]], dtype=torch.int64)
    out = OG.topk_ids_postprocess(ids, torch.tensor([10, 11, 12, 13], dtype=torch.int32), torch.tensor([2], dtype=torch.int32))
    assert out.tolist() == [[10, 12], [11, 13], [-1, -1]]


@pytest.mark.skipif(ref_extract.reference_root() is None, reason="no reference checkout")
def test_against_reference_model():
    model = ref_extract.reference_gate_model()
    g = torch.Generator().manual_seed(5)
    for (M, E, G, tg, k, sh, rsf) in [(50, 256, 8, 4, 8, 0, 2.5), (9, 256, 8, 3, 10, 2, 1.5), (31, 128, 4, 4, 16, 0, 1.0)]:
        x, b = torch.randn(M, E, generator=g), torch.randn(E, generator=g)
        wr, ir = canon(*model(x, b, G, tg, k, sh, rsf))
        w, i = canon(*OG.fused_gate(x, b, G, tg, k, sh, rsf))
        assert torch.equal(i, ir)
        torch.testing.assert_close(w, wr, rtol=1e-6, atol=1e-6)


def test_gate_variants_match_golden(golden_dir):
    mg = _golden_module(golden_dir)
    fx = torch.load(os.path.join(golden_dir, "gate_variant_cases.pt"))
    for entry in fx["kimi"]:
        M, E, k, renorm, rsf, apply, seed = entry["case"]
        x, b = mg.variant_inputs(M, E, seed)
        wc, ic = canon(*OG.kimi_k2_gate(x, b, k, renorm, rsf, apply))
        assert torch.equal(ic, entry["ids"]), entry["case"]
        torch.testing.assert_close(wc, entry["weights"], rtol=1e-6, atol=1e-7)
    for entry in fx["ssp"]:
        M, E, k, sh, renorm, rsf, apply, seed = entry["case"]
        x, b = mg.variant_inputs(M, E, seed)
        w, i = OG.sqrtsoftplus_gate(x, b, k, sh, renorm, rsf, apply)
        assert torch.equal(i, entry["ids"]), entry["case"]          # this model returns the descending order
        torch.testing.assert_close(w, entry["weights"], rtol=1e-6, atol=1e-7)


def test_gate_variants_known_answers():
    # Kimi-K2: without renormalisation the factor is never applied (test/ci_tests/test_kimi_k2_moe_fused_gate.py:37-41)
    x = torch.zeros(1, 8)
    b = torch.tensor([0.0, 0.3, 0.1, 0.0, 0.0, 0.2, 0.0, 0.0])
    w, i = OG.kimi_k2_gate(x, b, 3, renormalize=False, routed_scaling_factor=4.0, apply_routed_scaling_factor_on_output=True)
    assert i.tolist() == [[1, 5, 2]]
    torch.testing.assert_close(w, torch.full((1, 3), 0.5))
    w, _ = OG.kimi_k2_gate(x, b, 3, True, 4.0, True)
    torch.testing.assert_close(w, torch.full((1, 3), 4.0 / 3))
    # sqrt-softplus: score of logit 0 is sqrt(ln 2); the shared slot weighs routed sum / factor
    w, i = OG.sqrtsoftplus_gate(x, b, 4, 1, True, 2.0, False)
    assert i.tolist() == [[1, 5, 2, 8]]
    torch.testing.assert_close(w, torch.tensor([[1 / 3, 1 / 3, 1 / 3, 0.5]]))
    w, _ = OG.sqrtsoftplus_gate(x, b, 4, 1, False, 2.0, True)
    s = math.sqrt(math.log(2.0))
    torch.testing.assert_close(w, torch.tensor([[2 * s, 2 * s, 2 * s, 3 * s]]))


@pytest.mark.skipif(ref_extract.reference_root() is None, reason="no reference checkout")
def test_variants_against_reference_models():
    kimi, ssp = ref_extract.reference_gate_variant_models()
    g = torch.Generator().manual_seed(6)
    for (M, E, k, renorm, rsf, apply) in [(64, 384, 8, True, 2.0, True), (5, 384, 8, False, 2.0, True), (40, 128, 6, True, 1.0, False)]:
        x, b = torch.randn(M, E, generator=g), torch.randn(E, generator=g)
        wr, ir = canon(*kimi(None, x, b, k, renorm, rsf, apply))
        w, i = canon(*OG.kimi_k2_gate(x, b, k, renorm, rsf, apply))
        assert torch.equal(i, ir)
        torch.testing.assert_close(w, wr.float(), rtol=1e-6, atol=1e-7)
    for (M, E, k, sh, renorm, rsf, apply) in [(16, 256, 6, 0, True, 2.5, False), (512, 256, 6, 1, True, 2.5, True),
                                              (7, 256, 8, 2, False, 2.5, False)]:
        x, b = torch.randn(M, E, generator=g), torch.randn(E, generator=g)
        wr, ir = ssp(x, b, k, sh, renorm, rsf, apply)
        w, i = OG.sqrtsoftplus_gate(x, b, k, sh, renorm, rsf, apply)
        assert torch.equal(i, ir)
        torch.testing.assert_close(w, wr, rtol=1e-6, atol=1e-7)
