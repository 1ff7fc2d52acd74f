"""CPU tests: the oracle against the golden fixtures and against the reference's own functions."""
import os

import pytest
import torch

from lightop_b200 import synthetic
from oracle import moe_block_int8 as O
from oracle import ref_extract


@pytest.fixture(scope="module")
def c0(golden_dir):
    cfg = synthetic.CONFIGS["c0_tiny"]
    w1, w2, w1_s, w2_s = synthetic.make_weights(cfg["E"], cfg["H"], cfg["I"], seed=0)
    x, logits = synthetic.make_activations(cfg["M"], cfg["H"], cfg["E"], seed=1)
    gold = torch.load(os.path.join(golden_dir, "c0_tiny.pt"))
    return cfg, (w1, w2, w1_s, w2_s), x, logits, gold


@pytest.fixture(scope="module")
def small(golden_dir):
    return torch.load(os.path.join(golden_dir, "small_cases.pt"))


def test_routing_matches_golden(c0):
    cfg, _, _, logits, gold = c0
    w, ids = O.route_topk_softmax(logits, cfg["topk"], renormalize=True)
    assert torch.equal(ids, gold["topk_ids"])
    assert torch.equal(w, gold["topk_weights"])


def test_group_quant_matches_golden(c0, small):
    _, _, x, _, gold = c0
    q, s = O.group_quant_int8(x, 128)
    assert torch.equal(q, gold["xq"]) and torch.equal(s, gold["xs"])
    q6, s6 = O.group_quant_int8(small["x6"], 128)
    assert torch.equal(q6, small["q6"]) and torch.equal(s6, small["s6"])
    qe, se = O.group_quant_int8(small["xe"], 128)
    assert torch.equal(qe, small["qe"]) and torch.equal(se, small["se"])


def test_group_quant_truncates_not_rounds():
    # 1.9 / (2.54 / 127) = 95.0 exactly representable? use a case with a .5+ fraction
    x = torch.zeros(1, 128, dtype=torch.bfloat16)
    x[0, 0] = 127.0
    x[0, 1] = 1.75     # scale = 1 -> 1.75 truncates to 1, round-to-nearest would give 2
    x[0, 2] = -1.75
    q, s = O.group_quant_int8(x, 128)
    assert s.item() == 1.0
    assert q[0, :3].tolist() == [127, 1, -1]


def test_block_matmul_matches_golden(c0):
    _, (w1, _, w1_s, _), _, _, gold = c0
    e = gold["gemm1_expert"]
    rows = gold["gemm1_rows"]
    out = O.block_int8_matmul(gold["xq"][rows], w1[e], gold["xs"][rows], w1_s[e], (128, 128), torch.bfloat16)
    assert torch.equal(out, gold["gemm1_out"])


def test_align_matches_golden(c0, small):
    cfg, _, _, _, gold = c0
    s, e, n = O.align_block_size(gold["topk_ids"], cfg["E"], 16)
    assert torch.equal(s, gold["sorted_ids"]) and torch.equal(e, gold["expert_ids"]) and torch.equal(n, gold["num_tokens_post_pad"])
    s, e, n = O.align_block_size(small["doc_ids"], 5, 4)
    # the example of the reference wrapper's docstring (moe_align_block_size.py:65-78)
    assert s.tolist() == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]
    assert torch.equal(s, small["doc_sorted"]) and torch.equal(e, small["doc_expert_ids"]) and torch.equal(n, small["doc_npost"])
    s, e, n = O.align_block_size(small["rag_ids"], 16, 16)
    assert torch.equal(s, small["rag_sorted"]) and torch.equal(e, small["rag_expert_ids"]) and torch.equal(n, small["rag_npost"])


def test_align_expert_map_drops_non_local():
    ids = torch.tensor([[0, 3], [2, 1], [3, 3]])
    emap = torch.tensor([0, -1, 1, -1], dtype=torch.int32)
    s, e, n = O.align_block_size(ids, 4, 2, expert_map=emap)
    assert n.item() == 4 and e.tolist() == [0, 1] and s.tolist() == [0, 6, 2, 6]


def test_composed_moe_matches_golden(c0):
    cfg, (w1, w2, w1_s, w2_s), x, _, gold = c0
    y = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, gold["topk_weights"], gold["topk_ids"])
    assert torch.equal(y, gold["y"])
    # magnitudes the tolerances are normalised by
    assert 100 < float(y.float().abs().mean()) < 400


def test_ep_build_m_indices_known_answer():
    # known answer of the reference test (test/test_native_categorized_moe_api.py:32-43)
    ids = torch.tensor([[0, 1], [1, 2], [0, -1]])
    m, counts = O.ep_build_m_indices(ids, 3, 2, rows=6)
    assert m.tolist() == [0, 0, 1, 1, 2, -1]
    assert counts.tolist() == [2, 2, 1]


def test_moe_sum_oracle():
    g = torch.Generator().manual_seed(0)
    a = torch.randn(5, 4, 64, generator=g).to(torch.bfloat16)
    assert torch.equal(O.moe_sum(a), a.float().sum(1).to(torch.bfloat16))


@pytest.mark.skipif(ref_extract.reference_root() is None, reason="no reference checkout on this machine")
def test_oracle_equals_reference_functions_on_fresh_inputs():
    quant, blockmm = ref_extract.reference_block_functions()
    align = ref_extract.reference_align_python()
    moe = ref_extract.reference_composed_moe()
    g = torch.Generator().manual_seed(11)
    for (E, k, M, H, I) in [(4, 2, 9, 128, 128), (8, 3, 33, 384, 256)]:
        w1, w2, w1_s, w2_s = synthetic.make_weights(E, H, I, seed=5)
        x, logits = synthetic.make_activations(M, H, E, seed=7)
        w, ids = O.route_topk_softmax(logits, k)
        y = O.fused_moe_block_int8(x, w1, w2, w1_s, w2_s, w, ids)
        yr = moe(x, w1, w2, w1_s, w2_s, w, ids.long(), k)
        assert torch.equal(y, yr)
        q, s = O.group_quant_int8(x, 128)
        qr, sr = quant(x, 128)
        assert torch.equal(q, qr) and torch.equal(s, sr)
        for bs in (1, 4, 16, 128):
            a = O.align_block_size(ids, E, bs)
            b = align(ids.reshape(-1).long(), E, bs)
            assert all(torch.equal(u, v.cpu()) for u, v in zip(a, b))


def test_quantisers_match_the_reference_triton_kernels(golden_dir):
    """The two restated quantisers against the outputs of the reference's own Triton kernels
    (layers/gemm/int8_utils.py:21-71, 74-193), run in Triton's interpreter by tests/golden/make_triton_golden.py."""
    from oracle import moe_channel_int8 as OC
    cases = torch.load(os.path.join(golden_dir, "triton_quant_cases.pt"))
    assert len(cases) >= 6
    for name, c in cases.items():
        g = torch.Generator().manual_seed(c["seed"])
        x = (torch.randn(c["rows"], c["cols"], generator=g) * 3.0).to(getattr(torch, c["dtype"]))
        q, s = O.group_quant_int8(x, 128)
        assert torch.equal(q, c["group_q"]) and torch.equal(s, c["group_s"]), name
        q, s = OC.per_token_quant_int8(x)
        assert torch.equal(q, c["token_q"]) and torch.equal(s, c["token_s"]), name
