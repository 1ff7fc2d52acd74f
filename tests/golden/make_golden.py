"""Generate the golden fixtures of tests/golden/ from the reference's own torch functions.

Run where a reference checkout is available (``$LIGHTOP_REF``, see oracle/ref_extract.py):
    python tests/golden/make_golden.py            (all fixtures)
    python tests/golden/make_golden.py channel    (only channel_cases.pt)
    python tests/golden/make_golden.py gate       (only gate_cases.pt and gate_variant_cases.pt)
The outputs are produced by the reference code itself (loaded by oracle/ref_extract.py),
not by the restatement in oracle/moe_block_int8.py; the tests then hold both the oracle
and the CUDA kernels to these files.  Inputs are not stored: they are regenerated from
their seeds by lightop_b200.synthetic.
"""
from __future__ import annotations

import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from lightop_b200 import synthetic  # noqa: E402
from oracle import ref_extract  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    quant, blockmm = ref_extract.reference_block_functions()
    align = ref_extract.reference_align_python()
    moe = ref_extract.reference_composed_moe()

    # --- config 0: the reference-runnable tiny MoE -------------------------------------
    cfg = synthetic.CONFIGS["c0_tiny"]
    w1, w2, w1_s, w2_s = synthetic.make_weights(cfg["E"], cfg["H"], cfg["I"], seed=0)
    x, logits = synthetic.make_activations(cfg["M"], cfg["H"], cfg["E"], seed=1)
    # routing the way the reference's tests do (test_native_categorized_moe_api.py:188-190,
    # fuse_moegemm.py:449-450)
    w, ids = torch.topk(torch.softmax(logits.float(), dim=-1), cfg["topk"])
    w = w / w.sum(dim=-1, keepdim=True)
    y = moe(x, w1, w2, w1_s, w2_s, w, ids, cfg["topk"])
    xq, xs = quant(x, 128)
    sorted_ids, expert_ids, npost = align(ids.reshape(-1), cfg["E"], 16)
    # one expert's first GEMM, to pin the block matmul alone
    e0 = int(ids.reshape(-1)[0])
    rows = torch.nonzero(ids.reshape(-1) == e0).reshape(-1) // cfg["topk"]
    h0 = blockmm(xq[rows], w1[e0], xs[rows], w1_s[e0], [128, 128], torch.bfloat16)
    torch.save(dict(topk_weights=w, topk_ids=ids.to(torch.int32), y=y, xq=xq, xs=xs,
                    sorted_ids=sorted_ids, expert_ids=expert_ids, num_tokens_post_pad=npost,
                    gemm1_expert=e0, gemm1_rows=rows, gemm1_out=h0),
               os.path.join(HERE, "c0_tiny.pt"))

    # --- the reference's own pinned small cases ----------------------------------------
    # group quant, [3,256] bf16, seed 6, group 128 (test/test_quant_per_token_quant_int8.py:59-72)
    torch.manual_seed(6)
    xq6 = torch.randn(3, 256).to(torch.bfloat16)
    q6, s6 = quant(xq6, 128)
    # an all-zero group and a saturating group
    xe = torch.zeros(2, 256, dtype=torch.bfloat16)
    xe[1, :128] = torch.linspace(-3, 3, 128).to(torch.bfloat16)
    xe[1, 128:] = 1e-12
    qe, se = quant(xe, 128)
    # alignment example of the wrapper's docstring (moe_align_block_size.py:65-78), 1-based ids
    doc_ids = torch.tensor([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]])
    d_sorted, d_eids, d_npost = align(doc_ids.reshape(-1), 5, 4)
    # a ragged alignment case with empty experts
    g = torch.Generator().manual_seed(3)
    rag = torch.randint(0, 16, (37 * 3,), generator=g)
    rag[rag == 5] = 6
    r_sorted, r_eids, r_npost = align(rag, 16, 16)
    torch.save(dict(x6=xq6, q6=q6, s6=s6, xe=xe, qe=qe, se=se,
                    doc_ids=doc_ids, doc_sorted=d_sorted, doc_expert_ids=d_eids, doc_npost=d_npost,
                    rag_ids=rag, rag_sorted=r_sorted, rag_expert_ids=r_eids, rag_npost=r_npost),
               os.path.join(HERE, "small_cases.pt"))
    print("wrote", os.listdir(HERE))


def main_channel() -> None:
    """Fixtures of the per-channel W8A8 mode (tests/golden/channel_cases.pt)."""
    from oracle import moe_channel_int8 as och
    mm, moe = ref_extract.reference_channel_functions(och.per_token_quant_int8)
    cfg = synthetic.CONFIGS["c0_tiny"]
    w1, w2, _, _ = synthetic.make_weights(cfg["E"], cfg["H"], cfg["I"], seed=0)
    w1_s, w2_s = synthetic.make_channel_scales(cfg["E"], cfg["H"], cfg["I"], seed=0)
    x, logits = synthetic.make_activations(cfg["M"], cfg["H"], cfg["E"], seed=1)
    w, ids = torch.topk(torch.softmax(logits.float(), dim=-1), cfg["topk"])
    w = w / w.sum(dim=-1, keepdim=True)
    # the reference's matmul alone, on the rows of one expert (inputs from the restated quantiser)
    xq, xs = och.per_token_quant_int8(x)
    e0 = int(ids.reshape(-1)[0])
    rows = torch.nonzero(ids.reshape(-1) == e0).reshape(-1) // cfg["topk"]
    h0 = mm(xq[rows], w1[e0], xs[rows], w1_s[e0], output_dtype=torch.bfloat16)
    # the reference's composed per-channel layer
    y = moe(x, w1, w2, w1_s, w2_s, w, ids, cfg["topk"])
    torch.save(dict(topk_weights=w, topk_ids=ids.to(torch.int32), gemm1_expert=e0, gemm1_rows=rows,
                    gemm1_out=h0, y=y),
               os.path.join(HERE, "channel_cases.pt"))
    print("wrote channel_cases.pt")


GATE_CASES = [  # (tokens, experts, groups, topk_group, topk, shared, routed_scaling_factor, seed)
    (64, 256, 8, 4, 8, 0, 2.5, 21),       # DeepSeek-V3 layout
    (33, 256, 8, 4, 9, 1, 2.5, 22),       # with one fused shared expert
    (16, 128, 4, 2, 6, 0, 1.0, 23),
    (20, 384, 1, 1, 8, 0, 2.827, 24),     # single group
    (7, 128, 1, 1, 8, 1, 16.0, 25),
]


def gate_inputs(case):
    M, E, _, _, _, _, _, seed = case
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, E, generator=g), torch.randn(E, generator=g)


def main_gate() -> None:
    """Fixtures of the grouped sigmoid gate (tests/golden/gate_cases.pt): outputs of the reference's torch model,
    canonicalised by expert id as its own test does (test/ci_tests/test_fused_moe_gate.py:160-167)."""
    model = ref_extract.reference_gate_model()
    out = []
    for case in GATE_CASES:
        x, b = gate_inputs(case)
        w, i = model(x, b, *case[2:7])
        order = torch.argsort(i, dim=-1)
        out.append(dict(case=case, ids=torch.gather(i, 1, order), weights=torch.gather(w, 1, order)))
    torch.save(out, os.path.join(HERE, "gate_cases.pt"))
    print("wrote gate_cases.pt")


KIMI_CASES = [  # (tokens, experts, topk, renormalize, factor, apply on output, seed)
    (48, 384, 8, True, 2.0, True, 41), (17, 384, 8, True, 2.0, False, 42), (9, 256, 6, False, 3.0, True, 43)]
SSP_CASES = [   # (tokens, experts, topk, shared, renormalize, factor, apply on output, seed)
    (16, 256, 6, 0, True, 2.5, False, 51), (33, 256, 6, 1, True, 2.5, False, 52), (20, 256, 6, 1, True, 2.5, True, 53),
    (11, 128, 7, 2, False, 1.5, True, 54)]


def variant_inputs(M, E, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, E, generator=g), torch.randn(E, generator=g)


def main_gate_variants() -> None:
    """Fixtures of the Kimi-K2 and sqrt-softplus gates (tests/golden/gate_variant_cases.pt), canonicalised by id."""
    kimi, ssp = ref_extract.reference_gate_variant_models()
    out = {"kimi": [], "ssp": []}
    for case in KIMI_CASES:
        x, b = variant_inputs(case[0], case[1], case[-1])
        w, i = kimi(None, x, b, case[2], case[3], case[4], case[5])
        order = torch.argsort(i, dim=-1)
        out["kimi"].append(dict(case=case, ids=torch.gather(i, 1, order), weights=torch.gather(w, 1, order).float()))
    for case in SSP_CASES:
        x, b = variant_inputs(case[0], case[1], case[-1])
        w, i = ssp(x, b, case[2], case[3], case[4], case[5], case[6])
        out["ssp"].append(dict(case=case, ids=i, weights=w))        # this model's order is part of its contract
    torch.save(out, os.path.join(HERE, "gate_variant_cases.pt"))
    print("wrote gate_variant_cases.pt")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "channel":
        main_channel()
    elif len(sys.argv) > 1 and sys.argv[1] == "gate":
        main_gate()
        main_gate_variants()
    else:
        main()
        main_channel()
        main_gate()
        main_gate_variants()
