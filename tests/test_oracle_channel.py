"""CPU tests of the per-channel W8A8 oracle: against the fixture made from the reference's own
torch functions, against those functions when a reference checkout is present, and known answers
of the two restated quantisers."""
import os

import pytest
import torch

from lightop_b200 import synthetic
from oracle import moe_channel_int8 as OC
from oracle import ref_extract
from util import assert_out_close


@pytest.fixture(scope="module")
def c0(golden_dir):
    cfg = synthetic.CONFIGS["c0_tiny"]
    w1, w2, _, _ = synthetic.make_weights(cfg["E"], cfg["H"], cfg["I"], seed=0)
    w1_s, w2_s = synthetic.make_channel_scales(cfg["E"], cfg["H"], cfg["I"], seed=0)
    x, _ = synthetic.make_activations(cfg["M"], cfg["H"], cfg["E"], seed=1)
    gold = torch.load(os.path.join(golden_dir, "channel_cases.pt"))
    return cfg, (w1, w2, w1_s, w2_s), x, gold


def test_per_token_quant_known_answers():
    x = torch.zeros(3, 16, dtype=torch.bfloat16)
    x[0, 0] = 127.0
    x[0, 1] = 1.5      # scale 1: 1.5 rounds to 2 (half to even), 2.5 to 2, -0.5 to 0
    x[0, 2] = 2.5
    x[0, 3] = -0.5
    x[0, 4] = 1.75     # rounds to 2 where the group quantiser of the block mode truncates to 1
    x[2, :] = 3.0
    q, s = OC.per_token_quant_int8(x)
    assert s.shape == (3, 1) and s.dtype == torch.float32
    assert s[0].item() == 1.0
    assert q[0, :5].tolist() == [127, 2, 2, 0, 2]
    # a row of zeros: absmax clamps to 1e-10, q stays 0
    assert q[1].abs().max().item() == 0
    assert s[1].item() == pytest.approx(1e-10 / 127, rel=1e-6)
    assert q[2].tolist() == [127] * 16 and s[2].item() == pytest.approx(3.0 / 127)


def test_silu_mul_quant_known_answers():
    inter = torch.zeros(2, 32, dtype=torch.bfloat16)
    inter[0, :16] = 20.0          # silu(20) = 20 in bf16
    inter[0, 16:] = torch.linspace(-1, 1, 16).to(torch.bfloat16)
    q, s = OC.silu_mul_quant_int8(inter)
    act = (torch.tensor(20.0) * inter[0, 16:].float()).to(torch.bfloat16).float()
    assert s[0].item() == pytest.approx(act.abs().max().item() / 127)
    assert torch.equal(q[0], torch.round(act * (127.0 / act.abs().max())).to(torch.int8))
    # a row of zeros: scale 0 and q 0, no NaN
    assert s[1].item() == 0.0 and q[1].abs().max().item() == 0


def test_per_token_matmul_matches_golden(c0):
    _, (w1, _, w1_s, _), x, gold = c0
    xq, xs = OC.per_token_quant_int8(x)
    e, rows = gold["gemm1_expert"], gold["gemm1_rows"]
    out = OC.per_token_matmul(xq[rows], w1[e], xs[rows], w1_s[e], torch.bfloat16)
    assert torch.equal(out, gold["gemm1_out"])


def test_composed_layer_close_to_golden(c0):
    # The reference's composed torch model rounds to bf16 before the routed weight and sums in
    # bf16; the kernel order restated by the oracle weights in fp32 and sums in fp32: equal within
    # the layer tolerance, not bit for bit.
    _, (w1, w2, w1_s, w2_s), x, gold = c0
    y = OC.fused_moe_channel_int8(x, w1, w2, w1_s, w2_s, gold["topk_weights"], gold["topk_ids"])
    assert_out_close(y, gold["y"], "per-channel oracle vs reference model")


def test_expert_map_and_shared_output(c0):
    cfg, (w1, w2, w1_s, w2_s), x, gold = c0
    E = cfg["E"]
    half = E // 2
    emap = torch.full((E,), -1, dtype=torch.int32)
    emap[:half] = torch.arange(half, dtype=torch.int32)
    shared = torch.ones_like(x)
    y0 = OC.fused_moe_channel_int8(x, w1[:half], w2[:half], w1_s[:half], w2_s[:half], gold["topk_weights"],
                                   gold["topk_ids"], expert_map=emap)
    emap1 = torch.full((E,), -1, dtype=torch.int32)
    emap1[half:] = torch.arange(E - half, dtype=torch.int32)
    y1 = OC.fused_moe_channel_int8(x, w1[half:], w2[half:], w1_s[half:], w2_s[half:], gold["topk_weights"],
                                   gold["topk_ids"], expert_map=emap1)
    y = OC.fused_moe_channel_int8(x, w1, w2, w1_s, w2_s, gold["topk_weights"], gold["topk_ids"])
    assert_out_close(y0.float() + y1.float(), y, "two expert halves add up")
    ys = OC.fused_moe_channel_int8(x, w1, w2, w1_s, w2_s, gold["topk_weights"], gold["topk_ids"],
                                   routed_scaling_factor=0.5, shared_output=shared)
    assert_out_close(ys, 0.5 * y.float() + 1.0, "scaling factor and shared output")


@pytest.mark.skipif(ref_extract.reference_root() is None, reason="no reference checkout")
def test_against_reference_functions(c0):
    _, (w1, w2, w1_s, w2_s), x, gold = c0
    mm, moe = ref_extract.reference_channel_functions(OC.per_token_quant_int8)
    g = torch.Generator().manual_seed(11)
    A = torch.randint(-127, 128, (9, 256), generator=g, dtype=torch.int8)
    B = torch.randint(-127, 128, (384, 256), generator=g, dtype=torch.int8)
    As = torch.rand(9, 1, generator=g) * 0.05
    Bs = torch.rand(384, generator=g) * 1e-3
    assert torch.equal(OC.per_token_matmul(A, B, As, Bs, torch.bfloat16), mm(A, B, As, Bs, output_dtype=torch.bfloat16))
    y_ref = moe(x, w1, w2, w1_s, w2_s, gold["topk_weights"], gold["topk_ids"], gold["topk_ids"].shape[1])
    assert torch.equal(y_ref, gold["y"])


@pytest.mark.skipif(ref_extract.reference_root() is None, reason="no reference checkout")
def test_grouped_layouts_against_reference_models(capsys):
    contig, masked = ref_extract.reference_grouped_layout_models()
    g = torch.Generator().manual_seed(17)
    # contiguous: 3 experts, ranges padded to 8 rows here (the model has no alignment rule), tiny N and K
    M, N, K, E = 24, 6, 64, 3
    A = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    B = torch.randint(-127, 128, (E, N, K), generator=g, dtype=torch.int8)
    As = torch.rand(M, generator=g) * 0.05
    Bs = torch.rand(E, N, generator=g) * 1e-3
    m_indices = torch.tensor([0] * 5 + [-1] * 3 + [1] * 8 + [2] * 2 + [-1] * 6, dtype=torch.int32)
    base = torch.full((M, N), 7.0, dtype=torch.bfloat16)
    ref = contig(A, B, base, As, Bs, 1.0, 0.0, m_index_h=m_indices)
    assert torch.equal(OC.grouped_matmul_contig(A, As, B, Bs, m_indices, base), ref)
    # masked
    Em, T = 2, 5
    A3 = torch.randint(-127, 128, (Em, T, K), generator=g, dtype=torch.int8)
    B3 = torch.randint(-127, 128, (Em, N, K), generator=g, dtype=torch.int8)
    As3 = torch.rand(Em, T, 1, generator=g) * 0.05
    Bs3 = torch.rand(Em, N, 1, generator=g) * 1e-3
    full = masked(A3, B3, As3, Bs3, torch.bfloat16)
    capsys.readouterr()      # the reference function prints shapes
    mm = torch.tensor([5, 3], dtype=torch.int32)
    got = OC.grouped_matmul_masked(A3, As3, B3, Bs3, mm, torch.zeros(Em, T, N, dtype=torch.bfloat16))
    assert torch.equal(got[0], full[0]) and torch.equal(got[1, :3], full[1, :3]) and bool((got[1, 3:] == 0).all())
