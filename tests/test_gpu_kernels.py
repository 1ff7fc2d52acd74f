"""GPU parity tests of the routing, alignment, quantisation and reduction kernels against the oracle."""
import os

import pytest
import torch

from lightop_b200 import synthetic
from oracle import moe_block_int8 as O
from util import topk_ids_match

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def lo():
    import lightop_b200
    return lightop_b200


@pytest.fixture(scope="module")
def small(golden_dir):
    return torch.load(os.path.join(golden_dir, "small_cases.pt"))


# ------------------------------ group quant ------------------------------------

def test_group_quant_golden(lo, small, golden_dir):
    for x, q_ref, s_ref in [(small["x6"], small["q6"], small["s6"]), (small["xe"], small["qe"], small["se"])]:
        q, s = lo.quant.per_token_group_quant_int8(x.to(DEV), 128)
        assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    gold = torch.load(os.path.join(golden_dir, "c0_tiny.pt"))
    cfg = synthetic.CONFIGS["c0_tiny"]
    x, _ = synthetic.make_activations(cfg["M"], cfg["H"], cfg["E"], seed=1)
    q, s = lo.quant.per_token_group_quant_int8(x.to(DEV), 128)
    assert torch.equal(q.cpu(), gold["xq"]) and torch.equal(s.cpu(), gold["xs"])


def test_quantisers_match_the_reference_triton_kernels(lo, golden_dir):
    """Both quantisation kernels against the outputs of the reference's own Triton kernels
    (layers/gemm/int8_utils.py:21-71, 74-193; vectors produced by tests/golden/make_triton_golden.py): bit-equal."""
    cases = torch.load(os.path.join(golden_dir, "triton_quant_cases.pt"))
    for name, c in cases.items():
        g = torch.Generator().manual_seed(c["seed"])
        x = (torch.randn(c["rows"], c["cols"], generator=g) * 3.0).to(getattr(torch, c["dtype"])).to(DEV)
        q, s = lo.quant.per_token_group_quant_int8(x, 128)
        assert torch.equal(q.cpu(), c["group_q"]) and torch.equal(s.cpu(), c["group_s"]), name
        q, s = lo.quant.per_token_quant_int8(x)
        assert torch.equal(q.cpu(), c["token_q"]) and torch.equal(s.cpu(), c["token_s"]), name


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape,group", [((1, 128), 128), ((7, 384), 128), ((33, 7168), 128), ((5, 3, 256), 64), ((9, 512), 256)])
def test_group_quant_bit_exact(lo, dtype, shape, group):
    g = torch.Generator().manual_seed(hash((str(dtype), shape)) % 1000)
    x = (torch.randn(*shape, generator=g) * 3).to(dtype)
    q_ref, s_ref = O.group_quant_int8(x, group)
    q, s = lo.quant.per_token_group_quant_int8(x.to(DEV), group)
    assert q.shape == x.shape and s.shape == x.shape[:-1] + (x.shape[-1] // group,)
    assert torch.equal(q.cpu(), q_ref)
    assert torch.equal(s.cpu(), s_ref)


def test_group_quant_full_size(lo):
    # DeepSeek-V3 prefill activation: 4096 x 7168 bf16
    g = torch.Generator().manual_seed(3)
    x = torch.randn(4096, 7168, generator=g).to(torch.bfloat16)
    q_ref, s_ref = O.group_quant_int8(x, 128)
    q, s = lo.quant.per_token_group_quant_int8(x.to(DEV), 128)
    assert torch.equal(q.cpu(), q_ref) and torch.equal(s.cpu(), s_ref)
    # size-independent property: dequantised error is below one step, and codes never leave [-127,127]
    deq = q.float().view(4096, -1, 128) * s.unsqueeze(-1)
    err = (deq.view(4096, 7168) - x.to(DEV).float()).abs().view(4096, -1, 128)
    assert bool((err <= s.unsqueeze(-1) * 1.0001).all())
    assert int(q.abs().max()) <= 127


# ------------------------------ topk softmax -----------------------------------

@pytest.mark.parametrize("M,E,k", [(32, 8, 2), (8, 16, 4), (1, 256, 8), (7, 256, 8), (33, 160, 6), (4096, 256, 8), (50, 128, 8), (5, 512, 8), (3, 1024, 32)])
@pytest.mark.parametrize("renorm", [True, False])
def test_topk_softmax(lo, M, E, k, renorm):
    g = torch.Generator().manual_seed(2026 + M)
    logits = torch.randn(M, E, generator=g)
    w_ref, ids_ref = O.route_topk_softmax(logits, k, renormalize=renorm)
    w = torch.empty(M, k, dtype=torch.float32, device=DEV)
    ids = torch.empty(M, k, dtype=torch.int32, device=DEV)
    src = torch.empty(M, k, dtype=torch.int32, device=DEV)
    lo.moe.topk_softmax(w, ids, src, logits.to(DEV), renorm)
    assert topk_ids_match(ids, ids_ref, logits)
    same = (ids.cpu() == ids_ref).all(dim=1)
    # the reference's own bars (test/test_softmax_topk.py:55-60)
    torch.testing.assert_close(w.cpu()[same], w_ref[same], rtol=2e-5, atol=2e-6)
    expect_src = torch.arange(k).view(1, k) * M + torch.arange(M).view(M, 1)
    assert torch.equal(src.cpu(), expect_src.to(torch.int32))


@pytest.mark.parametrize("gdtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("idtype", [torch.int64, torch.int32])
def test_topk_softmax_dtypes(lo, gdtype, idtype):
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(64, 256, generator=g).to(gdtype)
    w_ref, ids_ref = O.route_topk_softmax(logits, 8, renormalize=True)
    w = torch.empty(64, 8, dtype=torch.float32, device=DEV)
    ids = torch.empty(64, 8, dtype=idtype, device=DEV)
    lo.moe.topk_softmax(w, ids, None, logits.to(DEV), True)
    # low-precision logits collide often: compare the selected logit multiset, as the reference's
    # test does (test/test_softmax_topk.py:45-53)
    sel = torch.gather(logits.float(), 1, ids.cpu().long()).sort(dim=1).values
    sel_ref = torch.gather(logits.float(), 1, ids_ref.long()).sort(dim=1).values
    assert torch.equal(sel, sel_ref)
    torch.testing.assert_close(w.cpu().sort(dim=1).values, w_ref.sort(dim=1).values, rtol=2e-5, atol=2e-6)


def test_topk_ties_go_to_lower_expert(lo):
    logits = torch.zeros(3, 64)
    w = torch.empty(3, 4, dtype=torch.float32, device=DEV)
    ids = torch.empty(3, 4, dtype=torch.int32, device=DEV)
    lo.moe.topk_softmax(w, ids, None, logits.to(DEV), True)
    assert ids.cpu().tolist() == [[0, 1, 2, 3]] * 3
    torch.testing.assert_close(w.cpu(), torch.full((3, 4), 0.25))


# ------------------------------ alignment --------------------------------------

def _check_align(lo, ids, E, bs, expert_map=None, ignore=False):
    s, e, n = lo.moe.moe_align_block_size(ids.to(DEV), bs, E, expert_map.to(DEV) if expert_map is not None else None,
                                          ignore_invalid_experts=ignore)
    if expert_map is not None and ignore:
        s_ref, e_ref, n_ref = O.align_block_size(ids, E, bs, expert_map=expert_map)
    else:
        s_ref, e_ref, n_ref = O.align_block_size(ids, E, bs)
        if expert_map is not None:
            e_ref = expert_map[e_ref.long()].to(torch.int32)
    total = int(n.item())
    assert total == int(n_ref.item())
    assert torch.equal(s.cpu()[:total], s_ref)
    assert torch.equal(e.cpu()[: total // bs], e_ref)
    assert bool((s.cpu()[total:] == ids.numel()).all())      # sentinel fill of the tail
    assert bool((e.cpu()[total // bs:] == -1).all())


def test_align_golden(lo, small):
    _check_align(lo, small["doc_ids"].to(torch.int32), 5, 4)
    _check_align(lo, small["rag_ids"].view(37, 3).to(torch.int64), 16, 16)


@pytest.mark.parametrize("num_tokens", [1, 5, 18, 90, 323, 1000, 4096, 5500])
@pytest.mark.parametrize("bs", [16, 128])
def test_align_dsv3_shapes(lo, num_tokens, bs):
    # E=256, top_k=8 as in the reference's test (test/test_moe_align_block_size.py:117-128)
    g = torch.Generator().manual_seed(num_tokens)
    ids = torch.randint(0, 256, (num_tokens, 8), generator=g, dtype=torch.int64)
    _check_align(lo, ids, 256, bs)


@pytest.mark.parametrize("E,k,bs", [(8, 2, 1), (64, 6, 64), (128, 8, 32), (1024, 4, 8)])
def test_align_other_shapes(lo, E, k, bs):
    g = torch.Generator().manual_seed(E)
    ids = torch.randint(0, E, (777, k), generator=g, dtype=torch.int32)
    ids[ids == 3] = 2          # an empty expert
    _check_align(lo, ids, E, bs)


def test_align_expert_map(lo):
    g = torch.Generator().manual_seed(0)
    E = 64
    ids = torch.randint(0, E, (300, 8), generator=g, dtype=torch.int32)
    emap = torch.full((E,), -1, dtype=torch.int32)
    emap[16:24] = torch.arange(8, dtype=torch.int32)      # rank 2 of 8 owns experts 16..23
    _check_align(lo, ids, E, 16, expert_map=emap, ignore=True)
    _check_align(lo, ids, E, 16, expert_map=emap, ignore=False)


@pytest.mark.parametrize("M,E,k,bs,dtype", [(8193, 8, 1, 16, torch.int32), (3000, 1024, 4, 8, torch.int64),
                                            (9001, 160, 6, 64, torch.int32), (65536, 32, 1, 16, torch.int32)])
def test_align_many_ids(lo, M, E, k, bs, dtype):
    # at and beyond 8192 ids the alignment runs as a cluster of CTAs: same stable order, ragged slices,
    # empty experts, many experts, and both expert-map modes
    g = torch.Generator().manual_seed(M + E)
    ids = torch.randint(0, E, (M, k), generator=g).to(dtype)
    ids[ids == 1] = 0          # an empty expert
    _check_align(lo, ids, E, bs)
    emap = torch.full((E,), -1, dtype=torch.int32)
    emap[E // 2:] = torch.arange(E - E // 2, dtype=torch.int32)
    _check_align(lo, ids, E, bs, expert_map=emap, ignore=True)
    _check_align(lo, ids, E, bs, expert_map=emap, ignore=False)


def test_align_is_deterministic(lo):
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 256, (8192, 8), generator=g, dtype=torch.int32).to(DEV)
    a = lo.moe.moe_align_block_size(ids, 128, 256)
    b = lo.moe.moe_align_block_size(ids, 128, 256)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


def test_align_out_variant(lo):
    ids = torch.tensor([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], dtype=torch.int32, device=DEV)
    s = torch.empty(12 + 5 * 3, dtype=torch.int32, device=DEV)
    e = torch.empty(7, dtype=torch.int32, device=DEV)
    n = torch.empty(1, dtype=torch.int32, device=DEV)
    lo.moe.moe_align_block_size_out(ids, 5, 4, s, e, n)
    assert n.item() == 16
    assert s.cpu()[:16].tolist() == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]


# ------------------------------ moe_sum ----------------------------------------

@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,k,H", [(1, 8, 7168), (37, 2, 256), (128, 8, 4096)])
def test_moe_sum(lo, dtype, M, k, H):
    g = torch.Generator().manual_seed(M)
    a = torch.randn(M, k, H, generator=g).to(dtype)
    bias = torch.randn(M, H, generator=g).to(dtype)
    out = torch.empty(M, H, dtype=dtype, device=DEV)
    lo.moe.moe_sum(a.to(DEV), out)
    # same bar as the reference's test (test/test_moe_sum_opt.py:31-56) and bit-equality with the oracle
    torch.testing.assert_close(out.cpu(), a.float().sum(1).to(dtype), rtol=1e-2, atol=1e-2)
    assert torch.equal(out.cpu(), O.moe_sum(a))
    lo.moe.moe_sum(a.to(DEV), out, bias=bias.to(DEV), factor=2.5)
    torch.testing.assert_close(out.cpu(), O.moe_sum(a, 2.5, bias), rtol=1e-2, atol=1e-2)


def test_moe_sum_mask(lo):
    g = torch.Generator().manual_seed(0)
    a = torch.randn(16, 4, 128, generator=g).to(torch.bfloat16)
    mask = torch.rand(16, 4, generator=g) > 0.5
    out = torch.empty(16, 128, dtype=torch.bfloat16, device=DEV)
    lo.moe.moe_sum(a.to(DEV), out, expert_mask=mask.to(DEV))
    ref = (a.float() * mask.unsqueeze(-1)).sum(1).to(torch.bfloat16)
    assert torch.equal(out.cpu(), ref)


# ------------------------------ expert-parallel local kernels ---------------------

def test_ep_build_m_indices_known_answer(lo):
    ids = torch.tensor([[0, 1], [1, 2], [0, -1]], device=DEV, dtype=torch.int64)
    m = torch.empty(6, device=DEV, dtype=torch.int32)
    lo.moe.ep_build_m_indices(ids, m, 3, 2)
    assert m.cpu().tolist() == [0, 0, 1, 1, 2, -1]


@pytest.mark.parametrize("T,k,E,world", [(2100, 4, 16, 2), (8192, 8, 256, 8), (9000, 1, 8, 1)])
def test_ep_scatter_many_rows(lo, T, k, E, world):
    # from 8192 (token, slot) pairs on the plan runs as a cluster of CTAs; rank-as-expert packing as the
    # expert-parallel driver uses it (the "expert" of a row is its destination rank)
    g = torch.Generator().manual_seed(T + E)
    H, align = 128, 1
    aq = torch.randint(-127, 128, (T, H), generator=g, dtype=torch.int8)
    scales = torch.rand(T, 1, generator=g)
    ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
    rank_of_expert = (torch.arange(E) // (E // world)).to(torch.int32)
    rows = T * k
    out = torch.zeros(rows, H, dtype=torch.int8, device=DEV)
    out_s = torch.zeros(rows, 1, device=DEV)
    m_idx = torch.empty(rows, dtype=torch.int32, device=DEV)
    inv = torch.empty(T, k, dtype=torch.int32, device=DEV)
    lo.moe.ep_scatter(aq.to(DEV), scales.to(DEV), ids.to(DEV), rank_of_expert.to(DEV), None, out, out_s, m_idx, inv, world, align)
    dest = rank_of_expert[ids.long()].reshape(-1)
    # stable counting sort by destination rank
    order = torch.sort(dest, stable=True).indices
    inv_ref = torch.empty(rows, dtype=torch.int64)
    inv_ref[order] = torch.arange(rows)
    assert torch.equal(inv.cpu().reshape(-1).long(), inv_ref)
    assert torch.equal(m_idx.cpu(), dest[order])
    tok = torch.arange(T).repeat_interleave(k)
    assert torch.equal(out.cpu()[inv_ref], aq[tok]) and torch.equal(out_s.cpu()[inv_ref], scales[tok])


def test_ep_scatter_gather_roundtrip(lo):
    # the structure of the reference's tests (test/test_native_categorized_moe_api.py:77-144)
    g = torch.Generator().manual_seed(0)
    T, k, H, E, align = 40, 4, 256, 8, 16
    aq = torch.randint(-127, 128, (T, H), generator=g, dtype=torch.int8)
    scales = torch.rand(T, H // 128, generator=g)
    ids = torch.stack([torch.randperm(16, generator=g)[:k] for _ in range(T)])
    emap = torch.full((16,), -1, dtype=torch.int32)
    emap[8:16] = torch.arange(8, dtype=torch.int32)
    loc = emap[ids]
    counts = torch.bincount(loc[loc >= 0].long(), minlength=E).to(torch.int32)
    rows = int(((counts + align - 1) // align * align).sum())
    out = torch.zeros(rows, H, dtype=torch.int8, device=DEV)
    out_s = torch.zeros(rows, H // 128, device=DEV)
    m_idx = torch.empty(rows, dtype=torch.int32, device=DEV)
    inv = torch.empty(T, k, dtype=torch.int32, device=DEV)
    lo.moe.ep_scatter(aq.to(DEV), scales.to(DEV), ids.to(DEV), emap.to(DEV), counts.to(DEV), out, out_s, m_idx, inv, E, align)
    inv_c = inv.cpu()
    assert bool(((inv_c >= 0) == (loc >= 0)).all())
    sel = inv_c >= 0
    tok = torch.arange(T).view(T, 1).expand(T, k)
    assert torch.equal(out.cpu()[inv_c[sel].long()], aq[tok[sel]])
    assert torch.equal(out_s.cpu()[inv_c[sel].long()], scales[tok[sel]])
    assert torch.equal(m_idx.cpu()[inv_c[sel].long()], loc[sel])
    m_ref, _ = O.ep_build_m_indices(ids, E, align, expert_map=emap, rows=rows)
    assert torch.equal(m_idx.cpu(), m_ref)
    # rows of one expert keep ascending (token, slot) order
    flat_inv = inv_c.reshape(-1)
    for e in range(E):
        r = flat_inv[(loc.reshape(-1) == e)]
        assert torch.equal(r, torch.sort(r).values)
    # gather
    a = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    w = torch.softmax(torch.randn(T, k, generator=g), dim=-1)
    y = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    lo.moe.ep_gather(a.to(DEV), ids.to(DEV), w.to(DEV), inv, emap.to(DEV), y)
    ref = O.ep_gather(a, ids, w, inv_c, emap)
    torch.testing.assert_close(y.cpu(), ref, rtol=1e-2, atol=1e-2)
