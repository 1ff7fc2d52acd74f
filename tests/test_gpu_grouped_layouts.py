"""GPU parity tests of the per-channel grouped GEMMs on expert-grouped rows (contiguous and masked layouts)
and of the masked SiLU*mul + quantisation, against the oracle."""
import pytest
import torch

from oracle import moe_channel_int8 as OC

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def lo():
    import lightop_b200
    return lightop_b200


def _contig_case(E, counts, align, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    m_idx = []
    for e, c in enumerate(counts):
        padded = -(-c // align) * align
        m_idx += [e] * c + [-1] * (padded - c)
    M = len(m_idx)
    A = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    As = torch.rand(M, generator=g) * 0.05 + 1e-3
    B = torch.randint(-127, 128, (E, N, K), generator=g, dtype=torch.int8)
    Bs = torch.rand(E, N, generator=g) * 9e-4 + 1e-4
    return A, As, B, Bs, torch.tensor(m_idx, dtype=torch.int32)


@pytest.mark.parametrize("E,counts,align,N,K", [
    (4, [100, 128, 1, 256], 128, 256, 256),          # partial, full, single row, two full blocks (merged chunk)
    (3, [300, 0, 129], 256, 128, 512),               # the reference test's 256-row alignment; an empty expert
    (8, [90, 180, 255, 257, 128, 384, 7, 200], 128, 384, 1024),
    (2, [5, 6], 128, 128, 7168)])
def test_contiguous_layout(lo, E, counts, align, N, K):
    A, As, B, Bs, m_idx = _contig_case(E, counts, align, N, K, seed=sum(counts) + N)
    M = A.shape[0]
    out = torch.full((M, N), 3.0, dtype=torch.bfloat16, device=DEV)
    ret = lo.gemm_ops.m_grouped_w8a8_gemm_nt_contig_asm((A.to(DEV), As.to(DEV)), (B.to(DEV), Bs.to(DEV)), out,
                                                        m_idx.to(DEV), {"MODE": 1000})
    torch.cuda.synchronize()
    lo.check_device_status()
    assert ret.data_ptr() == out.data_ptr()
    ref = OC.grouped_matmul_contig(A, As, B, Bs, m_idx, torch.full((M, N), 3.0, dtype=torch.bfloat16))
    assert torch.equal(out.cpu(), ref)          # integer sums exact, same fp32 scaling sequence; padding rows untouched


def test_contiguous_layout_contract_violation_is_reported(lo):
    A, As, B, Bs, m_idx = _contig_case(2, [128, 128], 128, 128, 256, seed=1)
    m_idx[100:128] = 1          # two experts inside one 128-row block
    out = torch.zeros(256, 128, dtype=torch.bfloat16, device=DEV)
    lo.gemm_ops.m_grouped_w8a8_gemm_nt_contig_asm((A.to(DEV), As.to(DEV)), (B.to(DEV), Bs.to(DEV)), out, m_idx.to(DEV))
    torch.cuda.synchronize()
    with pytest.raises(Exception):
        lo.check_device_status()
    assert bool((out[:128] == 0).all())         # the offending block was skipped, nothing was written for it


@pytest.mark.parametrize("E,max_m,masked,N,K", [
    (4, 128, [128, 0, 1, 77], 256, 256),
    (3, 300, [300, 129, 256], 128, 512),
    (2, 64, [10, 64], 384, 1024),
    (8, 512, [400, 512, 3, 0, 255, 257, 128, 129], 128, 256)])
def test_masked_layout(lo, E, max_m, masked, N, K):
    g = torch.Generator().manual_seed(E * max_m)
    A = torch.randint(-127, 128, (E, max_m, K), generator=g, dtype=torch.int8)
    As = torch.rand(E, max_m, 1, generator=g) * 0.05 + 1e-3
    B = torch.randint(-127, 128, (E, N, K), generator=g, dtype=torch.int8)
    Bs = torch.rand(E, N, 1, generator=g) * 9e-4 + 1e-4
    mm = torch.tensor(masked, dtype=torch.int32)
    d = torch.full((E, max_m, N), -5.0, dtype=torch.bfloat16, device=DEV)
    lo.gemm_ops.m_grouped_w8a8_gemm_nt_masked((A.to(DEV), As.to(DEV)), (B.to(DEV), Bs.to(DEV)), d, mm.to(DEV), 64)
    torch.cuda.synchronize()
    lo.check_device_status()
    ref = OC.grouped_matmul_masked(A, As, B, Bs, mm, torch.full((E, max_m, N), -5.0, dtype=torch.bfloat16))
    assert torch.equal(d.cpu(), ref)


def test_masked_silu_mul_quant(lo):
    g = torch.Generator().manual_seed(4)
    E, T, d = 4, 40, 256
    inter = (torch.randn(E, T, 2 * d, generator=g) * 3).to(torch.bfloat16)
    counts = torch.tensor([40, 0, 7, 33], dtype=torch.int32)
    q, s = lo.activation.fuse_silu_mul_quant_ep(inter.to(DEV), counts.to(DEV))
    assert q.shape == (E, T, d) and s.shape == (E, T, 1)
    q_ref, s_ref = OC.silu_mul_quant_int8(inter.reshape(E * T, 2 * d))
    q_ref, s_ref = q_ref.reshape(E, T, d), s_ref.reshape(E, T, 1)
    for e in range(E):
        c = int(counts[e])
        torch.testing.assert_close(s[e, :c].cpu(), s_ref[e, :c], rtol=1e-2, atol=0)
        same = (s[e, :c].cpu() == s_ref[e, :c]).reshape(-1)
        if c:
            assert float(same.float().mean()) >= 0.9
            dq = (q[e, :c].cpu().int() - q_ref[e, :c].int()).abs()[same]
            assert int(dq.max()) <= 1 and float((dq == 0).float().mean()) >= 0.999
    # without counts every row is processed
    q2, s2 = lo.activation.fuse_silu_mul_quant_ep(inter.to(DEV))
    torch.testing.assert_close(s2.cpu(), s_ref, rtol=1e-2, atol=0)


def test_expert_side_pipeline_on_masked_layout(lo):
    # gate_up GEMM -> SiLU*mul + quant -> down GEMM on the masked layout, the expert side of a low-latency
    # expert-parallel exchange, against the oracle's stage functions
    from util import assert_out_close
    g = torch.Generator().manual_seed(9)
    E, T, H, I = 4, 96, 512, 256
    counts = torch.tensor([96, 13, 0, 50], dtype=torch.int32)
    x = torch.randn(E, T, H, generator=g).to(torch.bfloat16)
    w1 = torch.randint(-127, 128, (E, 2 * I, H), generator=g, dtype=torch.int8)
    w2 = torch.randint(-127, 128, (E, H, I), generator=g, dtype=torch.int8)
    w1_s = torch.rand(E, 2 * I, 1, generator=g) * 9e-4 + 1e-4
    w2_s = torch.rand(E, H, 1, generator=g) * 9e-4 + 1e-4
    xq, xs = lo.quant.per_token_quant_int8(x.to(DEV))
    h = torch.zeros(E, T, 2 * I, dtype=torch.bfloat16, device=DEV)
    lo.gemm_ops.m_grouped_w8a8_gemm_nt_masked((xq, xs), (w1.to(DEV), w1_s.to(DEV)), h, counts.to(DEV), 64)
    aq, a_s = lo.activation.fuse_silu_mul_quant_ep(h, counts.to(DEV))
    y = torch.zeros(E, T, H, dtype=torch.bfloat16, device=DEV)
    lo.gemm_ops.m_grouped_w8a8_gemm_nt_masked((aq, a_s), (w2.to(DEV), w2_s.to(DEV)), y, counts.to(DEV), 64)
    torch.cuda.synchronize()
    lo.check_device_status()
    for e in range(E):
        c = int(counts[e])
        if c == 0:
            assert bool((y[e] == 0).all())
            continue
        xq_r, xs_r = OC.per_token_quant_int8(x[e, :c])
        h_r = OC.per_token_matmul(xq_r, w1[e], xs_r, w1_s[e].reshape(-1), torch.bfloat16)
        aq_r, as_r = OC.silu_mul_quant_int8(h_r)
        y_r = OC.per_token_matmul(aq_r, w2[e], as_r, w2_s[e].reshape(-1), torch.bfloat16)
        assert_out_close(y[e, :c], y_r, f"masked pipeline expert {e}")
        assert bool((y[e, c:] == 0).all())
