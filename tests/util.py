"""Helpers shared by the parity tests."""
from __future__ import annotations

import torch

# Parity bars of the bf16 layer output (normalised, because the outputs are O(1e2..1e3)
# at the benchmark's value distributions; the second one is the reference's own metric,
# test/moe_w8a8/benchmark_moe_int8.py:662).
MAX_ABS_NORM_TOL = 2e-2
MEAN_REL_TOL = 1e-2


def out_errors(y: torch.Tensor, ref: torch.Tensor):
    y = y.float().cpu()
    ref = ref.float().cpu()
    d = (y - ref).abs()
    return float(d.max() / ref.abs().max().clamp(min=1e-30)), float(d.mean() / ref.abs().mean().clamp(min=1e-30))


def assert_out_close(y, ref, what=""):
    max_norm, mean_rel = out_errors(y, ref)
    assert max_norm <= MAX_ABS_NORM_TOL and mean_rel <= MEAN_REL_TOL, \
        f"{what}: max|d|/max|ref|={max_norm:.3e} (tol {MAX_ABS_NORM_TOL}), mean|d|/mean|ref|={mean_rel:.3e} (tol {MEAN_REL_TOL})"
    return max_norm, mean_rel


def assert_gemm_close(got, ref, what="", max_flip_frac=1e-3):
    """bf16 GEMM output against the oracle's bf16 output.

    The kernels accumulate each K block as one fused multiply-add, fma(float(dot), a_s * b_s, acc), like the
    reference's Triton kernel (int8.py:507-519); the torch model rounds the product and the sum separately
    (benchmark_moe_int8.py:131-137).  The fp32 sums differ in their last bits, which moves a bf16 rounding now and
    then.  Bars: the reference's own allclose(rtol=1e-2, atol=1e-2) (test/moe_w8a8/release_moe_w8a8.py:550), no
    element further off than one bf16 step, and at most `max_flip_frac` of the elements different at all."""
    g = got.float().cpu()
    r = ref.float().cpu()
    assert g.shape == r.shape, f"{what}: shape {tuple(g.shape)} vs {tuple(r.shape)}"
    torch.testing.assert_close(g, r, rtol=1e-2, atol=1e-2)
    d = (g - r).abs()
    assert bool((d <= r.abs() * 2.0 ** -7 + 1e-3).all()), f"{what}: an element is more than one bf16 step off (max |d| {float(d.max())})"
    frac = float((d > 0).float().mean()) if d.numel() else 0.0
    assert frac <= max_flip_frac, f"{what}: {frac:.2e} of the elements differ from the oracle (bar {max_flip_frac:.0e})"
    return frac


def topk_ids_match(ids: torch.Tensor, ref_ids: torch.Tensor, logits: torch.Tensor) -> bool:
    """Exact match, except that positions whose oracle probabilities are bit-equal may swap."""
    ids = ids.cpu().long()
    ref_ids = ref_ids.cpu().long()
    if torch.equal(ids, ref_ids):
        return True
    p = torch.softmax(logits.float().cpu(), dim=-1)
    bad = (ids != ref_ids).any(dim=1).nonzero().reshape(-1)
    for r in bad.tolist():
        if not torch.equal(p[r][ids[r]], p[r][ref_ids[r]]):
            return False
    return True
