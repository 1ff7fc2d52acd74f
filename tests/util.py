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
