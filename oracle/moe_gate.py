"""Pure-torch CPU restatement of the reference's grouped, bias-corrected sigmoid gate.

TEST INFRASTRUCTURE ONLY -- the product never routes through this file.

Parity status: PINNED.  ``kimi_k2_gate`` and ``sqrtsoftplus_gate`` are checked against the reference's torch
models of those gates (test/ci_tests/test_kimi_k2_moe_fused_gate.py:14-43,
test/ci_tests/test_moe_fused_gate_sqrtsoftplus.py:9-45) and the fixture tests/golden/gate_variant_cases.pt;
``fused_gate`` is checked against the reference's own torch model of
``moe_fused_gate`` (``biased_grouped_topk_impl`` + ``requested_baseline_moe_gate``,
test/ci_tests/test_fused_moe_gate.py:9-117, loaded from a reference checkout by
``oracle/ref_extract.py``) and against the fixture generated from it
(tests/golden/gate_cases.pt).  The model selects with ``torch.topk(sorted=False)`` and the
reference's test compares after sorting by expert id; this restatement fixes the order the
kernel documents (descending selection score, lower id first on ties,
docs/moe_fused_gate_dispatch.md:59-64, csrc/kernels/moe_gate/moe_fused_gate.cu:259-295).
"""
from __future__ import annotations

from typing import Tuple

import torch


def _topk_lower_id_first(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest entries per row, descending, ties to the lower index."""
    order = torch.sort(scores, dim=-1, descending=True, stable=True).indices
    return order[..., :k]


def fused_gate(x: torch.Tensor, bias: torch.Tensor, num_expert_group: int, topk_group: int, topk: int,
               n_share_experts_fusion: int = 0, routed_scaling_factor: float = 1.0,
               apply_routed_scaling_factor_on_output: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(weights fp32 [M, topk], ids int32 [M, topk])``.

    Restates test/ci_tests/test_fused_moe_gate.py:9-117: ``p = sigmoid(x)`` in fp32; selection score
    ``p + bias``; group score = sum of the two largest selection scores of the group; the
    ``topk_group`` best groups stay, the rest is masked with -inf; ``topk - shared`` experts are
    taken; weights = ``p`` of the taken experts over their sum, times the scaling factor (when it
    is applied on the output and positive); shared experts get ids ``E + j`` and weight
    ``(1 / factor) * output factor`` (csrc/kernels/moe_gate/moe_fused_gate.cu:296-311).
    """
    M, E = x.shape
    p = torch.sigmoid(x.to(torch.float32))
    s = p + bias.to(torch.float32).unsqueeze(0)
    k_routed = topk - n_share_experts_fusion
    if num_expert_group > 1:
        gs = s.view(M, num_expert_group, -1).topk(2, dim=-1)[0].sum(dim=-1)
        gidx = _topk_lower_id_first(gs, topk_group)
        gmask = torch.zeros_like(gs, dtype=torch.bool)
        gmask.scatter_(1, gidx, True)
        emask = gmask.unsqueeze(-1).expand(M, num_expert_group, E // num_expert_group).reshape(M, E)
        s = s.masked_fill(~emask, float("-inf"))
    ids = _topk_lower_id_first(s, k_routed)
    w = p.gather(1, ids)
    w_sum = w.sum(dim=-1, keepdim=True)
    route_scale = float(routed_scaling_factor) if (apply_routed_scaling_factor_on_output
                                                   and routed_scaling_factor > 0) else 1.0
    w = (w / w_sum) * route_scale
    if n_share_experts_fusion > 0:
        shared_ids = torch.arange(E, E + n_share_experts_fusion).unsqueeze(0).expand(M, -1)
        base = 1.0 / routed_scaling_factor if routed_scaling_factor > 0 else 1.0
        shared_w = torch.full((M, n_share_experts_fusion), base * route_scale, dtype=torch.float32)
        ids = torch.cat([ids, shared_ids], dim=-1)
        w = torch.cat([w, shared_w], dim=-1)
    return w.to(torch.float32), ids.to(torch.int32)


def kimi_k2_gate(x: torch.Tensor, bias: torch.Tensor, topk: int, renormalize: bool = True,
                 routed_scaling_factor: float = 1.0, apply_routed_scaling_factor_on_output: bool = False
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Restates ``kimi_k2_biased_topk_impl_ref`` (test/ci_tests/test_kimi_k2_moe_fused_gate.py:14-43): sigmoid
    scores, top-k on score + bias, weights = scores of the chosen experts; when ``renormalize`` they are divided
    by ``sum + 1e-20`` and (only then) scaled on request.  Order: descending selection score, lower id on ties."""
    p = torch.sigmoid(x.to(torch.float32))
    ids = _topk_lower_id_first(p + bias.to(torch.float32).unsqueeze(0), topk)
    w = p.gather(1, ids)
    if renormalize:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
        if apply_routed_scaling_factor_on_output:
            w = w * routed_scaling_factor
    return w.to(torch.float32), ids.to(torch.int32)


def sqrtsoftplus_gate(x: torch.Tensor, bias: torch.Tensor, topk: int, num_fused_shared_experts: int = 0,
                      renormalize: bool = True, routed_scaling_factor: float = 1.0,
                      apply_routed_scaling_factor_on_output: bool = False,
                      softplus_linear_above_20: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Restates ``reference_moe_fused_gate_sqrtsoftplus`` (test/ci_tests/test_moe_fused_gate_sqrtsoftplus.py:9-45):
    scores ``sqrt(log1p(exp(x)))``, top-k (descending) on score + bias, shared experts with ids ``E + j`` and score
    ``routed sum / factor``, all weights over the routed sum when ``renormalize``, times the factor on request."""
    M, E = x.shape
    xf = x.to(torch.float32)
    softplus = torch.log1p(torch.exp(xf))
    if softplus_linear_above_20:        # csrc/kernels/moe_gate/moe_fused_gate_sqrtsoftplus.cu:66-69
        softplus = torch.where(xf > 20.0, xf, softplus)
    p = torch.sqrt(softplus)
    k_routed = topk - num_fused_shared_experts
    ids = _topk_lower_id_first(p + bias.to(torch.float32).reshape(-1, E), k_routed)   # bias [E] or [M, E]
    w = p.gather(1, ids)
    routed_sum = w.sum(dim=-1, keepdim=True)
    if num_fused_shared_experts > 0:
        shared_ids = torch.arange(E, E + num_fused_shared_experts).unsqueeze(0).expand(M, -1)
        ids = torch.cat([ids, shared_ids], dim=-1)
        w = torch.cat([w, (routed_sum / routed_scaling_factor).expand(M, num_fused_shared_experts)], dim=-1)
    if renormalize:     # the kernel leaves a row with a zero routed sum undivided (moe_fused_gate_sqrtsoftplus.cu:202)
        w = w / torch.where(routed_sum > 0, routed_sum, torch.ones_like(routed_sum))
    if apply_routed_scaling_factor_on_output:
        w = w * routed_scaling_factor
    return w.to(torch.float32), ids.to(torch.int32)


def mask_padded_rows(weights: torch.Tensor, ids: torch.Tensor, num_token_non_padded: int, padding_id: int
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rows at or beyond ``num_token_non_padded`` get weight 0 and id ``padding_id``; ids come back as int64: the
    final stores of the padded sqrt-softplus gates (csrc/kernels/moe_gate/moe_fused_gate_sqrtsoftplus.cu:205-212)."""
    w, i = weights.clone(), ids.to(torch.int64)
    w[num_token_non_padded:] = 0.0
    i[num_token_non_padded:] = padding_id
    return w, i


def topk_ids_postprocess(topk_ids: torch.Tensor, logical_to_physical_map=None, num_token_non_padded=None
                         ) -> torch.Tensor:
    """Restates csrc/kernels/topk/topk_ids_postprocess.cu:30-66 (returns a new tensor)."""
    out = topk_ids.clone()
    if logical_to_physical_map is not None:
        m = logical_to_physical_map.to(torch.int64)
        ok = (out >= 0) & (out < m.numel())
        out = torch.where(ok, m[out.clamp(0, m.numel() - 1).to(torch.int64)], torch.full_like(out, -1).to(torch.int64)
                          ).to(topk_ids.dtype)
    if num_token_non_padded is not None:
        nv = int(num_token_non_padded.reshape(-1)[0])
        out[nv:] = -1
    return out
