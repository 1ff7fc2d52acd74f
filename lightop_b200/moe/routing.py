"""Routing, expert alignment and top-k reduction (reference: python/lightop/moe/routing.py)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib


def _cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def _round_up(a: int, b: int) -> int:
    return _cdiv(a, b) * b


def topk_softmax(topk_weights: torch.Tensor, topk_indices: torch.Tensor,
                 token_expert_indices: Optional[torch.Tensor], gating_output: torch.Tensor,
                 Is_renormalize: bool = False) -> None:
    """Softmax over experts + top-k, written into the caller's tensors.

    Signature of the reference's ``op.topk_softmax`` (csrc/pybind/export.cpp:546,1437;
    host csrc/kernels/softmax/topk_softmax_kernels.cu:1716-1791).  ``topk_weights`` fp32
    ``[M,k]``; ``topk_indices`` int32 / uint32 / int64 ``[M,k]`` in descending score order;
    ``token_expert_indices`` int32 ``[M,k]`` receives ``slot * M + token``.
    """
    _lib.require_cuda(topk_weights, topk_indices, token_expert_indices, gating_output)
    if gating_output.dim() != 2:
        raise RuntimeError("gating_output must be [num_tokens, num_experts]")
    M, E = gating_output.shape
    k = topk_indices.shape[-1]
    if topk_weights.dtype != torch.float32:
        raise RuntimeError("topk_weights must be float32")
    if tuple(topk_weights.shape) != (M, k) or tuple(topk_indices.shape) != (M, k):
        raise RuntimeError("topk_weights / topk_indices must be [num_tokens, topk]")
    if token_expert_indices is not None and token_expert_indices.dtype != torch.int32:
        raise RuntimeError("token_expert_indices must be int32")
    if not (gating_output.is_contiguous() and topk_weights.is_contiguous() and topk_indices.is_contiguous()):
        raise RuntimeError("topk_softmax expects contiguous tensors")
    with torch.cuda.device(gating_output.device):
        st = _lib.load().lo_topk_softmax(_lib.ptr(gating_output), _lib.dtype_code(gating_output.dtype), M, E, k,
                                         int(bool(Is_renormalize)), _lib.ptr(topk_weights), _lib.ptr(topk_indices),
                                         _lib.dtype_code(topk_indices.dtype), _lib.ptr(token_expert_indices),
                                         _lib.current_stream(gating_output.device))
    _lib.check(st, "topk_softmax")


def moe_align_block_size_out(topk_ids, num_experts, block_size, sorted_ids, expert_ids, num_tokens_post_pad,
                             expert_map=None, expert_mask=None, num_local_tokens=None, is_ep=False,
                             is_fuse_fill=True):
    """Expert alignment into caller-provided tensors (reference: python/lightop/moe/routing.py:23-50).

    With an ``expert_map`` the ids are mapped before counting and ids mapping to -1 are
    dropped, as the reference's native kernel does when it is handed a map.  ``expert_mask``,
    ``num_local_tokens`` and ``is_ep`` select HCU-specific variants and are not supported;
    the sentinel fill is always done (``is_fuse_fill``).
    """
    if expert_mask is not None or num_local_tokens is not None:
        raise NotImplementedError("expert_mask / num_local_tokens variants are not part of this path")
    _lib.require_cuda(topk_ids, sorted_ids, expert_ids, num_tokens_post_pad, expert_map)
    if sorted_ids.dtype != torch.int32 or expert_ids.dtype != torch.int32 or num_tokens_post_pad.dtype != torch.int32:
        raise RuntimeError("sorted_ids, expert_ids and num_tokens_post_pad must be int32")
    ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
    if expert_map is not None and expert_map.dtype != torch.int32:
        expert_map = expert_map.to(torch.int32)
    with torch.cuda.device(ids.device):
        st = _lib.load().lo_moe_align_block_size(
            _lib.ptr(ids), _lib.dtype_code(ids.dtype), ids.numel(), int(num_experts), int(block_size),
            _lib.ptr(expert_map), 1 if expert_map is not None else 0, _lib.ptr(sorted_ids), sorted_ids.numel(),
            _lib.ptr(expert_ids), expert_ids.numel(), _lib.ptr(num_tokens_post_pad), _lib.current_stream(ids.device))
    _lib.check(st, "moe_align_block_size")


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int,
                         expert_map: Optional[torch.Tensor] = None, pad_sorted_ids: bool = False,
                         ignore_invalid_experts: bool = False
                         ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sort the flat ``(token, slot)`` indices by expert and pad every expert to ``block_size``.

    Signature, buffer sizes and the sentinel convention follow the reference wrapper
    (python/lightop/_lmslim_native/vllm_compat/moe_align_block_size.py:17-120).  With an
    ``expert_map``: ``ignore_invalid_experts=True`` drops ids that map to -1 before counting
    and returns local expert ids; otherwise all ids are counted and ``expert_ids`` holds
    ``expert_map[expert]`` (-1 for blocks of non-local experts).  Inside an expert the
    indices are ascending, the order of the reference's Python model
    (test/test_moe_align_block_size.py:79-87).
    """
    _lib.require_cuda(topk_ids, expert_map)
    numel = topk_ids.numel()
    max_num_tokens_padded = numel + num_experts * (block_size - 1)
    if pad_sorted_ids:
        max_num_tokens_padded = _round_up(max_num_tokens_padded, block_size)
    if numel < num_experts:
        max_num_tokens_padded = min(numel * block_size, max_num_tokens_padded)
    sorted_ids = torch.empty((max_num_tokens_padded,), dtype=torch.int32, device=topk_ids.device)
    expert_ids = torch.empty((_cdiv(max_num_tokens_padded, block_size),), dtype=torch.int32, device=topk_ids.device)
    num_tokens_post_pad = torch.empty((1,), dtype=torch.int32, device=topk_ids.device)
    ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
    mode = 0
    if expert_map is not None:
        if expert_map.dtype != torch.int32:
            expert_map = expert_map.to(torch.int32)
        mode = 1 if ignore_invalid_experts else 2
    with torch.cuda.device(ids.device):
        st = _lib.load().lo_moe_align_block_size(
            _lib.ptr(ids), _lib.dtype_code(ids.dtype), numel, int(num_experts), int(block_size),
            _lib.ptr(expert_map), mode, _lib.ptr(sorted_ids), sorted_ids.numel(), _lib.ptr(expert_ids),
            expert_ids.numel(), _lib.ptr(num_tokens_post_pad), _lib.current_stream(ids.device))
    _lib.check(st, "moe_align_block_size")
    return sorted_ids, expert_ids, num_tokens_post_pad


def moe_sum(input: torch.Tensor, output: torch.Tensor, bias: Optional[torch.Tensor] = None,
            expert_mask: Optional[torch.Tensor] = None, num_local_tokens: Optional[torch.Tensor] = None,
            factor: float = 1.0, expect_m: int = -1) -> None:
    """``output[t] = factor * sum_j input[t, j] (+ bias[t])`` (reference: python/lightop/moe_align_sum.py:12-29).

    fp32 accumulation and one rounding, as the reference's bf16 kernel
    (csrc/kernels/moe_align_sum_kernels.cu:604-760).  ``expert_mask`` (bool ``[M, topk]``)
    skips slots; ``num_local_tokens`` (int32 ``[1]``) limits the tokens written; ``expect_m``
    is a launch hint of the reference and is ignored.

    Deviation: fp16 and fp32 inputs follow the same rule (``sum * factor + bias``).  The reference's kernels for
    those dtypes invert the factor and scale the bias instead (``x * (1/factor)``, ``x + bias * (1/factor)``,
    moe_align_sum_kernels.cu:558-571, 680-686), which its bf16 kernel and its Python wrapper's description do not;
    parity with the reference is therefore pinned for bf16 only.
    """
    _lib.require_cuda(input, output, bias, expert_mask, num_local_tokens)
    if input.dim() != 3:
        raise RuntimeError("moe_sum input must be [num_tokens, topk, hidden]")
    M, topk, H = input.shape
    if tuple(output.shape) != (M, H) or output.dtype != input.dtype:
        raise RuntimeError("moe_sum output must be [num_tokens, hidden] of the input dtype")
    if not (input.is_contiguous() and output.is_contiguous()):
        raise RuntimeError("moe_sum expects contiguous tensors")
    if bias is not None and (tuple(bias.shape) != (M, H) or bias.dtype != input.dtype or not bias.is_contiguous()):
        raise RuntimeError("moe_sum bias must be a contiguous [num_tokens, hidden] tensor of the input dtype")
    if expert_mask is not None:
        expert_mask = expert_mask.to(torch.bool).contiguous()
    with torch.cuda.device(input.device):
        st = _lib.load().lo_moe_sum(_lib.ptr(input), _lib.ptr(output), _lib.ptr(bias), _lib.dtype_code(input.dtype),
                                    M, topk, H, float(factor), _lib.ptr(expert_mask), _lib.ptr(num_local_tokens),
                                    _lib.current_stream(input.device))
    _lib.check(st, "moe_sum")


def moe_fused_gate(x: torch.Tensor, bias: torch.Tensor, num_expert_group: int, topk_group: int, topk: int,
                   n_share_experts_fusion: int, routed_scaling_factor: float,
                   apply_routed_scaling_factor_on_output: bool = True,
                   output_indices_int64: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Grouped, bias-corrected sigmoid gate; returns ``(weights fp32 [M,topk], ids [M,topk])``.

    Signature of the reference (python/lightop/moe_fused_gate.py:10-31).  Selection and weights
    follow its kernel and test model (csrc/kernels/moe_gate/moe_fused_gate.cu:130-315,
    test/ci_tests/test_fused_moe_gate.py:9-117): scores ``sigmoid(x) + bias`` choose groups (sum of
    the two best scores per group) and then experts, in descending order with the lower id winning
    ties; weights are the unbiased ``sigmoid(x)`` of the chosen experts divided by their sum, times
    ``routed_scaling_factor`` when applied on the output; fused shared experts take ids
    ``num_experts + j``.  Any layout that satisfies the reference's argument rules is accepted.
    """
    _lib.require_cuda(x, bias)
    if x.dim() != 2:
        raise RuntimeError(f"moe_fused_gate: input must have shape [tokens, experts], got {tuple(x.shape)}")
    if bias.dim() != 1 or bias.numel() != x.shape[1]:
        raise RuntimeError(f"moe_fused_gate: bias must have shape [experts], got {tuple(bias.shape)}")
    if not (x.is_contiguous() and bias.is_contiguous()):
        raise RuntimeError("moe_fused_gate: input and bias must be contiguous")
    M, E = x.shape
    weights = torch.empty(M, topk, dtype=torch.float32, device=x.device)
    ids = torch.empty(M, topk, dtype=torch.int64 if output_indices_int64 else torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        st = _lib.load().lo_moe_fused_gate(_lib.ptr(x), _lib.dtype_code(x.dtype), _lib.ptr(bias),
                                           _lib.dtype_code(bias.dtype), M, E, int(num_expert_group), int(topk_group),
                                           int(topk), int(n_share_experts_fusion), float(routed_scaling_factor),
                                           int(bool(apply_routed_scaling_factor_on_output)), _lib.ptr(weights),
                                           _lib.ptr(ids), _lib.dtype_code(ids.dtype), _lib.current_stream(x.device))
    _lib.check(st, "moe_fused_gate")
    return weights, ids


def _gate_topk(x, bias, groups, topk_group, topk, n_shared, score_fn, renormalize, norm_eps, out_scale, shared_div,
               ids_dtype=torch.int32, num_token_non_padded=None, padding_id=0, per_token_bias=False, what="gate"):
    _lib.require_cuda(x, bias, num_token_non_padded)
    n = num_token_non_padded
    if n is not None and (n.dtype not in (torch.int32, torch.int64) or n.numel() != 1 or not n.is_contiguous()):
        raise RuntimeError(f"{what}: num_token_non_padded must be one contiguous int32 or int64 element")
    if x.dim() != 2:
        raise RuntimeError(f"{what}: input must have shape [tokens, experts], got {tuple(x.shape)}")
    M, E = x.shape
    if bias.dim() == 2 and per_token_bias:
        if tuple(bias.shape) != (M, E):
            raise RuntimeError(f"{what}: a 2D bias must have shape [tokens, experts], got {tuple(bias.shape)}")
    elif bias.dim() != 1 or bias.numel() != E:
        raise RuntimeError(f"{what}: bias must have shape [experts], got {tuple(bias.shape)}")
    if not (x.is_contiguous() and bias.is_contiguous()):
        raise RuntimeError(f"{what}: input and bias must be contiguous")
    weights = torch.empty(M, topk, dtype=torch.float32, device=x.device)
    ids = torch.empty(M, topk, dtype=ids_dtype, device=x.device)
    with torch.cuda.device(x.device):
        st = _lib.load().lo_moe_gate_topk(_lib.ptr(x), _lib.dtype_code(x.dtype), _lib.ptr(bias), _lib.dtype_code(bias.dtype),
                                          E if bias.dim() == 2 else 0, M, E, int(groups), int(topk_group), int(topk),
                                          int(n_shared), int(score_fn), int(bool(renormalize)), float(norm_eps),
                                          float(out_scale), float(shared_div), _lib.ptr(n) if n is not None else 0,
                                          _lib.dtype_code(n.dtype) if n is not None else 0, int(padding_id),
                                          _lib.ptr(weights), _lib.ptr(ids), _lib.dtype_code(ids.dtype),
                                          _lib.current_stream(x.device))
    _lib.check(st, what)
    return weights, ids


def kimi_k2_moe_fused_gate(x: torch.Tensor, bias: torch.Tensor, topk: int, renormalize: bool = True,
                           routed_scaling_factor: float = 1.0,
                           apply_routed_scaling_factor_on_output: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Ungrouped bias-corrected sigmoid gate (Kimi-K2): top-k on ``sigmoid(x) + bias``, weights ``sigmoid(x)`` of the
    chosen experts, divided by ``sum + 1e-20`` when ``renormalize`` and then (only then) scaled on request.

    Signature of the reference (python/lightop/moe_fused_gate.py:34-49); semantics of its torch model
    (test/ci_tests/test_kimi_k2_moe_fused_gate.py:14-43).  Ids come out in descending order of the selection
    score, ties to the lower id.
    """
    scale = float(routed_scaling_factor) if (renormalize and apply_routed_scaling_factor_on_output) else 1.0
    return _gate_topk(x, bias, 1, 1, topk, 0, _lib.LO_GATE_SIGMOID, renormalize, 1e-20, scale, 1.0,
                      what="kimi_k2_moe_fused_gate")


def _sqrtsoftplus(x, bias, topk, num_fused_shared_experts, renormalize, routed_scaling_factor,
                  apply_routed_scaling_factor_on_output, score_fn, what, ids_dtype=torch.int32,
                  num_token_non_padded=None, padding_id=0):
    # argument rules of csrc/kernels/moe_gate/moe_fused_gate_sqrtsoftplus.cu:267-294 (any expert count is accepted here)
    if not routed_scaling_factor > 0.0:
        raise RuntimeError(f"{what}: routed_scaling_factor must be positive")
    scale = float(routed_scaling_factor) if apply_routed_scaling_factor_on_output else 1.0
    return _gate_topk(x, bias, 1, 1, topk, num_fused_shared_experts, score_fn, renormalize, 0.0, scale,
                      float(routed_scaling_factor), ids_dtype=ids_dtype, num_token_non_padded=num_token_non_padded,
                      padding_id=padding_id, per_token_bias=True, what=what)


def moe_fused_gate_sqrtsoftplus(x: torch.Tensor, bias: torch.Tensor, topk: int, num_fused_shared_experts: int = 0,
                                renormalize: bool = True, routed_scaling_factor: float = 1.0,
                                apply_routed_scaling_factor_on_output: bool = False
                                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Ungrouped gate with scores ``sqrt(softplus(x))``: top-k on score + bias, weights = scores of the chosen experts
    over their sum (when ``renormalize``), shared experts as extra slots with ids ``E + j`` and score
    ``sum / routed_scaling_factor``, everything times the factor when it is applied on the output.  ``bias`` is
    ``[experts]`` or, per token, ``[tokens, experts]``.

    Signature of the reference (python/lightop/moe_fused_gate.py:52-69); semantics of its torch model
    (test/ci_tests/test_moe_fused_gate_sqrtsoftplus.py:9-45).
    """
    return _sqrtsoftplus(x, bias, topk, num_fused_shared_experts, renormalize, routed_scaling_factor,
                         apply_routed_scaling_factor_on_output, _lib.LO_GATE_SQRT_SOFTPLUS, "moe_fused_gate_sqrtsoftplus")


def moe_fused_gate_sqrtsoftplus_v41_hcu(x: torch.Tensor, bias: torch.Tensor, topk: int, num_fused_shared_experts: int = 0,
                                        renormalize: bool = True, routed_scaling_factor: float = 1.0,
                                        apply_routed_scaling_factor_on_output: bool = False
                                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The same gate with ``softplus(x) = x`` for ``x > 20`` (equal to fp32 precision, and free of the overflow of
    ``exp``): python/lightop/moe_fused_gate.py:72-88, csrc/kernels/moe_gate/moe_fused_gate_sqrtsoftplus.cu:66-69."""
    return _sqrtsoftplus(x, bias, topk, num_fused_shared_experts, renormalize, routed_scaling_factor,
                         apply_routed_scaling_factor_on_output, _lib.LO_GATE_SQRT_SOFTPLUS_SAFE,
                         "moe_fused_gate_sqrtsoftplus_v41_hcu")


def moe_fused_gate_sqrtsoftplus_v41_hcu_fused(x: torch.Tensor, bias: torch.Tensor, topk: int,
                                              num_fused_shared_experts: int = 0, renormalize: bool = True,
                                              routed_scaling_factor: float = 1.0,
                                              apply_routed_scaling_factor_on_output: bool = False,
                                              num_token_non_padded: Optional[torch.Tensor] = None
                                              ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The ``v41`` gate with int64 ids; rows at or beyond the device-side ``num_token_non_padded`` get weight 0 and
    id 0 (python/lightop/moe_fused_gate.py:91-107, csrc/kernels/moe_gate/moe_fused_gate_sqrtsoftplus.cu:378-399)."""
    return _sqrtsoftplus(x, bias, topk, num_fused_shared_experts, renormalize, routed_scaling_factor,
                         apply_routed_scaling_factor_on_output, _lib.LO_GATE_SQRT_SOFTPLUS_SAFE,
                         "moe_fused_gate_sqrtsoftplus_v41_hcu_fused", torch.int64, num_token_non_padded, 0)


def moe_fused_gate_sqrtsoftplus_v41_hcu_deepep(x: torch.Tensor, bias: torch.Tensor, topk: int,
                                               num_fused_shared_experts: int = 0, renormalize: bool = True,
                                               routed_scaling_factor: float = 1.0,
                                               apply_routed_scaling_factor_on_output: bool = False,
                                               num_token_non_padded: Optional[torch.Tensor] = None
                                               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """As the ``_fused`` form, with id -1 on the padded rows: the value an expert-parallel dispatch skips
    (python/lightop/moe_fused_gate.py:110-127, csrc/kernels/moe_gate/moe_fused_gate_sqrtsoftplus.cu:401-421)."""
    return _sqrtsoftplus(x, bias, topk, num_fused_shared_experts, renormalize, routed_scaling_factor,
                         apply_routed_scaling_factor_on_output, _lib.LO_GATE_SQRT_SOFTPLUS_SAFE,
                         "moe_fused_gate_sqrtsoftplus_v41_hcu_deepep", torch.int64, num_token_non_padded, -1)


def topk_ids_postprocess(topk_ids: torch.Tensor, logical_to_physical_map: Optional[torch.Tensor] = None,
                         num_token_non_padded: Optional[torch.Tensor] = None) -> None:
    """In place: padded tokens' ids become -1, the others are mapped logical -> physical
    (reference: csrc/kernels/topk/topk_ids_postprocess.cu:30-66, known answer in
    test/test_native_categorized_moe_api.py:147-169)."""
    if topk_ids.numel() == 0:
        return
    _lib.require_cuda(topk_ids, logical_to_physical_map, num_token_non_padded)
    if topk_ids.dim() != 2:
        raise RuntimeError("topk_ids_postprocess expects 2D topk_ids")
    if not topk_ids.is_contiguous():
        raise RuntimeError("topk_ids_postprocess expects contiguous topk_ids")
    for t, name in ((topk_ids, "topk_ids"), (logical_to_physical_map, "logical_to_physical_map"),
                    (num_token_non_padded, "num_token_non_padded")):
        if t is not None and t.dtype not in (torch.int32, torch.int64):
            raise RuntimeError(f"{name} expects int32 or int64 tensor")
    m = logical_to_physical_map
    n = num_token_non_padded
    with torch.cuda.device(topk_ids.device):
        st = _lib.load().lo_topk_ids_postprocess(
            _lib.ptr(topk_ids), _lib.dtype_code(topk_ids.dtype), topk_ids.shape[0], topk_ids.shape[1],
            _lib.ptr(m.contiguous()) if m is not None else 0, _lib.dtype_code(m.dtype) if m is not None else 0,
            m.numel() if m is not None else 0,
            _lib.ptr(n) if n is not None else 0, _lib.dtype_code(n.dtype) if n is not None else 0,
            _lib.current_stream(topk_ids.device))
    _lib.check(st, "topk_ids_postprocess")
