"""Expert-parallel local permutation kernels (reference: python/lightop/moe/expert_parallel.py:8-10)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib


def ep_build_m_indices(topk_ids: torch.Tensor, m_indices: torch.Tensor, local_num_experts: int,
                       alignment: int) -> None:
    """Expert id of every row of the aligned expert-contiguous layout, -1 on padding rows.

    Reference: ``ep_build_m_indices`` (csrc/kernels/deepgemm_moe_permute.cu:833,
    csrc/pybind/export.cpp:1137).  Negative ids are ignored.
    """
    _lib.require_cuda(topk_ids, m_indices)
    if m_indices.dtype != torch.int32:
        raise RuntimeError("m_indices must be int32")
    ids = topk_ids.contiguous()
    with torch.cuda.device(ids.device):
        st = _lib.load().lo_ep_build_m_indices(_lib.ptr(ids), _lib.dtype_code(ids.dtype), ids.numel(),
                                               _lib.ptr(m_indices), m_indices.numel(), int(local_num_experts),
                                               int(alignment), _lib.current_stream(ids.device))
    _lib.check(st, "ep_build_m_indices")


def ep_scatter(aq: torch.Tensor, aq_scale: torch.Tensor, topk_ids: torch.Tensor,
               expert_map: Optional[torch.Tensor], expert_num_tokens: torch.Tensor, aq_out: torch.Tensor,
               aq_scale_out: torch.Tensor, m_indices: torch.Tensor, inv_perm: torch.Tensor,
               local_num_experts: int, alignment: int) -> None:
    """Copy every local ``(token, slot)`` row into the expert-contiguous aligned layout.

    Reference: ``ep_scatter`` (csrc/kernels/deepgemm_moe_permute.cu:1080-1188,
    csrc/pybind/export.cpp:611,1765).  The reference carries one fp32 scale per token
    (``aq_scale [T, 1]``); group scales ``[T, H/128]`` are accepted too.  Destination rows are
    assigned in ascending ``(token, slot)`` order inside each expert, so the result is
    reproducible; ``inv_perm`` is -1 for non-local slots.
    """
    _lib.require_cuda(aq, aq_scale, topk_ids, expert_map, expert_num_tokens, aq_out, aq_scale_out, m_indices, inv_perm)
    if aq.dtype != torch.int8 or aq_out.dtype != torch.int8:
        raise RuntimeError("ep_scatter moves int8 rows")
    if aq_scale.dtype != torch.float32 or aq_scale_out.dtype != torch.float32:
        raise RuntimeError("ep_scatter scales must be float32")
    if m_indices.dtype != torch.int32 or inv_perm.dtype != torch.int32:
        raise RuntimeError("m_indices and inv_perm must be int32")
    T, H = aq.shape
    k = topk_ids.shape[1]
    S = aq_scale.shape[-1] if aq_scale.dim() == 2 else 1
    if aq_scale.numel() != T * S or aq_scale_out.numel() != aq_out.shape[0] * S:
        raise RuntimeError("scale tensors do not match the activation rows")
    if expert_map is not None and expert_map.dtype != torch.int32:
        expert_map = expert_map.to(torch.int32)
    counts = expert_num_tokens.to(torch.int32) if expert_num_tokens is not None else None
    ids = topk_ids.contiguous()
    with torch.cuda.device(aq.device):
        st = _lib.load().lo_ep_scatter(
            _lib.ptr(aq.contiguous()), _lib.ptr(aq_scale.contiguous()), S, _lib.ptr(ids), _lib.dtype_code(ids.dtype),
            _lib.ptr(expert_map), _lib.ptr(counts), _lib.ptr(aq_out), _lib.ptr(aq_scale_out), _lib.ptr(m_indices),
            _lib.ptr(inv_perm), T, k, H, aq_out.shape[0], int(local_num_experts), int(alignment),
            _lib.current_stream(aq.device))
    _lib.check(st, "ep_scatter")


def ep_gather(a: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, inv_perm: torch.Tensor,
              expert_map: Optional[torch.Tensor], output: torch.Tensor, specialize_k8: bool = False) -> None:
    """``output[t] = sum_j w[t,j] * a[inv_perm[t,j]]`` over local slots, fp32 accumulation.

    Reference: ``ep_gather`` (csrc/kernels/deepgemm_moe_permute.cu:1235, kernel :947-1022).
    ``specialize_k8`` selects a kernel variant in the reference and is ignored.
    """
    _lib.require_cuda(a, topk_ids, topk_weights, inv_perm, expert_map, output)
    if a.dtype != torch.bfloat16 or output.dtype != torch.bfloat16:
        raise RuntimeError("ep_gather works on bfloat16 rows")
    T, k = topk_ids.shape
    H = a.shape[1]
    if expert_map is not None and expert_map.dtype != torch.int32:
        expert_map = expert_map.to(torch.int32)
    ids = topk_ids.contiguous()
    w = topk_weights.to(torch.float32).contiguous()
    with torch.cuda.device(a.device):
        st = _lib.load().lo_ep_gather(_lib.ptr(a.contiguous()), _lib.ptr(ids), _lib.dtype_code(ids.dtype), _lib.ptr(w),
                                      _lib.ptr(inv_perm.contiguous()), _lib.ptr(expert_map), _lib.ptr(output), T, k, H,
                                      _lib.current_stream(a.device))
    _lib.check(st, "ep_gather")
