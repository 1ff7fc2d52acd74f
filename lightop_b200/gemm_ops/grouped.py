"""Per-channel grouped INT8 GEMMs on expert-grouped rows: the contiguous and the masked layout that
expert-parallel dispatchers hand over (reference: python/lightop/gemmopt.py:604-617, 744-751)."""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch

from .. import _lib, device_status_word


def _operands(a, b):
    inp, a_scale = a
    w, b_scale = b
    _lib.require_cuda(inp, a_scale, w, b_scale)
    if inp.dtype != torch.int8 or w.dtype != torch.int8:
        raise RuntimeError("the grouped W8A8 GEMM expects int8 activations and weights")
    if w.dim() != 3 or not (w.is_contiguous() and inp.is_contiguous()):
        raise RuntimeError("weights must be a contiguous [E, N, K] tensor and the activations contiguous")
    E, N, K = w.shape
    if inp.shape[-1] != K:
        raise RuntimeError("inner dimensions differ")
    if b_scale.numel() != E * N:
        raise RuntimeError("b_scale must hold one value per expert and output channel ([E, N])")
    return inp, a_scale.to(torch.float32).contiguous(), w, b_scale.to(torch.float32).contiguous(), E, N, K


def m_grouped_w8a8_gemm_nt_contig_asm(a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor],
                                      output: torch.Tensor, m_indices: torch.Tensor,
                                      config: Optional[Dict[str, Any]] = None) -> torch.Tensor:
    """``output[m] = (a_q[m] @ b_q[m_indices[m]].T) * a_s[m] * b_s[m_indices[m]]``; rows with index -1 are left as they are.

    Signature of the reference (python/lightop/gemmopt.py:744-751): ``a = (int8 [M, K], fp32 [M])``,
    ``b = (int8 [E, N, K], fp32 [E, N])``, ``output`` bf16 ``[M, N]``, ``m_indices`` int32 ``[M]``.  The
    rows of an expert must be consecutive and padded to a multiple of 128 rows
    (test/w8a8/test_w8a8_deepgemm_contig.py:75-103 pads to 256).  The reference's kernel takes the weights
    pre-shuffled for its matrix cores; this one takes them as they are.  ``config`` is accepted and ignored.
    """
    inp, a_scale, w, b_scale, E, N, K = _operands(a, b)
    _lib.require_cuda(output, m_indices)
    M = inp.shape[0]
    if inp.dim() != 2 or a_scale.numel() != M or m_indices.numel() != M:
        raise RuntimeError("a must be ([M, K], [M]) and m_indices [M]")
    if output.dtype != torch.bfloat16 or tuple(output.shape) != (M, N) or not output.is_contiguous():
        raise RuntimeError("output must be a contiguous bfloat16 [M, N] tensor")
    if m_indices.dtype != torch.int32:
        m_indices = m_indices.to(torch.int32)
    if M == 0:
        return output
    lib = _lib.load()
    ws_bytes = lib.lo_m_grouped_gemm_workspace_bytes(M, E)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=inp.device)
    status = device_status_word(inp.device)
    with torch.cuda.device(inp.device):
        st = lib.lo_m_grouped_w8a8_gemm_nt_contig(_lib.ptr(inp), _lib.ptr(a_scale), _lib.ptr(w), _lib.ptr(b_scale),
                                                  _lib.ptr(output), _lib.ptr(m_indices.contiguous()), M, E, N, K,
                                                  _lib.ptr(ws), ws_bytes, _lib.ptr(status),
                                                  _lib.current_stream(inp.device))
    _lib.check(st, "m_grouped_w8a8_gemm_nt_contig_asm")
    return output


def m_grouped_w8a8_gemm_nt_masked(a: Tuple[torch.Tensor, torch.Tensor], b: Tuple[torch.Tensor, torch.Tensor],
                                  d: torch.Tensor, masked_m: torch.Tensor, expected_m_per_group: int,
                                  config: Optional[Dict[str, Any]] = None) -> torch.Tensor:
    """``d[e, :masked_m[e]] = (a_q[e] @ b_q[e].T) * a_s[e] * b_s[e]``; the other rows of ``d`` are left as they are.

    Signature of the reference (python/lightop/gemmopt.py:604-617): ``a = (int8 [E, max_m, K], fp32
    [E, max_m, 1])``, ``b = (int8 [E, N, K], fp32 [E, N, 1])``, ``d`` bf16 ``[E, max_m, N]``, ``masked_m``
    int32 ``[E]``.  ``expected_m_per_group`` (a tile-selection hint there) and ``config`` are ignored.
    Weights in the plain layout (the reference's kernel takes them pre-shuffled).
    """
    inp, a_scale, w, b_scale, E, N, K = _operands(a, b)
    _lib.require_cuda(d, masked_m)
    if inp.dim() != 3 or inp.shape[0] != E:
        raise RuntimeError("a must be ([E, max_m, K], [E, max_m, 1])")
    max_m = inp.shape[1]
    if a_scale.numel() != E * max_m or masked_m.numel() != E:
        raise RuntimeError("a_scale must be [E, max_m, 1] and masked_m [E]")
    if d.dtype != torch.bfloat16 or tuple(d.shape) != (E, max_m, N) or not d.is_contiguous():
        raise RuntimeError("d must be a contiguous bfloat16 [E, max_m, N] tensor")
    if masked_m.dtype != torch.int32:
        masked_m = masked_m.to(torch.int32)
    if max_m == 0:
        return d
    lib = _lib.load()
    ws_bytes = lib.lo_m_grouped_gemm_workspace_bytes(E * max_m, E)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=inp.device)
    status = device_status_word(inp.device)
    with torch.cuda.device(inp.device):
        st = lib.lo_m_grouped_w8a8_gemm_nt_masked(_lib.ptr(inp), _lib.ptr(a_scale), _lib.ptr(w), _lib.ptr(b_scale),
                                                  _lib.ptr(d), _lib.ptr(masked_m.contiguous()), E, max_m, N, K,
                                                  _lib.ptr(ws), ws_bytes, _lib.ptr(status),
                                                  _lib.current_stream(inp.device))
    _lib.check(st, "m_grouped_w8a8_gemm_nt_masked")
    return d
