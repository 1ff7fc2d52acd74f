"""Gated-activation entry points of the per-channel W8A8 path
(reference: python/lightop/activation.py -> python/lightop/fuse_silu_mul_quant.py:44-62)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib


def fuse_silu_mul_quant(input: torch.Tensor, num_local_tokens_tensor: Optional[torch.Tensor] = None, topk: int = 1,
                        expect_m: int = -1, output: Optional[torch.Tensor] = None,
                        scales: Optional[torch.Tensor] = None, expert_ids: Optional[torch.Tensor] = None
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``silu(input[:, :d]) * input[:, d:]`` followed by per-token INT8 quantisation.

    Signature of the reference's wrapper (python/lightop/fuse_silu_mul_quant.py:44-62): returns
    ``(output int8 [rows, d], scales fp32 [rows, 1])``.  Semantics of its kernel
    (csrc/kernels/gated_activation/fuse_silu_mul_quant.cu:90-131): the activation is rounded to
    the element type after SiLU and after the product, ``scale = max|act| / 127`` and
    ``q = sat(rint(act * (127 / max)))``.  The expert-parallel masking arguments
    (``num_local_tokens_tensor``, ``expect_m``, ``expert_ids``) are not implemented.
    """
    if num_local_tokens_tensor is not None or expert_ids is not None:
        raise NotImplementedError("the expert-parallel masking arguments are not implemented")
    _lib.require_cuda(input, output, scales)
    if input.dim() != 2 or input.dtype != torch.bfloat16:
        raise RuntimeError("fuse_silu_mul_quant expects a 2-D bfloat16 tensor [rows, 2*d]")
    if not input.is_contiguous():
        input = input.contiguous()
    rows, d2 = input.shape
    d = d2 // 2
    if d2 % 16 != 0:
        raise RuntimeError("the row length must be a multiple of 16")
    if output is None:
        output = torch.empty(rows, d, dtype=torch.int8, device=input.device)
    if scales is None:
        scales = torch.empty((rows, 1), device=input.device, dtype=torch.float32)
    if output.dtype != torch.int8 or tuple(output.shape) != (rows, d) or not output.is_contiguous():
        raise RuntimeError("output must be a contiguous int8 tensor [rows, d]")
    if scales.dtype != torch.float32 or scales.numel() != rows or not scales.is_contiguous():
        raise RuntimeError("scales must be a contiguous float32 tensor with one value per row")
    if rows == 0:
        return output, scales
    with torch.cuda.device(input.device):
        st = _lib.load().lo_silu_mul_quant_int8(_lib.ptr(input), rows, d, _lib.ptr(output), _lib.ptr(scales),
                                                _lib.current_stream(input.device))
    _lib.check(st, "fuse_silu_mul_quant")
    return output, scales


def fuse_silu_mul_quant_ep(input: torch.Tensor, tokens_per_expert: Optional[torch.Tensor] = None,
                           num_local_tokens_tensor: Optional[torch.Tensor] = None, topk: int = 1,
                           expect_m: int = -1) -> Tuple[torch.Tensor, torch.Tensor]:
    """``fuse_silu_mul_quant`` on the masked layout ``[E, T, 2*d]``: only the first
    ``tokens_per_expert[e]`` rows of expert ``e`` are processed (all rows without it).

    Signature of the reference (python/lightop/fuse_silu_mul_quant.py:235-252): returns
    ``(int8 [E, T, d], fp32 [E, T, 1])``; rows that are not processed hold unspecified values.
    ``num_local_tokens_tensor`` / ``expect_m`` (launch-shaping hints there) are not implemented / ignored.
    """
    if input.dim() != 3:
        raise ValueError(f"Input tensor must be 3-dimensional [E, T, H], but got shape {input.shape}")
    if num_local_tokens_tensor is not None:
        raise NotImplementedError("num_local_tokens_tensor is not implemented")
    _lib.require_cuda(input, tokens_per_expert)
    if input.dtype != torch.bfloat16:
        raise RuntimeError("fuse_silu_mul_quant_ep expects bfloat16 input")
    if not input.is_contiguous():
        input = input.contiguous()
    E, T, H = input.shape
    d = H // 2
    if H % 16 != 0:
        raise RuntimeError("the row length must be a multiple of 16")
    output = torch.empty(E, T, d, dtype=torch.int8, device=input.device)
    scales = torch.empty((E, T, 1), device=input.device, dtype=torch.float32)
    if E * T == 0:
        return output, scales
    counts = None
    if tokens_per_expert is not None:
        if tokens_per_expert.numel() != E:
            raise RuntimeError("tokens_per_expert must hold one count per expert")
        counts = tokens_per_expert.to(torch.int32).contiguous()
    with torch.cuda.device(input.device):
        st = _lib.load().lo_silu_mul_quant_int8_masked(_lib.ptr(input), E, T, d, _lib.ptr(counts), _lib.ptr(output),
                                                       _lib.ptr(scales), _lib.current_stream(input.device))
    _lib.check(st, "fuse_silu_mul_quant_ep")
    return output, scales
