"""INT8 quantisation entry points (reference: python/lightop/quant/int8.py:13-16)."""
from __future__ import annotations

from typing import Tuple

import torch

from .. import _lib


def per_token_group_quant_int8(x: torch.Tensor, group_size: int, eps: float = 1e-10,
                               dtype: torch.dtype = torch.int8) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token-group symmetric INT8 quantisation of ``x`` along its last dimension.

    Same signature and return values as the reference
    (python/lightop/_lmslim_native/layers/gemm/int8_utils.py:125-193): ``x_q`` int8 with
    the shape of ``x`` and ``x_s`` fp32 ``[..., K / group_size]``.  The values follow the
    reference's torch model (test/moe_w8a8/benchmark_moe_int8.py:60-83): scale =
    amax / 127, ``q = trunc(clamp(x / scale, -128, 127))``.
    """
    assert x.shape[-1] % group_size == 0, \
        "the last dimension of `x` cannot be divisible by `group_size`"
    if dtype != torch.int8:
        raise ValueError("only torch.int8 is supported as the quantised type")
    _lib.require_cuda(x)
    if not x.is_contiguous():
        x = x.contiguous()
    x_q = torch.empty_like(x, dtype=torch.int8)
    x_s = torch.empty(x.shape[:-1] + (x.shape[-1] // group_size,), device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        st = _lib.load().lo_group_quant_int8(_lib.ptr(x), _lib.dtype_code(x.dtype), x.numel() // group_size,
                                             int(group_size), float(eps), _lib.ptr(x_q), _lib.ptr(x_s),
                                             _lib.current_stream(x.device))
    _lib.check(st, "per_token_group_quant_int8")
    return x_q, x_s


def per_token_quant_int8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Whole-row symmetric INT8 quantisation along the last dimension.

    Same signature and return values as the reference
    (python/lightop/_lmslim_native/layers/gemm/int8_utils.py:47-71): ``x_q`` int8 shaped like
    ``x`` and fp32 scales ``x.shape[:-1] + (1,)``; ``scale = max(max|x|, 1e-10) / 127`` and
    ``q = rint(x * (127 / absmax))`` (:38-41).
    """
    _lib.require_cuda(x)
    if not x.is_contiguous():
        x = x.contiguous()
    K = x.shape[-1]
    M = x.numel() // K if K else 0
    x_q = torch.empty_like(x, dtype=torch.int8)
    scales = torch.empty(x.shape[:-1] + (1,), device=x.device, dtype=torch.float32)
    if M == 0:
        return x_q, scales
    with torch.cuda.device(x.device):
        st = _lib.load().lo_per_token_quant_int8(_lib.ptr(x), _lib.dtype_code(x.dtype), M, K, _lib.ptr(x_q),
                                                 _lib.ptr(scales), _lib.current_stream(x.device))
    _lib.check(st, "per_token_quant_int8")
    return x_q, scales
