"""Grouped INT8 GEMM over expert-sorted row blocks (reference: python/lightop/gemmopt.py:437-457)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import _lib


def moe_gemm_w8a8(input: torch.Tensor, b_qweight: torch.Tensor, output: torch.Tensor, a_scale: torch.Tensor,
                  b_scale: torch.Tensor, topk_weights: Optional[torch.Tensor], sorted_token_ids: torch.Tensor,
                  experts_ids: torch.Tensor, num_tokens_post_pad: torch.Tensor, top_k: int, config=None
                  ) -> torch.Tensor:
    """``output[id] = (input_q[id // top_k] @ b_qweight[e].T)`` with block scales, per sorted row block.

    Argument order of the reference's ``moe_gemm_w8a8`` (python/lightop/gemmopt.py:437-457).
    Two scale formats are accepted.  Per-channel, the format of the reference's native kernel
    (csrc/moe_gemm/w8a8/moe_w8a8.cu:2389): ``a_scale`` ``[M, 1]``, ``b_scale`` ``[E, N, 1]``.
    Block INT8, the form its Triton ``fused_moe_kernel`` implements
    (python/lightop/_lmslim_native/layers/fused_moe/int8.py:485-541): ``a_scale``
    ``[M, K/128]``, ``b_scale`` ``[E, N/128, K/128]``.  ``topk_weights`` (or None) multiplies
    the fp32 sum before the cast (and before the scales in the per-channel form, :519-532).  ``output`` is ``[M, topk, N]`` (or ``[M*topk, N]``) bf16.
    The block size is taken from ``config['BLOCK_SIZE_M']`` when given, else it is inferred as
    ``sorted_token_ids.numel() // experts_ids.numel()`` rounded to what the buffers imply.
    """
    _lib.require_cuda(input, b_qweight, output, a_scale, b_scale, topk_weights, sorted_token_ids, experts_ids,
                      num_tokens_post_pad)
    if input.dtype != torch.int8 or b_qweight.dtype != torch.int8:
        raise RuntimeError("moe_gemm_w8a8 expects int8 activations and weights")
    if output.dtype != torch.bfloat16:
        raise RuntimeError("moe_gemm_w8a8 writes bfloat16 output")
    E, N, K = b_qweight.shape
    if not (input.is_contiguous() and b_qweight.is_contiguous() and output.is_contiguous()
            and a_scale.is_contiguous() and b_scale.is_contiguous()):
        raise RuntimeError("moe_gemm_w8a8 expects contiguous tensors")
    channel = a_scale.numel() == input.shape[0] and b_scale.numel() == E * N and K != 128
    if K == 128 and a_scale.numel() == input.shape[0] and b_scale.numel() == E * N:
        channel = b_scale.dim() != 3 or b_scale.shape[1] == N      # [E, N(, 1)] is per-channel, [E, N/128, 1] is block
    if not channel and (a_scale.dim() != 2 or a_scale.shape[1] != K // 128
                        or tuple(b_scale.shape) != (E, N // 128, K // 128)):
        raise NotImplementedError("scales must be per-channel (a_scale [M, 1], b_scale [E, N, 1]) or 128x128 blocks "
                                  "(a_scale [M, K/128], b_scale [E, N/128, K/128])")
    block_size = None
    if isinstance(config, dict):
        block_size = config.get("BLOCK_SIZE_M")
    if block_size is None:
        block_size = max(1, -(-sorted_token_ids.numel() // max(1, experts_ids.numel())))
    numel_valid = output.numel() // N
    lib = _lib.load()
    ws_bytes = lib.lo_grouped_gemm_workspace_bytes(sorted_token_ids.numel(), int(block_size), K)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=input.device)
    w = topk_weights.reshape(-1).contiguous() if topk_weights is not None else None
    with torch.cuda.device(input.device):
        entry = lib.lo_moe_grouped_gemm_i8_channel if channel else lib.lo_moe_grouped_gemm_i8_block
        st = entry(
            _lib.ptr(input), _lib.ptr(a_scale), input.shape[0], _lib.ptr(b_qweight), _lib.ptr(b_scale), E, N, K,
            _lib.ptr(output), _lib.ptr(w), _lib.LO_WEIGHT_FP32 if w is not None else _lib.LO_WEIGHT_NONE,
            _lib.ptr(sorted_token_ids), sorted_token_ids.numel(), _lib.ptr(experts_ids),
            _lib.ptr(num_tokens_post_pad), numel_valid, int(top_k), int(block_size), _lib.ptr(ws), ws_bytes,
            _lib.current_stream(input.device))
    _lib.check(st, "moe_gemm_w8a8")
    return output
