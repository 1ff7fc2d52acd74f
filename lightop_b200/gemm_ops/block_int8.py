"""Dense block-INT8 matmul: int8 activations with per-token-group scales times int8 weights with
128x128 block scales.  It is the grouped GEMM kernel of the MoE path run with a single expert."""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import _lib, device_status_word
from ..quant import per_token_group_quant_int8


def matmul_block_int8(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                      block_size: List[int], output_dtype: torch.dtype = torch.float16,
                      bias: Optional[torch.Tensor] = None, config: Optional[dict] = None) -> torch.Tensor:
    """``C = sum_kb (A_kb @ B_kb^T) * As[:, kb] * Bs[n/128, kb]`` (+ bias).

    Signature of the reference's ``matmul_block_int8``
    (python/lightop/_lmslim_native/layers/gemm/int8_utils.py:298-403).  ``A [..., K]`` int8,
    ``As [..., K/128]`` fp32, ``B [N, K]`` int8, ``Bs [ceil(N/128), K/128]`` fp32.  The kernel writes
    bf16; another ``output_dtype`` is produced by a cast of that result.  ``config`` (Triton tile
    sizes in the reference) is accepted and ignored.
    """
    assert len(block_size) == 2 and block_size[0] == 128 and block_size[1] == 128, "only [128, 128] blocks"
    _lib.require_cuda(A, B, As, Bs, bias)
    if A.dtype != torch.int8 or B.dtype != torch.int8:
        raise RuntimeError("matmul_block_int8 expects int8 operands")
    assert A.shape[-1] == B.shape[-1], "inner dimensions differ"
    assert B.dim() == 2 and B.is_contiguous(), "B must be a contiguous [N, K] matrix"
    N, K = B.shape
    M = A.numel() // K
    assert K % 128 == 0, "K must be a multiple of 128"
    assert As.shape[-1] == K // 128 and As.numel() == M * (K // 128), "As must be [..., K/128]"
    assert tuple(Bs.shape) == ((N + 127) // 128, K // 128), "Bs must be [ceil(N/128), K/128]"
    a2 = A.reshape(M, K).contiguous()
    as2 = As.reshape(M, K // 128).to(torch.float32).contiguous()
    bs2 = Bs.to(torch.float32).contiguous()
    C = torch.empty(M, N, dtype=torch.bfloat16, device=A.device)
    if M:
        lib = _lib.load()
        nbytes = lib.lo_block_int8_linear_workspace_bytes(M)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=A.device)
        with torch.cuda.device(A.device):
            st = lib.lo_block_int8_linear(_lib.ptr(a2), _lib.ptr(as2), _lib.ptr(B), _lib.ptr(bs2), M, N, K,
                                          _lib.ptr(C), _lib.ptr(ws), nbytes, _lib.ptr(device_status_word(A.device)),
                                          _lib.current_stream(A.device))
        _lib.check(st, "matmul_block_int8")
    C = C.reshape(A.shape[:-1] + (N,))
    if output_dtype != torch.bfloat16:
        C = C.to(output_dtype)
    if bias is not None:
        C = C + bias
    return C


def gemm_w8a8_asm(a, b, scale_a, scale_b, block_size, out_dtype, layout="TN"):
    """Dense block-INT8 GEMM with the argument convention of the reference's assembly kernel.

    Reference: ``gemm_w8a8_asm`` (python/lightop/gemmopt.py:633-639); its test passes the activation
    scales transposed, ``scale_a [K/128, M]`` (test/w8a8/test_w8a8_block.py:193-197).
    """
    assert a.dim() == 2 and b.dim() == 2 and a.is_contiguous() and b.is_contiguous()
    assert block_size[0] == 128 and block_size[1] == 128
    m, k = a.shape
    if tuple(scale_a.shape) == (k // 128, m):
        scale_a = scale_a.t()
    return matmul_block_int8(a, b, scale_a.contiguous(), scale_b, block_size, output_dtype=out_dtype)


def apply_w8a8_block_int8_linear(input: torch.Tensor, weight: torch.Tensor, block_size: List[int],
                                 weight_scale: torch.Tensor, input_scale: Optional[torch.Tensor] = None,
                                 bias: Optional[torch.Tensor] = None, config: Optional[dict] = None) -> torch.Tensor:
    """Quantise ``input`` per token per 128-group and multiply by the block-quantised ``weight``.

    Reference: ``apply_w8a8_block_int8_linear`` (int8_utils.py:406-429).
    """
    assert input_scale is None
    input_2d = input.reshape(-1, input.shape[-1])
    output_shape = [*input.shape[:-1], weight.shape[0]]
    q_input, x_scale = per_token_group_quant_int8(input_2d, block_size[1])
    output = matmul_block_int8(q_input, weight, x_scale, weight_scale, block_size, output_dtype=input.dtype,
                               config=config)
    if bias is not None:
        output = output + bias
    return output.to(dtype=input.dtype).view(*output_shape)
