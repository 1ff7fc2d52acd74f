"""Pure-torch CPU restatement of the reference's per-channel W8A8 INT8 MoE path
(one scale per token for activations, one per output channel for weights).

TEST INFRASTRUCTURE ONLY -- the product never routes through this file.

Parity status: PARTLY PINNED.
  * ``per_token_matmul`` is checked bit-for-bit against the reference's own torch
    function ``native_w8a8_per_token_matmul`` (test/moe_w8a8/benchmark_moe_int8.py:142-160)
    and against the fixture generated from it (tests/golden/channel_cases.pt).
  * ``fused_moe_channel_int8`` is checked against the reference's composed torch model
    ``torch_w8a8_per_column_moe`` (test/moe_w8a8/benchmark_moe_int8.py:163-201) within the
    bf16 tolerance of the layer (the two differ in where bf16 roundings fall, see below).
  * ``grouped_matmul_contig`` / ``grouped_matmul_masked`` are checked bit-for-bit against the reference's
    ``torch_gemm`` (test/w8a8/test_w8a8_deepgemm_contig.py:106-147) and
    ``native_w8a8_perChannel_batch_matmul``
    (test/deepgemm/w8a8_moe_groupgemm_mask_marlin_correctness.py:40-57) where a reference checkout exists.
  * ``per_token_quant_int8`` and ``silu_mul_quant_int8`` restate GPU-only code of the
    reference (a Triton kernel and a HIP kernel) that cannot run where the fixtures are
    made: PARITY UNPINNED for these two; they follow the formulas of the cited lines.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .moe_block_int8 import moe_sum


def per_token_quant_int8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Whole-row symmetric INT8 quantisation.

    Restates the Triton kernel ``_per_token_quant_int8``
    (python/lightop/_lmslim_native/layers/gemm/int8_utils.py:21-44): everything in
    fp32; ``absmax = max(max|x|, 1e-10)``; ``scale = absmax / 127``; the row is
    multiplied by the scalar ``127 / absmax`` and rounded with ``nearbyint`` (half to
    even).  Returns int8 ``x_q`` shaped like ``x`` and fp32 scales ``[..., 1]``.
    """
    xf = x.to(torch.float32)
    absmax = xf.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10)
    scale = absmax / 127.0
    inv = torch.tensor(127.0, dtype=torch.float32) / absmax
    x_q = torch.round(xf * inv).to(torch.int8)      # torch.round is round-half-to-even
    return x_q, scale


def per_token_matmul(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                     output_dtype=torch.bfloat16, row_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``C = (A_q @ B_q^T) * As * Bs`` with per-token ``As [M,1]`` and per-channel ``Bs [N]``.

    Restates ``native_w8a8_per_token_matmul`` (test/moe_w8a8/benchmark_moe_int8.py:142-160):
    the integer products are summed exactly (the reference sums them in an fp32 matmul,
    which is exact while partial sums stay below 2^24; the kernels sum in int32), the sum
    is converted to fp32 and multiplied by ``As`` first, then by ``Bs``.  ``row_weight``
    (fp32 ``[M]``), when given, multiplies the converted sum BEFORE the scales: the order
    of the reference's kernel when it applies the routed weight
    (python/lightop/_lmslim_native/layers/fused_moe/int8.py:519-532).
    """
    acc = torch.matmul(A.to(torch.float64), B.to(torch.float64).t()).to(torch.float32)
    if row_weight is not None:
        acc = acc * row_weight.to(torch.float32).reshape(-1, 1)
    C = As.to(torch.float32).reshape(-1, 1) * acc * Bs.to(torch.float32).reshape(1, -1)
    return C.to(output_dtype)


def silu_mul_quant_int8(inter: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``act = silu(gate) * up`` then per-token INT8 quantisation of bf16 rows ``[rows, 2d]``.

    Restates ``act_and_mul_kernel_quant``
    (csrc/kernels/gated_activation/fuse_silu_mul_quant.cu:90-131) with an exact fp32 SiLU
    (the reference's kernel uses approximate exp2 / reciprocal instructions of its GPU):
    SiLU is evaluated in fp32 and cast to the element type, the product with ``up`` is
    taken in the element type; ``scale = max|act| / 127`` without a lower clamp;
    ``q = sat(rint(act * (127 / max)))`` with the inverse taken as 0 for a row of zeros.
    """
    d = inter.shape[-1] // 2
    gate = inter[..., :d].to(torch.float32)
    silu = (gate / (1.0 + torch.exp(-gate))).to(inter.dtype)
    act = (silu * inter[..., d:]).to(torch.float32)
    amax = act.abs().amax(dim=-1, keepdim=True)
    scale = amax / 127.0
    inv = torch.where(amax == 0, torch.zeros_like(amax), torch.tensor(127.0, dtype=torch.float32) / amax)
    q = torch.round(act * inv).clamp(-128, 127).to(torch.int8)
    return q, scale


def fused_moe_channel_int8(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                           w1_s: torch.Tensor, w2_s: torch.Tensor,
                           topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                           expert_map: Optional[torch.Tensor] = None,
                           routed_scaling_factor: float = 1.0,
                           shared_output: Optional[torch.Tensor] = None,
                           return_intermediates: bool = False):
    """The per-channel fused expert layer, stage by stage as the reference runs it
    (python/lightop/_lmslim_native/layers/fused_moe/int8.py:735-905): per-token quant of
    ``x`` -> gate_up GEMM to bf16 -> ``fuse_silu_mul_quant`` -> down GEMM with the routed
    weight multiplied in fp32 before the scales -> ``moe_sum`` (fp32 accumulation over the
    top-k slots, times ``routed_scaling_factor``, plus ``shared_output``).

    ``w1 [E, 2I, H]`` / ``w2 [E, H, I]`` int8, ``w1_s [E, 2I]`` / ``w2_s [E, H]`` fp32 (a
    trailing singleton dimension is accepted).  ``expert_map`` maps global to local expert
    ids, -1 = not on this rank: such slots contribute nothing.
    """
    M, H = x.shape
    E = w1.shape[0]
    k = topk_ids.shape[1]
    w1_s = w1_s.reshape(E, -1)
    w2_s = w2_s.reshape(E, -1)
    x_q, x_s = per_token_quant_int8(x)
    ids = topk_ids.reshape(-1).to(torch.int64)
    local = ids if expert_map is None else expert_map.to(torch.int64)[ids]
    tok = torch.arange(M * k) // k
    wflat = topk_weights.reshape(-1).to(torch.float32)
    cache3 = torch.zeros(M * k, H, dtype=x.dtype)
    inter_all = {}
    for e in range(E):
        rows = torch.nonzero(local == e).reshape(-1)
        if rows.numel() == 0:
            continue
        h = per_token_matmul(x_q[tok[rows]], w1[e], x_s[tok[rows]], w1_s[e], x.dtype)
        a_q, a_s = silu_mul_quant_int8(h)
        cache3[rows] = per_token_matmul(a_q, w2[e], a_s, w2_s[e], x.dtype, row_weight=wflat[rows])
        if return_intermediates:
            inter_all[e] = (rows, h, a_q, a_s)
    valid = (local >= 0).reshape(M, k)
    y = moe_sum(cache3.reshape(M, k, H) * valid.unsqueeze(-1).to(x.dtype), routed_scaling_factor, shared_output)
    if return_intermediates:
        return y, dict(x_q=x_q, x_s=x_s, cache3=cache3.reshape(M, k, H), experts=inter_all)
    return y


def grouped_matmul_contig(A: torch.Tensor, As: torch.Tensor, B: torch.Tensor, Bs: torch.Tensor,
                          m_indices: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Contiguous grouped layout: ``out[m] = (A[m] . B[e]) * As[m] * Bs[e]`` with ``e = m_indices[m]``;
    rows with index -1 (or outside the expert range) keep the value they have in ``out``.

    Restates ``torch_gemm`` with alpha 1 and beta 0 (test/w8a8/test_w8a8_deepgemm_contig.py:106-147):
    fp32 dot product (exact here: summed in fp64 and rounded once), times the row scale, times the
    channel scale, cast to the output type.
    """
    res = out.clone()
    E = B.shape[0]
    for e in range(E):
        rows = torch.nonzero(m_indices == e).reshape(-1)
        if rows.numel():
            res[rows] = per_token_matmul(A[rows], B[e], As[rows], Bs[e], out.dtype)
    return res


def grouped_matmul_masked(A: torch.Tensor, As: torch.Tensor, B: torch.Tensor, Bs: torch.Tensor,
                          masked_m: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Masked grouped layout: ``out[e, :masked_m[e]] = (A[e] @ B[e]^T) * As[e] * Bs[e]``; other rows keep their value.

    Restates ``native_w8a8_perChannel_batch_matmul``
    (test/deepgemm/w8a8_moe_groupgemm_mask_marlin_correctness.py:40-57), which computes every row, limited
    to the rows the kernel is asked for (:139-147).
    """
    res = out.clone()
    for e in range(B.shape[0]):
        m = int(masked_m[e])
        if m > 0:
            res[e, :m] = per_token_matmul(A[e, :m], B[e], As[e, :m].reshape(-1, 1), Bs[e].reshape(-1), out.dtype)
    return res
