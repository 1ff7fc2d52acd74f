"""Pure-torch CPU restatement of the reference's block-INT8 (W8A8, 128x128) MoE path.

TEST INFRASTRUCTURE ONLY -- the product never routes through this file.

Parity status: PINNED.  Every function below is checked bit-for-bit against
the reference's own torch functions (loaded from a reference checkout by
``oracle/ref_extract.py`` when one is present) and against the committed
fixtures under ``tests/golden/`` that were generated from them.

Each function names the reference code it restates (paths are relative to the
reference project's root).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

INT8_MIN, INT8_MAX = -128, 127


def group_quant_int8(x: torch.Tensor, group_size: int = 128, eps: float = 1e-10
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token-group symmetric INT8 quantisation.

    Restates ``native_per_token_group_quant_int8``
    (test/moe_w8a8/benchmark_moe_int8.py:60-83): the group amax is taken and
    clamped to ``eps`` in the INPUT dtype, cast to fp32, divided by 127; the
    quotient ``x / scale`` is an fp32 division, clamped to [-128, 127] and
    converted with ``.to(int8)`` which TRUNCATES toward zero.
    """
    assert x.shape[-1] % group_size == 0
    assert x.is_contiguous()
    xg = x.reshape(x.numel() // group_size, group_size)
    amax = xg.abs().max(dim=-1, keepdim=True)[0].clamp(min=eps).to(torch.float32)
    x_s = amax / INT8_MAX
    x_q = (xg / x_s).clamp(min=INT8_MIN, max=INT8_MAX).to(torch.int8)
    return (x_q.reshape(x.shape),
            x_s.reshape(x.shape[:-1] + (x.shape[-1] // group_size,)))


def block_int8_matmul(A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor,
                      block_size=(128, 128), output_dtype=torch.bfloat16) -> torch.Tensor:
    """``C = sum_kb (A_kb @ B_kb^T) * (As[:, kb] * Bs[nb, kb])`` in fp32, K-block order.

    Restates ``native_w8a8_block_int8_matmul``
    (test/moe_w8a8/benchmark_moe_int8.py:87-139; same function in
    test/w8a8/test_w8a8_block.py:128-175).  The reference loops k-tile outer,
    n-tile inner; here the n-tiles of one k-tile are done in one matmul.  Every
    output element still sees the identical sequence of fp32 operations: an
    exact integer dot (|.| < 2^24), one multiply by the pre-formed scale
    product, one add into the running sum.
    """
    block_n, block_k = block_size
    A = A.to(torch.float32)
    B = B.to(torch.float32)
    M = A.numel() // A.shape[-1]
    N, K = B.shape
    out_shape = A.shape[:-1] + (N,)
    A = A.reshape(M, K)
    As = As.reshape(M, -1)
    k_tiles = (K + block_k - 1) // block_k
    n_tiles = (N + block_n - 1) // block_n
    assert As.shape[1] == k_tiles and Bs.shape == (n_tiles, k_tiles)
    C = torch.zeros((M, N), dtype=torch.float32)
    # per-column index of the n-tile, to expand Bs[:, i] over the N columns
    col_tile = torch.arange(N) // block_n
    for i in range(k_tiles):
        ks = slice(i * block_k, min((i + 1) * block_k, K))
        dot = A[:, ks] @ B[:, ks].t()                       # exact integers in fp32
        s = As[:, i:i + 1] * Bs[:, i][col_tile][None, :]    # fp32 product formed first
        C += dot * s                                         # separate mul, then add
    return C.reshape(out_shape).to(output_dtype)


def route_topk_softmax(logits: torch.Tensor, top_k: int, renormalize: bool = True
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 softmax over experts, top-k in descending order, optional renormalisation.

    Restates the torch side of the reference's routing tests
    (test/test_native_categorized_moe_api.py:188-190:
    ``torch.topk(torch.softmax(x.float(), -1), k)``) and the renormalisation of
    test/moe_w8a8/fuse_moegemm.py:449-450 (``w / w.sum(-1, keepdim=True)``).
    """
    p = torch.softmax(logits.to(torch.float32), dim=-1)
    w, ids = torch.topk(p, top_k, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, ids.to(torch.int32)


def align_block_size(topk_ids: torch.Tensor, num_experts: int, block_size: int,
                     expert_map: Optional[torch.Tensor] = None
                     ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Stable expert-major ordering of the flat ``(token, slot)`` indices, padded per expert.

    Restates ``moe_align_block_size_python`` (test/test_moe_align_block_size.py:26-98):
    counts per (mapped) expert, each count rounded up to ``block_size``,
    exclusive cumsum, sentinel ``numel`` everywhere, then flat indices placed in
    ascending order inside their expert's segment; ``expert_ids[b]`` is the
    expert owning block ``b``.  Returns tensors trimmed to the padded total.
    """
    flat = topk_ids.reshape(-1).to(torch.int64)
    if expert_map is not None:
        flat = expert_map.to(torch.int64)[flat]
    numel = flat.numel()
    counts = torch.bincount(flat[flat >= 0], minlength=num_experts)[:num_experts]
    padded = (counts + block_size - 1) // block_size * block_size
    cums = torch.zeros(num_experts + 1, dtype=torch.int64)
    cums[1:] = torch.cumsum(padded, 0)
    total = int(cums[-1])
    sorted_ids = torch.full((total,), numel, dtype=torch.int32)
    # stable sort by expert == ascending flat index within an expert
    valid = torch.nonzero(flat >= 0).reshape(-1)
    order = valid[torch.sort(flat[valid], stable=True)[1]]
    e_sorted = flat[order]
    start_unpadded = torch.zeros(num_experts + 1, dtype=torch.int64)
    start_unpadded[1:] = torch.cumsum(counts, 0)
    rank = torch.arange(order.numel()) - start_unpadded[e_sorted]
    sorted_ids[cums[e_sorted] + rank] = order.to(torch.int32)
    expert_ids = torch.repeat_interleave(torch.arange(num_experts, dtype=torch.int32),
                                         padded // block_size)
    return sorted_ids, expert_ids, torch.tensor([total], dtype=torch.int32)


def moe_sum(inp: torch.Tensor, factor: float = 1.0, bias: Optional[torch.Tensor] = None
            ) -> torch.Tensor:
    """``out[t] = factor * sum_j inp[t, j] (+ bias[t])`` with fp32 accumulation.

    Restates the contract of the reference's reducer
    (csrc/kernels/moe_align_sum_kernels.cu:604-637: fp32 accumulate over the
    top-k axis, scale, add bias, round once to the output dtype) and its test
    (test/test_moe_sum_opt.py:31-56, vs ``torch.sum(dim=1)``).
    """
    acc = inp.to(torch.float32).sum(dim=1) * factor
    if bias is not None:
        acc = acc + bias.to(torch.float32)
    return acc.to(inp.dtype)


def fused_moe_block_int8(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                         w1_s: torch.Tensor, w2_s: torch.Tensor,
                         topk_weight: torch.Tensor, topk_ids: torch.Tensor,
                         block_shape=(128, 128), return_intermediates: bool = False,
                         quant_fn=None, matmul_fn=None):
    """The composed block-INT8 MoE layer.

    ``quant_fn`` / ``matmul_fn`` replace this module's group quantisation and block matmul by functions of the
    same signatures (the benchmark's CPU arm passes the reference's own two functions when a checkout is found).

    The reference holds only a commented-out call of this function
    (test/moe_w8a8/benchmark_moe_int8.py:225-234); it is composed here exactly
    like its per-channel sibling ``torch_w8a8_per_column_moe`` (:163-201) with
    the two block functions substituted: quantise the input per 128-group,
    replicate rows top_k times, per expert run GEMM1 -> ``silu(gate) * up`` on
    bf16 tensors -> re-quantise -> GEMM2 into ``out[mask]``, then
    ``(out.view(B, k, H) * w.view(B, k, 1).to(bf16)).sum(dim=1)``.
    """
    B, D = x.shape
    topk = topk_ids.shape[1]
    group = block_shape[1]
    quant = quant_fn or group_quant_int8
    matmul = matmul_fn or block_int8_matmul
    a_q, a_s = quant(x, group)
    a_q = a_q.view(B, -1, D).repeat(1, topk, 1).reshape(-1, D)
    a_s = a_s.view(B, 1, -1).repeat(1, topk, 1).reshape(B * topk, -1)
    H = w2.shape[1]
    I = w2.shape[2]
    out = torch.zeros(B * topk, H, dtype=x.dtype)
    flat_w = topk_weight.reshape(-1)
    flat_ids = topk_ids.reshape(-1)
    act_q_all = torch.zeros(B * topk, I, dtype=torch.int8) if return_intermediates else None
    act_s_all = torch.zeros(B * topk, I // group, dtype=torch.float32) if return_intermediates else None
    for e in range(w1.shape[0]):
        mask = flat_ids == e
        if mask.sum():
            inter = matmul(a_q[mask], w1[e], a_s[mask], w1_s[e], list(block_shape), x.dtype)
            d = inter.shape[-1] // 2
            act = F.silu(inter[..., :d]) * inter[..., d:]
            act_q, act_s = quant(act.contiguous(), group)
            if return_intermediates:
                act_q_all[mask] = act_q
                act_s_all[mask] = act_s
            out[mask] = matmul(act_q, w2[e], act_s, w2_s[e], list(block_shape), x.dtype)
    y = (out.view(B, -1, H) * flat_w.view(B, -1, 1).to(out.dtype)).sum(dim=1)
    if return_intermediates:
        return y, dict(a_q=a_q.view(B, topk, D)[:, 0].contiguous(), a_s=a_s.view(B, topk, -1)[:, 0].contiguous(),
                       act_q=act_q_all, act_s=act_s_all, out=out)
    return y


# ---------------------------------------------------------------------------
# Expert-parallel local kernels (reference: csrc/kernels/deepgemm_moe_permute.cu)
# ---------------------------------------------------------------------------

def ep_build_m_indices(topk_ids: torch.Tensor, local_num_experts: int, alignment: int,
                       expert_map: Optional[torch.Tensor] = None, rows: Optional[int] = None
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Expert id of every row of the aligned contiguous layout (-1 for padding rows).

    Restates the layout rule of ``ep_scatter`` / ``ep_build_m_indices``
    (csrc/kernels/deepgemm_moe_permute.cu:833, :1156-1174; known answer in
    test/test_native_categorized_moe_api.py:32-43): per local expert the token
    count is rounded up to ``alignment`` and the segments are laid end to end.
    Returns ``(m_indices, counts)``.
    """
    flat = topk_ids.reshape(-1).to(torch.int64)
    if expert_map is not None:
        ok = flat >= 0
        mapped = torch.full_like(flat, -1)
        mapped[ok] = expert_map.to(torch.int64)[flat[ok]]
        flat = mapped
    ok = (flat >= 0) & (flat < local_num_experts)
    counts = torch.bincount(flat[ok], minlength=local_num_experts)[:local_num_experts]
    padded = (counts + alignment - 1) // alignment * alignment
    total = int(padded.sum())
    if rows is None:
        rows = total
    m = torch.full((rows,), -1, dtype=torch.int32)
    off = 0
    for e in range(local_num_experts):
        m[off:off + int(counts[e])] = e
        off += int(padded[e])
    return m, counts.to(torch.int32)


def ep_gather(a: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
              inv_perm: torch.Tensor, expert_map: Optional[torch.Tensor]) -> torch.Tensor:
    """``out[t] = sum_k w[t,k] * a[inv_perm[t,k]]`` over local experts, fp32 accumulate.

    Restates ``ep_gather`` (csrc/kernels/deepgemm_moe_permute.cu:947-1022).
    """
    T, K = topk_ids.shape
    ids = topk_ids.to(torch.int64)
    if expert_map is not None:
        loc = torch.where(ids >= 0, expert_map.to(torch.int64)[ids.clamp(min=0)], ids)
    else:
        loc = ids
    out = torch.zeros(T, a.shape[1], dtype=torch.float32)
    for k in range(K):
        sel = loc[:, k] >= 0
        rows = inv_perm[:, k].to(torch.int64)
        out[sel] += topk_weights[sel, k:k + 1].to(torch.float32) * a[rows[sel]].to(torch.float32)
    return out.to(a.dtype)
