"""The fused block-INT8 expert layer (reference: python/lightop/moe/native.py:7-23 ->
python/lightop/_lmslim_native/layers/fused_moe/int8.py:628-908)."""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from .. import _lib, device_status_word


def _chunk_size() -> int:
    # same environment knob and default as the reference (python/lightop/envs.py:50-53)
    return int(os.environ.get("LMSLIM_FUSED_MOE_CHUNK_SIZE", "16384"))


def fused_experts_impl_int8(hidden_states: torch.Tensor,
                            w1: torch.Tensor,
                            w2: torch.Tensor,
                            topk_weights: torch.Tensor,
                            topk_ids: torch.Tensor,
                            cache13: Optional[torch.Tensor],
                            inplace: bool = False,
                            activation: str = "silu",
                            apply_router_weight_on_input: bool = False,
                            use_fp8_w8a8: bool = False,
                            use_int8_w8a8: bool = False,
                            use_int8_w8a16: bool = False,
                            use_int4_w4a16: bool = False,
                            per_channel_quant: bool = False,
                            global_num_experts: int = -1,
                            expert_map: Optional[torch.Tensor] = None,
                            w1_scale: Optional[torch.Tensor] = None,
                            w2_scale: Optional[torch.Tensor] = None,
                            w1_zp: Optional[torch.Tensor] = None,
                            w2_zp: Optional[torch.Tensor] = None,
                            a1_scale: Optional[torch.Tensor] = None,
                            a2_scale: Optional[torch.Tensor] = None,
                            block_shape: Optional[List[int]] = None,
                            use_nn_moe: Optional[bool] = False,
                            routed_scaling_factor: Optional[float] = 1.0,
                            shared_output: Optional[torch.Tensor] = None,
                            i_q: Optional[torch.Tensor] = None,
                            i_s: Optional[torch.Tensor] = None, **_) -> torch.Tensor:
    """W8A8 INT8 fused experts: ``y[t] = factor * sum_j w[t,j] * down_e(silu(gate_e(x_t)) * up_e(x_t))``.

    Signature of the reference's ``fused_experts_impl_int8`` (int8.py:628-656); the checks
    below are its own (int8.py:658-667).  Supported configurations: ``use_int8_w8a8=True``,
    ``activation="silu"``, bf16 activations, and either ``block_shape=[128, 128]`` (block
    scales ``[E, N/128, K/128]``) or ``per_channel_quant=True`` with ``block_shape=None``
    (scales ``[E, N, 1]``; per-token activation scales, int8.py:735-905).  Tokens are processed in chunks of ``LMSLIM_FUSED_MOE_CHUNK_SIZE``
    (int8.py:703-721).  The top-k reduction is always performed (the reference's sibling
    path does so, int8_marlin.py:356-366); ``shared_output`` is added after scaling by
    ``routed_scaling_factor`` as in ``moe_sum`` (int8.py:882-888).  ``cache13`` is the
    caller's bf16 scratch of at least ``M * topk * hidden`` elements; None allocates it.
    """
    assert use_int8_w8a8 or use_fp8_w8a8
    assert hidden_states.shape[1] == w1.shape[2], "Hidden size mismatch"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.stride(-1) == 1, "Stride of last dimension must be 1"
    assert w2.stride(-1) == 1, "Stride of last dimension must be 1"
    assert hidden_states.dtype in [torch.float32, torch.float16, torch.bfloat16]
    if not use_int8_w8a8 or use_fp8_w8a8 or use_int8_w8a16 or use_int4_w4a16:
        raise NotImplementedError("only the W8A8 INT8 mode is implemented")
    if block_shape is None:
        # same rule as the reference's moe_kernel_prepare_input (int8.py:287-290)
        assert per_channel_quant, "int8 quantization only supports block or channel-wise"
        channel = True
    elif list(block_shape) == [128, 128] and not per_channel_quant:
        channel = False
    else:
        raise NotImplementedError("implemented: block_shape=[128, 128], or per_channel_quant=True with block_shape=None")
    if activation != "silu":
        raise ValueError(f"Unsupported FusedMoe activation: {activation}")
    if hidden_states.dtype != torch.bfloat16:
        raise NotImplementedError("activations must be bfloat16")
    if w1_zp is not None or w2_zp is not None or a1_scale is not None or a2_scale is not None:
        raise NotImplementedError("zero points and static activation scales do not apply to block INT8")
    if i_q is not None or i_s is not None:
        raise NotImplementedError("pre-quantised inputs (i_q / i_s) are not supported")
    if w1_scale is None or w2_scale is None:
        raise ValueError("w1_scale and w2_scale are required")
    _lib.require_cuda(hidden_states, w1, w2, topk_weights, topk_ids, cache13, expert_map, w1_scale, w2_scale,
                      shared_output)
    if w1.dtype != torch.int8 or w2.dtype != torch.int8:
        raise RuntimeError("w1 and w2 must be int8")
    if not (w1.is_contiguous() and w2.is_contiguous()):
        raise RuntimeError("w1 and w2 must be contiguous [E, N, K] tensors")

    num_tokens, H = hidden_states.shape
    E, N, K = w1.shape
    I = N // 2
    if tuple(w2.shape) != (E, H, I):
        raise RuntimeError(f"w2 must be [{E}, {H}, {I}]")
    if N % 256 != 0 or H % 128 != 0:
        raise NotImplementedError("hidden and intermediate sizes must be multiples of 128")
    if channel:
        if w1_scale.numel() != E * N or w2_scale.numel() != E * H:
            raise RuntimeError("per-channel scales must be [E, N, 1] (or [E, N])")
        if apply_router_weight_on_input and topk_ids.shape[1] != 1:
            raise AssertionError("apply_router_weight_on_input is only implemented for topk=1")
    elif tuple(w1_scale.shape) != (E, N // 128, H // 128) or tuple(w2_scale.shape) != (E, H // 128, I // 128):
        raise RuntimeError("block scales must be [E, N/128, K/128]")
    w1_scale = w1_scale.to(torch.float32).contiguous()
    w2_scale = w2_scale.to(torch.float32).contiguous()
    if global_num_experts == -1:
        global_num_experts = E
    top_k = topk_ids.shape[1]
    if apply_router_weight_on_input and top_k != 1:
        raise AssertionError("apply_router_weight_on_input is only implemented for topk=1")
    if topk_ids.dtype not in (torch.int32, torch.int64):
        topk_ids = topk_ids.to(torch.int32)
    topk_ids = topk_ids.contiguous()
    topk_weights = topk_weights.to(torch.float32).contiguous()
    if expert_map is not None and expert_map.dtype != torch.int32:
        expert_map = expert_map.to(torch.int32)
    if shared_output is not None:
        if tuple(shared_output.shape) != (num_tokens, H) or shared_output.dtype != hidden_states.dtype:
            raise RuntimeError("shared_output must match hidden_states")
        shared_output = shared_output.contiguous()

    CHUNK = _chunk_size()
    M = min(num_tokens, CHUNK)
    need = M * top_k * H
    if cache13 is None:
        cache13 = torch.empty(need, dtype=hidden_states.dtype, device=hidden_states.device)
    if cache13.dtype != hidden_states.dtype or cache13.numel() < need or not cache13.is_contiguous():
        raise RuntimeError(f"cache13 must be a contiguous {hidden_states.dtype} buffer of at least {need} elements")
    out = hidden_states if inplace else torch.empty_like(hidden_states)
    if num_tokens == 0:
        return out

    lib = _lib.load()
    dev = hidden_states.device
    ws_fn = lib.lo_fused_moe_channel_workspace_bytes if channel else lib.lo_fused_moe_workspace_bytes
    ws_bytes = ws_fn(M, E, int(global_num_experts), top_k, H, I)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    status = device_status_word(dev)
    factor = 1.0 if routed_scaling_factor is None else float(routed_scaling_factor)
    with torch.cuda.device(dev):
        stream = _lib.current_stream(dev)
        for begin in range(0, num_tokens, CHUNK):
            end = min(begin + CHUNK, num_tokens)
            m = end - begin
            x_c = hidden_states[begin:end]
            if channel:
                st = lib.lo_fused_moe_channel_int8(
                    _lib.ptr(x_c), _lib.dtype_code(x_c.dtype), _lib.ptr(w1), _lib.ptr(w2), _lib.ptr(w1_scale),
                    _lib.ptr(w2_scale), _lib.ptr(topk_weights[begin:end]), _lib.ptr(topk_ids[begin:end]),
                    _lib.dtype_code(topk_ids.dtype), _lib.ptr(expert_map), int(global_num_experts), m, E, top_k, H, I,
                    _lib.ptr(cache13),
                    _lib.ptr(shared_output[begin:end]) if shared_output is not None else 0, _lib.ptr(out[begin:end]),
                    int(bool(apply_router_weight_on_input)), factor, _lib.ptr(workspace), ws_bytes, _lib.ptr(status),
                    stream)
                _lib.check(st, "fused_experts_impl_int8")
                continue
            st = lib.lo_fused_moe_block_int8(
                _lib.ptr(x_c), _lib.ptr(w1), _lib.ptr(w2), _lib.ptr(w1_scale), _lib.ptr(w2_scale),
                _lib.ptr(topk_weights[begin:end]), _lib.ptr(topk_ids[begin:end]), _lib.dtype_code(topk_ids.dtype),
                _lib.ptr(expert_map), int(global_num_experts), m, E, top_k, H, I, _lib.ptr(cache13),
                _lib.ptr(shared_output[begin:end]) if shared_output is not None else 0, _lib.ptr(out[begin:end]),
                int(bool(apply_router_weight_on_input)), factor, _lib.ptr(workspace), ws_bytes, _lib.ptr(status),
                stream)
            _lib.check(st, "fused_experts_impl_int8")
    return out


def fused_experts_impl_int8_marlin(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
                                   topk_weights: torch.Tensor, topk_ids: torch.Tensor, inplace: bool = False,
                                   activation: str = "silu", apply_router_weight_on_input: bool = False,
                                   use_fp8_w8a8: bool = False, use_int8_w8a8: bool = False,
                                   use_int8_w8a16: bool = False, use_int4_w4a16: bool = False,
                                   per_channel_quant: bool = False, global_num_experts: int = -1,
                                   expert_map: Optional[torch.Tensor] = None,
                                   w1_scale: Optional[torch.Tensor] = None, w2_scale: Optional[torch.Tensor] = None,
                                   **kwargs) -> torch.Tensor:
    """Per-channel W8A8 fused experts with the signature of the reference's
    ``fused_experts_impl_int8_marlin`` (int8_marlin.py:165-195; no ``cache13`` argument, the
    scratch is allocated here as there, :213-222).  The reference's variant expects weights
    pre-shuffled for its matrix cores (``N = w2.shape[1] * 64``, :206); this one takes the plain
    ``[E, N, K]`` layout, everything else is the per-channel path of ``fused_experts_impl_int8``.
    """
    assert use_int8_w8a8 is True and per_channel_quant is True, "Unsupport quant method"
    if kwargs.get("gelu_clamp") is not None or kwargs.get("gelu_smooth_scale") is not None:
        raise NotImplementedError("GELU variants are not implemented")
    for name in ("gelu_clamp", "gelu_smooth_scale"):
        kwargs.pop(name, None)
    kwargs.pop("block_shape", None)
    return fused_experts_impl_int8(hidden_states, w1, w2, topk_weights, topk_ids, None, inplace=inplace,
                                   activation=activation,
                                   apply_router_weight_on_input=apply_router_weight_on_input,
                                   use_fp8_w8a8=use_fp8_w8a8, use_int8_w8a8=use_int8_w8a8,
                                   use_int8_w8a16=use_int8_w8a16, use_int4_w4a16=use_int4_w4a16,
                                   per_channel_quant=True, global_num_experts=global_num_experts,
                                   expert_map=expert_map, w1_scale=w1_scale, w2_scale=w2_scale,
                                   block_shape=None, **kwargs)
