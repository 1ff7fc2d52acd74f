"""ctypes binding of ``liblightop_b200.so`` (the C ABI declared in include/lightop_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# LIGHTOP_B200_LIB overrides the location of the shared library (e.g. an instrumented build)
LIB_PATH = os.environ.get("LIGHTOP_B200_LIB") or os.path.join(_HERE, "liblightop_b200.so")

LO_F32, LO_F16, LO_BF16, LO_I32, LO_I64, LO_U32 = 0, 1, 2, 3, 4, 5
LO_GATE_SIGMOID, LO_GATE_SQRT_SOFTPLUS, LO_GATE_SQRT_SOFTPLUS_SAFE = 0, 1, 2
LO_WEIGHT_NONE, LO_WEIGHT_FP32, LO_WEIGHT_BF16_PRODUCT = 0, 1, 2

_DTYPE_CODE = {
    torch.float32: LO_F32, torch.float16: LO_F16, torch.bfloat16: LO_BF16,
    torch.int32: LO_I32, torch.int64: LO_I64,
}
if hasattr(torch, "uint32"):
    _DTYPE_CODE[torch.uint32] = LO_U32

# name -> (restype, argtypes); mirrors include/lightop_b200.h one to one
PROTOTYPES = {
    "lo_version": (c_int, []),
    "lo_last_error": (c_char_p, []),
    "lo_sm_count": (c_int, []),
    "lo_launch_count": (ctypes.c_longlong, []),
    "lo_topk_softmax": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
                                c_void_p, c_void_p]),
    "lo_moe_align_block_size": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_int, c_void_p,
                                        c_int64, c_void_p, c_int64, c_void_p, c_void_p]),
    "lo_group_quant_int8": (c_int, [c_void_p, c_int, c_int64, c_int, c_float, c_void_p, c_void_p, c_void_p]),
    "lo_moe_sum": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int64, c_float, c_void_p,
                           c_void_p, c_void_p]),
    "lo_grouped_gemm_workspace_bytes": (c_size_t, [c_int64, c_int, c_int64]),
    "lo_moe_grouped_gemm_i8_block": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int64,
                                             c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p,
                                             c_void_p, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lo_fused_moe_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int, c_int64, c_int64]),
    "lo_fused_moe_workspace_layout": (c_int, [c_int64, c_int, c_int, c_int, c_int64, c_int64, c_void_p]),
    "lo_fused_moe_block_int8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_int, c_void_p, c_int, c_int64, c_int, c_int, c_int64, c_int64,
                                        c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_size_t,
                                        c_void_p, c_void_p]),
    "lo_fused_moe_block_int8_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_int, c_void_p, c_int, c_int64, c_int, c_int, c_int64, c_int64,
                                                c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p]),
    "lo_ep_dispatch_row_bytes": (c_int64, [c_int64]),
    "lo_ep_dispatch_pack": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int64,
                                    c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "lo_ep_dispatch_plan": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "lo_ep_dispatch_put": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                   c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "lo_expert_rows_block_int8_packed_put": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                     c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_size_t,
                                                     c_void_p, c_void_p]),
    "lo_peer_alloc": (c_int, [c_size_t, c_void_p]),
    "lo_words_to_host": (c_int, [c_void_p, c_void_p, c_int64, c_void_p]),
    "lo_peer_free": (c_int, [c_void_p]),
    "lo_peer_handle_bytes": (c_int, []),
    "lo_peer_export": (c_int, [c_void_p, c_void_p]),
    "lo_peer_open": (c_int, [c_void_p, c_void_p]),
    "lo_peer_close": (c_int, [c_void_p]),
    "lo_expert_rows_packed_workspace_bytes": (c_size_t, [c_int64, c_int, c_int64, c_int64]),
    "lo_expert_rows_block_int8_packed": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_int64, c_int64, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "lo_expert_rows_block_int8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p, c_void_p, c_size_t,
                                          c_void_p, c_void_p]),
    "lo_block_int8_linear_workspace_bytes": (c_size_t, [c_int64]),
    "lo_block_int8_linear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p,
                                     c_void_p, c_size_t, c_void_p, c_void_p]),
    "lo_moe_fused_gate": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "lo_moe_gate_topk": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_float, c_float, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "lo_topk_ids_postprocess": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int64, c_void_p, c_int,
                                        c_void_p]),
    "lo_per_token_quant_int8": (c_int, [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "lo_silu_mul_quant_int8": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "lo_moe_grouped_gemm_i8_channel": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int64,
                                               c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p,
                                               c_void_p, c_int64, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lo_fused_moe_channel_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int, c_int64, c_int64]),
    "lo_fused_moe_channel_int8": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int, c_void_p, c_int, c_int64, c_int, c_int, c_int64, c_int64,
                                          c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_size_t,
                                          c_void_p, c_void_p]),
    "lo_silu_mul_quant_int8_masked": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "lo_m_grouped_gemm_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "lo_m_grouped_w8a8_gemm_nt_contig": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                                 c_int, c_int64, c_int64, c_void_p, c_size_t, c_void_p, c_void_p]),
    "lo_m_grouped_w8a8_gemm_nt_masked": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_int64, c_int64, c_int64, c_void_p, c_size_t, c_void_p, c_void_p]),
    "lo_profile_enable": (c_int, [c_int]),
    "lo_profile_read": (c_int, [c_void_p]),
    "lo_ep_scatter": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64, c_int, c_int,
                              c_void_p]),
    "lo_ep_build_m_indices": (c_int, [c_void_p, c_int, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "lo_ep_gather": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                             c_int64, c_void_p]),
}

_lib = None


class LightopError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python lightop_b200/build.py` "
            "(there is no CPU or eager fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().lo_last_error()
        raise LightopError(f"{what}: status {status}: {msg.decode() if msg else ''}")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def ptr(t) -> int:
    """Device address of a tensor (None -> NULL)."""
    return 0 if t is None else t.data_ptr()


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("lightop_b200 runs on CUDA tensors only (no CPU fallback)")


def current_stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
