"""Mixture-of-experts APIs of the block-INT8 path (reference: python/lightop/moe/__init__.py:81-133)."""
from .expert_parallel import ep_build_m_indices, ep_gather, ep_scatter
from .gemm import moe_gemm_w8a8
from .native import fused_experts_impl_int8, fused_experts_impl_int8_marlin
from .routing import (kimi_k2_moe_fused_gate, moe_align_block_size, moe_align_block_size_out, moe_fused_gate,
                      moe_fused_gate_sqrtsoftplus, moe_fused_gate_sqrtsoftplus_v41_hcu,
                      moe_fused_gate_sqrtsoftplus_v41_hcu_deepep, moe_fused_gate_sqrtsoftplus_v41_hcu_fused, moe_sum, topk_ids_postprocess,
                      topk_softmax)

__all__ = [
    "ep_build_m_indices",
    "ep_gather",
    "ep_scatter",
    "fused_experts_impl_int8",
    "fused_experts_impl_int8_marlin",
    "moe_align_block_size",
    "moe_align_block_size_out",
    "kimi_k2_moe_fused_gate",
    "moe_fused_gate",
    "moe_fused_gate_sqrtsoftplus",
    "moe_fused_gate_sqrtsoftplus_v41_hcu",
    "moe_fused_gate_sqrtsoftplus_v41_hcu_deepep",
    "moe_fused_gate_sqrtsoftplus_v41_hcu_fused",
    "moe_gemm_w8a8",
    "moe_sum",
    "topk_ids_postprocess",
    "topk_softmax",
]
