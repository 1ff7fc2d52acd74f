"""Quantisation APIs of the INT8 MoE path (reference: python/lightop/quant/__init__.py:24-39)."""
from .int8 import per_token_group_quant_int8, per_token_quant_int8

__all__ = ["per_token_group_quant_int8", "per_token_quant_int8"]
