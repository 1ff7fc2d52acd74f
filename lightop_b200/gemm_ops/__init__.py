"""Dense block-INT8 (W8A8, 128x128) linear APIs (reference: python/lightop/gemm_ops/quantized.py:14-28)."""
from .block_int8 import apply_w8a8_block_int8_linear, gemm_w8a8_asm, matmul_block_int8

__all__ = ["apply_w8a8_block_int8_linear", "gemm_w8a8_asm", "matmul_block_int8"]
