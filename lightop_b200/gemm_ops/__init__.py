"""Dense block-INT8 (W8A8, 128x128) linear APIs and the grouped per-channel GEMMs on expert-grouped rows
(reference: python/lightop/gemm_ops/quantized.py:14-28, python/lightop/gemmopt.py:604-617, 744-751)."""
from .block_int8 import apply_w8a8_block_int8_linear, gemm_w8a8_asm, matmul_block_int8
from .grouped import m_grouped_w8a8_gemm_nt_contig_asm, m_grouped_w8a8_gemm_nt_masked

__all__ = ["apply_w8a8_block_int8_linear", "gemm_w8a8_asm", "matmul_block_int8",
           "m_grouped_w8a8_gemm_nt_contig_asm", "m_grouped_w8a8_gemm_nt_masked"]
