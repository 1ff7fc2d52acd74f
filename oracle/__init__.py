"""CPU oracle for the fused block-INT8 MoE path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is used by the tests, by the smoke check and by the CPU-baseline
leg of the benchmark as the checker the CUDA kernels are compared against.
"""
