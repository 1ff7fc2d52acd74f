"""CPU test of the drop-in name: ``lightop.*`` are the modules of ``lightop_b200`` themselves, with the names of the
reference's categorized API for this path (reference tests: test/test_moe_existing_api.py:175-214,306-330,
test/test_quant_per_token_quant_int8.py:22-25)."""
import importlib

import pytest


def test_modules_are_the_same_objects():
    import lightop
    import lightop_b200
    assert lightop.moe is lightop_b200.moe
    assert lightop.quant is lightop_b200.quant
    assert lightop.activation is lightop_b200.activation
    assert lightop.gemm_ops is lightop_b200.gemm_ops
    assert importlib.import_module("lightop.moe") is lightop_b200.moe
    assert importlib.import_module("lightop.moe.routing") is importlib.import_module("lightop_b200.moe.routing")
    assert importlib.import_module("lightop.quant.int8") is importlib.import_module("lightop_b200.quant.int8")


MOE_NAMES = ["topk_softmax", "moe_align_block_size", "moe_align_block_size_out", "moe_sum", "moe_gemm_w8a8",
             "fused_experts_impl_int8", "fused_experts_impl_int8_marlin", "ep_scatter", "ep_gather", "ep_build_m_indices",
             "moe_fused_gate", "topk_ids_postprocess", "kimi_k2_moe_fused_gate", "moe_fused_gate_sqrtsoftplus"]
QUANT_NAMES = ["per_token_group_quant_int8", "per_token_quant_int8"]


@pytest.mark.parametrize("name", MOE_NAMES)
def test_moe_inventory(name):
    from lightop import moe
    import lightop_b200
    assert callable(getattr(moe, name))
    assert getattr(moe, name) is getattr(lightop_b200.moe, name)


@pytest.mark.parametrize("name", QUANT_NAMES)
def test_quant_inventory(name):
    from lightop import quant
    import lightop_b200
    assert getattr(quant, name) is getattr(lightop_b200.quant, name)


def test_from_imports_work_as_in_the_reference():
    from lightop.moe import fused_experts_impl_int8, moe_align_block_size  # noqa: F401
    from lightop.quant import per_token_group_quant_int8  # noqa: F401
    from lightop.activation import fuse_silu_mul_quant  # noqa: F401
    from lightop.gemm_ops import gemm_w8a8_asm  # noqa: F401
