"""The reference's package name for this path.

``lightop.moe``, ``lightop.quant``, ``lightop.activation`` and ``lightop.gemm_ops`` are the modules of
:mod:`lightop_b200` themselves (the same objects, not copies), so that code written against the reference's
categorized API (python/lightop/moe/__init__.py:8-133, python/lightop/quant/__init__.py:6-39) imports unchanged:

    from lightop.moe import fused_experts_impl_int8, moe_align_block_size, topk_softmax
    from lightop.quant import per_token_group_quant_int8

Only the entry points of the fused block-INT8 / per-channel INT8 MoE path exist; the reference's other
operators are not provided under this name either.
"""
from __future__ import annotations

import sys

import lightop_b200 as _impl
from lightop_b200 import activation, gemm_ops, moe, quant  # noqa: F401
from lightop_b200 import check_device_status, device_status_word  # noqa: F401

__version__ = _impl.__version__

# every loaded module of the implementation answers to the reference's name as well (lightop.moe.routing, ...)
for _name, _mod in list(sys.modules.items()):
    if _name.startswith("lightop_b200.") and not _name.split(".")[1].startswith("_"):
        sys.modules.setdefault("lightop." + _name[len("lightop_b200."):], _mod)

__all__ = ["activation", "gemm_ops", "moe", "quant", "check_device_status", "device_status_word", "__version__"]
