"""Load the reference's own pure-torch functions without importing its package.

TEST INFRASTRUCTURE ONLY.  The reference's test modules import ray / vLLM /
the HIP extension at top level, so they cannot be imported on a CUDA or CPU
box.  The functions of interest are plain torch; this loader parses the file,
keeps only the requested ``FunctionDef`` nodes and executes them in a
namespace holding ``torch``, ``F`` and ``math`` (the reference's CI uses the
same trick, test/ci_tests/test_w8a8_small_m_config.py:63-76).

A reference checkout is looked for in ``$LIGHTOP_REF`` and then in ``baseline/_ref`` under the
repository root.  It exists only where the fixtures are generated; tests that need it skip when
it is absent.
"""
from __future__ import annotations

import ast
import math
import os
from typing import Dict, Iterable, Optional


def reference_root() -> Optional[str]:
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for cand in (os.environ.get("LIGHTOP_REF"), os.path.join(repo, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "test", "moe_w8a8")):
            return cand
    return None


def extract_functions(rel_path: str, names: Iterable[str]) -> Dict[str, object]:
    root = reference_root()
    if root is None:
        raise FileNotFoundError("no reference checkout available")
    import torch
    import torch.nn.functional as F
    with open(os.path.join(root, rel_path), "r", encoding="utf-8") as fh:
        tree = ast.parse(fh.read())
    wanted = set(names)
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in wanted]
    missing = wanted - {n.name for n in body}
    if missing:
        raise KeyError(f"{rel_path}: functions not found: {sorted(missing)}")
    ns = {"torch": torch, "F": F, "math": math, "Optional": Optional}
    exec(compile(ast.Module(body=body, type_ignores=[]), rel_path, "exec"), ns)
    return {n: ns[n] for n in wanted}


def reference_block_functions():
    """(group quant, block matmul) from test/moe_w8a8/benchmark_moe_int8.py:60-139."""
    fns = extract_functions("test/moe_w8a8/benchmark_moe_int8.py",
                            ["native_per_token_group_quant_int8", "native_w8a8_block_int8_matmul"])
    return fns["native_per_token_group_quant_int8"], fns["native_w8a8_block_int8_matmul"]


def reference_align_python():
    """``moe_align_block_size_python`` from test/test_moe_align_block_size.py:26-98."""
    return extract_functions("test/test_moe_align_block_size.py",
                             ["moe_align_block_size_python"])["moe_align_block_size_python"]


def reference_composed_moe():
    """The block MoE composed the way the reference composes its per-channel one.

    ``torch_w8a8_per_column_moe`` (test/moe_w8a8/benchmark_moe_int8.py:163-201)
    is executed with ``per_token_quant_int8`` / ``native_w8a8_per_token_matmul``
    bound to the reference's two *block* functions, i.e. its own expert loop,
    SiLU*mul and combine code run unmodified around its own block kernels.
    """
    quant, mm = reference_block_functions()
    import torch
    import torch.nn.functional as F
    root = reference_root()
    with open(os.path.join(root, "test/moe_w8a8/benchmark_moe_int8.py"), "r", encoding="utf-8") as fh:
        tree = ast.parse(fh.read())
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "torch_w8a8_per_column_moe"]

    # The per-channel loop carries ONE scale per row ([rows, 1]) through
    # ``repeat`` and ``a_s[mask]``.  Group scales ([rows, K/128]) do not fit that
    # shape, so the stubs hand the loop a [rows, 1] tensor of row HANDLES into a
    # table of the real group scales and resolve the handles inside the matmul.
    tables = []

    def per_token_quant_int8(a):
        q, s = quant(a.contiguous(), 128)
        base = sum(t.shape[0] for t in tables)
        tables.append(s.reshape(-1, s.shape[-1]))
        handles = torch.arange(base, base + q.shape[0], dtype=torch.float32).reshape(-1, 1)
        assert base + q.shape[0] < 2 ** 24
        return q, handles

    def native_w8a8_per_token_matmul(A, B, As, Bs, output_dtype=torch.bfloat16):
        idx = As.reshape(-1).to(torch.int64)
        bounds = [0]
        for t in tables:
            bounds.append(bounds[-1] + t.shape[0])
        which = max(i for i in range(len(tables)) if bounds[i] <= int(idx.min()))
        real = tables[which][idx - bounds[which]]
        return mm(A, B, real, Bs, [128, 128], output_dtype)

    ns = {"torch": torch, "F": F, "math": math,
          "per_token_quant_int8": per_token_quant_int8,
          "native_w8a8_per_token_matmul": native_w8a8_per_token_matmul}
    exec(compile(ast.Module(body=body, type_ignores=[]), "benchmark_moe_int8.py", "exec"), ns)
    return ns["torch_w8a8_per_column_moe"]


def reference_channel_functions(per_token_quant):
    """(per-token matmul, composed per-channel MoE) from test/moe_w8a8/benchmark_moe_int8.py:142-201.

    ``torch_w8a8_per_column_moe`` calls ``per_token_quant_int8``, which in the reference is a
    Triton kernel and cannot run on a CPU; the caller passes the restatement to bind under that
    name.  Everything else (the matmul, the expert loop, SiLU*mul, the weighted sum) is the
    reference's own code.
    """
    import torch
    import torch.nn.functional as F
    mm = extract_functions("test/moe_w8a8/benchmark_moe_int8.py", ["native_w8a8_per_token_matmul"])[
        "native_w8a8_per_token_matmul"]
    root = reference_root()
    with open(os.path.join(root, "test/moe_w8a8/benchmark_moe_int8.py"), "r", encoding="utf-8") as fh:
        tree = ast.parse(fh.read())
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "torch_w8a8_per_column_moe"]
    ns = {"torch": torch, "F": F, "math": math, "per_token_quant_int8": per_token_quant,
          "native_w8a8_per_token_matmul": mm}
    exec(compile(ast.Module(body=body, type_ignores=[]), "benchmark_moe_int8.py", "exec"), ns)
    return mm, ns["torch_w8a8_per_column_moe"]


def reference_gate_model():
    """``requested_baseline_moe_gate`` (with ``biased_grouped_topk_impl``) from
    test/ci_tests/test_fused_moe_gate.py:9-117: the reference's torch model of ``moe_fused_gate``."""
    fns = extract_functions("test/ci_tests/test_fused_moe_gate.py",
                            ["biased_grouped_topk_impl", "requested_baseline_moe_gate"])
    # the second function calls the first by name: give both the same globals
    fns["requested_baseline_moe_gate"].__globals__["biased_grouped_topk_impl"] = fns["biased_grouped_topk_impl"]
    return fns["requested_baseline_moe_gate"]


def reference_grouped_layout_models():
    """(``torch_gemm`` of the contiguous layout, ``native_w8a8_perChannel_batch_matmul`` of the masked one)."""
    contig = extract_functions("test/w8a8/test_w8a8_deepgemm_contig.py", ["torch_gemm"])["torch_gemm"]
    masked = extract_functions("test/deepgemm/w8a8_moe_groupgemm_mask_marlin_correctness.py",
                               ["native_w8a8_perChannel_batch_matmul"])["native_w8a8_perChannel_batch_matmul"]
    return contig, masked


def reference_gate_variant_models():
    """(Kimi-K2 gate model, sqrt-softplus gate model) from test/ci_tests/test_kimi_k2_moe_fused_gate.py:14-43 and
    test/ci_tests/test_moe_fused_gate_sqrtsoftplus.py:9-45."""
    kimi = extract_functions("test/ci_tests/test_kimi_k2_moe_fused_gate.py",
                             ["kimi_k2_biased_topk_impl_ref"])["kimi_k2_biased_topk_impl_ref"]
    ssp = extract_functions("test/ci_tests/test_moe_fused_gate_sqrtsoftplus.py",
                            ["reference_moe_fused_gate_sqrtsoftplus"])["reference_moe_fused_gate_sqrtsoftplus"]
    return kimi, ssp
