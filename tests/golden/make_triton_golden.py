"""Golden vectors of the reference's two Triton quantisation kernels, produced by the kernels themselves.

The reference has ``per_token_quant_int8`` and ``per_token_group_quant_int8`` only as Triton kernels
(python/lightop/_lmslim_native/layers/gemm/int8_utils.py:21-71 and :74-193).  Triton's interpreter mode
(``TRITON_INTERPRET=1``) executes a ``@triton.jit`` function on CPU tensors, so the kernels can be run where no
GPU is: this script copies nothing into the repository, it loads the four functions from a reference checkout
(``$LIGHTOP_REF``) into a temporary module (Triton needs a real source file), runs them on seeded inputs and
stores inputs' seeds and the outputs in ``triton_quant_cases.pt``.

One function of the per-token kernel has no interpreter implementation, ``libdevice.nearbyint``; the temporary
module binds that name to an explicit round-half-to-even built from ``tl.floor`` / ``tl.where``, which is what the
instruction does.  Everything else (maximum, scale, the multiplication by 127 / absmax, the conversions) is the
reference's own code.

    LIGHTOP_REF=<checkout> TRITON_INTERPRET=1 python tests/golden/make_triton_golden.py
"""
from __future__ import annotations

import ast
import importlib.util
import os
import sys
import tempfile

os.environ.setdefault("TRITON_INTERPRET", "1")

import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
REL = "python/lightop/_lmslim_native/layers/gemm/int8_utils.py"
NAMES = {"_per_token_quant_int8", "per_token_quant_int8", "_per_token_group_quant_int8", "per_token_group_quant_int8"}

HEADER = '''import torch
import triton
import triton.language as tl
from typing import Tuple


class _Libdevice:
    """libdevice.nearbyint for the interpreter: round half to even."""

    @staticmethod
    @triton.jit
    def nearbyint(x):
        r = tl.floor(x + 0.5)
        tie = (x + 0.5) == r
        odd = (r - 2.0 * tl.floor(r * 0.5)) != 0.0
        return tl.where(tie & odd, r - 1.0, r)


libdevice = _Libdevice

'''

# (name, rows, columns, dtype, seed): the reference test's pinned case first (test/test_quant_per_token_quant_int8.py:59-72),
# then one case per launch configuration of the group kernel (m <= 16, m <= 256, m > 256).  The element count is a
# multiple of the configuration's block (128 / 1024 / 2048): the kernel stores its scales without a mask, so a ragged last
# block writes past the end of the scale array
CASES = [("pinned_3x256", 3, 256, torch.bfloat16, 6), ("small_m", 16, 512, torch.bfloat16, 1), ("mid_m", 64, 256, torch.bfloat16, 2),
         ("large_m", 320, 128, torch.bfloat16, 3), ("fp16", 32, 384, torch.float16, 4), ("fp32", 40, 256, torch.float32, 5),
         ("hidden_7168", 9, 7168, torch.bfloat16, 7)]


def load_reference_kernels():
    root = os.environ.get("LIGHTOP_REF")
    if not root:
        raise SystemExit("set LIGHTOP_REF to a checkout of the reference")
    tree = ast.parse(open(os.path.join(root, REL), encoding="utf-8").read())
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in NAMES]
    assert {n.name for n in body} == NAMES
    code = HEADER + "\n\n".join(ast.unparse(n) for n in body) + "\n"
    tmp = tempfile.mkdtemp(prefix="lo_triton_ref_")
    path = os.path.join(tmp, "ref_triton_quant.py")
    with open(path, "w") as fh:
        fh.write(code)
    spec = importlib.util.spec_from_file_location("ref_triton_quant", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_triton_quant"] = mod
    spec.loader.exec_module(mod)
    return mod


def make_input(rows, cols, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * 3.0).to(dtype)


def main():
    ref = load_reference_kernels()
    out = {}
    for name, rows, cols, dtype, seed in CASES:
        x = make_input(rows, cols, dtype, seed)
        gq, gs = ref.per_token_group_quant_int8(x.clone(), 128)
        tq, ts = ref.per_token_quant_int8(x.clone())
        out[name] = dict(rows=rows, cols=cols, dtype=str(dtype).replace("torch.", ""), seed=seed,
                         group_q=gq.clone(), group_s=gs.clone(), token_q=tq.clone(), token_s=ts.clone())
        print(name, tuple(x.shape), dtype, "group", tuple(gq.shape), tuple(gs.shape), "token", tuple(tq.shape), tuple(ts.shape))
    torch.save(out, os.path.join(HERE, "triton_quant_cases.pt"))


if __name__ == "__main__":
    main()
