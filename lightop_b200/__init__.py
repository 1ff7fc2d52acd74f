"""lightop_b200 -- B200 (sm_100a) implementation of LightOp's fused block-INT8 MoE path.

Sub-packages mirror the reference's categorized API for this path
(``lightop.moe`` -> :mod:`lightop_b200.moe`, ``lightop.quant`` ->
:mod:`lightop_b200.quant`; reference: python/lightop/moe/__init__.py:8-133,
python/lightop/quant/__init__.py:6-39).  Importing the package loads the C-ABI
shared library and fails if it has not been built; nothing here computes on the CPU.
"""
from __future__ import annotations

import torch

from . import _lib

__version__ = "0.1.0"

_lib.load()

_status_words = {}


def device_status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels set when one of their bounded waits ran out."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w


def check_device_status(device=None) -> None:
    """Synchronise and raise if a kernel reported a timed-out wait since the last check."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    w = _status_words.get(idx)
    if w is None:
        return
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise _lib.LightopError(f"a grouped-GEMM wait timed out on the device (waiter code {code})")


from . import activation, gemm_ops, moe, quant  # noqa: E402

__all__ = ["activation", "gemm_ops", "moe", "quant", "check_device_status", "device_status_word", "__version__"]
