"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

These stand in for the reference's benchmark harness inputs
(test/moe_w8a8/moe_benchmark.py:853-967): bf16 activations ~ N(0,1), fp32 router logits
~ N(0,1) (plus a per-expert bias for the Zipf case), int8 weights uniform in [-127,127],
fp32 block scales uniform in [1e-3, 1e-2].
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

CONFIGS: Dict[str, dict] = {
    # E experts, top_k, M tokens, hidden H, intermediate I
    "c0_tiny": dict(E=8, topk=2, M=32, H=256, I=512),
    "c1_dsv3_prefill": dict(E=256, topk=8, M=4096, H=7168, I=2048),
    "c2_dsv3_decode": dict(E=256, topk=8, M=64, H=7168, I=2048),
    "c3_dsv3_ep_rank": dict(E=256, topk=8, M=8192, H=7168, I=2048),
    "c4_qwen3_zipf": dict(E=128, topk=8, M=2048, H=4096, I=1536, zipf=1.2),
}


def make_weights(E: int, H: int, I: int, seed: int = 0, device="cpu"):
    """w1 [E,2I,H] int8, w2 [E,H,I] int8, w1_s [E,2I/128,H/128], w2_s [E,H/128,I/128] fp32."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    w1 = torch.empty(E, 2 * I, H, dtype=torch.int8, device=dev)
    w2 = torch.empty(E, H, I, dtype=torch.int8, device=dev)
    for e in range(E):   # per expert: bounds the size of the int64 temporaries of randint
        w1[e] = torch.randint(-127, 128, (2 * I, H), generator=g, device=dev, dtype=torch.int8)
        w2[e] = torch.randint(-127, 128, (H, I), generator=g, device=dev, dtype=torch.int8)
    w1_s = torch.rand(E, 2 * I // 128, H // 128, generator=g, device=dev) * (1e-2 - 1e-3) + 1e-3
    w2_s = torch.rand(E, H // 128, I // 128, generator=g, device=dev) * (1e-2 - 1e-3) + 1e-3
    return w1, w2, w1_s, w2_s


def make_channel_scales(E: int, H: int, I: int, seed: int = 0, device="cpu"):
    """Per-output-channel weight scales of the per-channel W8A8 mode: w1_s [E,2I], w2_s [E,H] fp32."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed + 7919)
    w1_s = torch.rand(E, 2 * I, generator=g, device=dev) * (1e-3 - 1e-4) + 1e-4
    w2_s = torch.rand(E, H, generator=g, device=dev) * (1e-3 - 1e-4) + 1e-4
    return w1_s, w2_s


def make_activations(M: int, H: int, E: int, seed: int = 1, device="cpu", zipf: Optional[float] = None):
    """x [M,H] bf16 ~ N(0,1) and router logits [M,E] fp32 ~ N(0,1) (+ Zipf bias)."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(M, H, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(M, E, generator=g, device=dev)
    if zipf:
        gp = torch.Generator().manual_seed(seed + 1000)
        rank = torch.randperm(E, generator=gp).to(torch.float32) + 1.0
        logits = logits + (-zipf * torch.log(rank)).to(dev)
    return x, logits


def alg_flops(M: int, topk: int, H: int, I: int) -> float:
    """2 * M * k * (H*2I + I*H): the two grouped GEMMs only."""
    return 6.0 * M * topk * H * I


def alg_bytes(M: int, E: int, H: int, I: int, experts_hit: int) -> float:
    """Weights and block scales of the experts actually selected + x in + y out + logits."""
    w = experts_hit * 3.0 * H * I
    s = experts_hit * 4.0 * (2 * I // 128 * (H // 128) + H // 128 * (I // 128))
    return w + s + 2.0 * M * H + 2.0 * M * H + 4.0 * M * E
