"""Seeded synthetic MoE layers.  They stand in for the Qwen3-30B-A3B / Mixtral checkpoints the
reference's benchmarks load (absent here), taking their shapes; distributions follow the
reference's own test fixture (demo/tests/conftest.py:30-32): weights ~ N(0, 0.02^2),
activations ~ N(0, 1)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

CONFIGS = {
    # name: (H, E, K, I, dtype)
    "toy_fp32": (1024, 8, 2, 2816, torch.float32),
    "mixtral": (4096, 8, 2, 14336, torch.bfloat16),
    "qwen3": (2048, 128, 8, 768, torch.bfloat16),
    "tiny_fp16": (32, 4, 2, 16, torch.float16),   # the reference's unit-test config (conftest.py:108-128)
}


@dataclass
class SynthLayer:
    H: int
    E: int
    K: int
    I: int
    dtype: torch.dtype
    gate_w: torch.Tensor
    experts: Dict[int, Dict[str, torch.Tensor]]
    x: torch.Tensor


def make_layer(H: int, E: int, K: int, I: int, dtype: torch.dtype, T: int, *, seed: int = 0,
               device: str | torch.device = "cpu", gen_device: Optional[str] = None) -> SynthLayer:
    """Draws, in this fixed order and in fp32, the gate weight, experts 0..E-1 (gate, up, down)
    and x [T,H] from one generator seeded with `seed`; casts to `dtype`; moves to `device`.

    gen_device="cpu" (default) gives the same bits on every machine; gen_device="cuda" draws on
    the GPU (fast for multi-GB layers; a different but equally distributed stream)."""
    gen_device = gen_device or "cpu"
    g = torch.Generator(device=gen_device).manual_seed(seed)

    def draw(*shape, std=1.0):
        t = torch.randn(*shape, generator=g, device=gen_device, dtype=torch.float32)
        if std != 1.0:
            t = t * std
        return t.to(dtype).to(device)

    gate_w = draw(E, H, std=0.02)
    experts = {}
    for e in range(E):
        experts[e] = {"gate_proj": draw(I, H, std=0.02), "up_proj": draw(I, H, std=0.02), "down_proj": draw(H, I, std=0.02)}
    x = draw(T, H)
    return SynthLayer(H, E, K, I, dtype, gate_w, experts, x)


def make_named(name: str, T: int, **kw) -> SynthLayer:
    H, E, K, I, dtype = CONFIGS[name]
    return make_layer(H, E, K, I, dtype, T, **kw)


def zipf_bias(E: int, s: float = 1.1, seed: int = 0) -> torch.Tensor:
    """log-popularity bias b_e = log p_e, p_e ~ rank^-s over a seeded permutation of the experts
    (the load-imbalance stressor of the stacked benchmark configuration)."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(E, generator=g)
    p = (torch.arange(1, E + 1, dtype=torch.float64) ** (-s))
    p = p / p.sum()
    b = torch.empty(E, dtype=torch.float64)
    b[perm] = p.log()
    return b.float()
