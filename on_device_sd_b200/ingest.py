"""Per-layer weight slabs: all experts of a layer in ONE device allocation, registered once.

The reference keeps three separate tensors per expert per layer (ParameterLoader / ExpertCache,
demo/src/memory/parameter_loader.py:424-512, demo/src/memory/expert_cache.py:181-208): 3 x E x L
small allocations that the cache moves around, so the drop-in has to re-register pointers whenever
they change.  A model whose experts all live on the GPU can instead be ingested once: the matrices
are copied (host or device sources, any float dtype) into one slab per layer - dense in the model
dtype, or packed to int4 g128 on the device - and the library's expert table points into it for the
lifetime of the slab.  Nothing else changes: the kernels take row-major [out,in] matrices wherever
they lie, 16-byte aligned (every matrix of a slab starts on a 256-byte boundary).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ._lib import W_INT4_G128
from .context import MoEContext
from .quant import pack_int4

_NAMES = ("gate_proj", "up_proj", "down_proj")


def _round_up(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class LayerSlab:
    """One allocation holding every registered expert of one layer; keeps it alive."""

    def __init__(self, ctx: MoEContext, layer: int, experts: Dict[int, Dict[str, torch.Tensor]]):
        self.layer = layer
        H, I = ctx.H, ctx.I
        int4 = ctx.weight_mode == W_INT4_G128
        shapes = {"gate_proj": (I, H), "up_proj": (I, H), "down_proj": (H, I)}
        elem = torch.empty((), dtype=ctx.dtype).element_size()
        sizes: List[int] = []
        for name in _NAMES:
            o, i = shapes[name]
            sizes.append(_round_up(o * i // 2 if int4 else o * i * elem))
            if int4:
                sizes.append(_round_up(o * (i // 128) * 2))
        per_expert = sum(sizes)
        ids = sorted(experts)
        self.buffer = torch.empty(per_expert * len(ids), dtype=torch.uint8, device=ctx.device)
        self.bytes = self.buffer.numel()
        self.views: Dict[int, Dict[str, torch.Tensor]] = {}
        for n, e in enumerate(ids):
            off = n * per_expert
            params: Dict[str, torch.Tensor] = {}
            it = iter(sizes)
            for name in _NAMES:
                o, i = shapes[name]
                src = experts[e][name]
                if tuple(src.shape) != (o, i):
                    raise ValueError(f"expert {e} {name}: expected shape {(o, i)}, got {tuple(src.shape)}")
                if int4:
                    q, s = pack_int4(src.to(device=ctx.device, dtype=torch.bfloat16).contiguous())
                    nq = next(it)
                    params[name] = self.buffer[off:off + o * i // 2].view(o, i // 2)
                    params[name].copy_(q)
                    off += nq
                    ns = next(it)
                    params[name + "_scales"] = self.buffer[off:off + o * (i // 128) * 2].view(torch.bfloat16).view(o, i // 128)
                    params[name + "_scales"].copy_(s)
                    off += ns
                else:
                    nb = next(it)
                    params[name] = self.buffer[off:off + o * i * elem].view(ctx.dtype).view(o, i)
                    params[name].copy_(src.to(device=ctx.device, dtype=ctx.dtype))
                    off += nb
            self.views[e] = params
            ctx.set_expert(layer, e, params)


def ingest_layer(ctx: MoEContext, layer: int, experts: Dict[int, Dict[str, torch.Tensor]]) -> LayerSlab:
    """Copies (and, for an int4 context, quantises) the experts of one layer into a slab and registers them."""
    return LayerSlab(ctx, layer, experts)
