"""A stack of MoE blocks with the attention stubbed as identity: h <- x + MoE_l(h) for l = 0..L-1.

This is the shape of the engine's verify loop (demo/src/execution/cb_executor.py:406-450 of the
reference: per layer forward_attention -> route_experts -> forward_moe) with everything but the MoE
block removed, used to measure the block at model depth (48 layers of the Qwen3-30B-A3B shape).  The
residual add of forward_moe (demo/src/model/qwen3_runner.py:226) is kept and fused into the combine
kernel; norms are skipped.  Because there are no norms, the residual stream is re-anchored at the
input tokens x in every block (with random-init weights h <- h + MoE(h) squares its magnitude every
few layers through SiLU(g)*u and overflows bf16 long before layer 48); each block still consumes the
previous block's output, so the layers stay serially dependent.  Works on one GPU (MoEContext.forward_fused) and expert-parallel
(ExpertParallelMoE.forward)."""
from __future__ import annotations

from typing import Optional

import torch

from .context import MoEContext
from .ep import ExpertParallelMoE


class MoEStack:
    def __init__(self, ctx: MoEContext, num_layers: int, ep: Optional[ExpertParallelMoE] = None):
        self.ctx, self.L, self.ep = ctx, num_layers, ep

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        """h [T,H] (this rank's tokens when expert-parallel) -> [T,H] after L blocks."""
        x = h
        for layer in range(self.L):
            if self.ep is not None and self.ep.world > 1:
                h = self.ep.forward(layer, h, residual=x)
            else:
                h = self.ctx.forward_fused(layer, h, residual=x)
        return h
