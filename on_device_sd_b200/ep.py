"""Expert parallelism for the MoE block: experts sharded across ranks, tokens exchanged over NCCL.

Not in the reference (single GPU; "expert distribution across GPUs" is future work there,
demo/others.md:58-62).  One process per GPU, torch.distributed for the plumbing:

    rank r owns experts [r*E/G, (r+1)*E/G); the router weight is replicated.
    1. route        each rank routes its own T/G tokens                      (K1, local)
    2. dispatch     all-gather of x and of the ids: with top-8 over 8 ranks a token is needed by
                    ~5 ranks out of 8, so gathering every token everywhere IS the dispatch; both
                    collectives have fixed sizes, so no count exchange and no host sync
    3. experts      FFN of the local experts over every rank's tokens; outputs written in pair order
                    (row t*K+k), zeros for pairs served elsewhere                (K2, K3, scatter)
    4. return       sum reduce-scatter of the pair buffers: every row is non-zero on exactly one
                    rank, so the sum is exact, and each rank receives the rows of its own tokens
    5. combine      weighted accumulation in the model dtype, same order as on one GPU (K4, local)

The result is bit-identical to the single-GPU result for any number of ranks, because every
expert output row is computed by the same kernel on the same inputs and the combine sees the same
rows in the same order.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Sequence

import torch
import torch.distributed as dist


def expert_range(num_experts: int, world: int, rank: int) -> range:
    """Contiguous block of experts owned by `rank` (requires world | num_experts)."""
    if num_experts % world:
        raise ValueError(f"num_experts={num_experts} is not divisible by the number of ranks {world}")
    per = num_experts // world
    return range(rank * per, (rank + 1) * per)


def owner_of(expert: int, num_experts: int, world: int) -> int:
    return expert // (num_experts // world)


def split_tokens(T: int, world: int, rank: int) -> range:
    """Contiguous token slice of `rank`; T must be a multiple of world (callers pad)."""
    if T % world:
        raise ValueError(f"token count {T} must be a multiple of the number of ranks {world}")
    per = T // world
    return range(rank * per, (rank + 1) * per)


class ExpertParallelMoE:
    """One rank of an expert-parallel MoE block.

    `ctx` supplies the three local steps: route(layer, x) -> (ids, scores);
    ep_local_experts(layer, x_all, ids_all) -> y_pairs [T_all*K, H]; ep_combine(y_pairs, ids,
    scores, order=, residual=) -> out.  On a GPU that is a MoEContext; the CPU tests of the
    collective plumbing pass a stand-in with the same three methods.
    """

    def __init__(self, ctx: Any, num_experts: int, top_k: int, hidden_size: int, group: Optional[dist.ProcessGroup] = None):
        self.ctx, self.E, self.K, self.H = ctx, num_experts, top_k, hidden_size
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.local_experts = expert_range(num_experts, self.world, self.rank)

    def register_local_experts(self, layer: int, experts: Dict[int, Dict[str, torch.Tensor]]) -> None:
        """Registers the experts this rank owns (others in `experts` are ignored)."""
        for e in self.local_experts:
            if e in experts:
                self.ctx.set_expert(layer, e, experts[e])

    def forward(self, layer: int, x_local: torch.Tensor, *, residual: Optional[torch.Tensor] = None,
                order: Optional[Sequence[int]] = None) -> torch.Tensor:
        """x_local [T/G, H] (this rank's tokens) -> [T/G, H]."""
        Tl = x_local.shape[0]
        ids, scores = self.ctx.route(layer, x_local)
        if self.world == 1:
            y_pairs = self.ctx.ep_local_experts(layer, x_local, ids)
            return self.ctx.ep_combine(y_pairs, ids, scores, order=order, residual=residual)
        x_all = torch.empty(Tl * self.world, self.H, dtype=x_local.dtype, device=x_local.device)
        ids_all = torch.empty(Tl * self.world, self.K, dtype=torch.int64, device=x_local.device)
        dist.all_gather_into_tensor(x_all, x_local.contiguous(), group=self.group)
        dist.all_gather_into_tensor(ids_all, ids, group=self.group)
        y_pairs = self.ctx.ep_local_experts(layer, x_all, ids_all)          # [T*K, H], zeros where not served here
        y_own = torch.empty(Tl * self.K, self.H, dtype=x_local.dtype, device=x_local.device)
        dist.reduce_scatter_tensor(y_own, y_pairs, op=dist.ReduceOp.SUM, group=self.group)
        return self.ctx.ep_combine(y_own, ids, scores, order=order, residual=residual)
