"""Expert parallelism for the MoE block: experts sharded across ranks, tokens and results exchanged by
the library's own kernels through peer memory over NVLink.

Not in the reference (single GPU; "expert distribution across GPUs" is future work there,
demo/others.md:58-62).  One process per GPU; torch.distributed is the plumbing only - it carries the
64-byte buffer handles at set-up and the barriers around it, never a token:

    rank r owns experts [r*E/G, (r+1)*E/G); the router weight is replicated.
    1. route      each rank routes its own T/G tokens                                     (K1, local)
    2. dispatch   every (token, expert) pair's row is stored straight into the owner rank's receive
                  region for this source, then a count and an epoch flag                   (peer stores)
    3. experts    the owner waits for all sources' flags, groups the received rows by expert and runs
                  its local experts over its LOCAL receive buffer                          (K2, K3)
    4. return     every output row is stored straight into its source rank's return rows, then a flag
    5. combine    the source waits for all owners' flags and accumulates in the model dtype, in the
                  same order as on one GPU                                                 (K4, local)

The result is bit-identical to the single-GPU result: every expert output row is computed by the same
kernel on the same inputs and the combine sees the same rows in the same order.  Every rank must make
the same sequence of layer calls; a rank that never arrives makes the others' bounded waits run out
(status B200MOE_DEV_WAIT_EXPIRED), it cannot hang them.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

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


def exchange_handles(handle: bytes, group: Optional[dist.ProcessGroup] = None) -> List[bytes]:
    """All ranks' buffer handles, rank-major.  The one piece of host plumbing of the data plane."""
    world = dist.get_world_size(group)
    out: List[Any] = [None] * world
    dist.all_gather_object(out, bytes(handle), group=group)
    return [bytes(h) for h in out]


class ExpertParallelMoE:
    """One rank of an expert-parallel MoE block.

    `ctx` supplies ep_create(world, rank, max_local_tokens) -> handle, ep_attach(handles),
    ep_forward(layer, x_local, order=, residual=) -> out, ep_detach() and set_expert.  On a GPU that is a
    MoEContext; the CPU test of the exchange protocol passes a stand-in with the same methods.
    """

    def __init__(self, ctx: Any, num_experts: int, top_k: int, hidden_size: int, max_local_tokens: int,
                 group: Optional[dist.ProcessGroup] = None):
        self.ctx, self.E, self.K, self.H = ctx, num_experts, top_k, hidden_size
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.local_experts = expert_range(num_experts, self.world, self.rank)
        self.max_local_tokens = max_local_tokens
        handle = ctx.ep_create(self.world, self.rank, max_local_tokens)
        if self.world > 1:
            ctx.ep_attach(exchange_handles(handle, group))
            dist.barrier(group)          # every rank has mapped every buffer before anyone stores into one

    def register_local_experts(self, layer: int, experts: Dict[int, Dict[str, torch.Tensor]]) -> None:
        """Registers the experts this rank owns (others in `experts` are ignored)."""
        for e in self.local_experts:
            if e in experts:
                self.ctx.set_expert(layer, e, experts[e])

    def forward(self, layer: int, x_local: torch.Tensor, *, residual: Optional[torch.Tensor] = None,
                order: Optional[Sequence[int]] = None) -> torch.Tensor:
        """x_local [T/G, H] (this rank's tokens) -> [T/G, H]."""
        return self.ctx.ep_forward(layer, x_local, order=order, residual=residual)

    def close(self) -> None:
        """Unmaps the peers' buffers; call on every rank before the contexts go away."""
        if self.world > 1:
            dist.barrier(self.group)     # nobody is still storing into a buffer that is about to be unmapped
        self.ctx.ep_detach()
