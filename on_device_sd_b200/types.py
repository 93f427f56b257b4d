"""Data contracts of the ModelRunner boundary, mirrored field for field from the reference
(demo/src/core/model_runner.py:14-67 and demo/src/core/types.py:19-29) so that objects built by
the reference's engine and objects built here are interchangeable (duck typing)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Set

import torch


@dataclass
class ExpertID:
    layer_idx: int
    expert_idx: int

    def __hash__(self):
        return hash((self.layer_idx, self.expert_idx))

    def __str__(self):
        return f"L{self.layer_idx}_E{self.expert_idx}"


@dataclass
class RoutingResult:
    layer_idx: int
    topk_indices: torch.Tensor   # [tokens, top_k] int64
    topk_scores: torch.Tensor    # [tokens, top_k]
    activated_expert_ids: Set[Any]

    @property
    def top_k(self) -> int:
        return self.topk_indices.shape[-1]


@dataclass
class ExpertPlacement:
    gpu_expert_params: Dict[int, Dict[str, torch.Tensor]]
    cpu_expert_params: Dict[int, Dict[str, torch.Tensor]]
    substitution_map: Dict[int, int] = field(default_factory=dict)
    routing_result: Optional[RoutingResult] = None


@dataclass
class AttentionOutput:
    hidden_states: torch.Tensor
    post_attn_normed: torch.Tensor
    residual: torch.Tensor


@dataclass
class ExpertActivation:
    """demo/src/core/types.py:40-45."""
    expert_id: Any
    token_indices: torch.Tensor   # tokens that selected this expert at this rank, ascending
    scores: torch.Tensor          # their routing weights
    top_k_rank: int


@dataclass
class LayerExpertActivations:
    """demo/src/core/types.py:48-52."""
    layer_idx: int
    activations: List[ExpertActivation]
    routing_scores: torch.Tensor


@dataclass
class MoEShape:
    """The five numbers of the reference's MoEConfig that the MoE block consumes
    (demo/src/core/model.py:33-45).  Any object with these attributes works in its place."""
    hidden_size: int
    num_experts: int
    num_experts_per_token: int
    moe_intermediate_size: int
    torch_dtype: str = "bfloat16"
    num_hidden_layers: int = 1

    def get_dtype(self) -> torch.dtype:
        return {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}.get(self.torch_dtype, torch.float16)
