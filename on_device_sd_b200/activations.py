"""LayerExpertActivations from a RoutingResult with one device->host copy.

The reference builds the same object with a K x E loop of ``torch.where`` calls, each a device
synchronisation (demo/src/execution/model_runner_utils.py:13-41; up to 1024 per layer for the
128-expert model).  With a context (`ctx=`) the grouping kernel of the MoE block (K2) sorts the
(token, slot) pairs by expert on the device and its two tables cross to the host in one copy; without
one the ids themselves cross once and are grouped on the host.  Either way the token lists and scores
of all activations are slices of two tensors sent back in one copy and one gather.  Order and contents equal the reference's: activations sorted by
top-k rank, then expert index; ``token_indices`` ascending int64 on the ids' device; ``scores`` =
``topk_scores[token_indices, k]``; ``routing_scores`` is the RoutingResult's ``topk_scores``.
"""
from __future__ import annotations

from typing import Any, Callable, List, Optional

import numpy as np
import torch

from .types import ExpertActivation, ExpertID, LayerExpertActivations


def build_layer_activations(routing_result: Any, num_experts: int, *,
                            expert_id_cls: Optional[Callable[[int, int], Any]] = None, ctx: Any = None) -> LayerExpertActivations:
    ids = routing_result.topk_indices
    scores = routing_result.topk_scores
    layer = routing_result.layer_idx
    make_id = expert_id_cls or ExpertID
    T, K = ids.shape
    if T == 0 or K == 0:
        return LayerExpertActivations(layer_idx=layer, activations=[], routing_scores=scores)

    if ctx is not None and ids.is_cuda and ids.dtype == torch.int64 and ids.is_contiguous() and (ctx.E, ctx.K) == (num_experts, K) and T <= ctx.max_tokens:
        offsets, pairs = ctx.group_pairs(ids)                                        # K2's tables: the one device->host copy
        e_idx = np.repeat(np.arange(num_experts, dtype=np.int64), np.diff(offsets))  # pairs are grouped by expert, row-major inside
        t_idx, k_idx = np.divmod(pairs.astype(np.int64), K)
    else:
        ids_h = ids.detach().to("cpu", non_blocking=False).numpy()                   # the one device->host copy
        # ids outside [0, num_experts) never match the reference's `== expert_idx` test: drop them.
        t_idx, k_idx = np.nonzero((ids_h >= 0) & (ids_h < num_experts))
        e_idx = ids_h[t_idx, k_idx]
    key = k_idx.astype(np.int64) * num_experts + e_idx
    order = np.argsort(key, kind="stable")                                           # tokens stay ascending inside a key
    key, t_sorted, k_sorted = key[order], t_idx[order], k_idx[order]
    starts = np.flatnonzero(np.r_[True, key[1:] != key[:-1]]) if key.size else np.empty(0, np.int64)
    ends = np.r_[starts[1:], key.size]

    tok_dev = torch.from_numpy(np.ascontiguousarray(t_sorted, dtype=np.int64)).to(ids.device)
    flat_dev = torch.from_numpy(np.ascontiguousarray(t_sorted * K + k_sorted, dtype=np.int64)).to(ids.device)
    sc_dev = scores.reshape(-1)[flat_dev]                                            # one gather for every activation

    activations: List[ExpertActivation] = []
    for a, b in zip(starts.tolist(), ends.tolist()):
        k, e = divmod(int(key[a]), num_experts)
        activations.append(ExpertActivation(expert_id=make_id(layer, e), token_indices=tok_dev[a:b],
                                            scores=sc_dev[a:b], top_k_rank=k))
    return LayerExpertActivations(layer_idx=layer, activations=activations, routing_scores=scores)
