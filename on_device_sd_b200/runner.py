"""Drop-in for the MoE part of the reference's ModelRunner boundary.

`B200MoERunner` keeps the three signatures the engines call once per layer per step
(demo/src/core/model_runner.py:150-193; callers demo/src/execution/cb_executor.py:324-345,
:375-400, :427-448):

    route_experts(layer_idx, hidden_states) -> RoutingResult          (qwen3_runner.py:86-119)
    forward_moe(layer_idx, attn_output, expert_placement) -> Tensor   (qwen3_runner.py:212-226)
    _execute_moe_with_placement(hidden_states, expert_placement)      (qwen3_runner.py:269-385)

and adds `moe_block(layer_idx, hidden_states, residual=None)`, the same computation enqueued
with no host round trip (router, permute, expert FFN, combine back to back).  Everything runs
in libb200moe.so; a subclass of the reference's Qwen3ModelRunner can delegate these three
methods to an instance of this class unchanged.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Any, Dict, List, Optional, Sequence

import torch

from ._lib import FFN_AUTO, W_DENSE, W_INT4_G128
from .context import MoEContext
from .types import AttentionOutput, ExpertID, ExpertPlacement, RoutingResult

_PARAM_KEYS = ("gate_proj", "up_proj", "down_proj")


def plan_placement(expert_placement: Any, num_experts: int):
    """Host-side reading of an ExpertPlacement (qwen3_runner.py:298-333), with no tensor work.

    Returns (avail, slot, order):
      avail  {expert: params} usable this call - GPU-resident entries win over CPU-resident ones;
             CPU-resident experts are uploaded and executed on the GPU here (the reference runs
             those on host threads, :340-350)
      slot   slot[e] = expert whose parameters serve tokens routed to e: e itself, else its
             substitute from substitution_map (with the ORIGINAL routing weight, :322-329), else -1
             = skipped silently (:330-333).  Only activated experts get a slot.
      order  order[e] = position of e in the sequence in which the reference accumulates the
             per-expert results in the model dtype: every expert served from gpu_expert_params
             (directly or through its substitute) in the iteration order of
             routing.activated_expert_ids, THEN every expert served from cpu_expert_params in that
             same iteration order (the reference collects gpu_tasks and cpu_tasks in one pass, :303-333,
             and adds all GPU results before the CPU results, :352-383)
    """
    routing = expert_placement.routing_result
    E = num_experts
    gpu = expert_placement.gpu_expert_params or {}
    cpu = expert_placement.cpu_expert_params or {}
    avail: Dict[int, Dict[str, torch.Tensor]] = dict(cpu)
    avail.update(gpu)
    slot = [-1] * E
    sub = expert_placement.substitution_map or {}
    first: List[int] = []      # served from GPU-resident parameters
    second: List[int] = []     # served from CPU-resident parameters
    skipped: List[int] = []
    seen = [False] * E
    for eid in routing.activated_expert_ids:
        e = eid.expert_idx
        if not 0 <= e < E or seen[e]:
            continue
        seen[e] = True
        if e in gpu:
            slot[e] = e
            first.append(e)
        elif e in cpu:
            slot[e] = e
            second.append(e)
        elif e in sub and sub[e] in gpu:
            slot[e] = sub[e]
            first.append(e)
        elif e in sub and sub[e] in cpu:
            slot[e] = sub[e]
            second.append(e)
        else:
            skipped.append(e)
    order = [0] * E
    ranked = first + second + skipped
    for r, e in enumerate(ranked):
        order[e] = min(r, 255)
    for e in range(E):
        if not seen[e]:
            order[e] = min(len(ranked), 255)
    return avail, slot, order


class LazyRoutingResult(RoutingResult):
    """RoutingResult whose `activated_expert_ids` set is built when it is first read.

    The reference builds the set inside route_experts with .unique().tolist() - one device
    synchronisation per layer whether or not anybody looks at the set (qwen3_runner.py:110-112).
    Here the router kernel writes one bit per selected expert into pinned host memory; reading the
    attribute waits for that copy (an event, not the whole stream) and inserts ExpertID(layer, e) in
    ascending e, the insertion order of the reference, so the set iterates in the same order."""

    def __init__(self, layer_idx: int, topk_indices: torch.Tensor, topk_scores: torch.Tensor, bitmap: torch.Tensor,
                 ready: "torch.cuda.Event", expert_id_cls: type):
        self.layer_idx, self.topk_indices, self.topk_scores = layer_idx, topk_indices, topk_scores
        self._bitmap, self._ready, self._cls, self._set = bitmap, ready, expert_id_cls, None

    @property
    def activated_expert_ids(self):
        if self._set is None:
            self._ready.synchronize()
            s = set()
            for w in range(4):
                bits = int(self._bitmap[w]) & 0xFFFFFFFFFFFFFFFF
                while bits:
                    low = bits & -bits
                    s.add(self._cls(self.layer_idx, w * 64 + low.bit_length() - 1))
                    bits ^= low
            self._set = s
        return self._set

    @activated_expert_ids.setter
    def activated_expert_ids(self, value):
        self._set = value

    def __repr__(self):
        return f"LazyRoutingResult(layer_idx={self.layer_idx}, tokens={tuple(self.topk_indices.shape)})"


class B200MoERunner:
    def __init__(self, config: Any, *, device: Optional[torch.device] = None, max_tokens: int = 512,
                 weight_mode: int = W_DENSE, expert_id_cls: type = ExpertID, exact_logits: bool = False,
                 ffn_kind: int = FFN_AUTO, graph_blocks: bool = False):
        """`config` is the reference's MoEConfig or anything with hidden_size, num_experts,
        num_experts_per_token, moe_intermediate_size, num_hidden_layers and get_dtype().

        exact_logits=True computes the gate GEMM with torch's F.linear (the library GEMM the
        reference calls, moe_layer.py:44) and runs only top-k/softmax here, which reproduces the
        reference's logits roundings on the same GPU; the default computes the logits in the
        fused router kernel as correctly rounded dot products.

        graph_blocks=True makes `moe_block` capture its kernels into a CUDA graph the first time it sees
        an input buffer (keyed by layer, address, shape and residual address) and replay it afterwards:
        one launch per block instead of five.  The result then lives in a buffer owned by the runner that
        the next call with the same key overwrites.  A graph bakes the registered pointers in, so every
        graph is dropped as soon as a gate or an expert is registered, moved or cleared (the context
        counts such changes), and at most `max_graphs` graphs are kept, least recently used first out."""
        self.config = config
        self.dtype = config.get_dtype()
        self.expert_id_cls = expert_id_cls
        self.exact_logits = exact_logits
        self.ffn_kind = ffn_kind
        self.ctx = MoEContext(config.hidden_size, config.num_experts, config.num_experts_per_token,
                              config.moe_intermediate_size, self.dtype, num_layers=config.num_hidden_layers,
                              max_tokens=max_tokens, weight_mode=weight_mode, device=device)
        self.device = self.ctx.device
        # per layer: expert -> (params dict object, address of its gate_proj) as last registered through a placement
        self._placed: Dict[int, Dict[int, tuple]] = {}
        self._gate_w: Dict[int, torch.Tensor] = {}
        self._last_layer = 0
        self.graph_blocks = graph_blocks
        self.max_graphs = 64
        self._graphs: "OrderedDict[tuple, tuple]" = OrderedDict()
        self._graphs_generation = -1

    def get_config(self):
        return self.config

    @property
    def num_layers(self) -> int:
        return self.config.num_hidden_layers

    # -- weights ----------------------------------------------------------------------------
    def load_gate(self, layer_idx: int, gate_weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """What _load_static_weights does for `layer.mlp.gate` (qwen3_runner.py:387-405)."""
        self.ctx.set_gate(layer_idx, gate_weight, bias)
        self._gate_w[layer_idx] = self.ctx._gate[layer_idx][0]

    def register_experts(self, layer_idx: int, experts: Dict[int, Dict[str, torch.Tensor]]) -> None:
        self._placed.pop(layer_idx, None)
        for e, params in experts.items():
            self.ctx.set_expert(layer_idx, e, params)

    # -- ModelRunner boundary -----------------------------------------------------------------
    def route_experts(self, layer_idx: int, hidden_states: torch.Tensor) -> RoutingResult:
        h = self.config.hidden_size
        flat = hidden_states.reshape(-1, h)
        if not flat.is_contiguous():
            raise ValueError("hidden_states must be contiguous")
        bitmap = torch.empty(4, dtype=torch.int64, pin_memory=True)      # host-pinned blocks are recycled by torch's allocator
        if self.exact_logits:
            logits = torch.nn.functional.linear(flat, self._gate_w[layer_idx])
            bias = self.ctx._gate[layer_idx][1]
            if bias is not None:
                logits = logits + bias
            ids, scores = self.ctx.route(layer_idx, flat, bitmap=bitmap, logits=logits)
        else:
            ids, scores = self.ctx.route(layer_idx, flat, bitmap=bitmap)
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        self._last_layer = layer_idx
        return LazyRoutingResult(layer_idx, ids, scores, bitmap, ready, self.expert_id_cls)

    def build_layer_activations(self, routing_result: Any):
        """LayerExpertActivations of a routing (demo/src/execution/model_runner_utils.py:13-41) from the grouping kernel's tables."""
        from .activations import build_layer_activations
        return build_layer_activations(routing_result, self.config.num_experts, expert_id_cls=self.expert_id_cls, ctx=self.ctx)

    def forward_moe(self, layer_idx: int, attn_output: Any, expert_placement: Any) -> torch.Tensor:
        """residual + MoE(post_attn_normed); the add is fused into the combine kernel."""
        return self._execute_moe_with_placement(attn_output.post_attn_normed, expert_placement,
                                                residual=attn_output.residual, layer_idx=layer_idx)

    def _execute_moe_with_placement(self, hidden_states: torch.Tensor, expert_placement: Any, *,
                                    residual: Optional[torch.Tensor] = None, layer_idx: Optional[int] = None) -> torch.Tensor:
        routing = expert_placement.routing_result
        if routing is None:
            out = torch.zeros_like(hidden_states)
            return out if residual is None else residual + out
        layer = routing.layer_idx if layer_idx is None else layer_idx
        E = self.config.num_experts
        h = hidden_states.shape[-1]
        flat = hidden_states.reshape(-1, h)

        avail, slot, order = plan_placement(expert_placement, E)
        placed = self._placed.setdefault(layer, {})
        for e in {s for s in slot if s >= 0}:
            params = avail[e]
            hit = placed.get(e)
            # the engine hands over the same per-expert dict object call after call while the expert stays resident:
            # one identity check and one address check instead of three shape / device / pointer comparisons
            if hit is not None and hit[0] is params and hit[1] == params["gate_proj"].data_ptr():
                continue
            self.ctx.set_expert(layer, e, self._prepare_params(params))
            placed[e] = (params, params["gate_proj"].data_ptr())
        res2d = None if residual is None else residual.reshape(-1, h)
        out = self.ctx.forward(layer, flat, routing.topk_indices, routing.topk_scores, expert_slot=slot, order=order,
                               residual=res2d, ffn_kind=self.ffn_kind)
        return out.view(hidden_states.shape)

    def _prepare_params(self, params: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Same rule as the reference's _prepare_params (qwen3_runner.py:335-338): move / cast when needed."""
        if self.ctx.weight_mode == W_INT4_G128:
            return params
        p = params["gate_proj"]
        if p.device == self.device and p.dtype == self.dtype and all(params[k].is_contiguous() for k in _PARAM_KEYS):
            return params
        return {k: params[k].to(device=self.device, dtype=self.dtype).contiguous() for k in _PARAM_KEYS}

    # -- fused entry ---------------------------------------------------------------------------
    def moe_block(self, layer_idx: int, hidden_states: torch.Tensor, residual: Optional[torch.Tensor] = None,
                  return_routing: bool = False):
        """Router + experts + combine (+ residual) for registered experts, one enqueue, no sync.
        Accumulates per-expert results in ascending expert index (Qwen3MoELayer.forward's order)."""
        h = hidden_states.shape[-1]
        flat = hidden_states.reshape(-1, h)
        res2d = None if residual is None else residual.reshape(-1, h)
        if self.graph_blocks and not return_routing and flat.is_contiguous() and (res2d is None or res2d.is_contiguous()):
            key = (layer_idx, flat.data_ptr(), tuple(flat.shape), None if res2d is None else res2d.data_ptr())
            if self._graphs_generation != self.ctx.generation:     # a registered pointer changed: every captured graph is stale
                self._graphs.clear()
                self._graphs_generation = self.ctx.generation
            hit = self._graphs.get(key)
            if hit is not None:
                self._graphs.move_to_end(key)
            if hit is None:
                for _ in range(2):                       # warm-up outside the capture (lazy kernel attributes, tensor maps)
                    self.ctx.forward_fused(layer_idx, flat, residual=res2d, ffn_kind=self.ffn_kind)
                torch.cuda.current_stream(self.device).synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    out = self.ctx.forward_fused(layer_idx, flat, residual=res2d, ffn_kind=self.ffn_kind)
                hit = (g, out)
                self._graphs[key] = hit
                while len(self._graphs) > self.max_graphs:
                    self._graphs.popitem(last=False)
            hit[0].replay()
            return hit[1].view(hidden_states.shape)
        r = self.ctx.forward_fused(layer_idx, flat, residual=res2d, return_routing=return_routing, ffn_kind=self.ffn_kind)
        if return_routing:
            return r[0].view(hidden_states.shape), r[1], r[2]
        return r.view(hidden_states.shape)
