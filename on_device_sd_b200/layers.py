"""Module-level drop-ins with the reference's layer signatures
(demo/src/layers/moe_layer.py:14-254, demo/src/layers/mlp.py:209-231, demo/src/layers/layernorm.py:9-47)."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from ._lib import W_DENSE
from .context import MoEContext

_FFN_CTX: Dict[Tuple, MoEContext] = {}


def expert_forward_with_weights(x: torch.Tensor, gate_weight: torch.Tensor, up_weight: torch.Tensor,
                                down_weight: torch.Tensor) -> torch.Tensor:
    """SwiGLU FFN with external weights: x [*,H], gate/up [I,H], down [H,I] -> [*,H]  (mlp.py:209)."""
    H = x.shape[-1]
    I = gate_weight.shape[0]
    flat = x.reshape(-1, H).contiguous()
    n = flat.shape[0]
    key = (x.device.index, x.dtype, H, I)
    ctx = _FFN_CTX.get(key)
    if ctx is None or ctx.max_tokens < n:
        cap = max(64, 1 << max(n - 1, 0).bit_length())
        ctx = MoEContext(H, 1, 1, I, x.dtype, num_layers=1, max_tokens=cap, weight_mode=W_DENSE, device=x.device)
        _FFN_CTX[key] = ctx
    out = ctx.expert_ffn(flat, gate_weight.contiguous(), up_weight.contiguous(), down_weight.contiguous())
    return out.view(x.shape)


class Qwen3MoEGate(nn.Module):
    """Router gate: forward(hidden_states [B,S,H], top_k) -> (indices int64 [B,S,K], weights [B,S,K])  (moe_layer.py:14-65)."""

    def __init__(self, hidden_size: int, num_experts: int):
        super().__init__()
        self.hidden_size, self.num_experts = hidden_size, num_experts
        self.gate = nn.Linear(hidden_size, num_experts, bias=False)
        self._ctx: Optional[MoEContext] = None
        self._ctx_key = None

    def _context(self, top_k: int, tokens: int) -> MoEContext:
        w = self.gate.weight
        key = (w.data_ptr(), w.dtype, w.device, top_k, w._version)
        if self._ctx is None or self._ctx_key != key or self._ctx.max_tokens < tokens:
            cap = max(256, 1 << max(tokens - 1, 0).bit_length())
            self._ctx = MoEContext(self.hidden_size, self.num_experts, top_k, 8, w.dtype, max_tokens=cap, device=w.device)
            self._ctx.set_gate(0, w.detach())
            self._ctx_key = key
        return self._ctx

    def forward(self, hidden_states: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
        b, s, h = hidden_states.shape
        flat = hidden_states.reshape(-1, h).contiguous()
        ids, scores = self._context(top_k, flat.shape[0]).route(0, flat)
        return ids.view(b, s, top_k), scores.view(b, s, top_k)

    def load_weights(self, gate_weight: torch.Tensor):
        self.gate.weight.data = gate_weight.to(next(self.parameters()).dtype)


class Qwen3MoELayerWithWeights(nn.Module):
    """Stateless MoE layer: forward(hidden_states, gate_weight [E,H], expert_weights_dict)  (moe_layer.py:173-254)."""

    def __init__(self, hidden_size: int, num_experts: int, num_experts_per_token: int, moe_intermediate_size: int, layer_idx: int):
        super().__init__()
        self.hidden_size, self.num_experts = hidden_size, num_experts
        self.num_experts_per_token, self.moe_intermediate_size, self.layer_idx = num_experts_per_token, moe_intermediate_size, layer_idx
        self._ctx: Optional[MoEContext] = None
        self._gate_key = None

    def _run(self, hidden_states: torch.Tensor, gate_weight: torch.Tensor, expert_weights_dict) -> torch.Tensor:
        b, s, h = hidden_states.shape
        flat = hidden_states.reshape(-1, h).contiguous()
        T = flat.shape[0]
        if self._ctx is None or self._ctx.max_tokens < T or self._ctx.dtype != flat.dtype or self._ctx.device != flat.device:
            cap = max(256, 1 << max(T - 1, 0).bit_length())
            self._ctx = MoEContext(self.hidden_size, self.num_experts, self.num_experts_per_token, self.moe_intermediate_size,
                                   flat.dtype, max_tokens=cap, device=flat.device)
            self._gate_key = None
        ctx = self._ctx
        gkey = (gate_weight.data_ptr(), gate_weight._version)
        if gkey != self._gate_key:
            ctx.set_gate(0, gate_weight.detach())
            self._gate_key = gkey
        ids, scores = ctx.route(0, flat)
        # experts absent from the dict are skipped silently (moe_layer.py:136-137)
        slot = [-1] * self.num_experts
        for e, params in expert_weights_dict.items():
            if 0 <= e < self.num_experts:
                ctx.set_expert(0, e, {k: params[k].to(device=flat.device, dtype=flat.dtype).contiguous()
                                      for k in ("gate_proj", "up_proj", "down_proj")})
                slot[e] = e
        out = ctx.forward(0, flat, ids, scores, expert_slot=slot)
        return out.view(b, s, h)

    def forward(self, hidden_states: torch.Tensor, gate_weight: torch.Tensor, expert_weights_dict) -> torch.Tensor:
        return self._run(hidden_states, gate_weight, expert_weights_dict)


class Qwen3MoELayer(Qwen3MoELayerWithWeights):
    """MoE layer owning its gate: forward(hidden_states [B,S,H], expert_weights_dict) -> [B,S,H]  (moe_layer.py:68-170)."""

    def __init__(self, hidden_size: int, num_experts: int, num_experts_per_token: int, moe_intermediate_size: int, layer_idx: int):
        super().__init__(hidden_size, num_experts, num_experts_per_token, moe_intermediate_size, layer_idx)
        self.gate = Qwen3MoEGate(hidden_size, num_experts)

    def forward(self, hidden_states: torch.Tensor, expert_weights_dict) -> torch.Tensor:  # type: ignore[override]
        return self._run(hidden_states, self.gate.gate.weight, expert_weights_dict)


class RMSNorm(nn.Module):
    """The reference's RMSNorm (demo/src/layers/layernorm.py:9-47) with both forms in one kernel launch:
    `forward(x)` -> normed, `forward(x, residual)` -> (normed, x + residual).  The weight is used in the
    activation dtype, as it is once the reference has cast the model to its dtype."""

    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        H = x.shape[-1]
        flat = x.reshape(-1, H).contiguous()
        n = flat.shape[0]
        key = (x.device.index, x.dtype, H, 0)
        ctx = _FFN_CTX.get(key)
        if ctx is None:
            ctx = MoEContext(H, 1, 1, 8, x.dtype, num_layers=1, max_tokens=8, weight_mode=W_DENSE, device=x.device)
            _FFN_CTX[key] = ctx
        w = self.weight.detach().to(device=x.device, dtype=x.dtype).contiguous()
        if residual is None:
            return ctx.rmsnorm(flat, w, self.eps).view(x.shape)
        out, res = ctx.rmsnorm(flat, w, self.eps, residual.reshape(-1, H).contiguous())
        return out.view(x.shape), res.view(x.shape)
