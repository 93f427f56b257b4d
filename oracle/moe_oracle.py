"""CPU oracle for the MoE block forward of on_device_sd's demo engine.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file; only the
tests, the smoke check and the CPU-baseline legs of the benchmark may call it, and only as
the checker (or as the timed CPU baseline), never as the path that is shipped.

It restates, in plain PyTorch on whatever device the inputs live on (normally the CPU), the
algorithm of the reference's hot path:

  * router            demo/src/layers/moe_layer.py:25-60 (Qwen3MoEGate.forward) and the
                      stateless twin :207-219
  * route_experts     demo/src/model/qwen3_runner.py:86-119
  * expert FFN        demo/src/layers/mlp.py:209-231 (expert_forward_with_weights)
  * engine MoE block  demo/src/model/qwen3_runner.py:269-385 (_execute_moe_with_placement),
                      residual add :212-226 (forward_moe)       -> "path B"
  * layer MoE block   demo/src/layers/moe_layer.py:93-170 (Qwen3MoELayer.forward) -> "path A"

The arithmetic of the path lives in PyTorch (F.linear, topk, softmax, silu, index_put); the
reference pins no torch version, so the oracle runs on the torch that is installed (2.11 here).

Parity pin: the reference's own tests hold no golden vectors for this path (they only compare
one implementation with another on fresh random inputs).  This restatement is therefore pinned
against OUTPUTS OF THE REFERENCE ITSELF, produced by importing the reference's modules on the
CPU (oracle/pin_against_reference.py) and stored as fixtures under tests/golden/.

Two things are defined here more sharply than the reference defines them, because the
reference leaves them to the torch build it happens to run on:

  * tie order of the top-k.  torch.topk's order among equal logits is implementation defined
    and differs between torch's CPU and CUDA kernels.  `topk_cuda_order` states the order the
    CUDA implementation produces (the engine runs on CUDA), and `route(..., tie="torch")` keeps
    whatever torch.topk on the input's device does.
  * int4 group-wise weights (not in the reference): the format is defined in `quant_int4_g128`.
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

ExpertParams = Dict[str, torch.Tensor]


# --------------------------------------------------------------------------------------
# top-k with an explicit tie rule
# --------------------------------------------------------------------------------------
def _bitonic_pairs(n: int) -> List[List[Tuple[int, int, bool]]]:
    """Compare-exchange schedule of a bitonic sorting network over n = 2^m slots.

    Each stage is a list of (lo, hi, ascending_block) triples: slot `lo` < slot `hi`, and
    `ascending_block` tells whether this block of the network is sorted in the reverse sense.
    """
    stages = []
    size = 2
    while size < n:
        stride = size // 2
        while stride > 0:
            stage = []
            for t in range(n // 2):
                flag = (t & (size // 2)) != 0
                pos = 2 * t - (t & (stride - 1))
                stage.append((pos, pos + stride, flag))
            stages.append(stage)
            stride //= 2
        size *= 2
    stride = n // 2
    while stride > 0:
        stage = []
        for t in range(n // 2):
            pos = 2 * t - (t & (stride - 1))
            stage.append((pos, pos + stride, False))
        stages.append(stage)
        stride //= 2
    return stages


_NETWORK_CACHE: Dict[int, List[List[Tuple[int, int, bool]]]] = {}


def sort_network_descending(keys: List[float], vals: List[int], width: int = 32) -> Tuple[List[float], List[int]]:
    """Sort (key, value) pairs into descending key order with a bitonic network of `width` slots.

    Slots beyond len(keys) are padding that always sinks to the end.  The network is not
    stable; the permutation it applies to EQUAL keys is what fixes the order of tied experts
    inside a top-k result (torch's CUDA top-k sorts its k selected entries this way when
    1 < k <= 32; measured on a B200 with torch 2.11 for fp32, fp16 and bf16 logits).
    """
    n = width
    if n not in _NETWORK_CACHE:
        _NETWORK_CACHE[n] = _bitonic_pairs(n)
    k = list(keys) + [0.0] * (n - len(keys))
    v = list(vals) + [-1] * (n - len(vals))
    ok = [True] * len(keys) + [False] * (n - len(keys))
    for stage in _NETWORK_CACHE[n]:
        for lo, hi, flag in stage:
            # One compare-exchange.  `flag` marks the blocks of the merge phases that are built
            # in the opposite sense; padding always loses.  The predicate is strict, so the
            # exchange DOES happen for equal keys in the unflagged blocks - that is what moves
            # tied entries around.
            pred = (k[lo] > k[hi] and ok[lo]) or (not ok[hi])
            if pred == flag:
                k[lo], k[hi] = k[hi], k[lo]
                v[lo], v[hi] = v[hi], v[lo]
                ok[lo], ok[hi] = ok[hi], ok[lo]
    m = len(keys)
    return k[:m], v[:m]


def topk_cuda_order(logits: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k of each row with the tie order of torch's CUDA kernel, as a pure-Python loop.

    Selection: every entry strictly greater than the k-th largest value is taken, then entries
    EQUAL to the k-th value are taken in ascending index order until k are chosen.  Ordering:
    the chosen entries, in ascending index order (greater ones first, then the equal ones), go
    through `sort_network_descending`.  Only meant for the sizes the oracle finishes in
    seconds (T*E up to a few 100k).
    """
    assert logits.dim() == 2
    T, E = logits.shape
    vals = logits.float().cpu()
    out_v = torch.empty(T, top_k, dtype=torch.float32)
    out_i = torch.empty(T, top_k, dtype=torch.int64)
    for t in range(T):
        row = vals[t].tolist()
        kth = sorted(row, reverse=True)[top_k - 1]
        gt = [i for i, r in enumerate(row) if r > kth]
        eq = [i for i, r in enumerate(row) if r == kth][: top_k - len(gt)]
        chosen = gt + eq
        keys = [row[i] for i in chosen]
        if top_k == 1:
            pass
        elif top_k <= 32:
            keys, chosen = sort_network_descending(keys, chosen, 32)
        else:
            order = sorted(range(top_k), key=lambda j: (-keys[j], chosen[j]))
            keys, chosen = [keys[j] for j in order], [chosen[j] for j in order]
        out_v[t] = torch.tensor(keys)
        out_i[t] = torch.tensor(chosen)
    return out_v.to(logits.dtype).to(logits.device), out_i.to(logits.device)


# --------------------------------------------------------------------------------------
# router
# --------------------------------------------------------------------------------------
def router_logits(x2d: torch.Tensor, gate_w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  mode: str = "exact") -> torch.Tensor:
    """logits = x @ Wg^T in the model dtype (moe_layer.py:44, :211).

    mode="linear": F.linear, exactly what the reference calls.  Its low-order bits depend on the
      GEMM library's summation order (measured: for bf16 Qwen3-shaped inputs, ~0.1 % of cuBLAS
      logits on a B200 and ~0.02 % of oneDNN logits on the CPU differ by one bf16 ulp from the
      correctly rounded value), so two runs of the reference on different devices do not agree
      bit for bit with each other.
    mode="exact": the real-number dot product (fp64 accumulation; products of 16-bit values are
      exact) rounded to fp32 and then to the model dtype - the two roundings every
      fp32-accumulating GEMM applies, minus the summation-order noise.  This is the definition
      the CUDA router is held to, bit for bit.

    `bias` is not in the reference: it is the Zipf popularity stressor of the stacked config,
    added to the logits (in their dtype) between the linear and the top-k.
    """
    if mode == "linear":
        logits = F.linear(x2d, gate_w)
    elif mode == "exact":
        logits = (x2d.double() @ gate_w.double().t()).float().to(x2d.dtype)
    else:
        raise ValueError(mode)
    if bias is not None:
        logits = logits + bias.to(logits.dtype)
    return logits


def topk_softmax(logits: torch.Tensor, top_k: int, tie: str = "cuda") -> Tuple[torch.Tensor, torch.Tensor]:
    """moe_layer.py:49-54: top-k (descending), then softmax over the k kept logits."""
    if tie == "torch":
        vals, ids = torch.topk(logits, top_k, dim=-1)
    elif tie == "cuda":
        vals, ids = topk_cuda_order(logits, top_k)
    else:
        raise ValueError(tie)
    return ids, F.softmax(vals, dim=-1)


def route(x2d: torch.Tensor, gate_w: torch.Tensor, top_k: int, *, bias: Optional[torch.Tensor] = None,
          tie: str = "cuda", logits: str = "exact") -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Router of moe_layer.py:38-60.  Returns (ids int64 [T,K], scores [T,K] in the model dtype, logits [T,E])."""
    lg = router_logits(x2d, gate_w, bias, logits)
    ids, scores = topk_softmax(lg, top_k, tie)
    return ids, scores, lg


class _Key:
    """Stand-in for the reference's ExpertID (demo/src/core/types.py:19-29): same hash, same eq."""
    __slots__ = ("layer_idx", "expert_idx")

    def __init__(self, layer_idx: int, expert_idx: int):
        self.layer_idx, self.expert_idx = layer_idx, expert_idx

    def __hash__(self):
        return hash((self.layer_idx, self.expert_idx))

    def __eq__(self, other):
        return (self.layer_idx, self.expert_idx) == (other.layer_idx, other.expert_idx)


def activated_order(layer_idx: int, ids: torch.Tensor) -> List[int]:
    """Order in which the engine path visits the activated experts.

    qwen3_runner.py:110-112 inserts ExpertID(layer, e) for e in ascending unique order into a
    Python set; :303 iterates that set.  The iteration order is fixed by the hashes, so it is
    reproduced by building a set of objects with the same hash in the same insertion order.
    """
    s = set()
    for e in ids.flatten().unique().tolist():
        s.add(_Key(layer_idx, int(e)))
    return [k.expert_idx for k in s]


def layer_activations(ids: torch.Tensor, scores: torch.Tensor, num_experts: int) -> List[Tuple[int, int, torch.Tensor, torch.Tensor]]:
    """(top_k_rank, expert, token_indices, scores) per non-empty (rank, expert) cell, in the order
    demo/src/execution/model_runner_utils.py:21-35 appends ExpertActivation objects: rank outer,
    expert inner, tokens from ``torch.where`` (ascending), scores ``topk_scores[tokens, k]``."""
    out = []
    for k in range(ids.shape[1]):
        for e in range(num_experts):
            tok = torch.where(ids[:, k] == e)[0]
            if tok.numel():
                out.append((k, e, tok, scores[tok, k]))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None):
    """RMSNorm.rms_forward / add_rms_forward (demo/src/layers/layernorm.py:21-36): fp32 statistics, the
    normalised row rounded to the input dtype, then multiplied by the weight.  Returns out, or
    (out, new_residual) when `residual` is given."""
    orig = x.dtype
    s = x.float() if residual is None else x.float() + residual.float()
    var = s.pow(2).mean(dim=-1, keepdim=True)
    out = (s * torch.rsqrt(var + eps)).to(orig) * weight
    return out if residual is None else (out, s.to(orig))


# --------------------------------------------------------------------------------------
# expert FFN and the two MoE block paths
# --------------------------------------------------------------------------------------
def expert_ffn(x: torch.Tensor, gate_proj: torch.Tensor, up_proj: torch.Tensor, down_proj: torch.Tensor) -> torch.Tensor:
    """SwiGLU FFN, mlp.py:227-230: every intermediate is a tensor in the model dtype."""
    g = F.linear(x, gate_proj)
    u = F.linear(x, up_proj)
    h = F.silu(g) * u
    return F.linear(h, down_proj)


def moe_engine(x: torch.Tensor, ids: torch.Tensor, scores: torch.Tensor, experts: Dict[int, ExpertParams], *,
               layer_idx: int = 0, substitution: Optional[Dict[int, int]] = None,
               order: Optional[Sequence[int]] = None, residual: Optional[torch.Tensor] = None,
               cpu_experts: Optional[Dict[int, ExpertParams]] = None) -> torch.Tensor:
    """Path B: qwen3_runner.py:269-385.  `experts` plays gpu_expert_params, `cpu_experts` plays
    cpu_expert_params (both evaluated on x's device here: where an expert's arithmetic runs does not
    change the algorithm, only which of the two task lists it joins).

    One pass over the activated experts in set-iteration order (:303) sorts them into GPU tasks and
    CPU tasks - own GPU parameters, else own CPU parameters, else the substitute's GPU parameters,
    else the substitute's CPU parameters, else skipped (:316-333).  (tok, k) = where(ids == e) in
    row-major order, y = FFN(x[tok]), final[tok] += y * scores[tok, k][:, None]  (index-put without
    accumulation for repeated tok, exactly as torch does for `a[idx] += b`); every GPU task is
    accumulated before any CPU task (:352-383), each list in its collection order.  `residual` adds
    forward_moe's residual (:226).
    """
    shape = x.shape
    flat = x.reshape(-1, shape[-1])
    final = torch.zeros_like(flat)
    sub = substitution or {}
    cpu = cpu_experts or {}
    if order is None:
        order = activated_order(layer_idx, ids)
    gpu_tasks, cpu_tasks = [], []
    for e in order:
        tok, kk = torch.where(ids == e)
        if tok.numel() == 0:
            continue
        if e in experts:
            gpu_tasks.append((tok, kk, experts[e]))
        elif e in cpu:
            cpu_tasks.append((tok, kk, cpu[e]))
        elif e in sub and sub[e] in experts:
            gpu_tasks.append((tok, kk, experts[sub[e]]))
        elif e in sub and sub[e] in cpu:
            cpu_tasks.append((tok, kk, cpu[sub[e]]))
    for tok, kk, p in gpu_tasks + cpu_tasks:
        w = scores[tok, kk]
        y = expert_ffn(flat[tok], p["gate_proj"].to(flat.dtype), p["up_proj"].to(flat.dtype), p["down_proj"].to(flat.dtype))
        final[tok] += y * w.unsqueeze(1)
    out = final.view(shape)
    if residual is not None:
        out = residual + out
    return out


def moe_layer(x: torch.Tensor, gate_w: torch.Tensor, experts: Dict[int, ExpertParams], top_k: int, *,
              tie: str = "cuda", logits: str = "exact", bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Path A: moe_layer.py:93-170.  Experts in ascending index; per token, the routing weights
    of every slot that chose the expert are summed (:160-165) and `w * y` is accumulated."""
    shape = x.shape
    flat = x.reshape(-1, shape[-1])
    ids, scores, _ = route(flat, gate_w, top_k, tie=tie, logits=logits, bias=bias)
    final = torch.zeros_like(flat)
    E = gate_w.shape[0]
    for e in range(E):
        mask = (ids == e).any(dim=-1)
        if not bool(mask.any()) or e not in experts:
            continue
        tok = mask.nonzero(as_tuple=False).squeeze(1)
        p = experts[e]
        y = expert_ffn(flat[tok], p["gate_proj"], p["up_proj"], p["down_proj"])
        for i, t in enumerate(tok.tolist()):
            w = scores[t][(ids[t] == e)].sum()
            final[t] += w * y[i]
    return final.view(shape)


# --------------------------------------------------------------------------------------
# int4 g128 (format defined by this build; the reference has no quantised weights)
# --------------------------------------------------------------------------------------
GROUP = 128


def quant_int4_g128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Symmetric group-wise int4 along the `in` (last) dimension of a [out, in] matrix.

    amax over each group of 128 consecutive elements (fp32, from the bf16-rounded weights);
    scale = bf16(amax / 7), 1 when the group is all zero; q = clamp(rne(w / scale), -8, 7).
    Storage: uint8 [out, in/2], byte j = element 2j in the low nibble, 2j+1 in the high nibble,
    each stored as q + 8; scales bf16 [out, in/128].
    """
    assert w.dim() == 2 and w.shape[1] % GROUP == 0
    out_f, in_f = w.shape
    wf = w.to(torch.bfloat16).float().view(out_f, in_f // GROUP, GROUP)
    amax = wf.abs().amax(dim=-1)
    scale = (amax / 7.0).to(torch.bfloat16)
    scale = torch.where(amax == 0, torch.ones_like(scale), scale)
    q = torch.clamp(torch.round(wf / scale.float().unsqueeze(-1)), -8, 7).to(torch.int16) + 8
    q = q.view(out_f, in_f).to(torch.uint8)
    packed = q[:, 0::2] | (q[:, 1::2] << 4)
    return packed.contiguous(), scale.contiguous()


def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [out, in/2] -> int8 [out, in] holding q in [-8, 7]."""
    lo = (packed & 0xF).to(torch.int16) - 8
    hi = (packed >> 4).to(torch.int16) - 8
    return torch.stack([lo, hi], dim=-1).view(packed.shape[0], -1).to(torch.int8)


def dequant_int4_g128(packed: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """w = float(scale_g) * q, rounded to `dtype` (the weights the oracle's FFN then uses)."""
    q = unpack_int4(packed).float()
    out_f, in_f = q.shape
    w = q.view(out_f, in_f // GROUP, GROUP) * scale.float().unsqueeze(-1)
    return w.view(out_f, in_f).to(dtype)


# --------------------------------------------------------------------------------------
# error metrics the parity tests use
# --------------------------------------------------------------------------------------
def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).abs().max()) if a.numel() else 0.0


def mean_rel(a: torch.Tensor, b: torch.Tensor) -> float:
    """mean|a-b| / mean|b| (the element-wise ratio is dominated by near-zero elements)."""
    if not a.numel():
        return 0.0
    den = float(b.double().abs().mean())
    return float((a.double() - b.double()).abs().mean()) / (den if den > 0 else 1.0)
