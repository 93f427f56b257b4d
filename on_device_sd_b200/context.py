"""MoEContext: a thin, typed wrapper over one b200moe_ctx.  It passes data_ptr()s and the
current CUDA stream to the C ABI; torch is used for device memory and streams only."""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int, c_int32, c_void_p
from typing import Dict, Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import BF16, F16, F32, FFN_AUTO, W_DENSE, W_INT4_G128, Config, check

_DTYPE_TAG = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


def dtype_tag(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_TAG[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; the MoE block runs in float32, float16 or bfloat16") from None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _need_cuda(t: torch.Tensor, name: str, device: torch.device, dtype: Optional[torch.dtype] = None) -> None:
    if not t.is_cuda or t.device != device:
        raise ValueError(f"{name} must live on {device}, got {t.device} (this package has no CPU path)")
    if not t.is_contiguous():
        # the reference uses .view(-1, h) on these tensors (qwen3_runner.py:285): contiguity is its contract too
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")


class MoEContext:
    """Owns the library context of one device: workspace, registered gates and experts."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, intermediate_size: int, dtype: torch.dtype,
                 *, num_layers: int = 1, max_tokens: int = 512, weight_mode: int = W_DENSE,
                 device: Optional[torch.device] = None):
        self._lib = _lib.load()
        self._h = c_void_p()
        if not torch.cuda.is_available():
            raise RuntimeError("b200moe needs a CUDA device (B200); there is no CPU fallback")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.dtype = dtype
        self.H, self.E, self.K, self.I = hidden_size, num_experts, top_k, intermediate_size
        self.num_layers, self.max_tokens, self.weight_mode = num_layers, max_tokens, weight_mode
        cfg = Config(hidden_size, num_experts, top_k, intermediate_size, dtype_tag(dtype), weight_mode, num_layers,
                     max_tokens, self.device.index, 0)
        torch.cuda.init()
        with torch.cuda.device(self.device):
            check(None, self._lib.b200moe_create(byref(cfg), byref(self._h)))
        # keep registered tensors alive and remember their addresses (pointers are borrowed by the library)
        self._gate: Dict[int, Tuple[torch.Tensor, Optional[torch.Tensor]]] = {}
        self._experts: Dict[Tuple[int, int], Tuple[torch.Tensor, ...]] = {}
        self._expert_ptrs: Dict[Tuple[int, int], Tuple[int, ...]] = {}
        # bumped whenever a registered pointer changes: anything that baked pointers in (a captured CUDA graph) is stale then
        self.generation = 0

    # -- lifetime ---------------------------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h.value:
            self._lib.b200moe_destroy(self._h)
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, code: int) -> None:
        check(self._h, code)

    @property
    def launches(self) -> int:
        return int(self._lib.b200moe_launch_count(self._h))

    # -- registration -----------------------------------------------------------------------
    def set_gate(self, layer: int, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
        """Registers the router weight [E,H] (cast like Qwen3MoEGate.load_weights, moe_layer.py:62-65)."""
        weight = weight.to(device=self.device, dtype=self.dtype).contiguous()
        if weight.shape != (self.E, self.H):
            raise ValueError(f"gate weight must be [{self.E},{self.H}], got {tuple(weight.shape)}")
        if bias is not None:
            bias = bias.to(device=self.device, dtype=self.dtype).contiguous()
            if bias.shape != (self.E,):
                raise ValueError(f"gate bias must be [{self.E}]")
        self._gate[layer] = (weight, bias)
        self.generation += 1
        self._check(self._lib.b200moe_set_gate(self._h, layer, _ptr(weight), _ptr(bias), _stream(self.device)))

    def set_expert(self, layer: int, expert: int, params: Dict[str, torch.Tensor]) -> None:
        """Registers one expert.  Dense: {'gate_proj','up_proj','down_proj'} in the context dtype.
        Int4: the same keys hold uint8 [out,in/2] and '<name>_scales' holds bf16 [out,in/128]."""
        g, u, d = params["gate_proj"], params["up_proj"], params["down_proj"]
        if self.weight_mode == W_INT4_G128:
            sg, su, sd = params["gate_proj_scales"], params["up_proj_scales"], params["down_proj_scales"]
            shapes = ((g, (self.I, self.H // 2)), (u, (self.I, self.H // 2)), (d, (self.H, self.I // 2)),
                      (sg, (self.I, self.H // 128)), (su, (self.I, self.H // 128)), (sd, (self.H, self.I // 128)))
            for t in (g, u, d):
                _need_cuda(t, "int4 weight", self.device, torch.uint8)
            for t in (sg, su, sd):
                _need_cuda(t, "int4 scales", self.device, torch.bfloat16)
            tensors = (g, u, d, sg, su, sd)
        else:
            shapes = ((g, (self.I, self.H)), (u, (self.I, self.H)), (d, (self.H, self.I)))
            for t in (g, u, d):
                _need_cuda(t, "expert weight", self.device, self.dtype)
            tensors = (g, u, d, None, None, None)
        for t, shp in shapes:
            if tuple(t.shape) != shp:
                raise ValueError(f"expert {expert}: expected shape {shp}, got {tuple(t.shape)}")
        ptrs = tuple(_ptr(t) for t in tensors)
        key = (layer, expert)
        if self._expert_ptrs.get(key) == ptrs:
            self._experts[key] = tensors
            return
        self._check(self._lib.b200moe_set_expert(self._h, layer, expert, *ptrs))
        self._experts[key] = tensors
        self._expert_ptrs[key] = ptrs
        self.generation += 1

    def clear_expert(self, layer: int, expert: int) -> None:
        self._check(self._lib.b200moe_clear_expert(self._h, layer, expert))
        self._experts.pop((layer, expert), None)
        self._expert_ptrs.pop((layer, expert), None)
        self.generation += 1

    # -- compute ----------------------------------------------------------------------------
    def route(self, layer: int, x2d: torch.Tensor, *, bitmap: Optional[torch.Tensor] = None,
              logits: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """ids int64 [T,K], scores [T,K].  `logits` switches to the top-k/softmax stage on logits
        the caller computed (e.g. with F.linear, the GEMM the reference uses)."""
        src = logits if logits is not None else x2d
        _need_cuda(src, "router input", self.device, self.dtype)
        T = src.shape[0]
        ids = torch.empty(T, self.K, dtype=torch.int64, device=self.device)
        scores = torch.empty(T, self.K, dtype=self.dtype, device=self.device)
        if logits is not None:
            if logits.shape != (T, self.E):
                raise ValueError(f"logits must be [T,{self.E}]")
            self._check(self._lib.b200moe_route_from_logits(self._h, _ptr(logits), T, _ptr(ids), _ptr(scores), _ptr(bitmap), _stream(self.device)))
        else:
            if x2d.shape != (T, self.H):
                raise ValueError(f"x must be [T,{self.H}]")
            self._check(self._lib.b200moe_route(self._h, layer, _ptr(x2d), T, _ptr(ids), _ptr(scores), _ptr(bitmap), _stream(self.device)))
        return ids, scores

    def last_logits(self, T: int) -> torch.Tensor:
        """fp32 copy of the rounded logits [T,E] of the latest route / forward_fused call."""
        out = torch.empty(T, self.E, dtype=torch.float32, device=self.device)
        self._check(self._lib.b200moe_last_logits(self._h, T, _ptr(out), _stream(self.device)))
        return out

    def last_tables(self, T: int):
        """(offsets [E+1], sorted_pair [T*K], inv [T*K], act_list [n_act]) of the latest forward call, as int32 tensors."""
        i32 = dict(dtype=torch.int32, device=self.device)
        offsets, sp, inv = torch.empty(self.E + 1, **i32), torch.empty(T * self.K, **i32), torch.empty(T * self.K, **i32)
        act, n_act = torch.empty(self.E, **i32), torch.empty(1, **i32)
        self._check(self._lib.b200moe_last_tables(self._h, T, _ptr(offsets), _ptr(sp), _ptr(inv), _ptr(act), _ptr(n_act), _stream(self.device)))
        return offsets, sp, inv, act[: int(n_act.item())]

    def group_pairs(self, ids: torch.Tensor):
        """K2 on its own: (offsets [E+1], sorted_pair [valid pairs]) as int32 numpy arrays, through ONE device->host copy."""
        _need_cuda(ids, "ids", self.device, torch.int64)
        T = ids.shape[0]
        tables = torch.empty(self.E + 1 + T * self.K, dtype=torch.int32, pin_memory=True)
        self._check(self._lib.b200moe_group_pairs(self._h, _ptr(ids), T, _ptr(tables), _stream(self.device)))
        torch.cuda.current_stream(self.device).synchronize()
        t = tables.numpy()
        offsets = t[: self.E + 1]
        return offsets, t[self.E + 1: self.E + 1 + int(offsets[-1])]

    def forward(self, layer: int, x2d: torch.Tensor, ids: torch.Tensor, scores: torch.Tensor, *,
                expert_slot: Optional[Sequence[int]] = None, order: Optional[Sequence[int]] = None,
                residual: Optional[torch.Tensor] = None, ffn_kind: int = FFN_AUTO) -> torch.Tensor:
        _need_cuda(x2d, "x", self.device, self.dtype)
        T = x2d.shape[0]
        if x2d.shape != (T, self.H):
            raise ValueError(f"x must be [T,{self.H}]")
        ids = ids.to(device=self.device, dtype=torch.int64).contiguous()
        scores = scores.to(self.device).contiguous()
        if scores.dtype not in (self.dtype, torch.float32):
            scores = scores.to(torch.float32)
        if ids.shape != (T, self.K) or scores.shape != (T, self.K):
            raise ValueError(f"ids and scores must be [T,{self.K}]")
        if residual is not None:
            _need_cuda(residual, "residual", self.device, self.dtype)
        out = torch.empty_like(x2d)
        slot_arr = (c_int32 * self.E)(*expert_slot) if expert_slot is not None else None
        order_arr = (c_int32 * self.E)(*order) if order is not None else None
        self._check(self._lib.b200moe_forward(self._h, layer, _ptr(x2d), T, _ptr(ids), _ptr(scores), dtype_tag(scores.dtype),
                                              slot_arr, order_arr, _ptr(residual), _ptr(out), ffn_kind, _stream(self.device)))
        return out

    def forward_fused(self, layer: int, x2d: torch.Tensor, *, residual: Optional[torch.Tensor] = None,
                      return_routing: bool = False, ffn_kind: int = FFN_AUTO, out: Optional[torch.Tensor] = None):
        _need_cuda(x2d, "x", self.device, self.dtype)
        T = x2d.shape[0]
        if x2d.shape != (T, self.H):
            raise ValueError(f"x must be [T,{self.H}]")
        if residual is not None:
            _need_cuda(residual, "residual", self.device, self.dtype)
        if out is None:
            out = torch.empty_like(x2d)
        ids = scores = None
        if return_routing:
            ids = torch.empty(T, self.K, dtype=torch.int64, device=self.device)
            scores = torch.empty(T, self.K, dtype=self.dtype, device=self.device)
        self._check(self._lib.b200moe_forward_fused(self._h, layer, _ptr(x2d), T, _ptr(residual), _ptr(out), _ptr(ids), _ptr(scores),
                                                    ffn_kind, _stream(self.device)))
        return (out, ids, scores) if return_routing else out

    def forward_fused_norm(self, layer: int, hidden: torch.Tensor, norm_weight: torch.Tensor, eps: float, *,
                           residual: Optional[torch.Tensor] = None, return_parts: bool = False, ffn_kind: int = FFN_AUTO):
        """RMSNorm (+ residual add) -> router -> experts -> combine -> + new residual, one enqueue.
        Returns out, or (out, new_residual, normed, ids, scores) with return_parts."""
        _need_cuda(hidden, "hidden", self.device, self.dtype)
        _need_cuda(norm_weight, "norm_weight", self.device, self.dtype)
        if residual is not None:
            _need_cuda(residual, "residual", self.device, self.dtype)
        T = hidden.shape[0]
        if hidden.shape != (T, self.H) or norm_weight.shape != (self.H,):
            raise ValueError(f"hidden must be [T,{self.H}] and norm_weight [{self.H}]")
        out = torch.empty_like(hidden)
        res_out = normed = ids = scores = None
        if return_parts:
            res_out, normed = torch.empty_like(hidden), torch.empty_like(hidden)
            ids = torch.empty(T, self.K, dtype=torch.int64, device=self.device)
            scores = torch.empty(T, self.K, dtype=self.dtype, device=self.device)
        self._check(self._lib.b200moe_forward_fused_norm(self._h, layer, _ptr(hidden), _ptr(residual), _ptr(norm_weight), float(eps), T, _ptr(out),
                                                         _ptr(res_out), _ptr(normed), _ptr(ids), _ptr(scores), ffn_kind, _stream(self.device)))
        return (out, res_out, normed, ids, scores) if return_parts else out

    # -- expert parallelism (peer-store dispatch / return; include/b200moe.h) -----------------------
    def ep_create(self, world: int, rank: int, max_local_tokens: int) -> bytes:
        """Allocates this rank's exchange buffer and returns its 64-byte IPC handle for the other ranks."""
        buf = ctypes.create_string_buffer(_lib.EP_HANDLE_BYTES)
        with torch.cuda.device(self.device):
            self._check(self._lib.b200moe_ep_create(self._h, world, rank, max_local_tokens, buf))
        self.ep_world, self.ep_rank, self.ep_max_local = world, rank, max_local_tokens
        return buf.raw

    def ep_attach(self, handles: Sequence[bytes]) -> None:
        """Maps the other ranks' exchange buffers from their handles (rank-major; this rank's own entry is ignored)."""
        blob = b"".join(bytes(h) for h in handles)
        if len(blob) != self.ep_world * _lib.EP_HANDLE_BYTES:
            raise ValueError(f"expected {self.ep_world} handles of {_lib.EP_HANDLE_BYTES} bytes")
        with torch.cuda.device(self.device):
            self._check(self._lib.b200moe_ep_attach_ipc(self._h, blob))

    def ep_attach_local(self, ranks: Sequence["MoEContext"]) -> None:
        """The ranks are contexts of this process (one GPU emulating several ranks, or peer-accessible GPUs)."""
        arr = (c_void_p * len(ranks))(*[r._h.value for r in ranks])
        with torch.cuda.device(self.device):
            self._check(self._lib.b200moe_ep_attach_local(self._h, arr))

    def ep_set_wait_ms(self, ms: int) -> None:
        self._check(self._lib.b200moe_ep_set_wait_ms(self._h, ms))

    def ep_detach(self) -> None:
        self._check(self._lib.b200moe_ep_detach(self._h))

    def ep_dispatch(self, layer: int, x_local: torch.Tensor) -> None:
        _need_cuda(x_local, "x_local", self.device, self.dtype)
        if x_local.dim() != 2 or x_local.shape[1] != self.H:
            raise ValueError(f"x_local must be [T_local,{self.H}]")
        self._check(self._lib.b200moe_ep_dispatch(self._h, layer, _ptr(x_local), x_local.shape[0], _stream(self.device)))

    def ep_experts(self, layer: int, *, ffn_kind: int = FFN_AUTO) -> None:
        self._check(self._lib.b200moe_ep_experts(self._h, layer, ffn_kind, _stream(self.device)))

    def ep_combine(self, T_local: int, *, order: Optional[Sequence[int]] = None, residual: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if residual is not None:
            _need_cuda(residual, "residual", self.device, self.dtype)
        if out is None:
            out = torch.empty(T_local, self.H, dtype=self.dtype, device=self.device)
        order_arr = (c_int32 * self.E)(*order) if order is not None else None
        self._check(self._lib.b200moe_ep_combine(self._h, T_local, order_arr, _ptr(residual), _ptr(out), _stream(self.device)))
        return out

    def ep_forward(self, layer: int, x_local: torch.Tensor, *, order: Optional[Sequence[int]] = None,
                   residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, ffn_kind: int = FFN_AUTO) -> torch.Tensor:
        """One expert-parallel layer call for this rank's tokens: dispatch, local experts, combine in one enqueue."""
        _need_cuda(x_local, "x_local", self.device, self.dtype)
        if x_local.dim() != 2 or x_local.shape[1] != self.H:
            raise ValueError(f"x_local must be [T_local,{self.H}]")
        if residual is not None:
            _need_cuda(residual, "residual", self.device, self.dtype)
        if out is None:
            out = torch.empty_like(x_local)
        order_arr = (c_int32 * self.E)(*order) if order is not None else None
        self._check(self._lib.b200moe_ep_forward(self._h, layer, _ptr(x_local), x_local.shape[0], order_arr, _ptr(residual), _ptr(out),
                                                 ffn_kind, _stream(self.device)))
        return out

    def ep_last_routing(self, T_local: int) -> Tuple[torch.Tensor, torch.Tensor]:
        ids = torch.empty(T_local, self.K, dtype=torch.int64, device=self.device)
        scores = torch.empty(T_local, self.K, dtype=self.dtype, device=self.device)
        self._check(self._lib.b200moe_ep_last_routing(self._h, T_local, _ptr(ids), _ptr(scores), _stream(self.device)))
        return ids, scores

    def expert_ffn(self, x2d: torch.Tensor, gate_proj: torch.Tensor, up_proj: torch.Tensor, down_proj: torch.Tensor) -> torch.Tensor:
        for name, t in (("x", x2d), ("gate_proj", gate_proj), ("up_proj", up_proj), ("down_proj", down_proj)):
            _need_cuda(t, name, self.device, self.dtype)
        out = torch.empty_like(x2d)
        self._check(self._lib.b200moe_expert_ffn(self._h, _ptr(x2d), x2d.shape[0], _ptr(gate_proj), _ptr(up_proj), _ptr(down_proj),
                                                 _ptr(out), _stream(self.device)))
        return out

    def rmsnorm(self, x2d: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None):
        """RMSNorm of [T,H] rows, optionally fused with the residual add in front of it
        (demo/src/layers/layernorm.py:21-36).  Returns `out`, or `(out, new_residual)` when `residual` is given."""
        _need_cuda(x2d, "x", self.device, self.dtype)
        _need_cuda(weight, "weight", self.device, self.dtype)
        if residual is not None:
            _need_cuda(residual, "residual", self.device, self.dtype)
        out = torch.empty_like(x2d)
        res_out = torch.empty_like(x2d) if residual is not None else None
        self._check(self._lib.b200moe_rmsnorm(self._h, _ptr(x2d), _ptr(residual), _ptr(weight), float(eps), x2d.shape[0],
                                              _ptr(out), _ptr(res_out), _stream(self.device)))
        return out if residual is None else (out, res_out)

    def profile(self, enable: bool) -> None:
        """Turns per-kernel CUDA-event timing on or off (benchmarks only)."""
        self._check(self._lib.b200moe_profile(self._h, 1 if enable else 0))

    def profile_read(self):
        """{kernel class: (total ms, launches)} since profiling was enabled; waits for the events."""
        ms = (ctypes.c_float * _lib.KERNEL_CLASSES)()
        n = (c_int32 * _lib.KERNEL_CLASSES)()
        self._check(self._lib.b200moe_profile_read(self._h, ms, n))
        return {name: (float(ms[i]), int(n[i])) for i, name in enumerate(_lib.KERNEL_NAMES)}

    def set_token_kernel(self, enable: bool) -> None:
        """Single-token batches of `forward_fused` run as one cooperative launch (default) or through the kernel chain."""
        self._check(self._lib.b200moe_set_token_kernel(self._h, 1 if enable else 0))

    def status(self) -> int:
        """Synchronises the current stream and returns the device status word (0 = clean); raises when it is not."""
        v = c_int(0)
        self._check(self._lib.b200moe_status(self._h, byref(v), _stream(self.device)))
        return v.value
