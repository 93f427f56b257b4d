"""Int4 g128 expert weights: device packer / unpacker over the C ABI.

The reference has no quantised weights; the format is this library's (see include/b200moe.h):
symmetric scales per 128 consecutive input features, two values per byte."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from . import _lib
from ._lib import check
from .context import _ptr, _stream, dtype_tag

GROUP = 128


def pack_int4(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[out,in] float tensor on CUDA -> (uint8 [out,in/2], bf16 scales [out,in/128])."""
    if not w.is_cuda or w.dim() != 2 or not w.is_contiguous():
        raise ValueError("pack_int4 wants a contiguous 2-D CUDA tensor")
    out_f, in_f = w.shape
    if in_f % GROUP:
        raise ValueError(f"in_features must be a multiple of {GROUP}")
    q = torch.empty(out_f, in_f // 2, dtype=torch.uint8, device=w.device)
    s = torch.empty(out_f, in_f // GROUP, dtype=torch.bfloat16, device=w.device)
    with torch.cuda.device(w.device):
        check(None, _lib.load().b200moe_pack_int4(_ptr(w), out_f, in_f, dtype_tag(w.dtype), _ptr(q), _ptr(s), _stream(w.device)))
    return q, s


def unpack_int4(q: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (int8 [out,in] with values -8..7, dequantised [out,in] in `dtype`)."""
    if not q.is_cuda or q.dtype != torch.uint8 or not q.is_contiguous():
        raise ValueError("unpack_int4 wants a contiguous uint8 CUDA tensor")
    out_f, in_f = q.shape[0], q.shape[1] * 2
    scales = scales.contiguous()
    qi = torch.empty(out_f, in_f, dtype=torch.int8, device=q.device)
    w = torch.empty(out_f, in_f, dtype=dtype, device=q.device)
    with torch.cuda.device(q.device):
        check(None, _lib.load().b200moe_unpack_int4(_ptr(q), _ptr(scales), out_f, in_f, dtype_tag(dtype), _ptr(qi), _ptr(w), _stream(q.device)))
    return qi, w


def quantize_expert(params: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """{'gate_proj','up_proj','down_proj'} -> the int4 dict MoEContext.set_expert takes."""
    out: Dict[str, torch.Tensor] = {}
    for name in ("gate_proj", "up_proj", "down_proj"):
        q, s = pack_int4(params[name].contiguous())
        out[name] = q
        out[name + "_scales"] = s
    return out
