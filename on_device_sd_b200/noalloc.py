"""Expert FFN without any device allocation (b200moe_expert_ffn_noalloc).

For callers that own every byte of the GPU themselves - an engine whose pools already hold the
weights and the KV cache - or that run where cudaMalloc's device-wide synchronisation is not
acceptable: no context, no workspace, no output tensor is created here.  The caller passes the
output buffer; the library's built-in scratch (about 2 MiB per GPU) holds the intermediate.
Limits: at most 64 rows and rows * intermediate_size * element size <= 2 MiB.  Calls share that
scratch, so do not let two of them overlap on the GPU."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check
from .context import _ptr, _stream, dtype_tag


def expert_forward_noalloc(x: torch.Tensor, gate_weight: torch.Tensor, up_weight: torch.Tensor, down_weight: torch.Tensor,
                           out: torch.Tensor) -> torch.Tensor:
    """x [n,H] -> out [n,H] (written in place and returned); same math as expert_forward_with_weights."""
    for name, t in (("x", x), ("gate_weight", gate_weight), ("up_weight", up_weight), ("down_weight", down_weight), ("out", out)):
        if not t.is_cuda or not t.is_contiguous() or t.dtype != x.dtype or t.device != x.device:
            raise ValueError(f"{name} must be a contiguous CUDA tensor of x's dtype on x's device")
    n, H = x.shape
    I = gate_weight.shape[0]
    if gate_weight.shape != (I, H) or up_weight.shape != (I, H) or down_weight.shape != (H, I) or out.shape != (n, H):
        raise ValueError("shape mismatch: gate/up [I,H], down [H,I], out [n,H]")
    with torch.cuda.device(x.device):
        check(None, _lib.load().b200moe_expert_ffn_noalloc(_ptr(x), n, H, I, dtype_tag(x.dtype), _ptr(gate_weight), _ptr(up_weight),
                                                           _ptr(down_weight), _ptr(out), _stream(x.device)))
    return out


def noalloc_status(device: torch.device) -> int:
    """Waits for the current stream of `device` and returns the status word of the latest
    expert_forward_noalloc call there (0 = clean); raises B200MoEError when a kernel's bounded wait
    gave up.  Allocates nothing either."""
    import ctypes
    v = ctypes.c_int(0)
    with torch.cuda.device(device):
        check(None, _lib.load().b200moe_expert_ffn_noalloc_status(ctypes.byref(v), _stream(torch.device(device))))
    return v.value
