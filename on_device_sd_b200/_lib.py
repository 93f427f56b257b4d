"""ctypes binding of libb200moe.so (the C ABI declared in include/b200moe.h).

The library is the product; this module only loads it and fails loudly when it is missing or
cannot be loaded.  There is no eager-PyTorch or CPU fallback anywhere in the package.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, POINTER, Structure, c_char_p, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libb200moe.so"

OK, E_ARG, E_CUDA, E_STATE, E_DEVICE, E_UNSUPPORTED = 0, 1, 2, 3, 4, 5
F32, F16, BF16 = 0, 1, 2
W_DENSE, W_INT4_G128 = 0, 1
FFN_AUTO, FFN_GEMV, FFN_MMA = 0, 1, 2
MAX_EXPERTS, MAX_TOPK = 256, 32
EP_HANDLE_BYTES = 64
KERNEL_CLASSES = 8
KERNEL_NAMES = ("router", "permute", "ffn_gate_up", "ffn_down", "combine", "ep_dispatch", "ep_return", "token_block")
ABI_VERSION = 2


class Config(Structure):
    _fields_ = [
        ("hidden_size", c_int32), ("num_experts", c_int32), ("top_k", c_int32), ("intermediate_size", c_int32),
        ("act_dtype", c_int32), ("weight_mode", c_int32), ("num_layers", c_int32), ("max_tokens", c_int32),
        ("device", c_int32), ("reserved", c_int32),
    ]


# name -> (restype, argtypes); every symbol include/b200moe.h declares
PROTOTYPES = {
    "b200moe_abi_version": (c_int, []),
    "b200moe_last_error": (c_char_p, [c_void_p]),
    "b200moe_create": (c_int, [POINTER(Config), POINTER(c_void_p)]),
    "b200moe_destroy": (c_int, [c_void_p]),
    "b200moe_set_gate": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200moe_set_expert": (c_int, [c_void_p, c_int, c_int] + [c_void_p] * 6),
    "b200moe_clear_expert": (c_int, [c_void_p, c_int, c_int]),
    "b200moe_route": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200moe_route_from_logits": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200moe_last_logits": (c_int, [c_void_p, c_int, c_void_p, c_void_p]),
    "b200moe_forward": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, POINTER(c_int32),
                                POINTER(c_int32), c_void_p, c_void_p, c_int, c_void_p]),
    "b200moe_forward_fused": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "b200moe_forward_fused_norm": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int, c_void_p]),
    "b200moe_ep_create": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p]),
    "b200moe_ep_attach_ipc": (c_int, [c_void_p, c_void_p]),
    "b200moe_ep_attach_local": (c_int, [c_void_p, POINTER(c_void_p)]),
    "b200moe_ep_set_wait_ms": (c_int, [c_void_p, c_int]),
    "b200moe_ep_detach": (c_int, [c_void_p]),
    "b200moe_ep_dispatch": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "b200moe_ep_experts": (c_int, [c_void_p, c_int, c_int, c_void_p]),
    "b200moe_ep_combine": (c_int, [c_void_p, c_int, POINTER(c_int32), c_void_p, c_void_p, c_void_p]),
    "b200moe_ep_forward": (c_int, [c_void_p, c_int, c_void_p, c_int, POINTER(c_int32), c_void_p, c_void_p, c_int, c_void_p]),
    "b200moe_ep_last_routing": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200moe_expert_ffn": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200moe_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "b200moe_expert_ffn_noalloc": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200moe_expert_ffn_noalloc_status": (c_int, [POINTER(c_int), c_void_p]),
    "b200moe_last_tables": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "b200moe_group_pairs": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "b200moe_pack_int4": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b200moe_unpack_int4": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "b200moe_profile": (c_int, [c_void_p, c_int]),
    "b200moe_profile_read": (c_int, [c_void_p, c_void_p, c_void_p]),
    "b200moe_set_token_kernel": (c_int, [c_void_p, c_int]),
    "b200moe_status": (c_int, [c_void_p, POINTER(c_int), c_void_p]),
    "b200moe_launch_count": (c_int64, [c_void_p]),
}

_lib = None


class B200MoEError(RuntimeError):
    """A non-zero status from the library (the reference signals errors as exceptions, which
    ContinuousBatchEngine.step turns into per-sequence ERROR states, demo/src/execution/cb_engine.py:70-73)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"b200moe status {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    """Loads libb200moe.so from the package directory and binds every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m on_device_sd_b200.build` "
            "(needs nvcc with sm_100a support). There is no fallback path.")
    lib = ctypes.CDLL(os.fspath(LIB_PATH))
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    if lib.b200moe_abi_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH} has ABI version {lib.b200moe_abi_version()}, this binding expects {ABI_VERSION}; rebuild it")
    _lib = lib
    return lib


def check(ctx, code: int) -> None:
    if code != OK:
        msg = load().b200moe_last_error(ctx)
        raise B200MoEError(code, msg.decode() if msg else "unknown error")
