"""on_device_sd_b200 - the MoE block forward of on_device_sd's demo engine, rebuilt for B200.

Hot path: router -> token-to-expert permute -> grouped SwiGLU expert FFN -> weighted combine,
as hand-written sm_100a CUDA behind a C ABI (libb200moe.so, include/b200moe.h).  This package
is the host-side mirror of the reference's interfaces for that path and nothing else.
"""
from ._lib import (B200MoEError, BF16, F16, F32, FFN_AUTO, FFN_GEMV, FFN_MMA, W_DENSE, W_INT4_G128)
from .activations import build_layer_activations
from .context import MoEContext
from .ingest import LayerSlab, ingest_layer
from .layers import Qwen3MoEGate, Qwen3MoELayer, Qwen3MoELayerWithWeights, RMSNorm, expert_forward_with_weights
from .runner import B200MoERunner
from .types import AttentionOutput, ExpertActivation, ExpertID, LayerExpertActivations, ExpertPlacement, MoEShape, RoutingResult

__all__ = [
    "B200MoEError", "MoEContext", "B200MoERunner", "Qwen3MoEGate", "Qwen3MoELayer", "Qwen3MoELayerWithWeights", "RMSNorm",
    "expert_forward_with_weights", "build_layer_activations", "LayerSlab", "ingest_layer", "ExpertActivation", "LayerExpertActivations",
    "AttentionOutput", "ExpertID", "ExpertPlacement", "MoEShape", "RoutingResult",
    "F32", "F16", "BF16", "W_DENSE", "W_INT4_G128", "FFN_AUTO", "FFN_GEMV", "FFN_MMA",
]
