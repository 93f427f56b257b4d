"""The roofline arithmetic of bench.py: algorithmic bytes per layer forward must equal the figures of the
measurement plan (distinct experts x bytes per expert + gate weight + tokens in and out)."""
import importlib.util
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("b200moe_bench", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules.setdefault("b200moe_bench", mod)
    spec.loader.exec_module(mod)
    return mod


# (H, E, I, T, distinct experts, int4) -> MB of the layer; expected values with uniform routing:
# Mixtral-shaped T=1 hits K=2 experts, T=64 all 8; Qwen3-shaped T=1 hits 8, T=256 all 128.
@pytest.mark.parametrize("H,E,I,T,U,int4,mb", [
    (4096, 8, 14336, 1, 2, False, 704.7),
    (4096, 8, 14336, 64, 8, False, 2819.7),
    (4096, 8, 14336, 64, 8, True, 727.8),
    (2048, 128, 768, 1, 8, False, 76.0),
    (2048, 128, 768, 256, 128, False, 1210.6),
    (2048, 128, 768, 256, 128, True, 314.1),
])
def test_algorithmic_bytes_match_the_measurement_plan(H, E, I, T, U, int4, mb):
    layer, gate_up = _bench().algorithmic_bytes(H, E, I, T, U, int4)
    assert abs(layer / 1e6 - mb) < 0.06, layer / 1e6
    per_expert = (3 * H * I // 2 + 3 * H * I // 128 * 2) if int4 else 3 * H * I * 2
    assert gate_up == U * per_expert * 2 // 3 + T * H * 2          # two of the three matrices + the tokens read


def test_workload_tables_name_the_baseline_configs():
    b = _bench()
    assert b.WORKLOADS["mixtral_bf16"] == ("mixtral", "bf16", (1, 4, 8, 16, 64))
    assert b.WORKLOADS["qwen3_int4"][2] == (1, 2, 4, 8, 16, 32, 64, 128, 256)
    assert set(b.EP_WORKLOADS) == {"qwen3_bf16_ep", "qwen3_int4_ep", "qwen3_bf16_stack", "qwen3_int4_stack"}
    assert b.METRIC == "MoE-layer tokens/s at verify batch" and b.UNIT == "tokens/s"
