"""CPU: host-side logic of the drop-in layer (no kernels involved)."""
import torch

from on_device_sd_b200.runner import plan_placement
from on_device_sd_b200.synth import CONFIGS, make_layer, make_named, zipf_bias
from on_device_sd_b200.types import AttentionOutput, ExpertID, ExpertPlacement, MoEShape, RoutingResult
from oracle import moe_oracle as O


def _routing(layer, ids):
    act = {ExpertID(layer, i) for i in ids.flatten().unique().tolist()}
    return RoutingResult(layer_idx=layer, topk_indices=ids, topk_scores=torch.full(ids.shape, 0.5), activated_expert_ids=act)


def test_expert_id_hash_matches_reference_definition():
    # demo/src/core/types.py:19-29: hash((layer_idx, expert_idx)); the accumulation order depends on it
    assert hash(ExpertID(3, 17)) == hash((3, 17))
    assert ExpertID(1, 2) == ExpertID(1, 2) and str(ExpertID(1, 2)) == "L1_E2"


def test_plan_placement_order_is_set_iteration_order():
    ids = torch.tensor([[5, 1], [127, 64], [3, 9], [17, 100]])
    r = _routing(3, ids)
    p = ExpertPlacement(gpu_expert_params={e: {} for e in range(128)}, cpu_expert_params={}, routing_result=r)
    avail, slot, order = plan_placement(p, 128)
    visit = [eid.expert_idx for eid in r.activated_expert_ids]
    assert visit == O.activated_order(3, ids)      # the oracle's emulation of the same set
    for rank, e in enumerate(visit):
        assert order[e] == rank and slot[e] == e
    assert all(slot[e] == -1 for e in range(128) if e not in visit)
    assert all(order[e] == len(visit) for e in range(128) if e not in visit)


def test_plan_placement_substitution_skip_and_cpu_params():
    ids = torch.tensor([[0, 1], [2, 3]])
    r = _routing(0, ids)
    g0, c1, g2 = {"tag": "g0"}, {"tag": "c1"}, {"tag": "g2"}
    p = ExpertPlacement(gpu_expert_params={0: g0, 2: g2}, cpu_expert_params={1: c1, 2: {"tag": "c2"}},
                        substitution_map={3: 2, 1: 0}, routing_result=r)
    avail, slot, order = plan_placement(p, 4)
    assert avail[2] is g2 and avail[1] is c1            # GPU copy wins; CPU-resident experts are usable
    assert slot == [0, 1, 2, 2]                          # 3 -> substitute 2; 1 has its own params, substitution unused
    p = ExpertPlacement(gpu_expert_params={0: g0}, cpu_expert_params={}, substitution_map={3: 2}, routing_result=r)
    assert plan_placement(p, 4)[1] == [0, -1, -1, -1]    # substitute absent too -> skipped silently


def test_synth_is_deterministic_and_distributed_as_stated():
    a = make_layer(64, 4, 2, 32, torch.bfloat16, 5, seed=0)
    b = make_layer(64, 4, 2, 32, torch.bfloat16, 5, seed=0)
    assert torch.equal(a.gate_w, b.gate_w) and torch.equal(a.x, b.x)
    assert torch.equal(a.experts[3]["down_proj"], b.experts[3]["down_proj"])
    c = make_layer(64, 4, 2, 32, torch.bfloat16, 5, seed=1)
    assert not torch.equal(a.x, c.x)
    big = make_layer(256, 2, 1, 256, torch.float32, 64, seed=0)
    assert abs(float(big.experts[0]["gate_proj"].std()) - 0.02) < 1e-3 and abs(float(big.x.std()) - 1.0) < 2e-2
    assert CONFIGS["mixtral"][:4] == (4096, 8, 2, 14336) and CONFIGS["qwen3"][:4] == (2048, 128, 8, 768)
    assert make_named("tiny_fp16", 3).x.shape == (3, 32)


def test_zipf_bias_is_a_log_distribution():
    b = zipf_bias(128, 1.1, seed=0)
    p = b.double().exp()
    assert abs(float(p.sum()) - 1.0) < 1e-5
    top = p.sort(descending=True).values
    assert abs(float(top[0] / top[1]) - 2 ** 1.1) < 1e-3


def test_moe_shape_mirrors_config_dtype_rule():
    assert MoEShape(8, 2, 1, 8, "bfloat16").get_dtype() == torch.bfloat16
    assert MoEShape(8, 2, 1, 8, "float32").get_dtype() == torch.float32
    assert MoEShape(8, 2, 1, 8, "weird").get_dtype() == torch.float16   # demo/src/core/model.py:129 default
    a = AttentionOutput(torch.zeros(1), torch.zeros(1), torch.zeros(1))
    assert a.residual is not None
