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


def test_plan_placement_ranks_gpu_served_experts_before_cpu_served_ones():
    """The reference adds every GPU task before any CPU task (qwen3_runner.py:352-383): on its own mixed
    fixture the rank table must reproduce that sequence, which the oracle then turns into the stored output."""
    from test_oracle_golden import load_mixed_placement
    m = load_mixed_placement()
    act = set()
    for e in m["ids"].flatten().unique().tolist():
        act.add(ExpertID(m["layer_idx"], int(e)))
    r = RoutingResult(m["layer_idx"], m["ids"], m["scores"], act)
    avail, slot, order = plan_placement(ExpertPlacement(m["gpu"], m["cpu"], m["sub"], r), 12)
    visit = [eid.expert_idx for eid in act]
    assert visit == m["order"]
    gpu_served = [e for e in visit if e in m["gpu"] or (e not in m["cpu"] and m["sub"].get(e) in m["gpu"])]
    cpu_served = [e for e in visit if e not in gpu_served and (e in m["cpu"] or m["sub"].get(e) in m["cpu"])]
    assert cpu_served and gpu_served
    for rank, e in enumerate(gpu_served + cpu_served):
        assert order[e] == rank
    assert slot[6] == 1 and slot[9] == 4 and slot[10] == -1 and avail[7] is m["gpu"][7]     # resident in both: the GPU copy wins
    # the oracle, driven by that sequence and nothing else, reproduces the reference's output bit for bit
    served = {**m["cpu"], **m["gpu"]}
    table = {e: served[slot[e]] for e in visit if slot[e] >= 0}
    out = O.moe_engine(m["x"], m["ids"], m["scores"], table, order=sorted(table, key=lambda e: order[e]))
    assert torch.equal(out, m["ref"])


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


def _check_activations(acts, want, layer_idx, scores):
    assert acts.layer_idx == layer_idx and acts.routing_scores is scores
    assert len(acts.activations) == len(want)
    for a, (k, e, tok, sc) in zip(acts.activations, want):
        assert (a.top_k_rank, a.expert_id.layer_idx, a.expert_id.expert_idx) == (k, layer_idx, e)
        assert a.token_indices.dtype == torch.int64 and torch.equal(a.token_indices.cpu(), tok)
        assert a.scores.dtype == scores.dtype and torch.equal(a.scores.cpu(), sc)


def test_build_layer_activations_matches_reference_fixture():
    """Fixture written from the reference's own build_layer_activations
    (demo/src/execution/model_runner_utils.py:13-41): order, token lists and scores."""
    import numpy as np
    from conftest import GOLDEN, from_np
    from on_device_sd_b200 import build_layer_activations
    z = np.load(GOLDEN / "activations_bf16.npz")
    ids = torch.from_numpy(z["ids"].astype(np.int64))
    scores = from_np(z["scores"], torch.bfloat16)
    acts = build_layer_activations(RoutingResult(3, ids, scores, set()), int(z["num_experts"]))
    cuts = np.r_[0, np.cumsum(z["count"])]
    toks, asc = torch.from_numpy(z["tokens"].astype(np.int64)), from_np(z["act_scores"], torch.bfloat16)
    want = [(int(k), int(e), toks[a:b], asc[a:b]) for k, e, a, b in zip(z["rank"], z["expert"], cuts[:-1], cuts[1:])]
    _check_activations(acts, want, 3, scores)


def test_build_layer_activations_matches_oracle_on_random_and_edge_inputs():
    from on_device_sd_b200 import build_layer_activations
    g = torch.Generator().manual_seed(11)
    for T, K, E in [(1, 1, 4), (7, 2, 8), (64, 8, 128), (33, 4, 5)]:
        ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]) if K <= E else torch.randint(0, E, (T, K), generator=g)
        scores = torch.rand(T, K, generator=g).to(torch.float16)
        _check_activations(build_layer_activations(RoutingResult(1, ids, scores, set()), E), O.layer_activations(ids, scores, E), 1, scores)
    # duplicates inside a token, ids outside [0, E) (never matched by the reference's comparison), empty batch
    ids = torch.tensor([[0, 0], [5, 1], [-1, 2], [2, 2]])
    scores = torch.rand(4, 2, generator=g)
    _check_activations(build_layer_activations(RoutingResult(0, ids, scores, set()), 4), O.layer_activations(ids, scores, 4), 0, scores)
    empty = build_layer_activations(RoutingResult(0, torch.zeros(0, 2, dtype=torch.int64), torch.zeros(0, 2), set()), 4)
    assert empty.activations == []
