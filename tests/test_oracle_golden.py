"""CPU: the oracle against the fixtures produced from the reference itself."""
import hashlib

import numpy as np
import pytest
import torch

from conftest import GOLDEN, Golden, from_np
from oracle import moe_oracle as O


def test_oracle_reproduces_reference_outputs(golden):
    """Given the reference's two library choices (F.linear logits, torch.topk on this device) the
    restatement equals the stored reference outputs bit for bit (same torch build, CPU)."""
    g = golden
    ids, scores, _ = O.route(g.x, g.gate_w, g.K, tie="torch", logits="linear")
    assert torch.equal(ids, g.t("ref_ids"))
    assert torch.equal(scores, g.t("ref_scores"))
    order = O.activated_order(g.layer_idx, ids)
    assert order == g.t("ref_order").tolist()
    out_b = O.moe_engine(g.x, ids, scores, g.experts, layer_idx=g.layer_idx)
    assert torch.equal(out_b, g.t("ref_out_engine"))
    out_res = O.moe_engine(g.x, ids, scores, g.experts, layer_idx=g.layer_idx, residual=g.x)
    assert torch.equal(out_res, g.t("ref_out_engine_residual"))
    out_a = O.moe_layer(g.x, g.gate_w, g.experts, g.K, tie="torch", logits="linear")
    assert torch.equal(out_a, g.t("ref_out_layer"))
    assert torch.equal(O.expert_ffn(g.x, **g.experts[0]), g.t("ref_ffn0"))


def test_oracle_definition_outputs(golden):
    """The device-independent definition (exact logits, CUDA tie order) reproduces its stored outputs
    and stays within the path's tolerance of the reference's own outputs."""
    g = golden
    ids, scores, logits = O.route(g.x, g.gate_w, g.K)
    assert torch.equal(ids, g.t("def_ids"))
    assert torch.equal(scores, g.t("def_scores"))
    assert torch.equal(logits, g.t("def_logits"))
    out = O.moe_engine(g.x, ids, scores, g.experts, layer_idx=g.layer_idx)
    assert torch.equal(out, g.t("def_out_engine"))
    assert O.max_abs(out, g.t("ref_out_engine")) <= 2e-2
    assert O.mean_rel(out, g.t("ref_out_engine")) <= 5e-3
    # same expert sets as the reference chose, token by token
    assert torch.equal(ids.sort(-1).values, g.t("ref_ids").sort(-1).values)


def test_large_case_inputs_match_digest():
    g = Golden("toy_fp32")
    h = hashlib.sha256()
    h.update(g.gate_w.numpy().tobytes())
    for e in sorted(g.experts):
        for k in ("gate_proj", "up_proj", "down_proj"):
            h.update(g.experts[e][k].numpy().tobytes())
    h.update(g.x.numpy().tobytes())
    assert h.hexdigest() == str(g.z["input_sha256"])


def test_topk_tie_order_matches_cuda_fixture():
    """topk_cuda_order against indices torch.topk produced on a B200 for tie-heavy inputs."""
    z = np.load(GOLDEN / "topk_cuda_ties.npz")
    names = sorted(k[:-3] for k in z.files if k.endswith("_in"))
    assert len(names) >= 30
    for n in names:
        vin, idx = z[n + "_in"], z[n + "_idx"]
        _, got = O.topk_cuda_order(torch.from_numpy(vin.astype(np.float32)), idx.shape[1])
        assert np.array_equal(got.numpy(), idx.astype(np.int64)), n


def test_placement_semantics_fixture():
    """Substitution, silently skipped experts and fp32 scores with an fp16 model (qwen3_runner.py:298-333, :376)."""
    z = np.load(GOLDEN / "placement_fp16.npz")
    x = torch.from_numpy(z["x"])
    experts = {e: {k: torch.from_numpy(z[f"expert{e}_{k}"]) for k in ("gate_proj", "up_proj", "down_proj")} for e in range(4)}
    avail = {0: experts[0], 2: experts[2]}
    ids, scores = torch.from_numpy(z["ids"]), torch.from_numpy(z["scores"])
    assert O.activated_order(0, ids) == z["ref_order"].tolist()
    out = O.moe_engine(x, ids, scores, avail, substitution={1: 2})
    assert torch.equal(out, torch.from_numpy(z["ref_out_f32scores"]))
    out = O.moe_engine(x, ids, scores.half(), avail, substitution={1: 2})
    assert torch.equal(out, torch.from_numpy(z["ref_out_f16scores"]))


def test_int4_fixture_and_roundtrip():
    z = np.load(GOLDEN / "int4_g128.npz")
    w = from_np(z["w"], torch.bfloat16)
    q, s = O.quant_int4_g128(w)
    assert np.array_equal(q.numpy(), z["q"])
    assert torch.equal(s, from_np(z["scales"], torch.bfloat16))
    qi = O.unpack_int4(q)
    assert np.array_equal(qi.numpy(), z["unpacked"])
    assert int(qi.min()) >= -8 and int(qi.max()) <= 7
    dq = O.dequant_int4_g128(q, s)
    assert torch.equal(dq, from_np(z["dequant"], torch.bfloat16))
    # idempotence: quantising the dequantised weights returns the same nibbles and scales
    q2, s2 = O.quant_int4_g128(dq)
    assert torch.equal(q2, q) and torch.equal(s2, s)
    # the all-zero group gets scale 1 and stores the zero code (8)
    assert float(s[3, 1]) == 1.0 and bool((qi[3, 128:256] == 0).all())
    # error bound of symmetric rounding: |w - dq| <= scale/2, plus the bf16 rounding of scale*q (<= 7*scale*2^-9)
    err = (w.float() - dq.float()).abs().view(24, 3, 128)
    assert bool((err <= s.float().unsqueeze(-1) * 0.52 + 1e-6).all())


@pytest.mark.parametrize("T,E,K", [(0, 8, 2), (1, 8, 8), (5, 33, 7)])
def test_route_shapes_and_edge_cases(T, E, K):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(T, 64, generator=g)
    w = torch.randn(E, 64, generator=g) * 0.02
    ids, scores, logits = O.route(x, w, K)
    assert ids.shape == (T, K) and scores.shape == (T, K) and logits.shape == (T, E)
    if T:
        assert torch.allclose(scores.sum(-1), torch.ones(T), atol=1e-5)   # reference test_routing.py:18-24
        assert bool((ids.sort(-1).values == torch.topk(logits, K).indices.sort(-1).values).all())
        for t in range(T):
            assert len(set(ids[t].tolist())) == K


def test_rmsnorm_restatement_matches_reference_fixture():
    """tests/golden/rmsnorm.npz holds outputs of the reference's RMSNorm (demo/src/layers/layernorm.py:9-47)."""
    z = np.load(GOLDEN / "rmsnorm.npz")
    for name, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        x, r, w = (from_np(z[f"{name}_{k}"], dt) for k in ("x", "r", "w"))
        assert torch.equal(O.rmsnorm(x, w, 1e-6), from_np(z[f"{name}_out"], dt))
        out, res = O.rmsnorm(x, w, 1e-6, r)
        assert torch.equal(out, from_np(z[f"{name}_out_add"], dt)) and torch.equal(res, from_np(z[f"{name}_res"], dt))


def load_mixed_placement():
    """Fixture written from the reference's _execute_moe_with_placement on a placement that mixes
    GPU-resident and CPU-resident experts (demo/src/model/qwen3_runner.py:298-383)."""
    z = np.load(GOLDEN / "mixed_placement_bf16.npz")
    bf = torch.bfloat16
    experts = {e: {k: from_np(z[f"expert{e}_{k}"], bf) for k in ("gate_proj", "up_proj", "down_proj")} for e in range(12)}
    return dict(z=z, x=from_np(z["x"], bf), ids=torch.from_numpy(z["ids"].astype(np.int64)), scores=from_np(z["scores"], bf),
                gpu={int(e): experts[int(e)] for e in z["gpu_experts"]}, cpu={int(e): experts[int(e)] for e in z["cpu_experts"]},
                sub={int(a): int(b) for a, b in zip(z["sub_from"], z["sub_to"])}, ref=from_np(z["ref_out"], bf),
                order=z["ref_order"].tolist(), layer_idx=int(z["layer_idx"]))


def test_oracle_mixed_placement_accumulates_gpu_tasks_first():
    m = load_mixed_placement()
    assert O.activated_order(m["layer_idx"], m["ids"]) == m["order"]
    out = O.moe_engine(m["x"], m["ids"], m["scores"], m["gpu"], layer_idx=m["layer_idx"], substitution=m["sub"], cpu_experts=m["cpu"])
    assert torch.equal(out, m["ref"])
