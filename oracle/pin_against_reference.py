"""Pins oracle/moe_oracle.py against the reference itself and writes tests/golden/*.npz.

TEST INFRASTRUCTURE.  Run in a container that has the reference checked out:

    python oracle/pin_against_reference.py --reference <checkout of potatoZhx/on_device_sd>
    (or set ON_DEVICE_SD_REFERENCE to that directory)

It imports the reference's own modules (demo/src/layers/moe_layer.py, demo/src/model/
qwen3_runner.py, demo/src/core/*) on the CPU, runs both of its MoE paths on seeded inputs and
checks that the restatement reproduces them BIT FOR BIT when it is given the same two
library-defined choices the reference makes on that device (F.linear logits, torch.topk tie
order).  It then stores inputs and reference outputs as fixtures, together with the outputs of
the oracle's device-independent definition (exact logits, CUDA tie order), which is what the
CUDA kernels are compared with.  The reference's tests hold no golden vectors for this path,
so these fixtures are the pin.
"""
from __future__ import annotations

import argparse
import os
import hashlib
import sys
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import moe_oracle as O  # noqa: E402
from on_device_sd_b200.synth import make_layer  # noqa: E402


def to_np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().copy()
    return t.numpy().copy()


def digest(layer) -> str:
    h = hashlib.sha256()
    h.update(to_np(layer.gate_w).tobytes())
    for e in sorted(layer.experts):
        for k in ("gate_proj", "up_proj", "down_proj"):
            h.update(to_np(layer.experts[e][k]).tobytes())
    h.update(to_np(layer.x).tobytes())
    return h.hexdigest()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("ON_DEVICE_SD_REFERENCE"), required=os.environ.get("ON_DEVICE_SD_REFERENCE") is None,
                    help="directory of the reference checkout (the one that contains demo/)")
    args = ap.parse_args()
    sys.path.insert(0, str(Path(args.reference) / "demo"))
    from src.core.model_runner import AttentionOutput, ExpertPlacement, RoutingResult  # type: ignore
    from src.core.types import ExpertID  # type: ignore
    from src.layers.moe_layer import Qwen3MoEGate, Qwen3MoELayer, Qwen3MoELayerWithWeights  # type: ignore
    from src.layers.mlp import expert_forward_with_weights  # type: ignore
    from src.model.qwen3_runner import Qwen3ModelRunner  # type: ignore

    golden = ROOT / "tests" / "golden"
    golden.mkdir(parents=True, exist_ok=True)
    torch.set_num_threads(8)

    def reference_runner(layer, layer_idx=0):
        # the constructor hard-codes cuda; the reference's own tests bypass it the same way
        # (demo/tests/unit/test_engine_optimizations.py:634)
        r = Qwen3ModelRunner.__new__(Qwen3ModelRunner)
        gate = Qwen3MoEGate(layer.H, layer.E).to(layer.dtype)
        gate.load_weights(layer.gate_w)
        r.layers = [None] * layer_idx + [types.SimpleNamespace(mlp=types.SimpleNamespace(gate=gate))]
        r.config = types.SimpleNamespace(num_experts_per_token=layer.K)
        return r

    cases = {
        # name: (H, E, K, I, dtype, T, layer_idx, store_inputs)
        "toy_fp32": (1024, 8, 2, 2816, torch.float32, 64, 0, False),
        "tiny_fp16": (32, 4, 2, 16, torch.float16, 8, 0, True),
        "small_bf16": (256, 16, 4, 128, torch.bfloat16, 24, 3, True),
        "small_fp32": (64, 8, 3, 40, torch.float32, 5, 1, True),
    }
    for name, (H, E, K, I, dtype, T, li, store) in cases.items():
        layer = make_layer(H, E, K, I, dtype, T, seed=0)
        r = reference_runner(layer, li)
        with torch.no_grad():
            x3 = layer.x.unsqueeze(0)
            routing = r.route_experts(li, x3)
            placement = ExpertPlacement(gpu_expert_params=layer.experts, cpu_expert_params={}, routing_result=routing)
            attn = AttentionOutput(hidden_states=x3, post_attn_normed=x3, residual=x3)
            ref_b = r._execute_moe_with_placement(x3, placement)
            ref_b_res = r.forward_moe(li, attn, placement)
            mod_a = Qwen3MoELayer(H, E, K, I, li).to(dtype)
            mod_a.gate.load_weights(layer.gate_w)
            ref_a = mod_a(x3, layer.experts)
            ref_a2 = Qwen3MoELayerWithWeights(H, E, K, I, li)(x3, layer.gate_w, layer.experts)
            ref_ffn = expert_forward_with_weights(layer.x, **{k.replace("_proj", "_weight"): v for k, v in layer.experts[0].items()})
            ref_order = [eid.expert_idx for eid in routing.activated_expert_ids]

            # 1. restatement given the reference's library choices on this device: bit for bit
            ids, scores, _ = O.route(layer.x, layer.gate_w, K, tie="torch", logits="linear")
            assert torch.equal(ids, routing.topk_indices), name
            assert torch.equal(scores, routing.topk_scores), name
            assert O.activated_order(li, ids) == ref_order, name
            ob = O.moe_engine(layer.x, ids, scores, layer.experts, layer_idx=li)
            assert torch.equal(ob, ref_b[0]), (name, O.max_abs(ob, ref_b[0]))
            obr = O.moe_engine(layer.x, ids, scores, layer.experts, layer_idx=li, residual=layer.x)
            assert torch.equal(obr, ref_b_res[0]), name
            oa = O.moe_layer(layer.x, layer.gate_w, layer.experts, K, tie="torch", logits="linear")
            assert torch.equal(oa, ref_a[0]) and torch.equal(oa, ref_a2[0]), name
            assert torch.equal(O.expert_ffn(layer.x, **layer.experts[0]), ref_ffn), name

            # 2. the device-independent definition the CUDA path is held to
            ids_x, scores_x, logits_x = O.route(layer.x, layer.gate_w, K, tie="cuda", logits="exact")
            same_ids = bool(torch.equal(ids_x, ids))
            out_b = O.moe_engine(layer.x, ids_x, scores_x, layer.experts, layer_idx=li)
            out_a = O.moe_layer(layer.x, layer.gate_w, layer.experts, K)
            print(f"{name}: restatement == reference bit for bit (paths A, B, FFN, order {ref_order}); "
                  f"exact-logit ids equal reference ids: {same_ids}; "
                  f"|exact-def out - reference out| max {O.max_abs(out_b, ref_b[0]):.3g} mean-rel {O.mean_rel(out_b, ref_b[0]):.3g}")

        rec = dict(H=H, E=E, K=K, I=I, T=T, layer_idx=li, dtype=str(dtype).split(".")[-1], seed=0,
                   input_sha256=digest(layer),
                   ref_ids=to_np(routing.topk_indices), ref_scores=to_np(routing.topk_scores),
                   ref_out_engine=to_np(ref_b[0]), ref_out_engine_residual=to_np(ref_b_res[0]),
                   ref_out_layer=to_np(ref_a[0]), ref_ffn0=to_np(ref_ffn), ref_order=np.array(ref_order),
                   def_ids=to_np(ids_x), def_scores=to_np(scores_x), def_logits=to_np(logits_x),
                   def_out_engine=to_np(out_b), def_out_layer=to_np(out_a))
        if store:
            rec["gate_w"] = to_np(layer.gate_w)
            rec["x"] = to_np(layer.x)
            for e in layer.experts:
                for k, v in layer.experts[e].items():
                    rec[f"expert{e}_{k}"] = to_np(v)
        np.savez_compressed(golden / f"{name}.npz", **rec)

    # placement semantics on the reference's unit-test config: substitution, skipped experts,
    # fp32 scores with an fp16 model, duplicate ids (demo/tests/unit/test_forward_moe.py:44-92)
    layer = make_layer(32, 4, 2, 16, torch.float16, 6, seed=1)
    r = reference_runner(layer)
    ids = torch.tensor([[0, 1], [1, 2], [3, 0], [2, 3], [1, 0], [3, 2]])
    scores = torch.tensor([[0.5, 0.5], [0.75, 0.25], [0.1, 0.9], [0.6, 0.4], [1.0, 0.0], [0.3, 0.7]], dtype=torch.float32)
    act = {ExpertID(0, i) for i in ids.flatten().unique().tolist()}
    rr = RoutingResult(layer_idx=0, topk_indices=ids, topk_scores=scores, activated_expert_ids=act)
    avail = {0: layer.experts[0], 2: layer.experts[2]}      # expert 1 substituted by 2, expert 3 skipped
    pl = ExpertPlacement(gpu_expert_params=avail, cpu_expert_params={}, substitution_map={1: 2}, routing_result=rr)
    with torch.no_grad():
        ref = r._execute_moe_with_placement(layer.x, pl)
        mine = O.moe_engine(layer.x, ids, scores, avail, substitution={1: 2})
        assert torch.equal(ref, mine)
        refh = r._execute_moe_with_placement(layer.x, ExpertPlacement(gpu_expert_params=avail, cpu_expert_params={}, substitution_map={1: 2},
                                             routing_result=RoutingResult(0, ids, scores.half(), act)))
        mineh = O.moe_engine(layer.x, ids, scores.half(), avail, substitution={1: 2})
        assert torch.equal(refh, mineh)
        assert torch.equal(r._execute_moe_with_placement(layer.x, ExpertPlacement({}, {}, {}, None)), torch.zeros_like(layer.x))
    rec = dict(seed=1, gate_w=to_np(layer.gate_w), x=to_np(layer.x), ids=ids.numpy(), scores=scores.numpy(),
               ref_out_f32scores=to_np(ref), ref_out_f16scores=to_np(refh), ref_order=np.array([e.expert_idx for e in act]))
    for e in layer.experts:
        for k, v in layer.experts[e].items():
            rec[f"expert{e}_{k}"] = to_np(v)
    np.savez_compressed(golden / "placement_fp16.npz", **rec)
    print("placement_fp16: substitution / skip / fp32-score semantics == reference bit for bit")

    # mixed GPU-resident / CPU-resident placement with top-4 routing: the reference adds every GPU task
    # before any CPU task (demo/src/model/qwen3_runner.py:352-383), so the bf16 accumulation order is
    # "GPU-served experts in set order, then CPU-served experts in set order"
    layer = make_layer(64, 12, 4, 32, torch.bfloat16, 10, seed=6)
    r = reference_runner(layer, 2)
    with torch.no_grad():
        routing = r.route_experts(2, layer.x)
        gpu_p = {e: layer.experts[e] for e in (0, 3, 4, 7, 8, 11)}
        cpu_p = {e: layer.experts[e] for e in (1, 2, 5, 7)}                  # 7 is in both: the GPU copy wins
        subm = {6: 1, 9: 4, 10: 10}                                          # 6 -> CPU-resident 1, 9 -> GPU-resident 4, 10 -> nothing usable
        pl = ExpertPlacement(gpu_expert_params=gpu_p, cpu_expert_params=cpu_p, substitution_map=subm, routing_result=routing)
        ref = r._execute_moe_with_placement(layer.x, pl)
        ref_order = [eid.expert_idx for eid in routing.activated_expert_ids]
        mine = O.moe_engine(layer.x, routing.topk_indices, routing.topk_scores, gpu_p, layer_idx=2, substitution=subm, cpu_experts=cpu_p)
        assert torch.equal(ref, mine), O.max_abs(ref, mine)
        plain = O.moe_engine(layer.x, routing.topk_indices, routing.topk_scores, {**cpu_p, **gpu_p}, layer_idx=2, substitution=subm)
        assert not torch.equal(ref, plain)      # the case does distinguish the two orders
    rec = dict(seed=6, layer_idx=2, gate_w=to_np(layer.gate_w), x=to_np(layer.x), ids=routing.topk_indices.numpy(),
               scores=to_np(routing.topk_scores), ref_out=to_np(ref), ref_order=np.array(ref_order),
               gpu_experts=np.array(sorted(gpu_p)), cpu_experts=np.array(sorted(cpu_p)),
               sub_from=np.array(sorted(subm)), sub_to=np.array([subm[k] for k in sorted(subm)]))
    for e in layer.experts:
        for k, v in layer.experts[e].items():
            rec[f"expert{e}_{k}"] = to_np(v)
    np.savez_compressed(golden / "mixed_placement_bf16.npz", **rec)
    print("mixed_placement_bf16: GPU tasks before CPU tasks == reference bit for bit (and differs from plain set order)")

    # LayerExpertActivations (demo/src/execution/model_runner_utils.py:13-41) on a routed batch
    from src.execution.model_runner_utils import build_layer_activations
    layer = make_layer(64, 16, 4, 32, torch.bfloat16, 40, seed=5)
    with torch.no_grad():
        ids, scores, _ = O.route(layer.x, layer.gate_w, 4)
    ref_acts = build_layer_activations(RoutingResult(3, ids, scores, set()), 16)
    mine = O.layer_activations(ids, scores, 16)
    assert len(ref_acts.activations) == len(mine) and ref_acts.layer_idx == 3 and ref_acts.routing_scores is scores
    for a, (k, e, tok, sc) in zip(ref_acts.activations, mine):
        assert (a.top_k_rank, a.expert_id.expert_idx, a.expert_id.layer_idx) == (k, e, 3)
        assert torch.equal(a.token_indices, tok) and torch.equal(a.scores, sc)
    np.savez_compressed(golden / "activations_bf16.npz", ids=ids.numpy(), scores=to_np(scores), num_experts=16,
                        rank=np.array([m[0] for m in mine]), expert=np.array([m[1] for m in mine]),
                        count=np.array([m[2].numel() for m in mine]),
                        tokens=torch.cat([m[2] for m in mine]).numpy(), act_scores=to_np(torch.cat([m[3] for m in mine])))
    print(f"activations_bf16: {len(mine)} activations == reference")

    # RMSNorm in front of the MoE block (demo/src/layers/layernorm.py:9-47), both forms, weight in the model dtype
    from src.layers.layernorm import RMSNorm
    g = torch.Generator().manual_seed(9)
    rec = {}
    for name, dt in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        x = torch.randn(12, 256, generator=g).to(dt)
        r = torch.randn(12, 256, generator=g).to(dt)
        w = (1.0 + 0.1 * torch.randn(256, generator=g)).to(dt)
        m = RMSNorm(256, eps=1e-6)
        with torch.no_grad():
            m.weight.copy_(w.float())
            m = m.to(dt)
            ref1 = m(x)
            ref2, ref_res = m(x, r)
            o1 = O.rmsnorm(x, w, 1e-6)
            o2, ores = O.rmsnorm(x, w, 1e-6, r)
        assert ref1.dtype == dt and torch.equal(ref1, o1) and torch.equal(ref2, o2) and torch.equal(ref_res, ores), name
        rec.update({f"{name}_x": to_np(x), f"{name}_r": to_np(r), f"{name}_w": to_np(w), f"{name}_out": to_np(ref1),
                    f"{name}_out_add": to_np(ref2), f"{name}_res": to_np(ref_res)})
    np.savez_compressed(golden / "rmsnorm.npz", **rec)
    print("rmsnorm: restatement == reference bit for bit (bf16, f16, f32; with and without residual)")

    # int4 g128: the format is this build's; store a small packed example produced by the oracle
    g = torch.Generator().manual_seed(7)
    w = (torch.randn(24, 384, generator=g) * 0.02).to(torch.bfloat16)
    w[3, 128:256] = 0  # an all-zero group
    q, s = O.quant_int4_g128(w)
    assert torch.equal(O.unpack_int4(q), O.unpack_int4(O.quant_int4_g128(O.dequant_int4_g128(q, s))[0]))
    np.savez_compressed(golden / "int4_g128.npz", w=to_np(w), q=q.numpy(), scales=to_np(s),
                        unpacked=O.unpack_int4(q).numpy(), dequant=to_np(O.dequant_int4_g128(q, s)))
    print("int4_g128: fixture written")


if __name__ == "__main__":
    main()
