"""GPU: the drop-in layer (ModelRunner boundary and nn.Module signatures), written after the
reference's own tests for this path (demo/tests/unit/test_routing.py, test_forward_moe.py,
test_engine_optimizations.py:608-749)."""
import pytest
import torch

from conftest import OUT_TOL
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture()
def small():
    from on_device_sd_b200 import B200MoERunner, MoEShape
    from on_device_sd_b200.synth import make_named
    cfg = MoEShape(32, 4, 2, 16, "float16", num_hidden_layers=2)      # the reference's small_config (conftest.py:108-128)
    runner = B200MoERunner(cfg, max_tokens=16)
    layers = [make_named("tiny_fp16", 4, seed=s, device="cuda") for s in (0, 1)]
    for i, L in enumerate(layers):
        runner.load_gate(i, L.gate_w)
    return runner, cfg, layers


def test_route_experts_output_format(small):
    from on_device_sd_b200 import ExpertID, RoutingResult
    runner, cfg, layers = small
    hidden = torch.randn(1, 4, cfg.hidden_size, device="cuda", dtype=cfg.get_dtype())
    r = runner.route_experts(layer_idx=0, hidden_states=hidden)
    assert isinstance(r, RoutingResult) and r.layer_idx == 0
    assert r.topk_indices.shape == (4, 2) and r.topk_indices.dtype == torch.int64
    assert r.topk_scores.shape == r.topk_indices.shape and r.topk_scores.dtype == torch.float16
    s = r.topk_scores.float().sum(-1)
    assert torch.allclose(s, torch.ones_like(s), atol=2e-3)
    assert r.activated_expert_ids == {ExpertID(0, i) for i in r.topk_indices.flatten().unique().tolist()}
    r2 = runner.route_experts(1, hidden.view(4, -1))      # 2-D input is accepted too (qwen3_runner.py:98-99)
    assert r2.layer_idx == 1 and all(e.layer_idx == 1 for e in r2.activated_expert_ids)


def test_forward_moe_matches_oracle_with_residual(small):
    from on_device_sd_b200 import AttentionOutput, ExpertPlacement
    runner, cfg, layers = small
    L = layers[0]
    hidden = L.x.view(1, 4, -1)
    r = runner.route_experts(0, hidden)
    placement = ExpertPlacement(gpu_expert_params=L.experts, cpu_expert_params={}, routing_result=r)
    out = runner.forward_moe(0, AttentionOutput(hidden, hidden, hidden), placement)
    assert out.shape == hidden.shape
    cpu = {e: {k: v.cpu() for k, v in p.items()} for e, p in L.experts.items()}
    want = O.moe_engine(L.x.cpu(), r.topk_indices.cpu(), r.topk_scores.cpu(), cpu,
                        order=[e.expert_idx for e in r.activated_expert_ids], residual=L.x.cpu())
    assert O.max_abs(out.cpu().view(4, -1), want) <= 1e-3       # the reference's path-vs-path tolerance (test_forward_moe.py:66)
    assert torch.equal(runner._execute_moe_with_placement(hidden, ExpertPlacement({}, {}, {}, None)), torch.zeros_like(hidden))


def test_cpu_vs_gpu_placement_close(small):
    """test_forward_moe.py:44-66 with duplicate-free ids: CPU-resident parameters give the same result."""
    from on_device_sd_b200 import AttentionOutput, ExpertID, ExpertPlacement, RoutingResult
    runner, cfg, layers = small
    L = layers[0]
    hidden = L.x.view(1, 4, -1)
    ids = torch.tensor([[0, 1], [1, 2], [3, 0], [2, 3]], device="cuda")
    scores = torch.full((4, 2), 0.5, device="cuda", dtype=torch.float32)
    r = RoutingResult(0, ids, scores, {ExpertID(0, i) for i in range(4)})
    attn = AttentionOutput(hidden, hidden, hidden)
    gpu_out = runner.forward_moe(0, attn, ExpertPlacement(gpu_expert_params=L.experts, cpu_expert_params={}, routing_result=r))
    cpu = {e: {k: v.cpu() for k, v in p.items()} for e, p in L.experts.items()}
    cpu_out = runner.forward_moe(0, attn, ExpertPlacement(gpu_expert_params={}, cpu_expert_params=cpu, routing_result=r))
    assert torch.allclose(gpu_out, cpu_out, atol=1e-3)
    assert gpu_out.abs().sum() > 0


def test_substitution_uses_substitute_params(small):
    from on_device_sd_b200 import ExpertID, ExpertPlacement, RoutingResult
    runner, cfg, layers = small
    L = layers[0]
    ids = torch.tensor([[1, 3]] * 4, device="cuda")
    scores = torch.tensor([[0.25, 0.75]] * 4, device="cuda", dtype=torch.float16)
    r = RoutingResult(0, ids, scores, {ExpertID(0, 1), ExpertID(0, 3)})
    pl = ExpertPlacement(gpu_expert_params={0: L.experts[0]}, cpu_expert_params={}, substitution_map={1: 0}, routing_result=r)
    out = runner._execute_moe_with_placement(L.x, pl)
    want = (O.expert_ffn(L.x.cpu(), **{k: v.cpu() for k, v in L.experts[0].items()}) * 0.25).half()   # expert 3 skipped
    assert O.max_abs(out.cpu(), want) <= 1e-3 and out.abs().sum() > 0


def test_mixed_gpu_cpu_placement_matches_reference_fixture():
    """A placement mixing GPU-resident, CPU-resident and substituted experts with top-4 routing: the
    reference's own output (fixture) within the same-order tolerance, i.e. GPU tasks accumulate first."""
    from on_device_sd_b200 import B200MoERunner, ExpertID, ExpertPlacement, MoEShape, RoutingResult
    from test_oracle_golden import load_mixed_placement
    m = load_mixed_placement()
    runner = B200MoERunner(MoEShape(64, 12, 4, 32, "bfloat16", num_hidden_layers=3), max_tokens=16)
    act = set()
    for e in m["ids"].flatten().unique().tolist():
        act.add(ExpertID(m["layer_idx"], int(e)))
    r = RoutingResult(m["layer_idx"], m["ids"].cuda(), m["scores"].cuda(), act)
    gpu = {e: {k: v.cuda() for k, v in p.items()} for e, p in m["gpu"].items()}
    out = runner._execute_moe_with_placement(m["x"].cuda(), ExpertPlacement(gpu, m["cpu"], m["sub"], r))
    assert runner.ctx.status() == 0
    assert O.mean_rel(out.cpu(), m["ref"]) <= 1e-3 and O.max_abs(out.cpu(), m["ref"]) <= 2e-2


def test_module_dropins_match_oracle():
    from on_device_sd_b200 import Qwen3MoEGate, Qwen3MoELayer, Qwen3MoELayerWithWeights
    from on_device_sd_b200.synth import make_layer
    H, E, K, I, T = 128, 8, 2, 64, 12
    L = make_layer(H, E, K, I, torch.bfloat16, T, seed=2)
    x3 = L.x.cuda().view(2, 6, H)
    gate = Qwen3MoEGate(H, E).to(torch.bfloat16).cuda()
    gate.load_weights(L.gate_w.cuda())
    idx, w = gate(x3, K)
    o_ids, o_sc, _ = O.route(L.x, L.gate_w, K)
    assert idx.shape == (2, 6, K) and torch.equal(idx.view(T, K).cpu(), o_ids)
    assert O.max_abs(w.view(T, K).cpu().float(), o_sc.float()) <= 2 ** -8
    dev = {e: {k: v.cuda() for k, v in p.items()} for e, p in L.experts.items()}
    layer = Qwen3MoELayer(H, E, K, I, 0).to(torch.bfloat16).cuda()
    layer.gate.load_weights(L.gate_w.cuda())
    out = layer(x3, dev)
    want = O.moe_layer(L.x, L.gate_w, L.experts, K)
    tol_a, tol_r = OUT_TOL[torch.bfloat16]
    assert out.shape == x3.shape and O.max_abs(out.view(T, H).cpu(), want) <= tol_a and O.mean_rel(out.view(T, H).cpu(), want) <= 1e-3
    out2 = Qwen3MoELayerWithWeights(H, E, K, I, 0)(x3, L.gate_w.cuda(), dev)
    assert torch.equal(out2, out)
    # experts missing from the dict are skipped silently (moe_layer.py:136-137)
    part = {e: dev[e] for e in (0, 3, 5)}
    want = O.moe_layer(L.x, L.gate_w, {e: L.experts[e] for e in (0, 3, 5)}, K)
    got = layer(x3, part)
    assert O.mean_rel(got.view(T, H).cpu(), want) <= 1e-3


def test_exact_logits_mode_reproduces_torch_router():
    """exact_logits=True: ids equal torch's own router on this GPU for every token."""
    from on_device_sd_b200 import B200MoERunner, MoEShape
    cfg = MoEShape(2048, 128, 8, 768, "bfloat16")
    runner = B200MoERunner(cfg, max_tokens=256, exact_logits=True)
    g = torch.Generator(device="cuda").manual_seed(0)
    gate_w = (torch.randn(128, 2048, device="cuda", generator=g) * 0.02).bfloat16()
    x = torch.randn(256, 2048, device="cuda", generator=g).bfloat16()
    runner.load_gate(0, gate_w)
    r = runner.route_experts(0, x)
    vals, ids = torch.topk(torch.nn.functional.linear(x, gate_w), 8, dim=-1)
    assert torch.equal(r.topk_indices, ids)
    assert O.max_abs(r.topk_scores.float().cpu(), torch.softmax(vals, -1).float().cpu()) <= 2 ** -8


@pytest.mark.parametrize("mode", ["dense", "int4"])
def test_layer_slab_ingest_gives_identical_outputs(mode):
    """All experts of a layer copied into one allocation (host fp32 sources): same bits as separate tensors."""
    from on_device_sd_b200 import MoEContext, W_DENSE, W_INT4_G128, ingest_layer
    from on_device_sd_b200.quant import quantize_expert
    from on_device_sd_b200.synth import make_layer
    H, E, K, I, T = 256, 8, 2, 128, 24
    L = make_layer(H, E, K, I, torch.bfloat16, T, seed=41)
    wm = W_INT4_G128 if mode == "int4" else W_DENSE
    a = MoEContext(H, E, K, I, torch.bfloat16, max_tokens=32, weight_mode=wm)
    b = MoEContext(H, E, K, I, torch.bfloat16, max_tokens=32, weight_mode=wm)
    a.set_gate(0, L.gate_w.cuda()); b.set_gate(0, L.gate_w.cuda())
    keep = []
    for e, p in L.experts.items():
        dev = {k: v.cuda() for k, v in p.items()}
        keep.append(quantize_expert(dev) if mode == "int4" else dev)
        a.set_expert(0, e, keep[-1])
    slab = ingest_layer(b, 0, {e: {k: v.float() for k, v in p.items()} for e, p in L.experts.items()})   # CPU fp32 sources
    assert slab.buffer.data_ptr() % 256 == 0 and len(slab.views) == E
    x = L.x.cuda()
    assert torch.equal(a.forward_fused(0, x), b.forward_fused(0, x))
    assert a.status() == 0 and b.status() == 0


def test_moe_block_graph_replay_equals_eager_launches():
    """B200MoERunner(graph_blocks=True): the captured block replays with new contents of the same input buffer."""
    from on_device_sd_b200 import B200MoERunner, MoEShape
    from on_device_sd_b200.synth import make_layer
    H, E, K, I, T = 256, 8, 2, 128, 12
    L = make_layer(H, E, K, I, torch.bfloat16, T, seed=43)
    shape = MoEShape(H, E, K, I, "bfloat16", 1)
    eager = B200MoERunner(shape, max_tokens=16)
    graphed = B200MoERunner(shape, max_tokens=16, graph_blocks=True)
    for r in (eager, graphed):
        r.load_gate(0, L.gate_w.cuda())
        r.register_experts(0, {e: {k: v.cuda() for k, v in p.items()} for e, p in L.experts.items()})
    x = L.x.cuda().clone()
    res = torch.randn_like(x)
    for trial in range(3):
        want = eager.moe_block(0, x, residual=res)
        got = graphed.moe_block(0, x, residual=res)
        assert torch.equal(got, want), trial
        x.copy_(torch.randn(T, H, generator=torch.Generator().manual_seed(trial)).bfloat16())   # same buffer, new tokens
    assert len(graphed._graphs) == 1 and eager.ctx.status() == 0 and graphed.ctx.status() == 0
    # re-registering an expert at a new address drops the captured graphs: the replay must see the new weights
    moved = {k: (v.cuda() * 2).contiguous() for k, v in L.experts[0].items()}
    for r in (eager, graphed):
        r.register_experts(0, {0: moved})
    assert torch.equal(graphed.moe_block(0, x, residual=res), eager.moe_block(0, x, residual=res))
    assert len(graphed._graphs) == 1
    # the cache is bounded: least recently used graphs go first
    graphed.max_graphs = 2
    bufs = [x.clone() for _ in range(4)]
    for b in bufs:
        graphed.moe_block(0, b)
    assert len(graphed._graphs) == 2


def test_layer_activations_from_the_grouping_kernel_equal_the_reference_loop():
    """build_layer_activations fed by K2's tables (one device->host copy) against the oracle's restatement of the
    reference's K x E torch.where loop, on CUDA tensors: random routing, duplicates, ids outside [0, E), the fixture."""
    import numpy as np
    from conftest import GOLDEN, from_np
    from on_device_sd_b200 import B200MoERunner, MoEShape, RoutingResult
    from test_host_logic import _check_activations
    g = torch.Generator().manual_seed(13)
    for T, K, E in [(1, 1, 4), (7, 2, 8), (64, 8, 128), (33, 4, 5), (256, 8, 128)]:
        runner = B200MoERunner(MoEShape(64, E, K, 32, "bfloat16"), max_tokens=256)
        ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).cuda()
        scores = torch.rand(T, K, generator=g).to(torch.bfloat16).cuda()
        acts = runner.build_layer_activations(RoutingResult(1, ids, scores, set()))
        _check_activations(acts, O.layer_activations(ids.cpu(), scores.cpu(), E), 1, scores)
        assert all(a.token_indices.is_cuda and a.scores.is_cuda for a in acts.activations)
        assert runner.ctx.status() == 0
    runner = B200MoERunner(MoEShape(64, 4, 2, 32, "bfloat16"), max_tokens=8)
    ids = torch.tensor([[0, 0], [5, 1], [-1, 2], [2, 2]]).cuda()
    scores = torch.rand(4, 2, generator=g).cuda()
    _check_activations(runner.build_layer_activations(RoutingResult(0, ids, scores, set())), O.layer_activations(ids.cpu(), scores.cpu(), 4), 0, scores)
    assert runner.ctx.status() == 0                       # unknown ids are dropped quietly here, as the reference's comparison drops them
    z = np.load(GOLDEN / "activations_bf16.npz")
    runner = B200MoERunner(MoEShape(64, int(z["num_experts"]), z["ids"].shape[1], 32, "bfloat16"), max_tokens=64)
    ids = torch.from_numpy(z["ids"].astype(np.int64)).cuda()
    scores = from_np(z["scores"], torch.bfloat16).cuda()
    acts = runner.build_layer_activations(RoutingResult(3, ids, scores, set()))
    cuts = np.r_[0, np.cumsum(z["count"])]
    toks, asc = torch.from_numpy(z["tokens"].astype(np.int64)), from_np(z["act_scores"], torch.bfloat16)
    want = [(int(k), int(e), toks[a:b], asc[a:b]) for k, e, a, b in zip(z["rank"], z["expert"], cuts[:-1], cuts[1:])]
    _check_activations(acts, want, 3, scores)


def test_runner_subclass_of_the_integration_note_runs_the_engine_sequence():
    """The subclass a maintainer adds to the reference (the class body is the one shown in the integration
    note), on a stand-in for Qwen3ModelRunner that has the same constructor arguments and attributes: per layer
    route_experts -> placement from the loader's per-expert dicts -> forward_moe, as the engine loop does
    (demo/src/execution/cb_executor.py:427-448)."""
    import types
    from on_device_sd_b200 import AttentionOutput, B200MoERunner, ExpertID, ExpertPlacement, MoEShape
    from on_device_sd_b200.synth import make_layer

    class Qwen3ModelRunnerStandIn:                      # constructor and attributes of demo/src/model/qwen3_runner.py:28-69
        def __init__(self, config, parameter_loader):
            self.config, self.parameter_loader, self.device = config, parameter_loader, torch.device("cuda")

    class B200Qwen3ModelRunner(Qwen3ModelRunnerStandIn):
        def __init__(self, config, parameter_loader, max_tokens=512):
            super().__init__(config, parameter_loader)
            self._moe = B200MoERunner(config, device=self.device, max_tokens=max_tokens, expert_id_cls=ExpertID)
            for i in range(config.num_hidden_layers):
                self._moe.load_gate(i, parameter_loader.static_params_gpu[f"layer_{i}.router"])

        def route_experts(self, layer_idx, hidden_states):
            return self._moe.route_experts(layer_idx, hidden_states)

        def forward_moe(self, layer_idx, attn_output, expert_placement):
            return self._moe.forward_moe(layer_idx, attn_output, expert_placement)

        def _execute_moe_with_placement(self, hidden_states, expert_placement):
            return self._moe._execute_moe_with_placement(hidden_states, expert_placement)

    H, E, K, I, T, Ln = 128, 8, 2, 64, 10, 2
    layers = [make_layer(H, E, K, I, torch.bfloat16, T, seed=70 + l, device="cuda") for l in range(Ln)]
    loader = types.SimpleNamespace(static_params_gpu={f"layer_{l}.router": layers[l].gate_w for l in range(Ln)},
                                   expert_params_gpu={ExpertID(l, e): layers[l].experts[e] for l in range(Ln) for e in range(E)})
    runner = B200Qwen3ModelRunner(MoEShape(H, E, K, I, "bfloat16", num_hidden_layers=Ln), loader, max_tokens=16)
    hidden = layers[0].x.view(1, T, H)
    for step in range(2):                               # the second pass reuses the registered experts (same dict objects)
        h = hidden
        for l in range(Ln):
            routing = runner.route_experts(l, h)
            gpu = {eid.expert_idx: loader.expert_params_gpu[eid] for eid in routing.activated_expert_ids}
            placement = ExpertPlacement(gpu_expert_params=gpu, cpu_expert_params={}, routing_result=routing)
            out = runner.forward_moe(l, AttentionOutput(h, h, h), placement)
            cpu = {e: {k: v.cpu() for k, v in p.items()} for e, p in layers[l].experts.items()}
            ids, scores, _ = O.route(h.view(T, H).cpu(), layers[l].gate_w.cpu(), K)
            assert torch.equal(routing.topk_indices.cpu(), ids)
            want = O.moe_engine(h.view(T, H).cpu(), ids, scores, cpu, layer_idx=l, residual=h.view(T, H).cpu())
            assert O.mean_rel(out.view(T, H).cpu(), want) <= 1e-3 and O.max_abs(out.view(T, H).cpu(), want) <= 2e-2
            h = out
    assert runner._moe.ctx.status() == 0
