"""GPU: parity at the full benchmark sizes, with the measured numbers kept as data.

Every case evaluates the oracle's own functions on CUDA tensors (torch eager = the reference's
arithmetic on this device: F.linear through the vendor GEMM, torch.topk, index_put) next to the
kernels.  When the environment variable B200MOE_PARITY_RECORD names a file, each case appends one JSON
line with what it measured (mismatch counts of the routing, max-abs / mean-rel of the outputs, and the
same two figures between the reference's own two MoE paths on this device - the noise floor)."""
import json
import os

import pytest
import torch
import torch.nn.functional as F

from oracle import moe_oracle as O
from test_gpu_moe import _close

pytestmark = pytest.mark.gpu

MIXTRAL_T = (1, 4, 8, 16, 64)
QWEN3_T = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def _record(**kw):
    path = os.environ.get("B200MOE_PARITY_RECORD")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(kw) + "\n")


def _gate_and_tokens(name, T, seed=0):
    from on_device_sd_b200.synth import CONFIGS
    H, E, K, I, dtype = CONFIGS[name]
    g = torch.Generator(device="cuda").manual_seed(seed)
    gate_w = (torch.randn(E, H, device="cuda", generator=g) * 0.02).to(dtype)
    x = torch.randn(T, H, device="cuda", generator=g).to(dtype)
    return H, E, K, I, dtype, gate_w, x


@pytest.mark.parametrize("name,Ts", [("mixtral", MIXTRAL_T), ("qwen3", QWEN3_T)])
def test_routing_modes_against_torch_on_this_device(name, Ts):
    """Fused router: bit-exact to the correctly rounded definition; its distance to the reference's own
    router on this GPU (F.linear -> topk) is COUNTED.  Exact-logits mode: ordered ids equal torch's, always."""
    from on_device_sd_b200 import MoEContext
    for T in Ts:
        H, E, K, I, dtype, gate_w, x = _gate_and_tokens(name, T)
        ctx = MoEContext(H, E, K, 128, dtype, max_tokens=T)
        ctx.set_gate(0, gate_w)
        ids, scores = ctx.route(0, x)
        logits = ctx.last_logits(T)
        exact = (x.double() @ gate_w.double().t()).float().to(dtype)
        assert torch.equal(logits, exact.float())
        o_ids, _ = O.topk_softmax(exact.cpu(), K)
        assert torch.equal(ids.cpu(), o_ids)
        t_logits = F.linear(x, gate_w)                                   # what the reference computes here
        t_vals, t_ids = torch.topk(t_logits, K, dim=-1)
        ids2, scores2 = ctx.route(0, None, logits=t_logits)              # exact-logits mode
        assert torch.equal(ids2, t_ids)
        assert float((scores2.float() - F.softmax(t_vals, -1).float()).abs().max()) <= 2.0 ** -8
        _record(kind="routing", shape=name, T=T, fused_tokens_differing_from_torch=int((t_ids != ids).any(-1).sum()),
                fused_token_sets_differing=int((t_ids.sort(-1).values != ids.sort(-1).values).any(-1).sum()),
                vendor_gemm_logits_differing_from_correctly_rounded=int((t_logits.float() != logits).sum()), logits=T * E,
                exact_logits_mode_tokens_differing_from_torch=int((t_ids != ids2).any(-1).sum()))


@pytest.mark.parametrize("T", [160, 288])
def test_routing_modes_on_the_popularity_biased_gates(T):
    from on_device_sd_b200 import MoEContext
    from on_device_sd_b200.synth import zipf_bias
    H, E, K, I, dtype, _, x = _gate_and_tokens("qwen3", T, seed=7)
    ctx = MoEContext(H, E, K, 128, dtype, num_layers=48, max_tokens=T)
    g = torch.Generator(device="cuda").manual_seed(11)
    fused_diff = set_diff = exact_diff = 0
    for layer in range(48):
        gate_w = (torch.randn(E, H, device="cuda", generator=g) * 0.02).to(dtype)
        bias = zipf_bias(E, 1.1, seed=layer).to(dtype).cuda()
        ctx.set_gate(layer, gate_w, bias)
        ids, _ = ctx.route(layer, x)
        t_logits = F.linear(x, gate_w) + bias
        t_ids = torch.topk(t_logits, K, dim=-1).indices
        ids2, _ = ctx.route(layer, None, logits=t_logits)
        assert torch.equal(ids2, t_ids)
        exact = ((x.double() @ gate_w.double().t()).float().to(dtype) + bias)
        assert torch.equal(ids.cpu(), O.topk_softmax(exact.cpu(), K)[0])
        fused_diff += int((t_ids != ids).any(-1).sum())
        set_diff += int((t_ids.sort(-1).values != ids.sort(-1).values).any(-1).sum())
        exact_diff += int((t_ids != ids2).any(-1).sum())
    _record(kind="routing", shape="qwen3 48 layers, zipf(1.1) gate bias", T=T, tokens=48 * T, fused_tokens_differing_from_torch=fused_diff,
            fused_token_sets_differing=set_diff, exact_logits_mode_tokens_differing_from_torch=exact_diff)


def _noise_floor(L, ids, scores):
    """The reference's path A order (ascending experts) against its path B order (set iteration), both in torch on the device."""
    a = O.moe_engine(L.x, ids, scores, L.experts, order=sorted(set(ids.flatten().tolist())))
    b = O.moe_engine(L.x, ids, scores, L.experts, order=O.activated_order(0, ids.cpu()))
    return a, b, O.max_abs(a, b), O.mean_rel(a, b)


@pytest.mark.parametrize("name,T", [("qwen3", t) for t in (1, 8, 64, 256)] + [("mixtral", t) for t in MIXTRAL_T])
def test_block_in_exact_logits_mode_equals_reference_router_and_engine(name, T):
    """The drop-in sequence route_experts -> forward_moe with exact_logits=True against the reference's
    sequence on this device: F.linear logits, torch.topk, softmax (moe_layer.py:44-54), then the engine
    path (qwen3_runner.py:269-385).  Ordered ids must be EQUAL; outputs inside the tolerance."""
    from on_device_sd_b200 import AttentionOutput, B200MoERunner, ExpertPlacement, MoEShape
    from on_device_sd_b200.synth import make_named
    L = make_named(name, T, device="cuda", gen_device="cuda")
    runner = B200MoERunner(MoEShape(L.H, L.E, L.K, L.I, "bfloat16"), max_tokens=T, exact_logits=True)
    runner.load_gate(0, L.gate_w)
    r = runner.route_experts(0, L.x)
    o_ids, o_scores, _ = O.route(L.x, L.gate_w, L.K, tie="torch", logits="linear")
    assert torch.equal(r.topk_indices, o_ids)
    assert float((r.topk_scores.float() - o_scores.float()).abs().max()) <= 2.0 ** -8
    res = torch.randn_like(L.x)
    out = runner.forward_moe(0, AttentionOutput(L.x, L.x, res), ExpertPlacement(L.experts, {}, {}, r))
    assert runner.ctx.status() == 0
    order = [e.expert_idx for e in r.activated_expert_ids]
    assert order == O.activated_order(0, o_ids.cpu())
    want = O.moe_engine(L.x, o_ids, r.topk_scores, L.experts, order=order, residual=res)
    ma, mr = _close(out, want, torch.bfloat16, tight=True)
    if name == "qwen3":
        assert ma <= 2e-2                                        # plain max-abs: |y| stays small enough here that a bf16 ulp is below 2e-2
    _record(kind="block_exact_logits", shape=name, T=T, ids_equal_torch=True, max_abs=ma, mean_rel=mr, max_abs_y=float(want.abs().max()))


@pytest.mark.parametrize("name,T", [("qwen3", t) for t in (1, 8, 64, 256)] + [("mixtral", t) for t in MIXTRAL_T])
def test_fused_block_numbers_and_noise_floor(name, T):
    """Fused block (benchmarked mode) against the oracle on the device in both accumulation orders, with
    the reference's own path-A-versus-path-B difference measured beside it."""
    from on_device_sd_b200 import MoEContext
    from on_device_sd_b200.synth import make_named
    L = make_named(name, T, device="cuda", gen_device="cuda")
    ctx = MoEContext(L.H, L.E, L.K, L.I, L.dtype, max_tokens=T)
    ctx.set_gate(0, L.gate_w)
    for e, p in L.experts.items():
        ctx.set_expert(0, e, p)
    out, ids, scores = ctx.forward_fused(0, L.x, return_routing=True)
    assert ctx.status() == 0
    ref_a, ref_b, floor_ma, floor_mr = _noise_floor(L, ids, scores)
    ma_a, mr_a = _close(out, ref_a, L.dtype, tight=True)
    ma_b, mr_b = _close(out, ref_b, L.dtype)
    ymax = float(ref_a.abs().max())
    if name == "qwen3":
        assert ma_a <= 2e-2 and ma_b <= 2e-2                      # the plain bound of the target
    else:
        assert ma_a <= 2e-2 + 2 * 2.0 ** -8 * ymax                # |y| reaches ~16 here: one bf16 ulp is 0.0625
    _record(kind="block_fused", shape=name, T=T, max_abs_vs_same_order=ma_a, mean_rel_vs_same_order=mr_a, max_abs_vs_engine_order=ma_b,
            mean_rel_vs_engine_order=mr_b, reference_path_a_vs_b_max_abs=floor_ma, reference_path_a_vs_b_mean_rel=floor_mr, max_abs_y=ymax,
            bf16_ulp_at_max_y=2.0 ** (torch.tensor(ymax).log2().floor().item() - 7))


def _int4_qwen3_layer(ctx, layer, g, keep_dequant=True):
    """Registers one Qwen3-shaped layer of 128 int4 experts; returns (gate_w, dequantised experts for the oracle)."""
    from on_device_sd_b200.quant import quantize_expert, unpack_int4
    H, E, I = 2048, 128, 768
    gate_w = (torch.randn(E, H, device="cuda", generator=g) * 0.02).bfloat16()
    deq, packed = {}, []
    for e in range(E):
        p = {"gate_proj": (torch.randn(I, H, device="cuda", generator=g) * 0.02).bfloat16(),
             "up_proj": (torch.randn(I, H, device="cuda", generator=g) * 0.02).bfloat16(),
             "down_proj": (torch.randn(H, I, device="cuda", generator=g) * 0.02).bfloat16()}
        qp = quantize_expert(p)
        ctx.set_expert(layer, e, qp)
        packed.append(qp)
        if keep_dequant:
            deq[e] = {k: unpack_int4(qp[k], qp[k + "_scales"])[1] for k in ("gate_proj", "up_proj", "down_proj")}
    return gate_w, deq, packed


@pytest.mark.parametrize("T", [1, 64, 256])
def test_int4_qwen3_all_128_experts_against_device_oracle(T):
    """Qwen3-shaped layer with all 128 experts in int4 g128: oracle = the reference forward on dequant(quant(W)), on the device."""
    from on_device_sd_b200 import MoEContext, W_INT4_G128
    from on_device_sd_b200.quant import pack_int4
    ctx = MoEContext(2048, 128, 8, 768, torch.bfloat16, max_tokens=256, weight_mode=W_INT4_G128)
    g = torch.Generator(device="cuda").manual_seed(5)
    gate_w, deq, packed = _int4_qwen3_layer(ctx, 0, g)
    ctx.set_gate(0, gate_w)
    # the device packer agrees with the oracle's format on a full-size matrix, bit for bit
    w0 = deq[3]["down_proj"]
    q0, s0 = pack_int4(w0.contiguous())
    oq, os_ = O.quant_int4_g128(w0)
    assert torch.equal(q0, oq) and torch.equal(s0, os_)
    x = torch.randn(T, 2048, device="cuda", generator=g).bfloat16()
    out, ids, scores = ctx.forward_fused(0, x, return_routing=True)
    assert ctx.status() == 0
    want = O.moe_engine(x, ids, scores, deq, order=sorted(set(ids.flatten().tolist())))
    ma, mr = _close(out, want, torch.bfloat16, tight=True)
    assert ma <= 2e-2
    _record(kind="block_fused_int4", shape="qwen3 int4 g128, 128 experts", T=T, max_abs=ma, mean_rel=mr, experts_hit=int(ids.unique().numel()))


@pytest.mark.parametrize("T", [160, 288])
def test_int4_48_layer_stack_with_popularity_bias_layer_by_layer(T):
    """The stacked configuration at its own size on one GPU: 48 Qwen3-shaped int4 layers, Zipf(1.1) gate bias,
    T = 32 sequences x (k+1) verify tokens.  Every layer's kernel output is checked against the oracle fed with
    the SAME bf16 input (errors do not compound), and the chained outputs equal MoEStack.forward bit for bit."""
    from on_device_sd_b200 import MoEContext, W_INT4_G128
    from on_device_sd_b200.stack import MoEStack
    from on_device_sd_b200.synth import zipf_bias
    Lz, H, E, K = 48, 2048, 128, 8
    ctx = MoEContext(H, E, K, 768, torch.bfloat16, num_layers=Lz, max_tokens=T, weight_mode=W_INT4_G128)
    g = torch.Generator(device="cuda").manual_seed(100 + T)
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    cur, keep = x, []
    worst_ma = worst_mr = 0.0
    counts = torch.zeros(E, device="cuda")
    for layer in range(Lz):
        gate_w, deq, packed = _int4_qwen3_layer(ctx, layer, g)
        keep.append(packed)
        bias = zipf_bias(E, 1.1, seed=layer).bfloat16().cuda()
        ctx.set_gate(layer, gate_w, bias)
        got, ids, scores = ctx.forward_fused(layer, cur, residual=x, return_routing=True)
        exact = (cur.double() @ gate_w.double().t()).float().bfloat16() + bias
        assert torch.equal(ids.cpu(), O.topk_softmax(exact.cpu(), K)[0]), layer
        order = sorted(set(ids.flatten().tolist()))
        want = O.moe_engine(cur, ids, scores, deq, order=order, residual=x)
        _close(got, want, torch.bfloat16, tight=True)
        # the residual (|x| ~ 1) hides last-bit differences of the block itself: compare the bare block output too
        ma, mr = _close(ctx.forward(layer, cur, ids, scores), O.moe_engine(cur, ids, scores, deq, order=order), torch.bfloat16, tight=True)
        worst_ma, worst_mr = max(worst_ma, ma), max(worst_mr, mr)
        counts += torch.bincount(ids.flatten(), minlength=E)
        cur = got
        del deq
    assert ctx.status() == 0
    assert torch.equal(MoEStack(ctx, Lz).forward(x), cur)
    assert worst_ma <= 2e-2
    _record(kind="stack_int4", shape="48 x qwen3 int4 g128, zipf(1.1) gate bias", T=T, worst_layer_max_abs=worst_ma, worst_layer_mean_rel=worst_mr,
            max_over_mean_expert_load=float(counts.max() / counts.mean()))
