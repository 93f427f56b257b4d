"""GPU: expert execution (K2 permute, K3 FFN, K4 combine) and the fused block through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN, OUT_TOL, Golden
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
_QWEN_CACHE = {}


def _ctx(H, E, K, I, dtype, **kw):
    from on_device_sd_b200 import MoEContext
    return MoEContext(H, E, K, I, dtype, **kw)


def _register(ctx, experts, layer=0):
    dev = {}
    for e, p in experts.items():
        dev[e] = {k: v.cuda().contiguous() for k, v in p.items()}
        ctx.set_expert(layer, e, dev[e])
    return dev


def _close(got, want, dtype, tight=False, mean_rel_tol=None):
    """max-abs <= 2e-2 and mean-rel <= 5e-3 for 16-bit outputs (1e-5 for fp32).  The absolute bound
    is widened by two units in the last place of the expected value (2 * 2^-7 |y| for bf16,
    2 * 2^-10 |y| for fp16): with N(0, 0.02) weights the Mixtral-shaped layer produces |y| up to ~16,
    where ONE bf16 ulp is 0.0625 > 2e-2; a last-bit difference in one expert's output (fp32 summation
    order) can move the two-term bf16 accumulation by two ulps.  mean-rel is the sharp criterion."""
    got, want = got.cpu().double(), want.cpu().double()
    ma, mr = O.max_abs(got, want), O.mean_rel(got, want)
    tol_a, tol_r = OUT_TOL[dtype]
    if tight and dtype != torch.float32:
        tol_r = 1e-3     # same rounding points and same accumulation order: far inside the budget
    if mean_rel_tol is not None:
        tol_r = mean_rel_tol
    ulp = {torch.float32: 0.0, torch.float16: 2.0 ** -9, torch.bfloat16: 2.0 ** -6}[dtype]
    if not got.numel():
        return ma, mr
    # A token's output is a model-dtype sum of expert outputs that can cancel: the unit in the last
    # place that matters is that of the largest term, not of the (possibly tiny) result.  So every
    # element must lie within two ulps of the tensor's largest magnitude, and all but one in ten
    # thousand within two ulps of their own magnitude.
    diff = (got - want).abs()
    excess = float((diff - (tol_a + ulp * want.abs().max())).max())
    outliers = float((diff > tol_a + ulp * want.abs()).double().mean())
    assert excess <= 0 and outliers <= 1e-4 and mr <= tol_r, (ma, mr, excess, outliers)
    return ma, mr


def _rank(order, E):
    r = [len(order)] * E
    for i, e in enumerate(order):
        r[e] = i
    return r


def test_forward_matches_oracle_on_golden(golden):
    """Given the routing, experts + combine reproduce path B (engine order) and path A (ascending)."""
    g = golden
    ctx = _ctx(g.H, g.E, g.K, g.I, g.dtype, max_tokens=max(g.T, 8), num_layers=g.layer_idx + 1)
    _register(ctx, g.experts, g.layer_idx)
    ids, scores = g.t("def_ids"), g.t("def_scores")
    order = O.activated_order(g.layer_idx, ids)
    out = ctx.forward(g.layer_idx, g.x.cuda(), ids.cuda(), scores.cuda(), order=_rank(order, g.E))
    assert ctx.status() == 0
    _close(out, g.t("def_out_engine"), g.dtype, tight=True)
    _close(out, g.t("ref_out_engine"), g.dtype)                # the reference's own run of path B
    res = ctx.forward(g.layer_idx, g.x.cuda(), ids.cuda(), scores.cuda(), order=_rank(order, g.E), residual=g.x.cuda())
    _close(res, O.moe_engine(g.x, ids, scores, g.experts, layer_idx=g.layer_idx, residual=g.x), g.dtype, tight=True)
    asc = ctx.forward(g.layer_idx, g.x.cuda(), ids.cuda(), scores.cuda())
    _close(asc, g.t("def_out_layer"), g.dtype, tight=True)
    _close(asc, g.t("ref_out_layer"), g.dtype)


def test_fused_block_matches_oracle_on_golden(golden):
    g = golden
    ctx = _ctx(g.H, g.E, g.K, g.I, g.dtype, max_tokens=max(g.T, 8))
    ctx.set_gate(0, g.gate_w.cuda())
    _register(ctx, g.experts)
    out, ids, scores = ctx.forward_fused(0, g.x.cuda(), return_routing=True)
    assert ctx.status() == 0
    assert torch.equal(ids.cpu(), g.t("def_ids"))
    _close(out, g.t("def_out_layer"), g.dtype, tight=True)
    _close(out, g.t("ref_out_engine"), g.dtype)


def test_expert_ffn_matches_oracle(golden):
    g = golden
    from on_device_sd_b200 import expert_forward_with_weights
    p = {k: v.cuda() for k, v in g.experts[0].items()}
    out = expert_forward_with_weights(g.x.cuda(), p["gate_proj"], p["up_proj"], p["down_proj"])
    _close(out, g.t("ref_ffn0"), g.dtype, tight=True)
    out3 = expert_forward_with_weights(g.x.cuda().view(1, g.T, g.H), p["gate_proj"], p["up_proj"], p["down_proj"])
    assert out3.shape == (1, g.T, g.H) and torch.equal(out3.view(g.T, g.H), out)


def test_placement_fixture_substitution_skip_fp32_scores():
    z = np.load(GOLDEN / "placement_fp16.npz")
    x = torch.from_numpy(z["x"]).cuda()
    experts = {e: {k: torch.from_numpy(z[f"expert{e}_{k}"]) for k in ("gate_proj", "up_proj", "down_proj")} for e in range(4)}
    ctx = _ctx(32, 4, 2, 16, torch.float16, max_tokens=8)
    _register(ctx, {0: experts[0], 2: experts[2]})
    ids, scores = torch.from_numpy(z["ids"]).cuda(), torch.from_numpy(z["scores"]).cuda()
    slot = [0, 2, 2, -1]                       # 1 -> substitute 2, 3 skipped
    rank = _rank(z["ref_order"].tolist(), 4)
    out = ctx.forward(0, x, ids, scores, expert_slot=slot, order=rank)
    _close(out, torch.from_numpy(z["ref_out_f32scores"]), torch.float16, tight=True)
    out = ctx.forward(0, x, ids, scores.half(), expert_slot=slot, order=rank)
    _close(out, torch.from_numpy(z["ref_out_f16scores"]), torch.float16, tight=True)
    # an unregistered expert is skipped even with an identity slot table
    out2 = ctx.forward(0, x, ids, scores, order=rank)
    want = O.moe_engine(x.cpu(), ids.cpu(), scores.cpu(), {0: experts[0], 2: experts[2]}, order=z["ref_order"].tolist())
    _close(out2, want, torch.float16, tight=True)
    assert ctx.status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_edge_cases(dtype):
    H, E, K, I = 64, 8, 3, 48
    from on_device_sd_b200.synth import make_layer
    L = make_layer(H, E, K, I, dtype, 37, seed=5)
    ctx = _ctx(H, E, K, I, dtype, max_tokens=64)
    ctx.set_gate(0, L.gate_w.cuda())
    _register(ctx, L.experts)
    xc = L.x.cuda()
    # empty batch
    assert ctx.forward_fused(0, xc[:0]).shape == (0, H)
    # one token
    o_ids, o_sc, _ = O.route(L.x[:1], L.gate_w, K)
    _close(ctx.forward_fused(0, xc[:1].contiguous()), O.moe_engine(L.x[:1], o_ids, o_sc, L.experts, order=sorted(o_ids.flatten().tolist())), dtype, tight=True)
    # every token to the same experts (maximum ragged-ness: one group holds all pairs, others are empty)
    ids = torch.tensor([[5, 2, 7]] * 37)
    sc = torch.softmax(torch.randn(37, K, generator=torch.Generator().manual_seed(1)), -1).to(dtype)
    out = ctx.forward(0, xc, ids.cuda(), sc.cuda())
    _close(out, O.moe_engine(L.x, ids, sc, L.experts, order=[2, 5, 7]), dtype, tight=True)
    # duplicate ids in one token: contributions are summed (Qwen3MoELayer.forward, moe_layer.py:160-165)
    ids = torch.tensor([[1, 1, 4]] * 37)
    out = ctx.forward(0, xc, ids.cuda(), sc.cuda())
    y1 = O.expert_ffn(L.x, **L.experts[1]).float()
    y4 = O.expert_ffn(L.x, **L.experts[4]).float()
    want = (y1 * sc[:, 0:1].float()).to(dtype).float()
    want = (want + (y1 * sc[:, 1:2].float()).to(dtype).float()).to(dtype).float()
    want = (want + (y4 * sc[:, 2:3].float()).to(dtype).float()).to(dtype)
    _close(out, want, dtype, tight=True)
    assert ctx.status() == 0
    # an id outside [0,E) is skipped and reported through the status word, never dereferenced
    from on_device_sd_b200 import B200MoEError
    ids = torch.tensor([[1, 99, 4]] * 37)
    out = ctx.forward(0, xc, ids.cuda(), sc.cuda())
    with pytest.raises(B200MoEError, match="status word"):
        ctx.status()
    ids_ok = torch.tensor([[1, 4]] * 37)
    want = O.moe_engine(L.x, ids_ok, sc[:, [0, 2]].contiguous(), L.experts, order=[1, 4])
    _close(out, want, dtype, tight=True)
    assert ctx.status() == 0                   # the word is cleared by the read


@pytest.mark.parametrize("T", [1, 4, 16, 64])
def test_qwen3_shape_reduced_experts(T):
    """Qwen3-30B-A3B-shaped layer (H 2048, I 768, top-8) with 32 of its 128 experts so that the CPU
    oracle finishes in seconds; full-size runs are covered by the property tests below."""
    import copy
    from on_device_sd_b200.synth import make_layer
    if "L" not in _QWEN_CACHE:
        _QWEN_CACHE["L"] = make_layer(2048, 32, 8, 768, torch.bfloat16, 64, seed=0)
    L = copy.copy(_QWEN_CACHE["L"])
    L.x = L.x[:T].contiguous()
    ctx = _ctx(2048, 32, 8, 768, torch.bfloat16, max_tokens=64)
    ctx.set_gate(0, L.gate_w.cuda())
    _register(ctx, L.experts)
    out, ids, scores = ctx.forward_fused(0, L.x.cuda(), return_routing=True)
    o_ids, o_sc, _ = O.route(L.x, L.gate_w, 8)
    assert torch.equal(ids.cpu(), o_ids)
    want_a = O.moe_engine(L.x, o_ids, o_sc, L.experts, order=sorted(set(o_ids.flatten().tolist())))
    _close(out, want_a, torch.bfloat16, tight=True)
    want_b = O.moe_engine(L.x, o_ids, o_sc, L.experts, layer_idx=0)       # engine order: inside the path's tolerance
    _close(out, want_b, torch.bfloat16)
    order = O.activated_order(0, o_ids)
    out_b = ctx.forward(0, L.x.cuda(), ids, scores, order=_rank(order, 32))
    _close(out_b, want_b, torch.bfloat16, tight=True)
    assert ctx.status() == 0


def _device_oracle(L, ids, scores, order):
    """The oracle's own code on CUDA tensors (torch eager): the reference algorithm at full size."""
    return O.moe_engine(L.x, ids, scores, L.experts, order=order)


@pytest.mark.parametrize("name,T", [("qwen3", 256), ("qwen3", 8), ("mixtral", 64), ("mixtral", 1), ("mixtral", 16)])
def test_full_size_against_device_run_of_oracle(name, T):
    """The benchmark configurations at their full sizes: inputs drawn on the GPU, the oracle's functions evaluated on those
    CUDA tensors (torch eager = the reference's arithmetic on this device), same tolerance."""
    from on_device_sd_b200.synth import make_named
    L = make_named(name, T, device="cuda", gen_device="cuda")
    ctx = _ctx(L.H, L.E, L.K, L.I, L.dtype, max_tokens=256)
    ctx.set_gate(0, L.gate_w)
    for e, p in L.experts.items():
        ctx.set_expert(0, e, p)
    out, ids, scores = ctx.forward_fused(0, L.x, return_routing=True)
    assert ctx.status() == 0
    # routing: exact logits evaluated in fp64 on the device, tie rule from the oracle on the host
    logits = (L.x.double() @ L.gate_w.double().t()).float().to(L.dtype)
    assert torch.equal(ctx.last_logits(T), logits.float())
    o_ids, o_sc = O.topk_softmax(logits.cpu(), L.K)
    assert torch.equal(ids.cpu(), o_ids)
    want = _device_oracle(L, ids, scores, sorted(set(ids.flatten().tolist())))
    ma, mr = _close(out, want, L.dtype, tight=True)
    want_b = _device_oracle(L, ids, scores, O.activated_order(0, ids.cpu()))
    ma_b, mr_b = _close(out, want_b, L.dtype)
    print(f"\n[{name} T={T}] vs ascending-order oracle: max-abs {ma:.3g} mean-rel {mr:.3g}; vs engine-order oracle: {ma_b:.3g} / {mr_b:.3g}")
    # properties that need no oracle: permutation equivariance over tokens, and additivity over experts
    perm = torch.randperm(T, device="cuda")
    out_p = ctx.forward_fused(0, L.x[perm].contiguous())
    assert torch.equal(out_p, out[perm])
    if T > 1:
        half = [e if e < L.E // 2 else -1 for e in range(L.E)]
        other = [e if e >= L.E // 2 else -1 for e in range(L.E)]
        a = ctx.forward(0, L.x, ids, scores, expert_slot=half).float()
        b = ctx.forward(0, L.x, ids, scores, expert_slot=other).float()
        assert O.mean_rel((a + b).to(L.dtype), out) <= 5e-3


# ---------------------------------------------------------------------------------------------
# kernel families: the CUDA-core GEMV path and the tcgen05 tensor-core path must agree with the
# oracle on the same inputs, whatever the per-expert token count
# ---------------------------------------------------------------------------------------------
def _kinds():
    from on_device_sd_b200 import FFN_GEMV, FFN_MMA
    return {"gemv": FFN_GEMV, "mma": FFN_MMA}


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind", ["gemv", "mma"])
@pytest.mark.parametrize("T", [1, 3, 16, 17, 40])
def test_kernel_families_small_16bit(kind, T, dtype):
    """Both 16-bit model dtypes (the reference's default is float16, demo/src/core/model.py:122-129)."""
    from on_device_sd_b200.synth import make_layer
    H, E, K, I = 256, 16, 4, 192          # I is not a multiple of the 64-row tile of the tensor-core kernel
    L = make_layer(H, E, K, I, dtype, T, seed=11)
    ctx = _ctx(H, E, K, I, dtype, max_tokens=64)
    ctx.set_gate(0, L.gate_w.cuda())
    _register(ctx, L.experts)
    out, ids, scores = ctx.forward_fused(0, L.x.cuda(), return_routing=True, ffn_kind=_kinds()[kind])
    assert ctx.status() == 0
    want = O.moe_engine(L.x, ids.cpu(), scores.cpu(), L.experts, order=sorted(set(ids.flatten().tolist())))
    _close(out, want, dtype, tight=True)


@pytest.mark.parametrize("kind", ["gemv", "mma"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_kernel_families_many_tokens_one_expert(kind, dtype):
    """200 tokens all routed to the same two experts: more than one pass of 128 tokens in the
    tensor-core kernel, 50 passes of 4 in the GEMV kernel; K = 328 is not a multiple of 64."""
    from on_device_sd_b200.synth import make_layer
    H, E, K, I, T = 328, 4, 2, 136, 200
    L = make_layer(H, E, K, I, dtype, T, seed=12)
    ctx = _ctx(H, E, K, I, dtype, max_tokens=256)
    _register(ctx, L.experts)
    ids = torch.tensor([[3, 1]] * T)
    sc = torch.softmax(torch.randn(T, K, generator=torch.Generator().manual_seed(2)), -1).to(dtype)
    out = ctx.forward(0, L.x.cuda(), ids.cuda(), sc.cuda(), ffn_kind=_kinds()[kind])
    assert ctx.status() == 0
    _close(out, O.moe_engine(L.x, ids, sc, L.experts, order=[1, 3]), dtype, tight=True)


def test_expert_ffn_tensor_core_path():
    from on_device_sd_b200 import expert_forward_with_weights
    g = torch.Generator().manual_seed(3)
    H, I, n = 512, 320, 48
    x = torch.randn(n, H, generator=g).bfloat16()
    p = {"gate_proj": (torch.randn(I, H, generator=g) * 0.02).bfloat16(), "up_proj": (torch.randn(I, H, generator=g) * 0.02).bfloat16(),
         "down_proj": (torch.randn(H, I, generator=g) * 0.02).bfloat16()}
    out = expert_forward_with_weights(x.cuda(), p["gate_proj"].cuda(), p["up_proj"].cuda(), p["down_proj"].cuda())
    _close(out, O.expert_ffn(x, **p), torch.bfloat16, tight=True)


@pytest.mark.gpu
def test_popular_expert_exceeds_the_token_tile():
    """64 experts, every token picks the same two: the token tile is sized for the mean load (16 rows),
    so the two popular experts take four passes each in the tensor-core kernel."""
    from on_device_sd_b200.synth import make_layer
    H, E, K, I, T = 256, 64, 2, 192, 64
    L = make_layer(H, E, K, I, torch.bfloat16, T, seed=31)
    ctx = _ctx(H, E, K, I, torch.bfloat16, max_tokens=64)
    _register(ctx, L.experts)
    ids = torch.tensor([[9, 5]] * T)
    sc = torch.softmax(torch.randn(T, K, generator=torch.Generator().manual_seed(3)), -1).bfloat16()
    out = ctx.forward(0, L.x.cuda(), ids.cuda(), sc.cuda())
    assert ctx.status() == 0
    _close(out, O.moe_engine(L.x, ids, sc, L.experts, order=[5, 9]), torch.bfloat16, tight=True)
