"""GPU: K1 router through the C ABI against the oracle and against torch's CUDA ops."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import GOLDEN, Golden, ulp_tolerance
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _ctx(H, E, K, I, dtype, **kw):
    from on_device_sd_b200 import MoEContext
    return MoEContext(H, E, K, I, dtype, **kw)


def _check_scores(got, want, dtype):
    got, want = got.float().cpu(), want.float().cpu()
    tol = ulp_tolerance(dtype)
    assert float((got - want).abs().max()) <= tol, float((got - want).abs().max())
    if dtype != torch.float32:
        assert float((got == want).float().mean()) >= 0.98   # at most a stray last-bit difference


def test_router_matches_oracle_on_golden(golden):
    g = golden
    ctx = _ctx(g.H, g.E, g.K, g.I, g.dtype, max_tokens=max(g.T, 8))
    ctx.set_gate(0, g.gate_w.cuda())
    ids, scores = ctx.route(0, g.x.cuda())
    logits = ctx.last_logits(g.T)
    assert ctx.status() == 0
    want_logits = g.t("def_logits").float()
    if g.dtype == torch.float32:
        assert float((logits.cpu() - want_logits).abs().max()) <= 1e-6
    else:
        assert torch.equal(logits.cpu(), want_logits)          # bit-exact logits
    assert torch.equal(ids.cpu(), g.t("def_ids"))               # bit-exact ordered ids
    _check_scores(scores, g.t("def_scores"), g.dtype)
    # reference test_routing.py:18-24: the weights of a token sum to one
    assert torch.allclose(scores.float().sum(-1), torch.ones(g.T, device="cuda"), atol=2e-2 if g.dtype != torch.float32 else 1e-5)


def test_tie_order_matches_torch_cuda_fixture():
    z = np.load(GOLDEN / "topk_cuda_ties.npz")
    names = sorted(k[:-3] for k in z.files if k.endswith("_in"))
    dts = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}
    for n in names:
        vin, idx = z[n + "_in"], z[n + "_idx"]
        dtype = dts[n.split("_")[0]]
        T, E = vin.shape
        K = idx.shape[1]
        ctx = _ctx(8, E, K, 8, dtype, max_tokens=16)
        logits = torch.from_numpy(vin.astype(np.float32)).to(dtype).cuda()
        ids, scores = ctx.route(0, None, logits=logits)
        assert np.array_equal(ids.cpu().numpy(), idx.astype(np.int64)), n


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("E,K", [(8, 2), (128, 8), (60, 4), (256, 32), (16, 1)])
def test_topk_softmax_equals_torch_cuda_live(dtype, E, K):
    """Same logits in, same ordered ids out as torch.topk on this GPU - including ties - and the
    softmax of moe_layer.py:54 within one unit in the last place."""
    g = torch.Generator(device="cuda").manual_seed(E * 100 + K)
    T = 777
    logits = (torch.randn(T, E, device="cuda", generator=g) * 1.5).to(dtype)
    logits[::3] = (logits[::3].float() * 4).round().div(4).to(dtype)    # plant many exact ties
    ctx = _ctx(8, E, K, 8, dtype, max_tokens=T)
    ids, scores = ctx.route(0, None, logits=logits)
    vals, want = torch.topk(logits, K, dim=-1)
    assert torch.equal(ids, want)
    _check_scores(scores, F.softmax(vals, dim=-1), dtype)


@pytest.mark.parametrize("name,T", [("qwen3", 256), ("qwen3", 1), ("mixtral", 64), ("mixtral", 5)])
def test_router_seeded_benchmark_shapes(name, T):
    """Router of the benchmark shapes: logits bit-exact against the fp64 definition, ids bit-exact
    against the oracle; agreement with torch's own cuBLAS-based router is reported."""
    from on_device_sd_b200.synth import CONFIGS
    H, E, K, I, dtype = CONFIGS[name]
    g = torch.Generator().manual_seed(0)
    gate_w = (torch.randn(E, H, generator=g) * 0.02).to(dtype)
    x = torch.randn(T, H, generator=g).to(dtype)
    ctx = _ctx(H, E, K, 128, dtype, max_tokens=T)
    ctx.set_gate(0, gate_w.cuda())
    ids, scores = ctx.route(0, x.cuda())
    logits = ctx.last_logits(T).cpu()
    o_ids, o_scores, o_logits = O.route(x, gate_w, K)
    assert torch.equal(logits, o_logits.float())
    assert torch.equal(ids.cpu(), o_ids)
    _check_scores(scores, o_scores, dtype)
    # side by side with the reference's ops on this GPU (F.linear -> topk -> softmax)
    t_logits = F.linear(x.cuda(), gate_w.cuda())
    t_vals, t_ids = torch.topk(t_logits, K, dim=-1)
    differing_logits = int((t_logits.float().cpu() != logits).sum())
    differing_tokens = int((t_ids != ids).any(-1).sum())
    print(f"\n[{name} T={T}] cuBLAS logits differing from the correctly rounded ones: {differing_logits}/{T * E}; "
          f"tokens whose ordered ids differ from torch's: {differing_tokens}/{T}")
    # with torch's own logits the ids are identical
    ids2, scores2 = ctx.route(0, None, logits=t_logits)
    assert torch.equal(ids2, t_ids)
    _check_scores(scores2, F.softmax(t_vals, dim=-1), dtype)
    # every token that differs is explained by a logit that cuBLAS rounded the other way
    bad = (t_ids != ids).any(-1).cpu()
    changed = (t_logits.float().cpu() != logits).any(-1)
    assert bool((~bad | changed).all())


def test_router_bias_and_bitmap():
    from on_device_sd_b200.synth import zipf_bias
    H, E, K, T = 256, 128, 8, 40
    g = torch.Generator().manual_seed(4)
    gate_w = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    bias = zipf_bias(E).to(torch.bfloat16)
    ctx = _ctx(H, E, K, 128, torch.bfloat16, max_tokens=64)
    ctx.set_gate(0, gate_w.cuda(), bias.cuda())
    bitmap = torch.zeros(4, dtype=torch.int64).pin_memory()
    ids, scores = ctx.route(0, x.cuda(), bitmap=bitmap)
    torch.cuda.synchronize()
    o_ids, o_scores, _ = O.route(x, gate_w, K, bias=bias)
    assert torch.equal(ids.cpu(), o_ids)
    active = set()
    for w in range(4):
        v = int(bitmap[w]) & 0xFFFFFFFFFFFFFFFF
        active |= {w * 64 + b for b in range(64) if (v >> b) & 1}
    assert active == set(o_ids.flatten().tolist())      # reference test_routing.py:27-33


def test_router_fp16_extremes_take_the_exact_path():
    """Logits beyond fp16's normal range (overflow to inf, subnormal results) are still the
    correctly rounded values."""
    H, E, K = 64, 8, 2
    x = torch.zeros(3, H, dtype=torch.float16)
    w = torch.zeros(E, H, dtype=torch.float16)
    x[0, :] = 60000.0; w[0, :4] = 2.0; w[1, :4] = -2.0          # |dot| = 480000 -> +-inf in fp16
    x[1, 0] = 6e-5; w[:, 0] = torch.linspace(1e-3, 8e-3, E).half()   # subnormal fp16 results
    x[2, :] = 1.0; w[2, 8:16] = 0.5
    ctx = _ctx(H, E, K, 8, torch.float16, max_tokens=8)
    ctx.set_gate(0, w.cuda())
    ids, scores = ctx.route(0, x.cuda())
    logits = ctx.last_logits(3).cpu()
    want = (x.double() @ w.double().t()).float().half().float()
    assert torch.equal(torch.nan_to_num(logits, posinf=1e30, neginf=-1e30), torch.nan_to_num(want, posinf=1e30, neginf=-1e30))
    assert torch.equal(ids.cpu()[1:], O.route(x, w, K)[0][1:])


def test_router_empty_batch_and_errors():
    from on_device_sd_b200 import B200MoEError
    ctx = _ctx(64, 8, 2, 64, torch.bfloat16, max_tokens=4)
    with pytest.raises(B200MoEError, match="no gate weight"):
        ctx.route(0, torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda"))
    ctx.set_gate(0, torch.zeros(8, 64, dtype=torch.bfloat16, device="cuda"))
    ids, scores = ctx.route(0, torch.zeros(0, 64, dtype=torch.bfloat16, device="cuda"))
    assert ids.shape == (0, 2) and scores.shape == (0, 2)
    with pytest.raises(B200MoEError, match="max_tokens"):
        ctx.route(0, torch.zeros(5, 64, dtype=torch.bfloat16, device="cuda"))
    # all-zero logits: ids follow torch's tie order, scores are uniform
    ids, scores = ctx.route(0, torch.zeros(2, 64, dtype=torch.bfloat16, device="cuda"))
    assert ids.cpu().tolist() == [[1, 0], [1, 0]] and torch.equal(scores.float().cpu(), torch.full((2, 2), 0.5))


@pytest.mark.parametrize("T", [1, 2, 8, 32, 40])
@pytest.mark.parametrize("E,K,groups", [(128, 8, 16), (8, 2, 3), (60, 4, 60), (256, 32, 40)])
def test_tied_logits_follow_torch_order_in_every_router_form(T, E, K, groups):
    """Gate rows repeated in groups give exactly equal logits, so the kept set and its order are decided by the tie
    rules alone (lowest index first into the set, then the 32-slot network's permutation).  The batch sizes reach
    the one-launch block (T = 1, 2: routing read back from the fused entry), the one-token-per-CTA router (CTA-wide
    counting top-k) and the token-tile router (one warp per token); all must give the oracle's torch-CUDA order."""
    H, I = 256, 128
    g = torch.Generator().manual_seed(E + K + T)
    base = (torch.randn(groups, H, generator=g) * 0.05).to(torch.bfloat16)
    gate_w = base[torch.arange(E) % groups].contiguous()
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    ctx = _ctx(H, E, K, I, torch.bfloat16, max_tokens=64)
    ctx.set_gate(0, gate_w.cuda())
    want_ids, want_scores, _ = O.route(x, gate_w, K)
    ids, scores = ctx.route(0, x.cuda())
    assert torch.equal(ids.cpu(), want_ids) and torch.equal(scores.cpu(), want_scores)
    # the fused entry (no experts registered: the block contributes zeros) routes through the one-launch kernels for T <= 2
    out, ids2, scores2 = ctx.forward_fused(0, x.cuda(), return_routing=True)
    assert torch.equal(ids2.cpu(), want_ids) and torch.equal(scores2.cpu(), want_scores)
    assert ctx.status() == 0 and float(out.abs().max()) == 0.0
