"""GPU: the one-launch block of batches of one and two tokens (router, experts and combine in one cooperative
kernel) against the oracle and against the kernel chain it replaces, through the C ABI."""
import pytest
import torch

from conftest import OUT_TOL
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _layer(H, E, K, I, dtype, seed, served=None):
    g = torch.Generator().manual_seed(seed)
    gate_w = (torch.randn(E, H, generator=g) * 0.05).to(dtype)
    experts = {}
    for e in range(E):
        if served is not None and e not in served:
            continue
        experts[e] = {"gate_proj": (torch.randn(I, H, generator=g) * 0.03).to(dtype),
                      "up_proj": (torch.randn(I, H, generator=g) * 0.03).to(dtype),
                      "down_proj": (torch.randn(H, I, generator=g) * 0.03).to(dtype)}
    return gate_w, experts


def _ctx(H, E, K, I, dtype, gate_w, experts, bias=None):
    from on_device_sd_b200 import MoEContext
    ctx = MoEContext(H, E, K, I, dtype, max_tokens=8)
    ctx.set_gate(0, gate_w.cuda(), None if bias is None else bias.cuda())
    keep = []
    for e, p in experts.items():
        dev = {k: v.cuda().contiguous() for k, v in p.items()}
        keep.append(dev)
        ctx.set_expert(0, e, dev)
    ctx._keep = keep
    return ctx


def _launches(ctx, fn):
    ctx.profile(True)
    fn()
    torch.cuda.synchronize()
    ctx.profile(False)
    return {k: v[1] for k, v in ctx.profile_read().items() if v[1]}


def _check_close(got, want, dtype):
    tol_a, tol_r = OUT_TOL[dtype]
    ulp = {torch.float16: 2.0 ** -9, torch.bfloat16: 2.0 ** -6}[dtype]
    got, want = got.cpu().double(), want.cpu().double()
    diff = (got - want).abs()
    assert float((diff - (tol_a + ulp * want.abs().max())).max()) <= 0
    assert O.mean_rel(got, want) <= tol_r


# (H, E, K, I): Qwen3-like rows, a long-I shape (down_proj rows of several ring segments, as the Mixtral-shaped layer
# has them), a shape whose rows are ragged against the
# ring segments
# and a shape whose gate/up units the single-token kernel cuts in two along K to balance the warps
SHAPES = [(2048, 128, 8, 768), (512, 8, 2, 3072), (1032, 16, 4, 520), (4096, 8, 2, 1536)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("T", [1, 2])
def test_token_block_matches_oracle_and_chain(shape, dtype, T):
    H, E, K, I = shape
    gate_w, experts = _layer(H, E, K, I, dtype, seed=H + E)
    ctx = _ctx(H, E, K, I, dtype, gate_w, experts)
    g = torch.Generator().manual_seed(7 + T)
    for trial in range(3):
        x = torch.randn(T, H, generator=g).to(dtype)
        if trial == 2 and T > 1:
            x[1] = x[0]                                              # two tokens with the same routing: experts with two rows
        res = torch.randn(T, H, generator=g).to(dtype) if trial % 2 else None
        xd, rd = x.cuda(), (None if res is None else res.cuda())
        seen = _launches(ctx, lambda: ctx.forward_fused(0, xd, residual=rd))
        assert seen == {"token_block": 1}, seen                      # the one-launch path is the one that ran
        out, ids, scores = ctx.forward_fused(0, xd, residual=rd, return_routing=True)
        tables = ctx.last_tables(T)
        assert ctx.status() == 0
        want_ids, want_scores, _ = O.route(x, gate_w, K)
        assert torch.equal(ids.cpu(), want_ids) and torch.equal(scores.cpu(), want_scores)       # bit-exact routing
        want = O.moe_engine(x, want_ids, want_scores, experts, order=sorted(set(want_ids.flatten().tolist())), residual=res)
        _check_close(out, want, dtype)
        # the kernel chain on the same input: same routing, same tables, outputs equal to rounding
        ctx.set_token_kernel(False)
        seen = _launches(ctx, lambda: ctx.forward_fused(0, xd, residual=rd))
        assert "token_block" not in seen
        out2, ids2, scores2 = ctx.forward_fused(0, xd, residual=rd, return_routing=True)
        tables2 = ctx.last_tables(T)
        ctx.set_token_kernel(True)
        assert torch.equal(ids, ids2) and torch.equal(scores, scores2)
        for a, b in zip(tables, tables2):
            assert torch.equal(torch.as_tensor(a), torch.as_tensor(b))
        _check_close(out, out2.cpu(), dtype)
        assert O.mean_rel(out.cpu().double(), out2.cpu().double()) <= 1e-3


def test_token_block_skips_unserved_experts_and_adds_bias():
    H, E, K, I, dtype = 1024, 16, 4, 512, torch.bfloat16
    served = {0, 1, 2, 5, 7, 8, 11, 13}
    gate_w, experts = _layer(H, E, K, I, dtype, seed=3, served=served)
    bias = (torch.randn(E, generator=torch.Generator().manual_seed(4)) * 0.5).to(dtype)
    ctx = _ctx(H, E, K, I, dtype, gate_w, experts, bias=bias)
    g = torch.Generator().manual_seed(11)
    hit_unserved = 0
    for trial in range(8):
        x = torch.randn(1 + trial % 2, H, generator=g).to(dtype)
        out, ids, scores = ctx.forward_fused(0, x.cuda(), return_routing=True)
        assert ctx.status() == 0
        want_ids, want_scores, _ = O.route(x, gate_w, K, bias=bias)
        assert torch.equal(ids.cpu(), want_ids) and torch.equal(scores.cpu(), want_scores)
        chosen = want_ids.flatten().tolist()
        hit_unserved += sum(e not in served for e in chosen)
        want = O.moe_engine(x, want_ids, want_scores, experts, order=sorted(set(chosen)))      # experts without weights are skipped
        _check_close(out, want, dtype)
    assert hit_unserved > 0


def test_token_block_many_calls_and_graph_replay():
    """The grid barrier word returns to its resting state after every launch: hundreds of launches in a row, and
    the same launches replayed from a CUDA graph, keep giving the results of the first."""
    H, E, K, I, dtype = 2048, 128, 8, 768, torch.bfloat16
    gate_w, experts = _layer(H, E, K, I, dtype, seed=21)
    ctx = _ctx(H, E, K, I, dtype, gate_w, experts)
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(1 + i % 2, H, generator=g).to(dtype).cuda() for i in range(4)]
    first = [ctx.forward_fused(0, x).clone() for x in xs]
    for _ in range(100):
        for x, want in zip(xs, first):
            out = ctx.forward_fused(0, x)
        assert torch.equal(out, first[-1])
    assert ctx.status() == 0
    outs = [torch.empty_like(x) for x in xs]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for x, o in zip(xs, outs):
            ctx.forward_fused(0, x, out=o)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for x, o in zip(xs, outs):
                ctx.forward_fused(0, x, out=o)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(20):
        for o in outs:
            o.zero_()
        graph.replay()
    torch.cuda.synchronize()
    for o, want in zip(outs, first):
        assert torch.equal(o, want)
    assert ctx.status() == 0


def test_other_shapes_keep_the_chain():
    """fp32 models, int4 experts and explicit kernel kinds are not taken by the one-launch path."""
    from on_device_sd_b200 import FFN_GEMV
    H, E, K, I = 256, 8, 2, 128
    gate_w, experts = _layer(H, E, K, I, torch.float32, seed=9)
    ctx = _ctx(H, E, K, I, torch.float32, gate_w, experts)
    x = torch.randn(1, H, generator=torch.Generator().manual_seed(1))
    assert "token_block" not in _launches(ctx, lambda: ctx.forward_fused(0, x.cuda()))
    gate_w, experts = _layer(H, E, K, I, torch.bfloat16, seed=9)
    ctx = _ctx(H, E, K, I, torch.bfloat16, gate_w, experts)
    xb = x.to(torch.bfloat16).cuda()
    assert "token_block" not in _launches(ctx, lambda: ctx.forward_fused(0, xb, ffn_kind=FFN_GEMV))
    assert _launches(ctx, lambda: ctx.forward_fused(0, xb)) == {"token_block": 1}
    assert _launches(ctx, lambda: ctx.forward_fused(0, xb.repeat(2, 1))) == {"token_block": 1}
    assert "token_block" not in _launches(ctx, lambda: ctx.forward_fused(0, xb.repeat(3, 1)))
