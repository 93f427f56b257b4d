"""RMSNorm in front of the MoE block (b200moe_rmsnorm) against the reference's outputs and the oracle."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN, from_np
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
_DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def _ulp_close(got, want, dtype):
    """Equal except for at most 1e-3 of the elements, each off by one unit in the last place: the row's sum of
    squares is added in a different order than torch's CPU reduction, which can move a rounding boundary."""
    got, want = got.cpu(), want.cpu()
    if torch.equal(got, want):
        return
    if dtype == torch.float32:
        assert torch.allclose(got, want, rtol=2e-6, atol=1e-7)
        return
    gi, wi = got.view(torch.int16).int(), want.view(torch.int16).int()
    diff = (gi - wi).abs()
    assert int(diff.max()) <= 1, int(diff.max())
    assert float((diff > 0).float().mean()) <= 1e-3


@pytest.mark.parametrize("name", ["bf16", "f16", "f32"])
def test_rmsnorm_matches_reference_fixture(name):
    from on_device_sd_b200 import MoEContext
    dt = _DT[name]
    z = np.load(GOLDEN / "rmsnorm.npz")
    x, r, w = (from_np(z[f"{name}_{k}"], dt) for k in ("x", "r", "w"))
    ctx = MoEContext(x.shape[1], 1, 1, 8, dt, max_tokens=8)
    _ulp_close(ctx.rmsnorm(x.cuda(), w.cuda(), 1e-6), from_np(z[f"{name}_out"], dt), dt)
    out, res = ctx.rmsnorm(x.cuda(), w.cuda(), 1e-6, r.cuda())
    _ulp_close(out, from_np(z[f"{name}_out_add"], dt), dt)
    assert torch.equal(res.cpu(), from_np(z[f"{name}_res"], dt))          # the residual sum has no reduction: bit-exact


@pytest.mark.parametrize("T,H", [(1, 2048), (33, 2048), (7, 4096), (5, 16384), (3, 8)])
def test_rmsnorm_module_matches_oracle(T, H):
    from on_device_sd_b200 import RMSNorm
    g = torch.Generator().manual_seed(T * 31 + H)
    x = torch.randn(2, T, H, generator=g).bfloat16()
    r = torch.randn(2, T, H, generator=g).bfloat16()
    m = RMSNorm(H, eps=1e-6)
    with torch.no_grad():
        m.weight.copy_(1.0 + 0.1 * torch.randn(H, generator=g))
    w = m.weight.detach().bfloat16()
    _ulp_close(m(x.cuda()), O.rmsnorm(x, w, 1e-6), torch.bfloat16)
    out, res = m(x.cuda(), r.cuda())
    want, want_res = O.rmsnorm(x, w, 1e-6, r)
    _ulp_close(out, want, torch.bfloat16)
    assert torch.equal(res.cpu(), want_res) and out.shape == x.shape


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("T", [1, 2, 5, 32, 33, 40])
@pytest.mark.parametrize("with_residual", [True, False])
def test_norm_fused_into_the_router_equals_norm_then_block(dtype, T, with_residual):
    """b200moe_forward_fused_norm (the norm applied inside the router kernel's load of the tokens) against the
    two-step form b200moe_rmsnorm -> b200moe_forward_fused: normalised rows, new residual, ids and output all
    bit-identical, for the single-token-per-CTA router (T <= 32) and the tile router (T > 32)."""
    from on_device_sd_b200 import MoEContext
    from on_device_sd_b200.synth import make_layer
    H, E, K, I = 256, 16, 4, 128
    L = make_layer(H, E, K, I, dtype, T, seed=61)
    ctx = MoEContext(H, E, K, I, dtype, max_tokens=64)
    ctx.set_gate(0, L.gate_w.cuda())
    for e, p in L.experts.items():
        ctx.set_expert(0, e, {k: v.cuda() for k, v in p.items()})
    g = torch.Generator().manual_seed(T)
    hidden = (L.x * 3).to(dtype).cuda()
    res = torch.randn(T, H, generator=g).to(dtype).cuda() if with_residual else None
    w = (1.0 + 0.1 * torch.randn(H, generator=g)).to(dtype).cuda()
    if with_residual:
        normed, new_res = ctx.rmsnorm(hidden, w, 1e-6, res)
    else:
        normed, new_res = ctx.rmsnorm(hidden, w, 1e-6), hidden
    want, want_ids, want_scores = ctx.forward_fused(0, normed, residual=new_res, return_routing=True)
    out, r_out, n_out, ids, scores = ctx.forward_fused_norm(0, hidden, w, 1e-6, residual=res, return_parts=True)
    assert ctx.status() == 0
    assert torch.equal(n_out, normed) and torch.equal(r_out, new_res)
    assert torch.equal(ids, want_ids) and torch.equal(scores, want_scores)
    assert torch.equal(out, want)
    assert torch.equal(ctx.forward_fused_norm(0, hidden, w, 1e-6, residual=res), want)      # internal buffers for the parts
    # and against the oracle's norm + block
    o_norm = O.rmsnorm(hidden.cpu(), w.cpu(), 1e-6, res.cpu() if with_residual else None)
    o_n, o_r = o_norm if with_residual else (o_norm, hidden.cpu())
    assert torch.equal(r_out.cpu(), o_r)
    assert float((n_out.cpu().float() - o_n.float()).abs().max()) <= (1e-6 if dtype == torch.float32 else 2.0 ** -6)
