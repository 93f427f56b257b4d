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
