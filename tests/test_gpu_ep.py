"""GPU: expert-parallel legs of the C ABI.  On one GPU the ranks are emulated by contexts that each
register a block of the experts (the sum over their pair buffers plays the reduce-scatter); with two
or more GPUs the same check runs as NCCL ranks (one process per GPU)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from conftest import ROOT
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("mode", ["bf16", "int4"])
def test_emulated_ranks_are_bit_identical_to_one_gpu(world, mode):
    from on_device_sd_b200 import MoEContext, W_DENSE, W_INT4_G128
    from on_device_sd_b200.ep import expert_range
    from on_device_sd_b200.quant import quantize_expert
    from on_device_sd_b200.synth import make_layer
    H, E, K, I, T = 256, 16, 4, 128, 24
    L = make_layer(H, E, K, I, torch.bfloat16, T, seed=31)
    wm = W_INT4_G128 if mode == "int4" else W_DENSE
    dev = {e: {k: v.cuda() for k, v in p.items()} for e, p in L.experts.items()}
    if mode == "int4":
        dev = {e: quantize_expert(p) for e, p in dev.items()}
    full = MoEContext(H, E, K, I, torch.bfloat16, max_tokens=32, weight_mode=wm)
    full.set_gate(0, L.gate_w.cuda())
    for e, p in dev.items():
        full.set_expert(0, e, p)
    x = L.x.cuda()
    want, ids, scores = full.forward_fused(0, x, return_routing=True)
    total = None
    for r in range(world):
        ctx = MoEContext(H, E, K, I, torch.bfloat16, max_tokens=32, weight_mode=wm)
        for e in expert_range(E, world, r):
            ctx.set_expert(0, e, dev[e])
        y = ctx.ep_local_experts(0, x, ids)
        assert ctx.status() == 0
        served = torch.tensor([int(e) in expert_range(E, world, r) for e in ids.flatten().tolist()], device="cuda")
        assert bool((y[~served] == 0).all())              # rows of pairs served elsewhere are zeros
        total = y if total is None else total + y         # what the sum reduce-scatter computes
    out = full.ep_combine(total, ids, scores)
    assert torch.equal(out, want)
    # token shards combine independently
    half = T // 2
    out2 = full.ep_combine(total[half * K:].contiguous(), ids[half:].contiguous(), scores[half:].contiguous())
    assert torch.equal(out2, want[half:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_nccl_ranks_match_single_gpu():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), str(ROOT / "tests" / "ep_nccl_check.py")], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "EP_NCCL_CHECK PASS" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_stack_with_popularity_bias_matches_oracle_layer_by_layer():
    """Three stacked blocks h <- x + MoE_l(h) with the Zipf gate bias of the stacked benchmark; each
    layer's kernel output is checked against the oracle fed with the SAME bf16 input, so errors do not compound."""
    from on_device_sd_b200 import MoEContext
    from on_device_sd_b200.stack import MoEStack
    from on_device_sd_b200.synth import make_layer, zipf_bias
    from test_gpu_moe import _close
    H, E, K, I, T, L = 256, 16, 4, 128, 20, 3
    ctx = MoEContext(H, E, K, I, torch.bfloat16, num_layers=L, max_tokens=32)
    layers = []
    for l in range(L):
        Ll = make_layer(H, E, K, I, torch.bfloat16, T, seed=50 + l)
        bias = zipf_bias(E, 1.1, seed=l).to(torch.bfloat16)
        ctx.set_gate(l, Ll.gate_w.cuda(), bias.cuda())
        for e, p in Ll.experts.items():
            ctx.set_expert(l, e, {k: v.cuda() for k, v in p.items()})
        layers.append((Ll, bias))
    h = layers[0][0].x.cuda()
    out = MoEStack(ctx, L).forward(h)
    assert ctx.status() == 0
    cur = h
    counts = torch.zeros(E)
    for l, (Ll, bias) in enumerate(layers):
        got = ctx.forward_fused(l, cur, residual=h)
        ids, scores, _ = O.route(cur.cpu(), Ll.gate_w, K, bias=bias)
        counts += torch.bincount(ids.flatten(), minlength=E)
        want = O.moe_engine(cur.cpu(), ids, scores, Ll.experts, order=list(range(E)), residual=h.cpu())
        _close(got, want, torch.bfloat16, tight=True)
        cur = got
    assert torch.equal(cur, out)
    assert counts.max() >= 2 * counts.mean() and counts.min() == 0    # the bias really skews the expert load
