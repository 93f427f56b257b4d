"""GPU: the expert-parallel path of the C ABI (peer-store dispatch / return).  On one GPU the ranks are
contexts of one process whose exchange buffers point at one another and whose phases are enqueued one
after the other; with two or more GPUs the same check runs as one process per GPU over CUDA IPC."""
import os
import socket
import subprocess
import sys

import pytest
import torch

from conftest import ROOT
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _full_and_ranks(world, mode, H, E, K, I, T, seed, max_local):
    from on_device_sd_b200 import MoEContext, W_DENSE, W_INT4_G128
    from on_device_sd_b200.ep import expert_range
    from on_device_sd_b200.quant import quantize_expert
    from on_device_sd_b200.synth import make_layer
    L = make_layer(H, E, K, I, torch.bfloat16, T, seed=seed)
    wm = W_INT4_G128 if mode == "int4" else W_DENSE
    dev = {e: {k: v.cuda() for k, v in p.items()} for e, p in L.experts.items()}
    if mode == "int4":
        dev = {e: quantize_expert(p) for e, p in dev.items()}
    full = MoEContext(H, E, K, I, torch.bfloat16, max_tokens=world * max_local, weight_mode=wm)
    full.set_gate(0, L.gate_w.cuda())
    for e, p in dev.items():
        full.set_expert(0, e, p)
    ranks = []
    for r in range(world):
        ctx = MoEContext(H, E, K, I, torch.bfloat16, max_tokens=world * max_local, weight_mode=wm)
        ctx.set_gate(0, L.gate_w.cuda())
        for e in expert_range(E, world, r):
            ctx.set_expert(0, e, dev[e])
        ctx.ep_create(world, r, max_local)
        ranks.append(ctx)
    for ctx in ranks:
        ctx.ep_attach_local(ranks)
    return L, full, ranks


def _run_phases(ranks, xs, residuals=None, order=None):
    """One layer call of every rank, phase by phase on one stream: a kernel that waits for a flag is
    always enqueued after the kernel that raises it, so no two of them ever have to run at the same time."""
    for ctx, x in zip(ranks, xs):
        ctx.ep_dispatch(0, x)
    for ctx in ranks:
        ctx.ep_experts(0)
    return [ctx.ep_combine(x.shape[0], order=order, residual=None if residuals is None else residuals[i])
            for i, (ctx, x) in enumerate(zip(ranks, xs))]


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", ["bf16", "int4"])
def test_emulated_ranks_are_bit_identical_to_one_gpu(world, mode):
    """Ranks emulated by contexts of one process on one GPU whose exchange buffers are plain device
    pointers to one another: same kernels, same protocol, one call after the other."""
    H, E, K, I, T = 256, 16, 4, 128, 48
    per = T // world
    L, full, ranks = _full_and_ranks(world, mode, H, E, K, I, T, 31, 2 * per)
    x = L.x.cuda()
    want, ids, scores = full.forward_fused(0, x, return_routing=True)
    xs = [x[r * per:(r + 1) * per].contiguous() for r in range(world)]
    for call in range(3):                                   # later calls reuse every buffer and the epoch counters
        outs = _run_phases(ranks, xs)
        assert all(ctx.status() == 0 for ctx in ranks)
        assert torch.equal(torch.cat(outs), want), call
    r_ids, r_scores = ranks[1].ep_last_routing(per)
    assert torch.equal(r_ids, ids[per:2 * per]) and torch.equal(r_scores, scores[per:2 * per])
    # residual and a caller-given accumulation order, as on one GPU
    order = list(reversed(range(E)))
    res = torch.randn_like(x)
    want2 = full.forward(0, x, ids, scores, order=order, residual=res)
    outs = _run_phases(ranks, xs, residuals=[res[r * per:(r + 1) * per].contiguous() for r in range(world)], order=order)
    assert torch.equal(torch.cat(outs), want2)
    # ragged: ranks hold different numbers of tokens, one of them none at all
    sizes = [per] * world
    sizes[0] += 2
    sizes[1] -= 2
    if world >= 4:
        sizes[3] += sizes[2]
        sizes[2] = 0
    cuts = [0]
    for n in sizes:
        cuts.append(cuts[-1] + n)
    xs2 = [x[a:b].contiguous() for a, b in zip(cuts[:-1], cuts[1:])]
    outs = _run_phases(ranks, xs2)
    assert all(ctx.status() == 0 for ctx in ranks)
    # the token tile is sized from each rank's own slice here, so only closeness is promised
    assert O.mean_rel(torch.cat(outs).cpu(), want.cpu()) <= 1e-3


def test_one_rank_world_equals_the_fused_block():
    L, full, ranks = _full_and_ranks(1, "bf16", 256, 16, 4, 128, 24, 7, 24)
    x = L.x.cuda()
    want = full.forward_fused(0, x)
    got = ranks[0].ep_forward(0, x)
    assert ranks[0].status() == 0 and torch.equal(got, want)


def test_a_rank_that_never_arrives_makes_the_wait_run_out_not_hang():
    """Rank 1 never dispatches: rank 0's bounded waits (set to 20 ms here) give up, its kernels finish,
    the status word says so and the context stays usable."""
    from on_device_sd_b200 import B200MoEError
    import time
    L, full, ranks = _full_and_ranks(2, "bf16", 256, 16, 4, 128, 16, 9, 8)
    x = L.x.cuda()
    for ctx in ranks:
        ctx.ep_set_wait_ms(20)
    t0 = time.time()
    ranks[0].ep_dispatch(0, x[:8].contiguous())
    ranks[0].ep_experts(0)                        # waits for rank 1's dispatch flag, which nothing raises
    ranks[0].ep_combine(8)                        # waits for rank 1's return flag
    with pytest.raises(B200MoEError, match="status word = 4"):
        ranks[0].status()
    assert time.time() - t0 < 5.0
    # the late rank catches up; from the next call on both are in step again
    ranks[1].ep_dispatch(0, x[8:].contiguous())
    ranks[1].ep_experts(0)
    ranks[1].ep_combine(8)
    try:
        ranks[1].status()                         # reads and clears whatever the late rank recorded
    except B200MoEError:
        pass
    want = full.forward_fused(0, x)
    outs = _run_phases(ranks, [x[:8].contiguous(), x[8:].contiguous()])
    assert all(ctx.status() == 0 for ctx in ranks)
    assert torch.equal(torch.cat(outs), want)


def test_ep_argument_errors():
    from on_device_sd_b200 import B200MoEError, MoEContext
    ctx = MoEContext(64, 8, 2, 32, torch.bfloat16, max_tokens=16)
    with pytest.raises(B200MoEError, match="no exchange buffer"):
        ctx.ep_experts(0)
    with pytest.raises(B200MoEError, match="not divisible"):
        ctx.ep_create(3, 0, 4)
    with pytest.raises(B200MoEError, match="exceeds the context's max_tokens"):
        ctx.ep_create(2, 0, 9)
    ctx.ep_create(2, 1, 8)
    with pytest.raises(B200MoEError, match="not attached"):
        ctx.ep_dispatch(0, torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ranks_on_separate_gpus_match_single_gpu():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), str(ROOT / "tests" / "ep_ranks_check.py")], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "EP_RANKS_CHECK PASS" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


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
