"""GPU: int4 g128 expert weights - packer / unpacker bit-exactness and the int4 FFN kernels."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN, from_np
from oracle import moe_oracle as O
from test_gpu_moe import _close

pytestmark = pytest.mark.gpu


def test_pack_unpack_bit_exact_against_oracle_fixture():
    from on_device_sd_b200.quant import pack_int4, unpack_int4
    z = np.load(GOLDEN / "int4_g128.npz")
    w = from_np(z["w"], torch.bfloat16)
    q, s = pack_int4(w.cuda())
    assert np.array_equal(q.cpu().numpy(), z["q"])
    assert torch.equal(s.cpu(), from_np(z["scales"], torch.bfloat16))
    qi, dq = unpack_int4(q, s)
    assert np.array_equal(qi.cpu().numpy(), z["unpacked"])
    assert torch.equal(dq.cpu(), from_np(z["dequant"], torch.bfloat16))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(768, 2048), (64, 128), (33, 1280)])
def test_pack_unpack_random_matches_oracle_and_roundtrips(dtype, shape):
    from on_device_sd_b200.quant import pack_int4, unpack_int4
    g = torch.Generator().manual_seed(shape[0])
    w = (torch.randn(*shape, generator=g) * 0.02).to(dtype)
    w[0, :128] = 0
    q, s = pack_int4(w.cuda())
    oq, os_ = O.quant_int4_g128(w)
    assert torch.equal(q.cpu(), oq) and torch.equal(s.cpu(), os_)
    qi, dq = unpack_int4(q, s, dtype)
    assert torch.equal(qi.cpu(), O.unpack_int4(oq))
    assert torch.equal(dq.cpu(), O.dequant_int4_g128(oq, os_, dtype))
    # unpack(pack(q)) == q: quantising the dequantised weights gives the same nibbles
    q2, s2 = pack_int4(dq.to(torch.bfloat16).contiguous())
    if dtype == torch.bfloat16:
        assert torch.equal(q2, q) and torch.equal(s2, s)


def _int4_layer(H, E, K, I, T, seed):
    from on_device_sd_b200 import MoEContext, W_INT4_G128
    from on_device_sd_b200.quant import quantize_expert
    from on_device_sd_b200.synth import make_layer
    L = make_layer(H, E, K, I, torch.bfloat16, T, seed=seed)
    ctx = MoEContext(H, E, K, I, torch.bfloat16, max_tokens=max(T, 8), weight_mode=W_INT4_G128)
    ctx.set_gate(0, L.gate_w.cuda())
    deq = {}
    for e, p in L.experts.items():
        qp = quantize_expert({k: v.cuda() for k, v in p.items()})
        ctx.set_expert(0, e, qp)
        deq[e] = {k: O.dequant_int4_g128(*O.quant_int4_g128(v)) for k, v in p.items()}
    return L, ctx, deq


@pytest.mark.parametrize("kind", ["gemv", "mma"])
@pytest.mark.parametrize("T", [1, 5, 8, 20, 40])
def test_int4_moe_matches_oracle_on_dequantised_weights(T, kind):
    """The oracle for int4 is the reference forward on dequant(quant(W)); K = 384 exercises a last
    TMA box that is half beyond the matrix, I = 136... is not allowed (multiples of 128), so rows use 16-row tails via H."""
    H, E, K, I = 384, 8, 2, 256
    L, ctx, deq = _int4_layer(H, E, K, I, T, seed=21)
    from on_device_sd_b200 import FFN_GEMV, FFN_MMA
    # "gemv": per-warp tiles with register-fragment MMAs (any token count); "mma": the tcgen05 kernel
    out, ids, scores = ctx.forward_fused(0, L.x.cuda(), return_routing=True, ffn_kind={"gemv": FFN_GEMV, "mma": FFN_MMA}[kind])
    assert ctx.status() == 0
    o_ids, o_sc, _ = O.route(L.x, L.gate_w, K)
    assert torch.equal(ids.cpu(), o_ids)
    want = O.moe_engine(L.x, o_ids, o_sc, deq, order=sorted(set(o_ids.flatten().tolist())))
    _close(out, want, torch.bfloat16, tight=True)


@pytest.mark.parametrize("T", [1, 16, 64])
def test_int4_qwen3_shape_reduced_experts(T):
    L, ctx, deq = _int4_layer(2048, 16, 8, 768, T, seed=22)
    out, ids, scores = ctx.forward_fused(0, L.x.cuda(), return_routing=True)
    assert ctx.status() == 0
    want = O.moe_engine(L.x, ids.cpu(), scores.cpu(), deq, order=sorted(set(ids.flatten().tolist())))
    _close(out, want, torch.bfloat16, tight=True)


@pytest.mark.parametrize("kind", ["gemv", "mma"])
def test_int4_all_tokens_one_expert_many_passes(kind):
    from on_device_sd_b200 import FFN_GEMV, FFN_MMA
    H, E, K, I, T = 256, 4, 2, 128, 200
    L, ctx, deq = _int4_layer(H, E, K, I, T, seed=23)
    ids = torch.tensor([[2, 0]] * T)
    sc = torch.softmax(torch.randn(T, K, generator=torch.Generator().manual_seed(2)), -1).bfloat16()
    out = ctx.forward(0, L.x.cuda(), ids.cuda(), sc.cuda(), ffn_kind={"gemv": FFN_GEMV, "mma": FFN_MMA}[kind])
    assert ctx.status() == 0
    _close(out, O.moe_engine(L.x, ids, sc, deq, order=[0, 2]), torch.bfloat16, tight=True)


def test_int4_mixtral_full_size_against_device_run_of_oracle():
    from on_device_sd_b200 import MoEContext, W_INT4_G128
    from on_device_sd_b200.quant import quantize_expert, unpack_int4
    from on_device_sd_b200.synth import make_named
    T = 16
    L = make_named("mixtral", T, device="cuda", gen_device="cuda")
    ctx = MoEContext(L.H, L.E, L.K, L.I, L.dtype, max_tokens=64, weight_mode=W_INT4_G128)
    ctx.set_gate(0, L.gate_w)
    deq = {}
    for e, p in L.experts.items():
        qp = quantize_expert(p)
        ctx.set_expert(0, e, qp)
        deq[e] = {k: unpack_int4(qp[k], qp[k + "_scales"])[1] for k in ("gate_proj", "up_proj", "down_proj")}
        L.experts[e] = None            # free the bf16 originals
    out, ids, scores = ctx.forward_fused(0, L.x, return_routing=True)
    assert ctx.status() == 0
    want = O.moe_engine(L.x, ids, scores, deq, order=sorted(set(ids.flatten().tolist())))
    _close(out, want, L.dtype, tight=True)


@pytest.mark.gpu
def test_int4_popular_expert_exceeds_the_token_tile():
    """As the bf16 case: tile of 16 rows, two experts with 64 tokens each -> four passes; I = 128 gives the
    down projection a single k-stage, so the second MMA issuer never starts its accumulators."""
    H, E, K, I, T = 256, 64, 2, 128, 64
    L, ctx, deq = _int4_layer(H, E, K, I, T, seed=29)
    ids = torch.tensor([[9, 5]] * T)
    sc = torch.softmax(torch.randn(T, K, generator=torch.Generator().manual_seed(3)), -1).bfloat16()
    out = ctx.forward(0, L.x.cuda(), ids.cuda(), sc.cuda())
    assert ctx.status() == 0
    _close(out, O.moe_engine(L.x, ids, sc, deq, order=[5, 9]), torch.bfloat16, tight=True)


@pytest.mark.gpu
@pytest.mark.parametrize("T", [3, 24, 70])
def test_int4_odd_number_of_k_stages(T):
    """H = 384 and I = 640 give 3 and 5 k-stages of 128 per work item: the two MMA issuers alternate over the
    running stage index, so which issuer starts a work item changes from item to item."""
    H, E, K, I = 384, 8, 2, 640
    L, ctx, deq = _int4_layer(H, E, K, I, T, seed=37)
    out, ids, scores = ctx.forward_fused(0, L.x.cuda(), return_routing=True)
    assert ctx.status() == 0
    want = O.moe_engine(L.x, ids.cpu(), scores.cpu(), deq, order=sorted(set(ids.flatten().tolist())))
    _close(out, want, torch.bfloat16, tight=True)
