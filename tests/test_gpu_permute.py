"""GPU: K2 (token-to-expert grouping) checked as integers against a host restatement of the reference's
per-expert `torch.where(topk_indices == e)` (demo/src/model/qwen3_runner.py:305-314)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _host_grouping(ids: torch.Tensor, E: int, usable):
    """offsets, sorted pairs, inverse map and active list as the reference's loop implies them."""
    T, K = ids.shape
    offsets, sorted_pair = [0], []
    inv = torch.full((T * K,), -1, dtype=torch.int64)
    act = []
    for e in range(E):
        tok, k = torch.where(ids == e)                  # row-major order of (token, slot)
        pairs = (tok * K + k).tolist()
        for p in pairs:
            inv[p] = len(sorted_pair)
            sorted_pair.append(p)
        offsets.append(len(sorted_pair))
        if pairs and e in usable:
            act.append(e)
    return torch.tensor(offsets), torch.tensor(sorted_pair, dtype=torch.int64), inv, torch.tensor(act, dtype=torch.int64)


def _cases():
    g = torch.Generator().manual_seed(3)
    E, K = 24, 4
    yield "uniform", torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(37)]), E
    yield "single token", torch.tensor([[5, 1, 23, 0]]), E
    yield "all tokens to the same experts (everything else empty)", torch.tensor([[7, 3, 9, 11]] * 50), E
    yield "duplicates inside a token", torch.tensor([[2, 2, 2, 5], [5, 5, 1, 1], [0, 0, 0, 0]]), E
    yield "ragged: expert 0 takes most pairs", torch.cat([torch.tensor([[0, 1, 2, 3]] * 90), torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(11)])]), E
    yield "more than 1024 pairs", torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(300)]), E
    yield "ids outside [0, E)", torch.tensor([[1, 99, 4, -3], [99, 99, 2, 1]]), E


@pytest.mark.parametrize("name,ids,E", list(_cases()), ids=[c[0] for c in _cases()])
def test_grouping_tables_equal_host_restatement(name, ids, E):
    from on_device_sd_b200 import B200MoEError, MoEContext
    H, I, K = 64, 32, ids.shape[1]
    T = ids.shape[0]
    ctx = MoEContext(H, E, K, I, torch.bfloat16, max_tokens=max(T, 8))
    usable = set(range(E)) - {3, 17}                      # two experts are never registered: they hold pairs but are not active
    w = {k: torch.zeros(s, dtype=torch.bfloat16, device="cuda") for k, s in (("gate_proj", (I, H)), ("up_proj", (I, H)), ("down_proj", (H, I)))}
    for e in usable:
        ctx.set_expert(0, e, w)
    x = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    scores = torch.full((T, K), 0.25, dtype=torch.bfloat16, device="cuda")
    ctx.forward(0, x, ids.cuda(), scores)
    offsets, sp, inv, act = ctx.last_tables(T)
    bad = bool(((ids < 0) | (ids >= E)).any())
    if bad:
        with pytest.raises(B200MoEError, match="status word"):
            ctx.status()
    else:
        assert ctx.status() == 0
    w_off, w_sp, w_inv, w_act = _host_grouping(ids, E, usable)
    assert torch.equal(offsets.cpu().long(), w_off)
    n = int(w_off[-1])
    assert torch.equal(sp.cpu().long()[:n], w_sp)
    assert torch.equal(inv.cpu().long(), w_inv)
    assert torch.equal(act.cpu().long(), w_act)


def test_grouping_of_an_empty_batch_is_a_no_op():
    from on_device_sd_b200 import MoEContext
    ctx = MoEContext(64, 8, 2, 32, torch.bfloat16, max_tokens=8)
    out = ctx.forward(0, torch.zeros(0, 64, dtype=torch.bfloat16, device="cuda"), torch.zeros(0, 2, dtype=torch.int64, device="cuda"),
                      torch.zeros(0, 2, dtype=torch.bfloat16, device="cuda"))
    assert out.shape == (0, 64) and ctx.status() == 0
