"""CPU, world_size 2 over gloo: the expert-parallel plumbing (sharding, all-gather dispatch, pair-ordered
return buffers, sum reduce-scatter, local combine) reproduces the single-process oracle exactly.
The three local steps are played by a torch stand-in built from the oracle (test infrastructure);
on GPUs the same ExpertParallelMoE drives libb200moe.so (tests/test_gpu_ep.py)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from on_device_sd_b200.ep import ExpertParallelMoE, expert_range, owner_of, split_tokens
from on_device_sd_b200.synth import make_layer
from oracle import moe_oracle as O


class OracleBackedContext:
    """Stand-in for MoEContext on the CPU: same three methods, arithmetic from the oracle."""

    def __init__(self, layer, K):
        self.gate_w, self.K, self.experts = layer.gate_w, K, {}

    def set_expert(self, layer, e, params):
        self.experts[e] = params

    def route(self, layer, x):
        ids, scores, _ = O.route(x, self.gate_w, self.K)
        return ids, scores

    def ep_local_experts(self, layer, x_all, ids_all):
        T, H = x_all.shape
        out = torch.zeros(T * self.K, H, dtype=x_all.dtype)
        for e, p in self.experts.items():
            tok, kk = torch.where(ids_all == e)
            if tok.numel():
                out[tok * self.K + kk] = O.expert_ffn(x_all[tok], **p)
        return out

    def ep_combine(self, y_pairs, ids, scores, order=None, residual=None):
        T, K = ids.shape
        out = torch.zeros(T, y_pairs.shape[1], dtype=y_pairs.dtype)
        for t in range(T):
            ks = sorted(range(K), key=lambda k: (order[int(ids[t, k])] if order is not None else int(ids[t, k]), k))
            for k in ks:
                out[t] += y_pairs[t * K + k] * scores[t, k]
        return out if residual is None else residual + out


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        H, E, K, I, T = 64, 8, 3, 32, 12
        L = make_layer(H, E, K, I, torch.float32, T, seed=3)
        ctx = OracleBackedContext(L, K)
        ep = ExpertParallelMoE(ctx, E, K, H)
        ep.register_local_experts(0, L.experts)
        assert sorted(ctx.experts) == list(expert_range(E, world, rank))
        sl = split_tokens(T, world, rank)
        out = ep.forward(0, L.x[sl.start:sl.stop].contiguous())
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_ranks_reproduce_single_process_oracle():
    world, port = 2, _free_port()
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    procs = [ctxm.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=100) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    H, E, K, I, T = 64, 8, 3, 32, 12
    L = make_layer(H, E, K, I, torch.float32, T, seed=3)
    ids, scores, _ = O.route(L.x, L.gate_w, K)
    want = O.moe_engine(L.x, ids, scores, L.experts, order=list(range(E)))
    out = torch.cat([got[0], got[1]])
    assert torch.equal(out, want)      # fp32 on both sides, same operations in the same order


def test_partition_helpers():
    assert list(expert_range(128, 8, 3)) == list(range(48, 64))
    assert owner_of(47, 128, 8) == 2 and owner_of(48, 128, 8) == 3
    assert list(split_tokens(256, 8, 7)) == list(range(224, 256))
    with pytest.raises(ValueError):
        expert_range(10, 4, 0)
    with pytest.raises(ValueError):
        split_tokens(10, 4, 0)
