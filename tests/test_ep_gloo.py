"""CPU, world_size 2 over gloo: the expert-parallel exchange protocol and its host plumbing.

`ExpertParallelMoE` (handle exchange through torch.distributed, barriers, sharding) is the product code
under test.  The context it drives is a stand-in that restates the library's exchange protocol over
POSIX shared memory instead of peer GPU memory - one receive region per (destination, source), dense
rows in pair order, a count and an epoch flag per source, return rows in pair order and an epoch flag
per owner, bounded waits - with the arithmetic taken from the oracle (test infrastructure).  The
result must equal the single-process oracle exactly.  On GPUs the same class drives libb200moe.so
(tests/test_gpu_ep.py, tests/ep_ranks_check.py)."""
import os
import socket
import time
from multiprocessing import shared_memory

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from on_device_sd_b200.ep import ExpertParallelMoE, exchange_handles, expert_range, owner_of, split_tokens
from on_device_sd_b200.synth import make_layer
from oracle import moe_oracle as O


class _Exchange:
    """Views into one rank's exchange buffer (same sections as the device buffer)."""

    def __init__(self, shm, G, cap, H):
        self.shm = shm
        n_hdr, n_meta, n_x = 3 * G * 8, G * cap * 2 * 4, G * cap * H * 4
        buf = shm.buf
        self.hdr = np.ndarray((3, G), dtype=np.int64, buffer=buf, offset=0)          # disp_flag, disp_count, ret_flag
        self.meta = np.ndarray((G, cap, 2), dtype=np.int32, buffer=buf, offset=n_hdr)
        self.x = np.ndarray((G, cap, H), dtype=np.float32, buffer=buf, offset=n_hdr + n_meta)
        self.ret = np.ndarray((cap, H), dtype=np.float32, buffer=buf, offset=n_hdr + n_meta + n_x)

    @staticmethod
    def size(G, cap, H):
        return 3 * G * 8 + G * cap * 2 * 4 + G * cap * H * 4 + cap * H * 4


class SharedMemoryContext:
    """Stand-in for MoEContext's expert-parallel methods on the CPU (fp32)."""

    def __init__(self, layer, K, wait_s=30.0):
        self.gate_w, self.K, self.H, self.E = layer.gate_w, K, layer.H, layer.E
        self.experts, self.epoch, self.wait_s = {}, 0, wait_s

    def set_expert(self, layer, e, params):
        self.experts[e] = params

    def ep_create(self, world, rank, max_local_tokens):
        self.G, self.me, self.cap, self.epr = world, rank, max_local_tokens * self.K, self.E // world
        self.own_shm = shared_memory.SharedMemory(create=True, size=_Exchange.size(world, self.cap, self.H))
        self.own_shm.buf[:] = bytes(len(self.own_shm.buf))
        self.peers = [None] * world
        self.peers[rank] = _Exchange(self.own_shm, world, self.cap, self.H)
        return self.own_shm.name.encode().ljust(64, b"\0")

    def ep_attach(self, handles):
        assert len(handles) == self.G and all(len(h) == 64 for h in handles)
        for r, h in enumerate(handles):
            if r != self.me:
                self.peers[r] = _Exchange(shared_memory.SharedMemory(name=h.rstrip(b"\0").decode()), self.G, self.cap, self.H)

    def _wait(self, row):
        t0 = time.time()
        while not bool((self.peers[self.me].hdr[row] >= self.epoch).all()):
            if time.time() - t0 > self.wait_s:
                raise TimeoutError("a peer never arrived")     # the device kernels set a status bit instead
            time.sleep(0.001)

    def ep_forward(self, layer, x_local, order=None, residual=None):
        T, K, me = x_local.shape[0], self.K, self.me
        assert T * K <= self.cap
        ids, scores, _ = O.route(x_local, self.gate_w, K)
        self.epoch += 1
        # dispatch: pair p -> owner d, dense rows in pair order in region [d][me]
        cnt = [0] * self.G
        for p, e in enumerate(ids.flatten().tolist()):
            d = e // self.epr
            self.peers[d].x[me, cnt[d]] = x_local[p // K].numpy()
            self.peers[d].meta[me, cnt[d]] = (e, p)
            cnt[d] += 1
        for d in range(self.G):
            self.peers[d].hdr[1, me] = cnt[d]
            self.peers[d].hdr[0, me] = self.epoch
        # experts: wait for every source, group the received rows by expert, return each output row to its source
        self._wait(0)
        own = self.peers[me]
        rows = [(int(own.meta[s, j, 0]), s, j, int(own.meta[s, j, 1])) for s in range(self.G) for j in range(int(own.hdr[1, s]))]
        for e in sorted(self.experts):
            mine = [r for r in rows if r[0] == e]
            if mine:
                y = O.expert_ffn(torch.from_numpy(np.stack([own.x[s, j] for _, s, j, _ in mine])), **self.experts[e])
                for (_, s, _, pair), yr in zip(mine, y):
                    self.peers[s].ret[pair] = yr.numpy()
        for s in range(self.G):
            self.peers[s].hdr[2, me] = self.epoch
        # combine: wait for every owner, accumulate in rank order
        self._wait(2)
        out = torch.zeros(T, self.H)
        for t in range(T):
            ks = sorted(range(K), key=lambda k: (order[int(ids[t, k])] if order is not None else int(ids[t, k]), k))
            for k in ks:
                out[t] += torch.from_numpy(own.ret[t * K + k].copy()) * scores[t, k]
        return out if residual is None else residual + out

    def ep_detach(self):
        own = self.own_shm
        self.peers = []
        for _ in range(2):
            try:
                own.close()
                break
            except BufferError:
                import gc
                gc.collect()
        if hasattr(self, "own_shm"):
            try:
                own.unlink()
            except FileNotFoundError:
                pass


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
        ctx = SharedMemoryContext(L, K)
        ep = ExpertParallelMoE(ctx, E, K, H, max_local_tokens=T // world)
        ep.register_local_experts(0, L.experts)
        assert sorted(ctx.experts) == list(expert_range(E, world, rank))
        sl = split_tokens(T, world, rank)
        x_local = L.x[sl.start:sl.stop].contiguous()
        out = ep.forward(0, x_local)
        out2 = ep.forward(0, x_local, residual=x_local)        # second call: same buffers, next epoch
        q.put((rank, out, out2))
        dist.barrier()
        ep.close()
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
    got = {r: (a, b) for r, a, b in (q.get(timeout=100) for _ in range(world))}
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    H, E, K, I, T = 64, 8, 3, 32, 12
    L = make_layer(H, E, K, I, torch.float32, T, seed=3)
    ids, scores, _ = O.route(L.x, L.gate_w, K)
    want = O.moe_engine(L.x, ids, scores, L.experts, order=list(range(E)))
    assert torch.equal(torch.cat([got[0][0], got[1][0]]), want)      # fp32 on both sides, same operations in the same order
    assert torch.equal(torch.cat([got[0][1], got[1][1]]), L.x + want)


def test_partition_helpers():
    assert list(expert_range(128, 8, 3)) == list(range(48, 64))
    assert owner_of(47, 128, 8) == 2 and owner_of(48, 128, 8) == 3
    assert list(split_tokens(256, 8, 7)) == list(range(224, 256))
    with pytest.raises(ValueError):
        expert_range(10, 4, 0)
    with pytest.raises(ValueError):
        split_tokens(10, 4, 0)
