"""Run under torchrun on N GPUs of one node: the expert-parallel MoE block (peer-store dispatch / return
over CUDA IPC mappings) against the single-GPU result of the same library (bit-identical) and the
oracle (tolerance).  Prints EP_RANKS_CHECK PASS on rank 0."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main():
    from on_device_sd_b200 import MoEContext
    from on_device_sd_b200.ep import ExpertParallelMoE, split_tokens
    from on_device_sd_b200.synth import make_layer
    from oracle import moe_oracle as O
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    H, E, K, I, T = 512, 32, 8, 256, 16 * world
    L = make_layer(H, E, K, I, torch.bfloat16, T, seed=41)             # same seed on every rank
    ctx = MoEContext(H, E, K, I, torch.bfloat16, max_tokens=T)
    ctx.set_gate(0, L.gate_w.cuda())
    ep = ExpertParallelMoE(ctx, E, K, H, max_local_tokens=T // world)
    ep.register_local_experts(0, {e: {k: v.cuda() for k, v in p.items()} for e, p in L.experts.items()})
    sl = split_tokens(T, world, rank)
    x_local = L.x[sl.start:sl.stop].cuda().contiguous()
    dist.barrier()
    out = ep.forward(0, x_local)
    outs = [ep.forward(0, x_local) for _ in range(20)]                 # later calls reuse every buffer and the epoch counters
    torch.cuda.synchronize()
    status_ok = True
    try:
        ctx.status()
    except Exception as exc:  # noqa: BLE001
        print(f"rank {rank}: {exc}", flush=True)
        status_ok = False
    ok = status_ok and all(torch.equal(out, o) for o in outs)
    # single-GPU result of the same library on this rank's GPU
    full = MoEContext(H, E, K, I, torch.bfloat16, max_tokens=T)
    full.set_gate(0, L.gate_w.cuda())
    for e, p in L.experts.items():
        full.set_expert(0, e, {k: v.cuda() for k, v in p.items()})
    want = full.forward_fused(0, L.x.cuda())[sl.start:sl.stop]
    ok = ok and torch.equal(out, want)
    ids, scores, _ = O.route(L.x, L.gate_w, K)
    ref = O.moe_engine(L.x, ids, scores, L.experts, order=list(range(E)))[sl.start:sl.stop]
    mr = O.mean_rel(out.cpu(), ref)
    ok = ok and mr <= 1e-3
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"EP_RANKS_CHECK {'PASS' if int(flag) else 'FAIL'} world={world} mean_rel_vs_oracle={mr:.3g}", flush=True)
    ep.close()
    dist.destroy_process_group()
    sys.exit(0 if int(flag) else 1)


if __name__ == "__main__":
    main()
