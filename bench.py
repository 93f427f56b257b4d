#!/usr/bin/env python
"""Benchmark of the MoE block forward (router -> permute -> grouped SwiGLU FFN -> combine).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Workload `mixtral_bf16` (default): one Mixtral-8x7B-shaped MoE layer (hidden 4096, 8 experts,
top-2, intermediate 14336, bf16, random-init weights ~N(0,0.02), activations ~N(0,1)); one step =
one forward of the layer for each speculative-verify batch T in {1,4,8,16,64} (93 tokens).
Other workloads: mixtral_int4, qwen3_bf16, qwen3_int4 (T in {1..256}).

Prints ONE JSON line.  `value` = tokens/s with inputs resident in HBM; `e2e` = the same through
the public runner API with host buffers (H2D + D2H inside the timed region); `roofline` = the
dominant kernel's algorithmic bytes over its CUDA-event duration against the measured HBM peak;
`cpu_baseline` = the reference algorithm (oracle port, torch CPU) on this box's host cores.
With N > 1 (torchrun) every rank runs an independent replica of the layer on its own batch
(weak scaling; the layer's experts fit one GPU, so there is no data-path collective).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (synth config, weight mode, token batches)
    "mixtral_bf16": ("mixtral", "bf16", (1, 4, 8, 16, 64)),
    "mixtral_int4": ("mixtral", "int4", (1, 4, 8, 16, 64)),
    "qwen3_bf16": ("qwen3", "bf16", (1, 2, 4, 8, 16, 32, 64, 128, 256)),
    "qwen3_int4": ("qwen3", "int4", (1, 2, 4, 8, 16, 32, 64, 128, 256)),
}
EP_WORKLOADS = {
    # expert-parallel runs of the 128-expert layer: the batch is split across the ranks (strong scaling)
    "qwen3_bf16_ep": ("qwen3", "bf16", (8, 16, 32, 64, 128, 256)),
    "qwen3_int4_ep": ("qwen3", "int4", (8, 16, 32, 64, 128, 256)),
    # 48 stacked blocks, attention = identity, Zipf(1.1) gate bias; verify of k = 4 / 8 drafts for 32 sequences
    # (T = 32*(k+1) as the reference builds the verify batch, demo/src/execution/cb_executor.py:236-243)
    "qwen3_int4_stack": ("qwen3", "int4", (160, 288)),
    "qwen3_bf16_stack": ("qwen3", "bf16", (160, 288)),
}
# DRAM bytes (read + write) of the gate/up kernel over its algorithmic bytes, from one ncu capture per workload
# (a smaller case of the same kernel: one batch of 16 tokens, 8 experts hit); the kernel reads every weight byte
# once whatever the batch, so the ratio carries over to the mean launch of the sweep.
NCU_TRAFFIC_RATIO = {
    "mixtral_bf16": (1.0023, "ncu capture at T=16: 1.879 GB read + 4.2 MB written against 1.879 GB algorithmic (profiles/ffn_umma_mixtral_bf16_T16.md), scaled to the mean launch"),
    "mixtral_int4": (1.0082, "ncu capture at T=16: 484.8 MB read + 3.8 MB written against 484.6 MB algorithmic (profiles/ffn_int4_umma_mixtral_int4_T16.md), scaled to the mean launch"),
}
METRIC = "MoE-layer tokens/s at verify batch"
UNIT = "tokens/s"


def measured_peak_gbs() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs (read-only queries)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc, self.thread = index, [], None, None
        self.mark_begin = self.mark_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        def pump():
            for line in self.proc.stdout:
                self.samples.append((time.time(), line.strip()))
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = [(t, [c.strip() for c in l.split(",")]) for t, l in self.samples]
        inside = [r for t, r in rows if self.mark_begin and self.mark_begin <= t <= (self.mark_end or 1e300)]
        use, where = (inside, "timed region") if len(inside) >= 2 else ([r for _, r in rows], "whole run (timed region shorter than the sampling period)")
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in use:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": where}


def algorithmic_bytes(H, E, I, T, n_active, int4: bool):
    """Bytes an ideal implementation moves per layer forward: the distinct selected experts' weights,
    the gate weight, x in and y out (routing tables and the [T*K, I] intermediate stay on chip)."""
    per_expert = 3 * H * I // 2 + 3 * H * I // 128 * 2 if int4 else 3 * H * I * 2
    layer = n_active * per_expert + E * H * 2 + 2 * T * H * 2
    gate_up = n_active * per_expert * 2 // 3 + T * H * 2
    return layer, gate_up


def cpu_reference_sweep(layer_cpu, batches, K, repeats_budget_s: float, steps: int | None = None):
    """Times the oracle's engine path (route + per-expert FFN + accumulate, torch CPU, all host
    threads) on the same sweep.  Returns (tokens/s, seconds, sweeps)."""
    from oracle import moe_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    xs = layer_cpu["xs"]
    def sweep():
        for T in batches:
            x = xs[T]
            ids, scores, _ = O.route(x, layer_cpu["gate_w"], K, tie="torch", logits="linear")
            O.moe_engine(x, ids, scores, layer_cpu["experts"])
    with torch.inference_mode():
        sweep()  # warm-up
        t0 = time.time(); n = 0
        while True:
            sweep(); n += 1
            if steps is not None:
                if n >= steps:
                    break
            elif time.time() - t0 >= repeats_budget_s:
                break
        dt = time.time() - t0
    return sum(batches) * n / dt, dt, n


def make_cpu_layer(cfg_name, batches, int4: bool, src=None):
    """CPU copy of the layer for the baseline.  With int4 the CPU path runs on the dequantised weights."""
    from on_device_sd_b200.synth import CONFIGS, make_layer
    from oracle import moe_oracle as O
    H, E, K, I, dtype = CONFIGS[cfg_name]
    if src is not None:
        gate_w = src.gate_w.cpu(); experts = {e: {k: v.cpu() for k, v in p.items()} for e, p in src.experts.items()}
    else:
        L = make_layer(H, E, K, I, dtype, 1, seed=0)
        gate_w, experts = L.gate_w, L.experts
    if int4:
        experts = {e: {k: O.dequant_int4_g128(*O.quant_int4_g128(v)) for k, v in p.items()} for e, p in experts.items()}
    g = torch.Generator().manual_seed(1)
    xs = {T: torch.randn(T, H, generator=g).to(dtype) for T in batches}
    return {"gate_w": gate_w, "experts": experts, "xs": xs}, K


def run_reference(args, workload):
    cfg_name, wmode, batches = WORKLOADS[workload]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from on_device_sd_b200.synth import CONFIGS
    H, E, K, I, dtype = CONFIGS[cfg_name]
    t0 = time.time()
    layer_cpu, K = make_cpu_layer(cfg_name, batches, wmode == "int4")
    gen_s = time.time() - t0
    # one sweep is seconds of CPU work: run K sweeps unless that would pass ~150 s, then as many as fit
    from oracle import moe_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    t1 = time.time()
    with torch.inference_mode():
        for T in batches:
            ids, scores, _ = O.route(layer_cpu["xs"][T], layer_cpu["gate_w"], K, tie="torch", logits="linear")
            O.moe_engine(layer_cpu["xs"][T], ids, scores, layer_cpu["experts"])
    sweep_s = time.time() - t1
    steps = max(1, min(args.steps, int(150.0 / max(sweep_s, 1e-3))))
    val, dt, n = cpu_reference_sweep(layer_cpu, batches, K, 0, steps=steps)
    cores = os.cpu_count() or 1
    sample = f"{n} sweeps of T in {list(batches)} ({sum(batches)} tokens each), full layer, torch CPU {torch.get_num_threads()} threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": n, "warmup": max(args.warmup, 1),
        "ms_per_step": dt / n * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if dtype == torch.bfloat16 else str(dtype), "data": "synthetic",
        "config": {"workload": workload, "layer": cfg_name, "hidden": H, "experts": E, "top_k": K, "intermediate": I,
                   "token_batches": list(batches), "weights": wmode, "note": "reference algorithm (oracle port of demo/src/model/qwen3_runner.py:269-385) on host cores"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "setup_s": round(gen_s, 1),
    }
    print(json.dumps(line), flush=True)


def run_ours(args, workload):
    import torch.distributed as dist
    from on_device_sd_b200 import B200MoERunner, MoEShape, W_DENSE, W_INT4_G128
    from on_device_sd_b200.quant import quantize_expert
    from on_device_sd_b200.synth import CONFIGS, make_named

    cfg_name, wmode, batches = WORKLOADS[workload]
    H, E, K, I, dtype = CONFIGS[cfg_name]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    int4 = wmode == "int4"
    L = make_named(cfg_name, 1, seed=rank, device=dev, gen_device="cuda")
    shape = MoEShape(H, E, K, I, "bfloat16")
    from on_device_sd_b200 import FFN_AUTO, FFN_GEMV, FFN_MMA
    kind = {"auto": FFN_AUTO, "gemv": FFN_GEMV, "mma": FFN_MMA}[args.ffn_kind]
    runner = B200MoERunner(shape, device=dev, max_tokens=max(batches), weight_mode=W_INT4_G128 if int4 else W_DENSE, ffn_kind=kind,
                           graph_blocks=not args.no_graph)
    runner.load_gate(0, L.gate_w)
    dense_experts = L.experts
    if int4:
        runner.register_experts(0, {e: quantize_expert(p) for e, p in L.experts.items()})
    else:
        runner.register_experts(0, L.experts)
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    xs = {T: torch.randn(T, H, device=dev, generator=g).to(dtype) for T in batches}
    outs = {T: torch.empty_like(xs[T]) for T in batches}
    ctx = runner.ctx

    def step_eager():
        for T in batches:
            ctx.forward_fused(0, xs[T], out=outs[T], ffn_kind=kind)

    def capture(fn):
        """One step as a CUDA graph (the calls enqueue kernels only, so they capture as they are)."""
        if args.no_graph:
            return None
        try:
            fn(); torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            g.replay(); torch.cuda.synchronize()
            return g
        except Exception as exc:  # noqa: BLE001
            print(f"[bench] CUDA graph capture failed ({exc}); timing eager launches", file=sys.stderr)
            torch.cuda.synchronize()
            return None

    # distinct experts selected per batch (for the algorithmic byte count)
    n_active = {}
    for T in batches:
        _, ids, _ = ctx.forward_fused(0, xs[T], return_routing=True)
        n_active[T] = int(ids.unique().numel())
    ctx.status()

    graph = capture(step_eager)
    step = graph.replay if graph is not None else step_eager
    launches_per_step = None
    l_before = ctx.launches
    step_eager(); torch.cuda.synchronize()
    launches_per_step = ctx.launches - l_before
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    l0 = ctx.launches
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark_begin = time.time()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    sampler.mark_end = time.time()
    if world > 1:
        dist.barrier()
    ms = ev0.elapsed_time(ev1)
    launches = (ctx.launches - l0) if graph is None else launches_per_step * args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tokens_per_step = sum(batches)
    value = world * tokens_per_step * args.steps / (ms * 1e-3)

    if args.quick:
        if rank == 0:
            sampler.stop()
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "ms_per_step": ms / args.steps,
                              "gpu_launches": launches, "config": {"workload": workload, "token_batches": list(batches)}, "quick": True}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # per-kernel CUDA-event durations: the same steps again with every launch bracketed by events
    ctx.profile(True)
    for _ in range(args.steps):
        step_eager()
    torch.cuda.synchronize()
    ctx.profile(False)
    prof = ctx.profile_read()

    # end to end through the public runner API: pinned host x -> device, moe_block, result -> pinned host
    hx = {T: xs[T].cpu().pin_memory() for T in batches}
    hy = {T: torch.empty(T, H, dtype=dtype).pin_memory() for T in batches}
    dx = {T: torch.empty_like(xs[T]) for T in batches}
    def e2e_step():
        for T in batches:
            dx[T].copy_(hx[T], non_blocking=True)
            y = runner.moe_block(0, dx[T])
            hy[T].copy_(y, non_blocking=True)
        torch.cuda.synchronize()
    for _ in range(3):
        e2e_step()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * tokens_per_step * args.steps / (e2e_ms * 1e-3)
    clocks = sampler.stop() if rank == 0 else None
    ctx.status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # roofline of the dominant kernel (gate/up weight streaming): bytes per launch / mean launch time
    peak, peak_kind = measured_peak_gbs()
    gu_bytes = sum(algorithmic_bytes(H, E, I, T, n_active[T], int4)[1] for T in batches) / len(batches)
    layer_bytes = sum(algorithmic_bytes(H, E, I, T, n_active[T], int4)[0] for T in batches)
    gu_ms, gu_n = prof["ffn_gate_up"]
    achieved = gu_bytes / (gu_ms / max(gu_n, 1) * 1e-3) / 1e9 if gu_ms > 0 else None
    total_kernel_ms = sum(v[0] for v in prof.values())
    roofline = {"bound": "hbm", "kernel": "ffn_gate_up (expert gate_proj/up_proj streaming + SwiGLU)",
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": (achieved / peak) if achieved else None,
                "peak_kind": f"{peak_kind} copy bandwidth", "traffic": (gu_bytes * NCU_TRAFFIC_RATIO[workload][0]) if workload in NCU_TRAFFIC_RATIO else None,
                "traffic_source": NCU_TRAFFIC_RATIO[workload][1] if workload in NCU_TRAFFIC_RATIO else None,
                "algorithmic_bytes_per_launch": gu_bytes, "mean_launch_us": gu_ms / max(gu_n, 1) * 1e3,
                "timing": "CUDA events around every launch, separate pass of the same steps right after the timed region",
                "layer": {"algorithmic_bytes_per_step": layer_bytes, "achieved_gbs": layer_bytes * args.steps / (ms * 1e-3) / 1e9,
                          "frac": layer_bytes * args.steps / (ms * 1e-3) / 1e9 / peak},
                "kernel_share": {k: (v[0] / total_kernel_ms if total_kernel_ms else None) for k, v in prof.items()},
                "kernel_mean_us": {k: (v[0] / v[1] * 1e3 if v[1] else None) for k, v in prof.items()}}

    # CPU baseline: the reference algorithm on the host cores, bounded sample of the same workload
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        src = type("S", (), {"gate_w": L.gate_w, "experts": dense_experts})
        layer_cpu, _ = make_cpu_layer(cfg_name, batches, int4, src=src)
        layer_cpu["xs"] = {T: xs[T].cpu() for T in batches}
        v, dt, n = cpu_reference_sweep(layer_cpu, batches, K, 10.0)
        cpu = {"value": v, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
               "sample": f"{n} sweep(s) of T in {list(batches)} on the full layer in {dt:.1f} s, torch CPU {torch.get_num_threads()} threads"}

    per_T = {}
    for T in batches:   # short individual timings, reported for context only
        one = lambda T=T: ctx.forward_fused(0, xs[T], out=outs[T], ffn_kind=kind)
        gT = capture(one)
        runT = gT.replay if gT is not None else one
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            runT()
        b.record(); torch.cuda.synchronize()
        us = a.elapsed_time(b) / 20 * 1e3
        lb = algorithmic_bytes(H, E, I, T, n_active[T], int4)[0]
        ctx.profile(True)
        for _ in range(10):
            ctx.forward_fused(0, xs[T], out=outs[T], ffn_kind=kind)
        torch.cuda.synchronize()
        ctx.profile(False)
        kp = {k: round(v[0] / max(v[1], 1) * 1e3, 1) for k, v in ctx.profile_read().items()}
        per_T[str(T)] = {"us": round(us, 1), "tokens_per_s": round(T / us * 1e6), "experts_hit": n_active[T],
                         "layer_gbs": round(lb / us / 1e3, 1), "frac_of_peak": round(lb / us / 1e3 / peak, 3), "kernel_us": kp}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload, "layer": cfg_name, "hidden": H, "experts": E, "top_k": K, "intermediate": I,
                   "token_batches": list(batches), "weights": wmode, "ffn_kind": args.ffn_kind,
                   "launch": "one CUDA graph replay per step" if graph is not None else "eager launches", "parallelism": "single GPU" if world == 1 else f"{world} independent replicas",
                   "l2": "expert weights of one step (0.7-2.8 GB for mixtral) exceed the 126 MB L2, no flush needed" if cfg_name == "mixtral"
                         else "weights of the larger batches exceed L2; the smallest batches can be L2-resident"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": tokens_per_step * H * 2, "d2h_bytes_per_step": tokens_per_step * H * 2,
                "api": "B200MoERunner(graph_blocks=%s).moe_block with pinned host buffers: H2D copy, block, D2H copy per batch, one synchronize per step" % (not args.no_graph)},
        "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu, "per_T": per_T,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_ep(args, workload):
    """Expert-parallel layer: experts sharded over the ranks, token rows and results exchanged by the
    library's own kernels through peer memory (on_device_sd_b200/ep.py).  Eager launches; time = max over
    ranks, device events."""
    import torch.distributed as dist
    from on_device_sd_b200 import MoEContext, W_DENSE, W_INT4_G128
    from on_device_sd_b200.ep import ExpertParallelMoE, expert_range, split_tokens
    from on_device_sd_b200.quant import quantize_expert
    from on_device_sd_b200.synth import CONFIGS
    cfg_name, wmode, batches = EP_WORKLOADS[workload]
    H, E, K, I, dtype = CONFIGS[cfg_name]
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if "RANK" in os.environ:
        import datetime
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")     # plain rings for the few control collectives: no buffer stays bound to a multicast object
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))   # a stuck collective is aborted, not waited for
    else:   # plain `python bench.py`: a one-rank group, no collectives are issued
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29555", rank=0, world_size=1, device_id=dev)
    batches = tuple(T for T in batches if T % world == 0)
    int4 = wmode == "int4"
    stack = workload.endswith("_stack")
    n_layers = 48 if stack else 1
    ctx = MoEContext(H, E, K, I, dtype, num_layers=n_layers, max_tokens=max(batches), weight_mode=W_INT4_G128 if int4 else W_DENSE, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)                      # same gate and tokens on every rank
    ctx.set_gate(0, (torch.randn(E, H, device=dev, generator=g) * 0.02).to(dtype))
    xs_full = {T: torch.randn(T, H, device=dev, generator=g).to(dtype) for T in batches}
    ep = ExpertParallelMoE(ctx, E, K, H, max_local_tokens=max(batches) // world)
    gl = torch.Generator(device=dev).manual_seed(100 + rank)
    keep = []
    for layer in range(n_layers):
        if layer > 0:
            from on_device_sd_b200.synth import zipf_bias
            ctx.set_gate(layer, (torch.randn(E, H, device=dev, generator=g) * 0.02).to(dtype), None)
        for e in expert_range(E, world, rank):                          # only the local shard is ever materialised
            p = {"gate_proj": (torch.randn(I, H, device=dev, generator=gl) * 0.02).to(dtype),
                 "up_proj": (torch.randn(I, H, device=dev, generator=gl) * 0.02).to(dtype),
                 "down_proj": (torch.randn(H, I, device=dev, generator=gl) * 0.02).to(dtype)}
            p = quantize_expert(p) if int4 else p
            keep.append(p)
            ctx.set_expert(layer, e, p)
    if stack:
        from on_device_sd_b200.synth import zipf_bias
        for layer in range(n_layers):                                   # popularity skew: b_e = log p_e, p ~ rank^-1.1
            gw = ctx._gate[layer][0] if layer in ctx._gate else None
            ctx.set_gate(layer, gw, zipf_bias(E, 1.1, seed=layer).to(dev))
    xl = {}
    for T in batches:
        sl = split_tokens(T, world, rank)
        xl[T] = xs_full[T][sl.start:sl.stop].contiguous()
    from on_device_sd_b200.stack import MoEStack
    model = MoEStack(ctx, n_layers, ep)
    eager = (lambda T: model.forward(xl[T])) if stack else (lambda T: ep.forward(0, xl[T]))
    graphs = {}
    launches_per_T = {}
    for T in batches:                                  # kernels of this library one forward enqueues (a graph replay launches the same ones)
        l_ = ctx.launches
        eager(T)
        launches_per_T[T] = ctx.launches - l_
    one = (lambda T: graphs[T][0].replay()) if graphs else eager
    def step():
        for T in batches:
            one(T)
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record(); torch.cuda.synchronize(); dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    per_T = {}
    for T in batches:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(); dist.barrier()
        a.record()
        reps = 3 if stack else 20
        for _ in range(reps):
            one(T)
        b.record(); torch.cuda.synchronize()
        tt = torch.tensor([a.elapsed_time(b) / reps * 1e3], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        per_T[str(T)] = {"us": round(float(tt.item()), 1), "tokens_per_s": round(T / float(tt.item()) * 1e6)}
    ctx.status()
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": sum(batches) * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                          "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": workload, "layer": cfg_name, "hidden": H, "experts": E, "top_k": K, "intermediate": I,
                                     "token_batches": list(batches), "weights": wmode, "parallelism": f"ep{world}: {E // world} experts per GPU, "
                                     "peer-store dispatch and return over NVLink (the library's own kernels)", "launch": "one CUDA graph replay per batch" if graphs else "eager", "layers": n_layers,
                                     "gate_bias": "zipf s=1.1 over a seeded permutation" if stack else None},
                          "gpu_launches": args.steps * sum(launches_per_T.values()), "per_T": per_T}), flush=True)
    ep.close()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="mixtral_bf16", choices=sorted(WORKLOADS) + sorted(EP_WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batches", default=None, help="comma-separated token batches replacing the workload's sweep (profiling runs)")
    ap.add_argument("--ffn-kind", default="auto", choices=["auto", "gemv", "mma"], help="force one expert-FFN kernel family")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of CUDA graph replays")
    ap.add_argument("--quick", action="store_true", help="timed region only: no e2e, per-T or CPU-baseline legs (for ncu captures)")
    args = ap.parse_args()
    if args.workload in EP_WORKLOADS:
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference has no expert-parallel path (single GPU, demo/others.md:58-62)"}))
            return
        if args.batches:
            cfg, wm, _ = EP_WORKLOADS[args.workload]
            EP_WORKLOADS[args.workload] = (cfg, wm, tuple(int(b) for b in args.batches.split(",")))
        return run_ep(args, args.workload)
    if args.batches:
        cfg, wm, _ = WORKLOADS[args.workload]
        WORKLOADS[args.workload] = (cfg, wm, tuple(int(b) for b in args.batches.split(",")))
    if args.impl == "reference":
        run_reference(args, args.workload)
    else:
        run_ours(args, args.workload)


if __name__ == "__main__":
    main()
