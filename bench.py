#!/usr/bin/env python
"""Benchmark of the MoE block forward (router -> permute -> grouped SwiGLU FFN -> combine).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Workload `mixtral_bf16` (default): one Mixtral-8x7B-shaped MoE layer (hidden 4096, 8 experts,
top-2, intermediate 14336, bf16, random-init weights ~N(0,0.02), activations ~N(0,1)); one step =
one forward of the layer for each speculative-verify batch T in {1,4,8,16,64} (93 tokens).
Other workloads: mixtral_int4, qwen3_bf16, qwen3_int4 (T in {1..256}), and the expert-parallel ones.

Prints ONE JSON line.
  value          tokens/s with inputs resident in HBM.  The timed region is `timed_blocks` blocks of exactly
                 --steps steps each, as many blocks as it takes to run for about a second (so that clock
                 samples fall inside it); ms_per_step is the mean over all of them.
  e2e            the same through the public runner API with pinned host buffers (H2D + D2H inside the region)
  roofline       the dominant kernel's algorithmic bytes over its CUDA-event duration against the measured HBM peak
  cpu_baseline   the reference algorithm (oracle port, torch CPU) on this box's host cores
  gpu_eager_baseline  the reference algorithm as eager PyTorch on this same GPU (the like-for-like "before")
  engine_path    the drop-in call sequence of the reference's engine (route_experts -> placement -> forward_moe)
  routing        how many tokens' ordered expert ids differ between the fused router and torch's own router on
                 this GPU, and the throughput of the exact-logits mode that never differs
  other_workloads   compact records of the int4 and Qwen3-shaped workloads measured in the same run (N = 1)
  ep             (N > 1) the expert-parallel Qwen3-shaped layer and the 48-layer stack over the N GPUs
With N > 1 (torchrun) `value` is N independent replicas of the default layer (weak scaling; its 8 experts
fit one GPU, so there is no data-path collective); the sharded path is what `ep` reports.
"""
from __future__ import annotations

import argparse
import json
import math
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
    "mixtral_bf16": (1.0023, "ncu capture at T=16: 1.879 GB read + 4.2 MB written against 1.879 GB algorithmic, scaled to the mean launch"),
    "mixtral_int4": (1.0082, "ncu capture at T=16: 484.8 MB read + 3.8 MB written against 484.6 MB algorithmic, scaled to the mean launch"),
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


def shared_config(workload: str, world: int) -> dict:
    """The workload description both arms print (same keys, same values)."""
    from on_device_sd_b200.synth import CONFIGS
    cfg_name, wmode, batches = WORKLOADS[workload]
    H, E, K, I, _ = CONFIGS[cfg_name]
    return {"workload": workload, "layer": cfg_name, "hidden": H, "experts": E, "top_k": K, "intermediate": I,
            "token_batches": list(batches), "weights": wmode,
            "parallelism": "single GPU" if world == 1 else f"{world} independent replicas",
            "l2": ("expert weights of one step (0.7-2.8 GB for the Mixtral shape) exceed the 126 MB L2, no flush needed" if cfg_name == "mixtral"
                   else "the batches of one step together touch > 1 GB of expert weights, more than the 126 MB L2; no flush")}


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
        "config": shared_config(workload, int(os.environ.get("WORLD_SIZE", "1"))),
        "note": "reference algorithm (oracle port of demo/src/model/qwen3_runner.py:269-385) on host cores",
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "setup_s": round(gen_s, 1),
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# one single-GPU workload
# ---------------------------------------------------------------------------------------------------
class Workload:
    """A layer of one workload on this rank's GPU, its runner and the sweep inputs."""

    def __init__(self, workload, dev, seed, kind, no_graph):
        from on_device_sd_b200 import B200MoERunner, MoEShape, W_DENSE, W_INT4_G128
        from on_device_sd_b200.quant import quantize_expert
        from on_device_sd_b200.synth import CONFIGS, make_named
        self.name = workload
        self.cfg_name, self.wmode, self.batches = WORKLOADS[workload]
        self.H, self.E, self.K, self.I, self.dtype = CONFIGS[self.cfg_name]
        self.int4 = self.wmode == "int4"
        self.kind, self.no_graph, self.dev = kind, no_graph, dev
        self.L = make_named(self.cfg_name, 1, seed=seed, device=dev, gen_device="cuda")
        shape = MoEShape(self.H, self.E, self.K, self.I, "bfloat16")
        self.runner = B200MoERunner(shape, device=dev, max_tokens=max(self.batches), weight_mode=W_INT4_G128 if self.int4 else W_DENSE,
                                    ffn_kind=kind, graph_blocks=not no_graph)
        self.runner.load_gate(0, self.L.gate_w)
        if self.int4:
            self.runner.register_experts(0, {e: quantize_expert(p) for e, p in self.L.experts.items()})
        else:
            self.runner.register_experts(0, self.L.experts)
        g = torch.Generator(device=dev).manual_seed(1000 + seed)
        self.xs = {T: torch.randn(T, self.H, device=dev, generator=g).to(self.dtype) for T in self.batches}
        self.outs = {T: torch.empty_like(self.xs[T]) for T in self.batches}
        self.ctx = self.runner.ctx
        self.n_active = {}
        for T in self.batches:
            _, ids, _ = self.ctx.forward_fused(0, self.xs[T], return_routing=True)
            self.n_active[T] = int(ids.unique().numel())
        self.ctx.status()

    def step_eager(self):
        for T in self.batches:
            self.ctx.forward_fused(0, self.xs[T], out=self.outs[T], ffn_kind=self.kind)

    def capture(self, fn):
        """`fn` as a CUDA graph (the calls enqueue kernels only, so they capture as they are)."""
        if self.no_graph:
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


def timed_blocks(step, steps, warmup, min_seconds, world, sampler=None):
    """W warm-up steps, then B blocks of exactly `steps` steps, B chosen from the warm-up so that the region
    lasts about `min_seconds`; device events at the block boundaries; barrier + synchronize on both sides;
    max over ranks.  Returns (total ms, blocks, per-block ms list)."""
    import torch.distributed as dist
    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(3):
        step()
    b.record(); torch.cuda.synchronize()
    est = max(a.elapsed_time(b) / 3, 1e-3)
    blocks = max(1, min(2000, math.ceil(min_seconds * 1e3 / (est * steps))))
    if world > 1:
        t = torch.tensor([blocks], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        blocks = int(t.item())
        dist.barrier()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    if sampler is not None:
        sampler.mark_begin = time.time()
    evs[0].record()
    for blk in range(blocks):
        for _ in range(steps):
            step()
        evs[blk + 1].record()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.mark_end = time.time()
    if world > 1:
        dist.barrier()
    per_block = [evs[i].elapsed_time(evs[i + 1]) for i in range(blocks)]
    total = evs[0].elapsed_time(evs[blocks])
    if world > 1:
        t = torch.tensor([total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total = float(t.item())
    return total, blocks, per_block


def kernel_profile(w: Workload, steps: int):
    """Per-kernel CUDA-event durations: the same steps again with every launch bracketed by events."""
    w.ctx.profile(True)
    for _ in range(steps):
        w.step_eager()
    torch.cuda.synchronize()
    w.ctx.profile(False)
    return w.ctx.profile_read()


def per_batch_table(w: Workload, peak: float):
    per_T = {}
    for T in w.batches:   # short individual timings, reported for context only
        one = lambda T=T: w.ctx.forward_fused(0, w.xs[T], out=w.outs[T], ffn_kind=w.kind)
        gT = w.capture(one)
        runT = gT.replay if gT is not None else one
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            runT()
        a.record()
        for _ in range(20):
            runT()
        b.record(); torch.cuda.synchronize()
        us = a.elapsed_time(b) / 20 * 1e3
        lb = algorithmic_bytes(w.H, w.E, w.I, T, w.n_active[T], w.int4)[0]
        w.ctx.profile(True)
        for _ in range(10):
            w.ctx.forward_fused(0, w.xs[T], out=w.outs[T], ffn_kind=w.kind)
        torch.cuda.synchronize()
        w.ctx.profile(False)
        kp = {k: round(v[0] / max(v[1], 1) * 1e3, 1) for k, v in w.ctx.profile_read().items() if v[1]}
        per_T[str(T)] = {"us": round(us, 1), "tokens_per_s": round(T / us * 1e6), "experts_hit": w.n_active[T],
                         "layer_gbs": round(lb / us / 1e3, 1), "frac_of_peak": round(lb / us / 1e3 / peak, 3), "kernel_us": kp}
    return per_T


def roofline_record(w: Workload, prof, ms_per_step, peak, peak_kind):
    """Roofline of the dominant kernel (gate/up weight streaming): bytes per launch / mean launch time."""
    # a batch that ran as the one-launch block has no gate/up launch of its own: every batch of a sweep gives
    # exactly one launch of either kind, and the one-launch block takes the smallest batches
    tb_n, gu_n0 = prof.get("token_block", (0.0, 0))[1], prof["ffn_gate_up"][1]
    n_tok = round(len(w.batches) * tb_n / (tb_n + gu_n0)) if (tb_n + gu_n0) else 0
    gu_batches = sorted(w.batches)[n_tok:] or list(w.batches)
    gu_bytes = sum(algorithmic_bytes(w.H, w.E, w.I, T, w.n_active[T], w.int4)[1] for T in gu_batches) / len(gu_batches)
    layer_bytes = sum(algorithmic_bytes(w.H, w.E, w.I, T, w.n_active[T], w.int4)[0] for T in w.batches)
    gu_ms, gu_n = prof["ffn_gate_up"]
    achieved = gu_bytes / (gu_ms / max(gu_n, 1) * 1e-3) / 1e9 if gu_ms > 0 else None
    total_kernel_ms = sum(v[0] for v in prof.values())
    ratio = NCU_TRAFFIC_RATIO.get(w.name)
    return {"bound": "hbm", "kernel": "ffn_gate_up (expert gate_proj/up_proj streaming + SwiGLU)",
            "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": (achieved / peak) if achieved else None,
            "peak_kind": f"{peak_kind} copy bandwidth", "traffic": (gu_bytes * ratio[0]) if ratio else None,
            "traffic_source": ratio[1] if ratio else None,
            "algorithmic_bytes_per_launch": gu_bytes, "mean_launch_us": gu_ms / max(gu_n, 1) * 1e3,
            "timing": "CUDA events around every launch, separate pass of the same steps right after the timed region",
            "layer": {"algorithmic_bytes_per_step": layer_bytes, "achieved_gbs": layer_bytes / (ms_per_step * 1e-3) / 1e9,
                      "frac": layer_bytes / (ms_per_step * 1e-3) / 1e9 / peak},
            "kernel_share": {k: (v[0] / total_kernel_ms if total_kernel_ms else None) for k, v in prof.items() if v[1]},
            "kernel_mean_us": {k: (v[0] / v[1] * 1e3) for k, v in prof.items() if v[1]}}


def eager_gpu_baseline(w: Workload, budget_s=2.0):
    """The reference's path on this GPU: F.linear -> topk -> softmax (moe_layer.py:44-54), then the per-expert
    loop of _execute_moe_with_placement (qwen3_runner.py:269-385), as eager PyTorch on CUDA tensors."""
    from oracle import moe_oracle as O
    if w.int4:
        return None
    experts = w.L.experts
    def sweep():
        for T in w.batches:
            ids, scores, _ = O.route(w.xs[T], w.L.gate_w, w.K, tie="torch", logits="linear")
            O.moe_engine(w.xs[T], ids, scores, experts)
    with torch.inference_mode():
        sweep(); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time(); n = 0
        a.record()
        while n < 3 or (time.time() - t0 < budget_s and n < 50):
            sweep(); n += 1
        b.record(); torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    return {"value": sum(w.batches) * n / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms / n, "sweeps": n,
            "what": "the reference algorithm (oracle restatement of moe_layer.py:44-54 + qwen3_runner.py:269-385) as eager PyTorch on this GPU, inputs resident, CUDA events"}


def engine_path_record(w: Workload, steps: int):
    """The drop-in sequence the reference's engine runs per layer (cb_executor.py:427-448): route_experts ->
    ExpertPlacement -> forward_moe, with the host round trip that building the activated-expert set implies."""
    from on_device_sd_b200 import AttentionOutput, ExpertPlacement
    names = ("gate_proj", "up_proj", "down_proj", "gate_proj_scales", "up_proj_scales", "down_proj_scales")
    params = {e: {k: v for k, v in zip(names, t) if v is not None} for (l, e), t in w.runner.ctx._experts.items() if l == 0}
    def sweep():
        for T in w.batches:
            x = w.xs[T]
            r = w.runner.route_experts(0, x)
            pl = ExpertPlacement(gpu_expert_params=params, cpu_expert_params={}, routing_result=r)
            w.runner.forward_moe(0, AttentionOutput(x, x, x), pl)
    for _ in range(3):
        sweep()
    torch.cuda.synchronize()
    n = max(5, min(steps, 50))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    a.record()
    for _ in range(n):
        sweep()
    b.record(); torch.cuda.synchronize()
    wall = time.time() - t0
    ms = a.elapsed_time(b)
    return {"value": sum(w.batches) * n / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms / n, "host_wall_ms_per_step": wall / n * 1e3,
            "us_per_layer_call": ms / n / len(w.batches) * 1e3,
            "what": "route_experts -> ExpertPlacement -> forward_moe per batch (eager launches, one event wait per layer for the activated-expert set)"}


def routing_record(w: Workload, steps: int):
    """Fused router against torch's own router on this GPU for the sweep's tokens, and the exact-logits mode."""
    import torch.nn.functional as F
    differ = sets = total = 0
    for T in w.batches:
        ids, _ = w.ctx.route(0, w.xs[T])
        t_ids = torch.topk(F.linear(w.xs[T], w.L.gate_w), w.K, dim=-1).indices
        differ += int((t_ids != ids).any(-1).sum()); total += T
        sets += int((t_ids.sort(-1).values != ids.sort(-1).values).any(-1).sum())
    def sweep():
        for T in w.batches:
            logits = F.linear(w.xs[T], w.L.gate_w)
            ids, scores = w.ctx.route(0, None, logits=logits)
            w.ctx.forward(0, w.xs[T], ids, scores, ffn_kind=w.kind)
    g = w.capture(sweep)
    run = g.replay if g is not None else sweep
    for _ in range(3):
        run()
    n = max(5, min(steps, 100))
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        run()
    b.record(); torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    return {"mode": "fused router: logits are the correctly rounded dot products (bit-exact to that definition)",
            "tokens": total, "tokens_differing_from_torch": differ, "token_sets_differing_from_torch": sets,
            "exact_logits_mode": {"tokens_differing_from_torch": 0, "value": sum(w.batches) * n / (ms * 1e-3), "unit": UNIT,
                                  "what": "torch F.linear logits -> b200moe_route_from_logits -> b200moe_forward; ordered ids equal torch.topk's on this GPU by construction (asserted in the GPU tests)"}}


def compact_record(args, name, dev, peak, peak_kind):
    """One of the other single-GPU workloads, measured in the same run: throughput, gate/up roofline, layer fraction per batch."""
    w = Workload(name, dev, 0, 0, args.no_graph)
    graph = w.capture(w.step_eager)
    step = graph.replay if graph is not None else w.step_eager
    total, blocks, _ = timed_blocks(step, args.steps, args.warmup, 0.3, 1)
    ms_per_step = total / (blocks * args.steps)
    prof = kernel_profile(w, min(args.steps, 10))
    roof = roofline_record(w, prof, ms_per_step, peak, peak_kind)
    per_T = per_batch_table(w, peak)
    w.ctx.status()
    rec = {"value": sum(w.batches) / (ms_per_step * 1e-3), "unit": UNIT, "ms_per_step": ms_per_step, "steps": blocks * args.steps,
           "token_batches": list(w.batches), "roofline_frac_gate_up": roof["frac"], "gate_up_gbs": roof["achieved"], "layer_frac": roof["layer"]["frac"],
           "layer_frac_per_T": {T: v["frac_of_peak"] for T, v in per_T.items()}, "layer_us_per_T": {T: v["us"] for T, v in per_T.items()},
           "kernel_mean_us": {k: round(v, 1) for k, v in roof["kernel_mean_us"].items()}}
    del w, graph
    torch.cuda.empty_cache()
    return rec


def build_stack(dev, n_layers, int4, world, rank, max_tokens):
    """Qwen3-shaped layers with this rank's shard of the experts (all of them when world == 1); gates replicated."""
    from on_device_sd_b200 import MoEContext, W_DENSE, W_INT4_G128
    from on_device_sd_b200.ep import expert_range
    from on_device_sd_b200.quant import quantize_expert
    from on_device_sd_b200.synth import CONFIGS, zipf_bias
    H, E, K, I, dtype = CONFIGS["qwen3"]
    ctx = MoEContext(H, E, K, I, dtype, num_layers=n_layers, max_tokens=max_tokens, weight_mode=W_INT4_G128 if int4 else W_DENSE, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)                      # same gates on every rank
    keep = []
    for layer in range(n_layers):
        bias = zipf_bias(E, 1.1, seed=layer).to(dev) if n_layers > 1 else None
        ctx.set_gate(layer, (torch.randn(E, H, device=dev, generator=g) * 0.02).to(dtype), bias)
        for e in expert_range(E, world, rank):
            ge = torch.Generator(device=dev).manual_seed(1_000_000 + layer * 1000 + e)     # an expert's weights do not depend on who holds it
            p = {"gate_proj": (torch.randn(I, H, device=dev, generator=ge) * 0.02).to(dtype),
                 "up_proj": (torch.randn(I, H, device=dev, generator=ge) * 0.02).to(dtype),
                 "down_proj": (torch.randn(H, I, device=dev, generator=ge) * 0.02).to(dtype)}
            p = quantize_expert(p) if int4 else p
            keep.append(p)
            ctx.set_expert(layer, e, p)
    return ctx, keep


def stack_record(args, dev, n_layers=48):
    """48 stacked Qwen3-shaped int4 blocks on ONE GPU (attention = identity, Zipf(1.1) gate bias), T = 160 and 288."""
    from on_device_sd_b200.stack import MoEStack
    ctx, keep = build_stack(dev, n_layers, True, 1, 0, 288)
    model = MoEStack(ctx, n_layers)
    g = torch.Generator(device=dev).manual_seed(5)
    out = {}
    for T in (160, 288):
        x = torch.randn(T, 2048, device=dev, generator=g).bfloat16()
        for _ in range(2):
            model.forward(x)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            model.forward(x)
        b.record(); torch.cuda.synchronize()
        out[str(T)] = {"ms_per_stack_forward": round(a.elapsed_time(b) / 5, 3), "tokens_per_s": round(T / (a.elapsed_time(b) / 5 * 1e-3))}
    ctx.status()
    del model, ctx, keep
    torch.cuda.empty_cache()
    return {"layers": n_layers, "weights": "int4 g128", "gate_bias": "zipf s=1.1 over a seeded permutation", "launch": "eager", "per_T": out,
            "ms_per_step_T160_plus_T288": round(sum(v["ms_per_stack_forward"] for v in out.values()), 3)}


def ep_record(args, dev, world, rank):
    """The sharded path over the N GPUs of this run: the Qwen3-shaped layer (bf16 and int4) expert-parallel against
    the same layer on rank 0's GPU alone, and the 48-layer int4 stack.  Device events, max over ranks."""
    import torch.distributed as dist
    from on_device_sd_b200.ep import ExpertParallelMoE
    from on_device_sd_b200.stack import MoEStack
    from on_device_sd_b200.synth import CONFIGS
    H, E, K, I, dtype = CONFIGS["qwen3"]
    batches = tuple(T for T in (16, 64, 256) if T % world == 0)
    rec = {"data_plane": "peer stores over NVLink issued by the library's own dispatch / return kernels (CUDA IPC mappings); "
                         "torch.distributed (NCCL) carries the 64-byte buffer handles, barriers and the timing reductions only",
           "experts_per_gpu": E // world, "token_split": "contiguous, T/N per rank"}
    g = torch.Generator(device=dev).manual_seed(77)
    xs = {T: torch.randn(T, H, device=dev, generator=g).to(dtype) for T in batches}

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record(); torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / reps * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for wname, int4 in (("qwen3_bf16_ep", False), ("qwen3_int4_ep", True)):
        ctx, keep = build_stack(dev, 1, int4, world, rank, 256)
        ep = ExpertParallelMoE(ctx, E, K, H, max_local_tokens=256 // world)
        alone = alone_keep = None
        if rank == 0:
            alone, alone_keep = build_stack(dev, 1, int4, 1, 0, 256)
        per_T = {}
        for T in batches:
            xl = xs[T][rank * (T // world):(rank + 1) * (T // world)].contiguous()
            us = timed(lambda: ep.forward(0, xl), 30)
            out = ep.forward(0, xl)
            gathered = [torch.empty_like(out) for _ in range(world)] if rank == 0 else None
            dist.gather(out, gathered, dst=0)
            entry = {"us": round(us, 1), "tokens_per_s": round(T / us * 1e6)}
            if rank == 0:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                for _ in range(3):
                    alone.forward_fused(0, xs[T])
                a.record()
                for _ in range(30):
                    alone.forward_fused(0, xs[T])
                b.record(); torch.cuda.synchronize()
                us1 = a.elapsed_time(b) / 30 * 1e3
                want, ids, _ = alone.forward_fused(0, xs[T], return_routing=True)
                load = torch.bincount(ids.flatten() // (E // world), minlength=world).float()
                entry.update({"us_rank0_alone": round(us1, 1), "speedup": round(us1 / us, 2), "bit_identical_to_1gpu": bool(torch.equal(torch.cat(gathered), want)),
                              "max_over_mean_gpu_load": round(float(load.max() / load.mean()), 2)})
            dist.barrier()
            per_T[str(T)] = entry
        ctx.status()
        rec[wname] = {"per_T": per_T, "launch": "eager: one library call per layer enqueues router, dispatch, permute, expert kernels, return, combine"}
        ep.close()
        del ctx, keep, ep, alone, alone_keep
        torch.cuda.empty_cache()

    # 48-layer int4 stack, verify batches of 32 sequences x (k+1) tokens, Zipf(1.1) gate bias
    stack_T = tuple(T for T in (160, 288) if T % world == 0)
    ctx, keep = build_stack(dev, 48, True, world, rank, 288)
    ep = ExpertParallelMoE(ctx, E, K, H, max_local_tokens=288 // world)
    model = MoEStack(ctx, 48, ep)
    per_T = {}
    for T in stack_T:
        x = torch.randn(T, H, device=dev, generator=torch.Generator(device=dev).manual_seed(T)).to(dtype)
        xl = x[rank * (T // world):(rank + 1) * (T // world)].contiguous()
        us = timed(lambda: model.forward(xl), 5)
        per_T[str(T)] = {"ms_per_stack_forward": round(us / 1e3, 3), "tokens_per_s": round(T / us * 1e6)}
    ctx.status()
    rec["qwen3_int4_stack"] = {"layers": 48, "per_T": per_T, "ms_per_step_T160_plus_T288": round(sum(v["ms_per_stack_forward"] for v in per_T.values()), 3),
                               "gate_bias": "zipf s=1.1 over a seeded permutation", "launch": "eager"}
    ep.close()
    del model, ep, ctx, keep
    torch.cuda.empty_cache()
    return rec


def run_ours(args, workload):
    import torch.distributed as dist
    from on_device_sd_b200 import FFN_AUTO, FFN_GEMV, FFN_MMA

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")     # plain rings for the few control collectives: no buffer stays bound to a multicast object
        dist.init_process_group("nccl", device_id=dev)

    kind = {"auto": FFN_AUTO, "gemv": FFN_GEMV, "mma": FFN_MMA}[args.ffn_kind]
    w = Workload(workload, dev, rank, kind, args.no_graph)
    batches, H, dtype = w.batches, w.H, w.dtype
    ctx, runner = w.ctx, w.runner
    graph = w.capture(w.step_eager)
    step = graph.replay if graph is not None else w.step_eager
    l_before = ctx.launches
    w.step_eager(); torch.cuda.synchronize()
    launches_per_step = ctx.launches - l_before

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    total_ms, blocks, per_block = timed_blocks(step, args.steps, args.warmup, 0.0 if args.quick else args.min_seconds, world, sampler)
    n_steps = blocks * args.steps
    ms_per_step = total_ms / n_steps
    tokens_per_step = sum(batches)
    value = world * tokens_per_step / (ms_per_step * 1e-3)
    launches = launches_per_step * n_steps

    if args.quick:
        if rank == 0:
            sampler.stop()
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "ms_per_step": ms_per_step,
                              "gpu_launches": launches, "config": {"workload": workload, "token_batches": list(batches)}, "quick": True}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    prof = kernel_profile(w, min(args.steps, 20))

    # end to end through the public runner API: pinned host x -> device, moe_block, result -> pinned host
    hx = {T: w.xs[T].cpu().pin_memory() for T in batches}
    hy = {T: torch.empty(T, H, dtype=dtype).pin_memory() for T in batches}
    dx = {T: torch.empty_like(w.xs[T]) for T in batches}
    def e2e_step():
        for T in batches:
            dx[T].copy_(hx[T], non_blocking=True)
            y = runner.moe_block(0, dx[T])
            hy[T].copy_(y, non_blocking=True)
        torch.cuda.synchronize()
    e2e_total, e2e_blocks, _ = timed_blocks(e2e_step, args.steps, 3, min(args.min_seconds, 0.5), world)
    e2e_value = world * tokens_per_step * e2e_blocks * args.steps / (e2e_total * 1e-3)
    clocks = sampler.stop() if rank == 0 else None
    ctx.status()

    ep = None
    if world > 1 and workload == "mixtral_bf16" and not args.no_ep:
        try:
            ep = ep_record(args, dev, world, rank)
        except Exception as exc:  # noqa: BLE001
            ep = {"error": f"{type(exc).__name__}: {exc}"}

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak_gbs()
    roofline = roofline_record(w, prof, ms_per_step, peak, peak_kind)

    extras = {}
    def leg(name, fn):
        try:
            extras[name] = fn()
        except Exception as exc:  # noqa: BLE001
            extras[name] = {"error": f"{type(exc).__name__}: {exc}"}
    per_T = per_batch_table(w, peak)
    leg("routing", lambda: routing_record(w, args.steps))
    leg("engine_path", lambda: engine_path_record(w, args.steps))
    leg("gpu_eager_baseline", lambda: eager_gpu_baseline(w))

    # CPU baseline: the reference algorithm on the host cores, bounded sample of the same workload
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        src = type("S", (), {"gate_w": w.L.gate_w, "experts": w.L.experts})
        layer_cpu, _ = make_cpu_layer(w.cfg_name, batches, w.int4, src=src)
        layer_cpu["xs"] = {T: w.xs[T].cpu() for T in batches}
        v, dt, n = cpu_reference_sweep(layer_cpu, batches, w.K, 10.0)
        cpu = {"value": v, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
               "sample": f"{n} sweep(s) of T in {list(batches)} on the full layer in {dt:.1f} s, torch CPU {torch.get_num_threads()} threads"}
        del layer_cpu

    others = None
    if world == 1 and workload == "mixtral_bf16" and not args.no_others:
        w.runner._graphs.clear()
        others = {}
        for name in ("mixtral_int4", "qwen3_bf16", "qwen3_int4"):
            try:
                others[name] = compact_record(args, name, dev, peak, peak_kind)
            except Exception as exc:  # noqa: BLE001
                others[name] = {"error": f"{type(exc).__name__}: {exc}"}
        try:
            others["qwen3_int4_stack"] = stack_record(args, dev)
        except Exception as exc:  # noqa: BLE001
            others["qwen3_int4_stack"] = {"error": f"{type(exc).__name__}: {exc}"}
        if "error" not in others["mixtral_int4"]:
            others["mixtral_int4"]["speedup_over_bf16_layer_per_T"] = {T: round(per_T[T]["us"] / others["mixtral_int4"]["layer_us_per_T"][T], 2) for T in per_T}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": shared_config(workload, world),
        "timed_blocks": blocks, "timed_region_s": total_ms * 1e-3,
        "ms_per_step_blocks": {"min": min(per_block) / args.steps, "median": statistics.median(per_block) / args.steps, "max": max(per_block) / args.steps},
        "run": {"ffn_kind": args.ffn_kind, "launch": "one CUDA graph replay per step" if not args.no_graph else "eager launches"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": tokens_per_step * H * 2, "d2h_bytes_per_step": tokens_per_step * H * 2,
                "api": "B200MoERunner(graph_blocks=%s).moe_block with pinned host buffers: H2D copy, block, D2H copy per batch, one synchronize per step" % (not args.no_graph)},
        "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
        "gpu_eager_baseline": extras.get("gpu_eager_baseline"), "engine_path": extras.get("engine_path"), "routing": extras.get("routing"),
        "per_T": per_T, "other_workloads": others, "ep": ep,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_ep(args, workload):
    """Expert-parallel layer: experts sharded over the ranks, token rows and results exchanged by the
    library's own kernels through peer memory (on_device_sd_b200/ep.py).  Eager launches; time = max over
    ranks, device events."""
    import torch.distributed as dist
    from on_device_sd_b200.ep import ExpertParallelMoE, split_tokens
    from on_device_sd_b200.stack import MoEStack
    from on_device_sd_b200.synth import CONFIGS
    cfg_name, wmode, batches = EP_WORKLOADS[workload]
    H, E, K, I, dtype = CONFIGS[cfg_name]
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")     # plain rings for the few control collectives: no buffer stays bound to a multicast object
    if "RANK" in os.environ:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))   # a stuck collective is aborted, not waited for
    else:   # plain `python bench.py`: a one-rank group, no collectives are issued
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29555", rank=0, world_size=1, device_id=dev)
    batches = tuple(T for T in batches if T % world == 0)
    int4 = wmode == "int4"
    stack = workload.endswith("_stack")
    n_layers = 48 if stack else 1
    ctx, keep = build_stack(dev, n_layers, int4, world, rank, max(batches))
    ep = ExpertParallelMoE(ctx, E, K, H, max_local_tokens=max(batches) // world)
    g = torch.Generator(device=dev).manual_seed(0)
    xs_full = {T: torch.randn(T, H, device=dev, generator=g).to(dtype) for T in batches}
    xl = {}
    for T in batches:
        sl = split_tokens(T, world, rank)
        xl[T] = xs_full[T][sl.start:sl.stop].contiguous()
    model = MoEStack(ctx, n_layers, ep)
    one = (lambda T: model.forward(xl[T])) if stack else (lambda T: ep.forward(0, xl[T]))
    launches_per_T = {}
    for T in batches:                                  # kernels of this library one forward enqueues
        l_ = ctx.launches
        one(T)
        launches_per_T[T] = ctx.launches - l_
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
        entry = {"us": round(float(tt.item()), 1), "tokens_per_s": round(T / float(tt.item()) * 1e6)}
        if not stack:
            dist.barrier()
            ctx.profile(True)
            for _ in range(10):
                one(T)
            torch.cuda.synchronize()
            ctx.profile(False)
            entry["kernel_us_rank0"] = {k: round(v[0] / max(v[1], 1) * 1e3, 1) for k, v in ctx.profile_read().items() if v[1]}
        per_T[str(T)] = entry
    ctx.status()
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": sum(batches) * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                          "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": workload, "layer": cfg_name, "hidden": H, "experts": E, "top_k": K, "intermediate": I,
                                     "token_batches": list(batches), "weights": wmode, "parallelism": f"ep{world}: {E // world} experts per GPU, "
                                     "peer-store dispatch and return over NVLink (the library's own kernels)", "launch": "eager", "layers": n_layers,
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
    ap.add_argument("--min-seconds", type=float, default=1.0, help="the timed region repeats blocks of --steps steps until it has run about this long")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="skip the compact records of the other single-GPU workloads")
    ap.add_argument("--no-ep", action="store_true", help="N > 1: skip the expert-parallel record")
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
