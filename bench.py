#!/usr/bin/env python
"""Benchmark of the MoE layer hot path: tokens/s of one forward+backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

Prints ONE JSON line (rank 0).  ``value`` is device-timed throughput with inputs
resident in HBM; ``e2e`` is the same step through the host-buffer entry point
(H2D of x and dy, D2H of y and dx inside the timed region); ``roofline`` scores
the dominant kernel against the measured peaks; ``cpu_baseline`` is the
reference's own CPU code (or the C restatement of it) timed on a bounded sample.
For N > 1 launch under torchrun: one rank per GPU.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "moe_layer_fwd_bwd_tokens_per_sec"
# DRAM bytes (read + write) per launch from ncu captures, keyed by (workload, stage); see profiles/.
# c4 is too large to capture with many passes: its figures are those of c4q (a quarter of the tokens and of the
# experts, same rows per expert) times four -- every term of the traffic is proportional to the number of experts.
TRAFFIC = {
    ("c3", "wgrad_gemm"): 827.5e6, ("c3", "gateup_gemm"): 337.8e6, ("c3", "dhh_gemm"): 397.0e6,
    ("c3", "down_gemm"): 177.2e6, ("c3", "dxg_gemm"): 282.2e6,
    ("c4q", "wgrad_gemm"): 1413.9e6, ("c4q", "gateup_gemm"): 373.7e6, ("c4q", "dhh_gemm"): 344.1e6,
    ("c4q", "down_gemm"): 188.5e6, ("c4q", "dxg_gemm"): 339.5e6,
    ("c4", "wgrad_gemm"): 4 * 1413.9e6, ("c4", "gateup_gemm"): 4 * 373.7e6, ("c4", "dhh_gemm"): 4 * 344.1e6,
    ("c4", "down_gemm"): 4 * 188.5e6, ("c4", "dxg_gemm"): 4 * 339.5e6,
}
UNIT = "tokens/s"


def describe(w) -> str:
    return (f"{w.name}: {w.n_tokens} tokens, C={w.C}, H={w.H}, E={w.E}, top-{w.k}, "
            f"{'fwd+bwd' if w.backward else 'fwd only'}, {w.dtype}" + (", skewed router" if w.skew else ""))


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------- CPU arm
def cpu_reference_step(w, sample_tokens: int, threads: int = 1, iters: int = 1):
    """Forward+backward of the reference's CPU code on `sample_tokens` tokens of workload w
    (layer construction and parameter loading untimed).  Returns (seconds per iteration list, kind, cores)."""
    from mgpt_b200 import synth
    from oracle import oracle

    ws = w.scaled(sample_tokens)
    x, params, dy = synth.make_inputs(ws, seed=1234)
    d = oracle.Dims(ws.n_tokens, ws.C, ws.H, ws.E, ws.k, ws.alpha)
    if oracle.have_ref():
        which, kind, cores = "ref", "reference", 1      # the reference has no threads of its own
    else:
        which, kind, cores = "oracle", "port", threads
    secs = oracle.bench(d, x, params, dy if w.backward else None, which=which, iters=iters, threads=cores)
    return secs, kind, cores


def cpu_step_estimate_s(w, sample_tokens: int) -> float:
    """Rough seconds per forward+backward of the reference's CPU code: it walks every expert's weights and
    weight gradients once per step whatever the sample (~30 ns per weight element on one core) and does
    18 flop per (row, weight element of one expert) at a few GFLOP/s.  Used only to bound the run."""
    weights = 3.0 * w.E * w.C * w.H
    return 30e-9 * weights + 18.0 * sample_tokens * w.k * w.C * w.H / 4e9


def run_reference_arm(args, w):
    """--impl reference: the reference's CPU implementation of the path on bounded samples.

    Every CPU step has a fixed cost whatever the sample (it walks all experts' weights and weight gradients,
    2.2 GB each at the 64-expert configuration) plus a cost per token, so one small sample divided by its time
    understates the full configuration's throughput.  Two sample sizes are timed; the fixed and the per-token
    cost are fitted through the two means and ``value`` is the full configuration's tokens/s extrapolated from
    them (``ms_per_step`` likewise).  Both raw points are in ``sample``.  The run is held to about four minutes:
    when the requested steps would take longer, fewer are run and the line says how many."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    small = min(w.n_tokens, args.cpu_sample or 256)
    large = min(w.n_tokens, 4 * small)
    sizes = [small] if large == small else [small, large]
    per_step = sum(cpu_step_estimate_s(w, n) for n in sizes)
    allowed = max(2, int(240.0 / per_step))            # steps (warm-up included) per size
    warmup = min(args.warmup, max(1, allowed // 4))
    steps = max(1, min(args.steps, allowed - warmup))
    points, kind, cores = [], None, 1
    for n in sizes:
        secs, kind, cores = cpu_reference_step(w, n, threads=os.cpu_count() or 1, iters=warmup + steps)
        t = secs[warmup:]
        points.append((n, sum(t) / len(t)))
    if len(points) == 2 and points[1][1] > points[0][1]:
        (n0, t0), (n1, t1) = points
        per_token = (t1 - t0) / (n1 - n0)
        fixed = max(0.0, t0 - per_token * n0)
    else:                                              # one size (the workload is that small): no extrapolation
        per_token, fixed = points[0][1] / points[0][0], 0.0
    sec_full = fixed + per_token * w.n_tokens
    value = w.n_tokens / sec_full
    sample_txt = ("forward+backward of " + " and ".join(f"{n} tokens ({t:.2f} s/step, {n / t:.1f} tok/s)" for n, t in points)
                  + f" of {w.name} (same C,H,E,k); fitted {fixed:.2f} s fixed + {per_token * 1e3:.3f} ms per token -> "
                  f"{sec_full:.1f} s per step of all {w.n_tokens} tokens (value and ms_per_step are this extrapolation)")
    if steps != args.steps or warmup != args.warmup:
        sample_txt += f"; {steps} timed steps after {warmup} warm-up per size (of {args.steps}/{args.warmup} asked) to bound the run"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec_full * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": describe(w), "sample": sample_txt},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample_txt,
                         "points": [{"tokens": n, "s_per_step": round(t, 3)} for n, t in points],
                         "fixed_s": round(fixed, 3), "per_token_ms": round(per_token * 1e3, 4)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in out.strip().splitlines():
            f = [c.strip() for c in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- our arm
def stage_model(w):
    """Algorithmic work per launch of each stage: flops for the products, bytes for the rest."""
    N, C, H, E, k = w.n_tokens, w.C, w.H, w.E, w.k
    R, b = N * k, 2
    flops = {"gateup_gemm": 4.0 * R * C * H, "down_gemm": 2.0 * R * C * H, "dhh_gemm": 2.0 * R * C * H,
             "dxg_gemm": 4.0 * R * C * H, "wgrad_gemm": 6.0 * R * C * H}
    byts = {
        "router": N * C * b + C * E * 4 + N * k * 8 + N * E * 4,
        "dispatch": N * C * b + R * C * b + R * 4,
        "combine": R * C * b + N * k * 4 + N * C * b,
        "combine_bwd": N * C * b + R * C * b + R * C * b + N * k * 4,
        "router_bwd": R * C * b + N * C * b + N * C * b + N * E * 8 + C * E * 4,
    }
    return flops, byts


SEED = 1234


def load_synth_params(params, w, dev, global_index):
    """Weights of the workload from the seeded generator the oracle uses (mgpt_b200/synth.py: Philox keyed by
    seed and tensor id; N(0, 0.02), biases 0, the skewed workload's router bias; rounded to bf16 for bf16
    workloads), so a bench run can be re-checked against the CPU oracle afterwards.  global_index(i) maps this
    process's parameter i to the index in the full 2+6E list."""
    import torch

    from mgpt_b200 import synth
    for i, p in enumerate(params):
        a = synth.make_param(w, global_index(i), seed=SEED)
        p.copy_(torch.from_numpy(a).reshape(p.shape))


def host_tokens(w, rank):
    """Pinned host x and dy of this rank (seed + rank: rank 0's are the oracle's own inputs) plus output buffers."""
    import torch

    from mgpt_b200 import synth
    io = torch.bfloat16 if w.dtype == "bf16" else torch.float32
    x, dy = synth.make_tokens(w, seed=SEED + rank)
    x_host = torch.from_numpy(x).to(io).pin_memory()
    dy_host = torch.from_numpy(dy).to(io).pin_memory()
    return x_host, dy_host, torch.empty_like(x_host).pin_memory(), torch.empty_like(x_host).pin_memory()


def measure(args, w, world, rank, dev, step, step_host, host_checksum, stage_ms, set_profiling, barrier, N, io_bytes,
            graph_ok=False, steps=None, warmup=None, sample_clocks=True, pipe=None):
    """Warm-up, K timed steps (CUDA events, L2 flushed between steps, max over ranks), then the host-buffer path."""
    import torch
    import torch.distributed as dist

    from mgpt_b200 import launch_count

    steps = steps or args.steps
    warmup = max(warmup if warmup is not None else args.warmup, 3)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # > 126 MB L2
    sampler = ClockSampler(dev.index) if rank == 0 and sample_clocks else None   # samples every 100 ms from here on
    for _ in range(warmup):
        flush.zero_()
        step()
    set_profiling(True)
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    stage_sum = {}
    launch_count(reset=True)
    for s, e in ev:
        flush.zero_()                      # L2 flush between timed iterations, outside the events
        if world > 1:
            dist.barrier()                 # ranks enter each timed step together
        s.record()
        step()
        e.record()
        e.synchronize()
        for name, ms in stage_ms().items():
            stage_sum[name] = stage_sum.get(name, 0.0) + ms
    launches = launch_count()
    barrier()
    set_profiling(False)
    total_ms = sum(s.elapsed_time(e) for s, e in ev)
    launch_mode = "stream launches"
    stream_ms = total_ms / steps
    if graph_ok and world == 1:
        # The whole forward+backward enqueues without a host synchronisation, so it can be replayed as one
        # CUDA graph; the timed value is then free of launch gaps.  Stage times above come from the stream pass.
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            gms = 0.0
            for s, e in ev:
                flush.zero_()
                s.record()
                g.replay()
                e.record()
                e.synchronize()
                gms += s.elapsed_time(e)
            total_ms = gms
            launch_mode = "CUDA graph replay of the whole step"
            step = g.replay
        except Exception as exc:        # capture not possible here: keep the stream numbers
            launch_mode = f"stream launches (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / steps
    clocks = None
    if sample_clocks:
        # a short run can end before nvidia-smi has printed a sample: keep the same load up (untimed) for
        # about 0.7 s in total; the count is derived from the all-reduced step time, so every rank runs the same
        extra = min(2000, max(0, int(700.0 / max(ms_per_step, 1e-3)) - steps - warmup))
        for _ in range(extra):
            step()
        barrier()
        clocks = sampler.stop() if sampler else None

    for _ in range(2):
        step_host()
    barrier()
    e2e_ms = 0.0
    for _ in range(steps):
        flush.zero_()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        step_host()
        e2e_ms += (time.perf_counter() - t0) * 1e3
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / steps
    n_dir = 2 if w.backward else 1
    checksum = host_checksum()             # of the last step's output, computed outside the timed region
    e2e = {"value": world * N / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": io_bytes * n_dir, "d2h_bytes_per_step": io_bytes * n_dir, "checksum": checksum,
           "steps_in_flight": 1}
    if pipe is not None:
        # The same K steps through the pipelined call: every step still uploads its x and dy from pinned host memory
        # and downloads its y and dx inside the timed region, but one step's copies overlap another's kernels (two
        # steps in flight).  Inputs (134 MB at c4) exceed L2, so consecutive steps do not find them cached.
        enqueue, wait = pipe
        for i in range(3):
            enqueue(i)
        wait()
        barrier()
        t0 = time.perf_counter()
        for i in range(steps):
            enqueue(i)
        wait()
        pms = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([pms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pms = float(t.item()) / steps
        e2e.update({"value": world * N / (pms * 1e-3), "ms_per_step": pms, "steps_in_flight": 2,
                    "call": ("mgpt_moe_step_host_async" if world == 1 else "the same pipeline around the expert-parallel layer")
                            + " (the next step's uploads and the previous step's downloads overlap this step's "
                              "kernels), timed over all K steps and the final wait",
                    "one_step_alone_ms": e2e_ms, "checksum": host_checksum()})
    return {"ms_per_step": ms_per_step, "stage_sum": stage_sum, "steps": steps, "launches": int(launches),
            "clocks": clocks, "e2e": e2e, "launch_mode": launch_mode, "stream_ms": stream_ms}


def single_gpu_pass(args, w, rank, dev, *, light=False):
    """One replica of the whole layer on this GPU (all experts local).  ``light``: a short pass for the
    secondary workloads (fewer steps, no clock sampling, no optimiser / recompute timing)."""
    import torch

    from mgpt_b200 import MoELayer

    N, C = w.n_tokens, w.C
    layer = MoELayer(w.C, w.H, w.E, w.k, mode=w.dtype, device=dev.index, lb_alpha=w.alpha)
    load_synth_params(layer.get_parameters(), w, dev, lambda i: i)
    layer.sync_weights()
    x_host, dy_host, y_host, dx_host = host_tokens(w, rank)
    x, dy = x_host.to(dev), dy_host.to(dev)
    y, dx = torch.empty_like(x), torch.empty_like(x)

    def step():
        if w.backward:
            layer.forward_into(x, y)
            layer.backward_into(dy, dx)
        else:
            layer.forward_inference_into(x, y)         # the generator's call: forward only, nothing kept

    def step_host():
        layer.step_host(x_host, dy_host if w.backward else None, y_host, dx_host if w.backward else None)

    def host_checksum():
        return float(y_host[:4096].float().abs().mean())

    def barrier():
        torch.cuda.synchronize()

    # second set of pinned outputs: with two steps in flight, consecutive steps must not share their y / dx
    y_host2, dx_host2 = (torch.empty_like(y_host).pin_memory(), torch.empty_like(dx_host).pin_memory()) if not light else (None, None)

    def enqueue(i):
        yo, dxo = (y_host, dx_host) if i % 2 == 0 else (y_host2, dx_host2)
        layer.step_host_async(x_host, dy_host if w.backward else None, yo, dxo if w.backward else None)

    layer.zero_grad()
    step()
    counts = layer.get_expert_counts()                 # also reads the layer's error word
    res = measure(args, w, 1, 0, dev, step, step_host, host_checksum, layer.stage_ms, layer.set_profiling, barrier, N,
                  x_host.numel() * x_host.element_size(), graph_ok=not args.no_graph,
                  steps=min(args.steps, 10) if light else None, warmup=3 if light else None, sample_clocks=not light,
                  pipe=None if light else (enqueue, layer.step_host_wait))
    layer.check_status()
    res["experts_touched"] = sum(1 for c in counts if c > 0)
    if w.dtype == "bf16":
        # tokens whose routing the tensor-core pass of the router could not prove and the exact pass recomputed
        rc = layer.workspace_view("router_recompute", torch.int32)       # absent from the inference workspace
        res["router_recomputed"] = int(rc.cpu()[0]) if rc.numel() else None
    res["counts"] = counts
    res["y"], res["dx"] = y, (dx if w.backward else None)          # of the last timed step (device tensors)
    res["overwrite"] = time_overwrite(layer, w, step) if w.backward and not light and w.dtype == "bf16" else None
    res["recompute"] = time_recompute(layer, x, torch.empty_like(y)) if w.backward and not args.no_optimizer and not light else None
    res["optimizer"] = time_optimizer(layer, w) if w.backward and not args.no_optimizer and not light else None
    layer.close()
    return res


def time_overwrite(layer, w, step):
    """Outside the timed steps: the weight-gradient stage when the caller has said its gradient tensors are freshly
    zeroed (first backward after the trainer's zero fill), so that the library stores instead of read-modify-writes."""
    import torch
    layer.set_weight_grad_overwrite(True)
    layer.set_profiling(True)
    ms = []
    for _ in range(4):
        step()
        torch.cuda.synchronize()
        ms.append(layer.stage_ms().get("wgrad_gemm", 0.0))
    layer.set_profiling(False)
    layer.set_weight_grad_overwrite(False)
    best = min(ms[1:])
    flop = 6.0 * w.n_tokens * w.k * w.C * w.H
    return {"wgrad_ms": round(best, 4), "wgrad_tflops": round(flop / (best * 1e-3) / 1e12, 1),
            "note": "not part of the timed step: weight gradients stored instead of accumulated "
                    "(mgpt_moe_set_weight_grad_overwrite; equals accumulation into zeroed tensors bit for bit)"}


def time_recompute(layer, x, y):
    """Outside the timed steps: forward alone against the recompute forward that takes the saved routing
    (activation checkpointing runs the forward twice per step).  CUDA events, best of three."""
    import torch

    def timed(fn, reps=3):
        fn()
        torch.cuda.synchronize()
        best = None
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            t = a.elapsed_time(b)
            best = t if best is None else min(best, t)
        return best

    fwd_ms = timed(lambda: layer.forward_into(x, y))
    routing = layer.save_routing()
    re_ms = timed(lambda: layer.recompute_into(x, y, routing))
    return {"forward_ms": round(fwd_ms, 4), "recompute_forward_ms": round(re_ms, 4),
            "routing_state_bytes": int(routing.numel()),
            "note": "not part of the timed step; the recompute skips router and plan"}


def time_optimizer(layer, w):
    """Outside the timed steps: the fused AdamW + BF16-copy refresh against the copy refresh alone
    (what an engine-side AdamW would have to be followed by).  CUDA events, three runs after one warm-up."""
    import torch

    def timed(fn, reps=3):
        fn()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * reps)]
        for i in range(reps):
            ev[2 * i].record()
            fn()
            ev[2 * i + 1].record()
        torch.cuda.synchronize()
        return min(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(reps))

    try:
        step_no = [0]

        def adamw():
            step_no[0] += 1
            layer.adamw_step(step_no[0])

        adamw_ms = timed(adamw)
        sync_ms = timed(layer.sync_weights)
    except torch.OutOfMemoryError:
        return None
    n_w = sum(p.numel() for p in layer.get_parameters())
    byts = n_w * (28 + (4 if w.dtype == "bf16" else 0))      # read w,g,m,v; write w,m,v (+ two BF16 copies)
    return {"adamw_fused_ms": round(adamw_ms, 4), "adamw_fused_gbs": round(byts / (adamw_ms * 1e-3) / 1e9, 1),
            "bytes": byts, "sync_weights_alone_ms": round(sync_ms, 4),
            "note": "not part of the timed step; one optimiser step over all 2+6E tensors, copies refreshed in the same pass"}


def bind_to_gpu_numa_node(index: int) -> None:
    """Restricts this process to the CPU cores NVML reports as local to GPU `index` (read-only query), so that
    the pinned host buffers of the end-to-end path are first touched on that GPU's NUMA node.  With one rank
    per GPU and no binding, every rank's buffers can end up on one socket and all copies cross the
    socket interconnect.  Best effort: any failure leaves the affinity as it was."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        n_cpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (n_cpu + 63) // 64)
        cpus = {64 * i + b for i, wd in enumerate(words) for b in range(64) if (int(wd) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
        pynvml.nvmlShutdown()
    except Exception:
        pass


def score(w, res, peaks, world):
    """Per-stage achieved TFLOP/s or GB/s and the roofline of the dominant kernel, from the stage times."""
    flops, byts = stage_model(w)
    stages = {}
    for name, ms in res["stage_sum"].items():
        ms /= res["steps"]
        if ms <= 0:
            continue
        ent = {"ms": round(ms, 4)}
        if name in flops:
            ent["tflops"] = round(flops[name] / (ms * 1e-3) / 1e12, 1)
        elif name in byts and world == 1:
            ent["gbs"] = round(byts[name] / (ms * 1e-3) / 1e9, 1)
        if name == "router" and "router_recomputed" in res:
            ent["tokens_recomputed_exactly"] = res["router_recomputed"]
        stages[name] = ent
    gemm = {k: v for k, v in stages.items() if k in flops}
    roofline = None
    if gemm:
        dom = max(gemm, key=lambda k: gemm[k]["ms"])
        achieved = flops[dom] / (gemm[dom]["ms"] * 1e-3) / 1e12
        peak = peaks["bf16_tflops"]
        roofline = {"bound": "tensor", "kernel": dom, "achieved": round(achieved, 1), "peak": peak,
                    "peak_source": f"{peaks['source']} cuBLAS bf16 burst", "unit": "TFLOP/s",
                    "frac": round(achieved / peak, 4), "traffic": TRAFFIC.get((w.name, dom)),
                    "all_gemms_tflops": round(sum(flops[k] for k in gemm) / (sum(v["ms"] for v in gemm.values()) * 1e-3) / 1e12, 1)}
    if not w.backward and gemm and world == 1:
        # decode shapes stream the touched experts' weights once: HBM-bound, scored in GB/s
        touched = res.get("experts_touched", w.E)
        wbytes = touched * 3.0 * w.C * w.H * 2
        ms = sum(v["ms"] for v in gemm.values())
        ach = wbytes / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "gateup_gemm+down_gemm", "achieved": round(ach, 1), "peak": peaks["hbm_gbs"],
                    "peak_source": f"{peaks['source']} copy bandwidth", "unit": "GB/s", "frac": round(ach / peaks["hbm_gbs"], 4),
                    "traffic": None, "experts_touched": touched}
    return stages, roofline


def rel_l2(a, b) -> float:
    import torch
    a, b = a.double().reshape(-1), b.double().reshape(-1)
    den = float(torch.linalg.vector_norm(b))
    err = float(torch.linalg.vector_norm(a - b))
    return err / den if den > 0 else err


def oracle_check(w, y, sample):
    """The bench's own outputs against the CPU oracle: forward of the first `sample` tokens (tokens are independent
    in forward, and the seeded generator's first rows are the same whatever the token count)."""
    import numpy as np
    import torch

    from mgpt_b200 import synth
    from oracle import oracle
    ws = w.scaled(sample)
    x, params, _ = synth.make_inputs(ws, seed=SEED)
    d = oracle.Dims(ws.n_tokens, ws.C, ws.H, ws.E, ws.k, ws.alpha)
    ref = oracle.run(d, x, params, None, which="ref" if oracle.have_ref() else "oracle", threads=os.cpu_count() or 1)
    got = y[:sample].float().cpu()
    return {"tokens": sample, "y_rel_l2": rel_l2(got, torch.from_numpy(np.ascontiguousarray(ref["y"]))),
            "against": "the reference's CPU MoELayer" if oracle.have_ref() else "the C restatement", "bar": 2e-2}


def run_ours(args, w):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    peaks = load_peaks()
    N, C = w.n_tokens, w.C
    reference_1gpu = None
    ep_phases = None
    ep_check = None
    single = None

    bind_to_gpu_numa_node(local)            # before any pinned allocation: host buffers land next to this rank's GPU
    if world == 1:
        res = single = single_gpu_pass(args, w, rank, dev)
        parallelism = "single GPU"
    else:
        from mgpt_b200.ep import ExpertParallelMoE

        # NCCL's stream at high priority: an exchange that becomes ready together with a persistent compute kernel is
        # placed first (the compute CTAs that find their SM taken start late and take fewer work items)
        try:
            opts = dist.ProcessGroupNCCL.Options()
            opts.is_high_priority_stream = True
            dist.init_process_group("nccl", device_id=dev, pg_options=opts)
        except Exception:
            dist.init_process_group("nccl", device_id=dev)
        if w.E % world:
            raise SystemExit(f"workload {w.name}: {w.E} experts do not divide over {world} GPUs")
        if rank == 0 and not args.no_single:
            # the same per-GPU problem on one GPU with every expert local: the reference point of the scaling,
            # and (same seeded weights and tokens) the check of the expert-parallel result below
            single = single_gpu_pass(args, w, rank, dev)
            reference_1gpu = {"n_gpus": 1, "value": N / (single["ms_per_step"] * 1e-3), "unit": UNIT,
                              "ms_per_step": single["ms_per_step"],
                              "workload": describe(w), "note": "all experts local, no exchange"}
            torch.cuda.empty_cache()
        dist.barrier()
        E_local = w.E // world
        chunks = args.ep_chunks if E_local % max(1, args.ep_chunks) == 0 else 1
        native = args.ep_impl == "native"
        if args.ep_transport == "peer" and not all(torch.cuda.can_device_access_peer(local, o)
                                                   for o in range(world) if o != local):
            args.ep_transport = "collective"       # no peer access between these GPUs (same answer on every rank of a node)
        if native:
            # the whole exchange behind the C ABI (mgpt_moe_ep_*: the library's own NCCL communicator and stream)
            from mgpt_b200.ep import NativeExpertParallelMoE
            layer = NativeExpertParallelMoE(w.C, w.H, w.E, w.k, rank=rank, world=world,
                                            nccl_id=NativeExpertParallelMoE.create_id(), mode=w.dtype, device=local,
                                            lb_alpha=w.alpha, n_chunks=chunks,
                                            max_tokens=N if args.ep_transport == "peer" else 0)
        else:
            layer = ExpertParallelMoE(w.C, w.H, w.E, w.k, mode=w.dtype, device=local, lb_alpha=w.alpha,
                                      n_chunks=chunks, sm_budget=args.ep_sm_budget, transport=args.ep_transport)
        # router: the same tensors on every rank; experts: those this rank owns, by their global index
        load_synth_params(layer.get_parameters(), w, dev,
                          lambda i: i if i < 2 else 2 + 6 * layer.global_expert((i - 2) // 6) + (i - 2) % 6)
        if native:
            # parameters are bound in place; only the BF16 copies need building
            layer._lib_mod.check(layer.lib.mgpt_moe_ep_sync_weights(layer._h, layer._stream()))
        else:
            layer.stages.sync_weights()
        x_host, dy_host, y_host, dx_host = host_tokens(w, rank)
        x, dy = x_host.to(dev), dy_host.to(dev)
        last = {}

        def step():
            last["y"] = layer.forward(x)
            if w.backward:
                last["dx"] = layer.backward(dy)

        xd, dyd = torch.empty_like(x), torch.empty_like(dy)
        copy_stream = torch.cuda.Stream(device=dev)

        def step_host():
            # as in mgpt_moe_step_host: dy goes up while forward runs, y comes down while backward runs
            cur = torch.cuda.current_stream()
            xd.copy_(x_host, non_blocking=True)
            up = torch.cuda.Event()
            if w.backward:
                copy_stream.wait_stream(cur)           # the previous step's backward has finished with dyd
                with torch.cuda.stream(copy_stream):
                    dyd.copy_(dy_host, non_blocking=True)
                    up.record()
            y = layer.forward(xd)
            copy_stream.wait_stream(cur)
            with torch.cuda.stream(copy_stream):
                y_host.copy_(y, non_blocking=True)
            y.record_stream(copy_stream)
            if w.backward:
                cur.wait_event(up)
                dx_host.copy_(layer.backward(dyd), non_blocking=True)
            torch.cuda.synchronize()

        # The pipelined form of the same step (what mgpt_moe_step_host_async does for the one-GPU layer): two slots
        # of device staging, uploads and downloads on streams of their own, compute in call order.
        slots = [{"xd": xd, "dyd": dyd}, {"xd": torch.empty_like(x), "dyd": torch.empty_like(dy)}]
        outs = [(y_host, dx_host), (torch.empty_like(y_host).pin_memory(), torch.empty_like(dx_host).pin_memory())]
        up_stream, down_stream = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

        def enqueue(i):
            sl, (yo, dxo) = slots[i % 2], outs[i % 2]
            cur = torch.cuda.current_stream()
            if sl.get("out_done") is not None:
                sl["out_done"].synchronize()           # the step before last: its results are in host memory
                up_stream.wait_event(sl["compute_done"])
            in_x, in_dy = torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(up_stream):
                sl["xd"].copy_(x_host, non_blocking=True)
                in_x.record()
                if w.backward:
                    sl["dyd"].copy_(dy_host, non_blocking=True)
                    in_dy.record()
            cur.wait_event(in_x)
            y = layer.forward(sl["xd"])
            down_stream.wait_stream(cur)
            with torch.cuda.stream(down_stream):
                yo.copy_(y, non_blocking=True)
            y.record_stream(down_stream)
            if w.backward:
                cur.wait_event(in_dy)
                dxd = layer.backward(sl["dyd"])
                down_stream.wait_stream(cur)
                with torch.cuda.stream(down_stream):
                    dxo.copy_(dxd, non_blocking=True)
                dxd.record_stream(down_stream)
            sl["compute_done"] = torch.cuda.Event()
            sl["compute_done"].record(cur)
            sl["out_done"] = torch.cuda.Event()
            sl["out_done"].record(down_stream)

        def wait_all():
            torch.cuda.synchronize()

        def host_checksum():
            return float(y_host[:4096].float().abs().mean())

        def barrier():
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()

        layer.zero_grad()
        if native:
            res = measure(args, w, world, rank, dev, step, step_host, host_checksum, lambda: {}, lambda on: None, barrier, N,
                          x_host.numel() * x_host.element_size(), pipe=(enqueue, wait_all))
            layer.check_status()
        else:
            res = measure(args, w, world, rank, dev, step, step_host, host_checksum, layer.stages.stage_ms,
                          layer.stages.set_profiling, barrier, N, x_host.numel() * x_host.element_size(),
                          pipe=(enqueue, wait_all))
            # one more step with CUDA events around every phase (exchange vs compute), outside the timed region
            layer.phase_events = {}
            step()
            torch.cuda.synchronize()
            ep_phases = {k: round(v, 3) for k, v in layer.phase_ms().items()}
            layer.phase_events = None
            layer.stages.check_status()
        counts_native = None
        if native:
            # what every rank received from rank 0, per local expert: together, rank 0's counts over all experts
            try:
                mine = layer.last_recv_counts[0].to(dev)
                gathered = torch.empty(world * mine.numel(), dtype=mine.dtype, device=dev)
                dist.all_gather_into_tensor(gathered, mine)
                gathered = gathered.view(world, -1).cpu().tolist()
                Ec = E_local // chunks
                counts_native = [0] * w.E
                for r in range(world):
                    for l in range(E_local):
                        c, j = divmod(l, Ec)
                        counts_native[c * (w.E // chunks) + r * Ec + j] = int(gathered[r][l])
            except Exception:
                counts_native = None
        if rank == 0 and single is not None:
            # rank 0's tokens through the expert-parallel layer against the same tokens through the one-GPU layer
            # (same weights; the load-balance term uses this rank's own counts in both)
            if native:
                counts_ep = counts_native
            else:
                counts_ep = layer.stages.routing_view("counts", torch.int32).cpu().tolist()
            ep_check = {"y_rel_l2": rel_l2(last["y"], single["y"]),
                        "dx_rel_l2": rel_l2(last["dx"], single["dx"]) if w.backward else None,
                        "counts_equal": None if counts_ep is None else counts_ep == [int(c) for c in single["counts"]],
                        "note": "rank 0: expert-parallel result vs the one-GPU layer on the same seeded tokens and weights"}
        if not native:
            layer.close_peer()
        dist.barrier()
        parallelism = (f"expert parallel: {E_local} of {w.E} experts per GPU, {N} tokens per GPU, "
                       + (("copy-engine pulls from peer buffers" if args.ep_transport == "peer" else "NCCL point-to-point groups")
                          + " inside the library (mgpt_moe_ep_*)" if native else
                          "rows pulled from the producers' buffers by copy engines over NVLink (CUDA IPC, mgpt_moe_peer_*), "
                          "NCCL for the counts and the barriers" if args.ep_transport == "peer" else
                          "NCCL all-to-all (torch.distributed)")
                       + f" for dispatch and combine, experts in {chunks} chunk(s) "
                       "(a chunk's exchange overlaps the previous chunk's expert work)")

    ms_per_step = res["ms_per_step"]
    value = world * N / (ms_per_step * 1e-3)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    stages, roofline = score(w, res, peaks, world)
    if roofline is None and world > 1 and single is not None:
        # the C-ABI expert-parallel driver has no per-stage events: the same kernels, timed stage by stage in the
        # one-GPU pass of this job (rank 0, same workload and weights)
        stages, roofline = score(w, single, peaks, 1)
        roofline["measured_in"] = "the one-GPU pass of the same job (same kernels, all experts local)"
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": res["steps"], "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": w.dtype, "data": "synthetic",
        "config": {"workload": describe(w), "parallelism": parallelism,
                   "l2": "flushed between timed steps by a 256 MiB write", "hbm_peak_gbs": peaks["hbm_gbs"],
                   "launch": res["launch_mode"], "ms_per_step_stream_launches": round(res["stream_ms"], 4),
                   "inputs": f"seeded synthetic (Philox, seed {SEED} + rank for tokens), the CPU oracle's generator"},
        "clocks": res["clocks"], "e2e": res["e2e"], "gpu_launches": res["launches"], "roofline": roofline, "stages": stages,
    }

    cpu = None
    if world == 1 and not args.no_cpu:
        sample = min(N, args.cpu_sample or (1024 if cpu_step_estimate_s(w, 1024) < 10 else 512))
        secs, kind, cores = cpu_reference_step(w, sample, threads=os.cpu_count() or 1,
                                               iters=2 if cpu_step_estimate_s(w, sample) < 10 else 1)
        sec = min(secs)
        cpu = {"value": sample / sec, "unit": UNIT, "cores": cores, "kind": kind,
               "sample": f"{sample} tokens of {w.name} (same C,H,E,k), one forward+backward, {sec:.1f} s "
                         "(includes the fixed cost of walking every expert's weights; --impl reference fits it out)"}
        line["oracle_check"] = oracle_check(w, single["y"], min(sample, 512))
    line["cpu_baseline"] = cpu
    if world == 1 and single.get("optimizer"):
        line["optimizer"] = single["optimizer"]
    if world == 1 and single.get("overwrite"):
        line["weight_gradients_stored"] = single["overwrite"]
    if world == 1 and single.get("recompute"):
        line["checkpointing"] = single["recompute"]
    if reference_1gpu:
        line["same_workload_on_one_gpu"] = reference_1gpu
    if world > 1:
        line["ep_phases_ms"] = ep_phases
        line["ep_check"] = ep_check
    if world == 1 and not args.no_others and args.workload is None:
        # the other configurations of the baseline, each a short pass after the timed run (not part of `value`)
        from mgpt_b200 import synth
        single = None
        torch.cuda.empty_cache()
        others = {}
        for name in ("c2", "c3", "c5-8", "c5-64", "c5-256"):
            ow = synth.WORKLOADS[name]
            r = single_gpu_pass(args, ow, 0, dev, light=True)
            st, rf = score(ow, r, peaks, 1)
            others[name] = {"workload": describe(ow), "ms_per_step": round(r["ms_per_step"], 4),
                            "tokens_per_s": round(ow.n_tokens / (r["ms_per_step"] * 1e-3), 1), "steps": r["steps"],
                            "launch": r["launch_mode"],
                            "roofline": None if rf is None else {k: rf[k] for k in ("bound", "kernel", "achieved", "unit", "frac", "traffic") if k in rf},
                            "e2e": {"value": round(r["e2e"]["value"], 1), "ms_per_step": round(r["e2e"]["ms_per_step"], 4)},
                            "stages_ms": {k: v["ms"] for k, v in st.items()}}
            del r
            torch.cuda.empty_cache()
        line["other_workloads"] = others
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, help="c1 c2 c3 c4 c5-8 c5-64 c5-256 (default c4)")
    ap.add_argument("--ep-chunks", type=int, default=2, help="N>1: expert chunks whose exchange overlaps compute")
    ap.add_argument("--ep-impl", default="native", choices=["python", "native"],
                    help="N>1: exchange driven from Python over torch.distributed, or entirely inside the C library")
    ap.add_argument("--ep-transport", default="peer", choices=["collective", "peer"],
                    help="N>1, --ep-impl python: rows by all_to_all_single, or pulled by copy engines from peer buffers")
    ap.add_argument("--ep-sm-budget", type=int, default=0,
                    help="N>1: CTAs of the persistent expert kernels (0 = every SM); leaves SMs to the exchange kernels")
    ap.add_argument("--cpu-sample", type=int, default=0, help="tokens per CPU-baseline step")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="time plain stream launches instead of a CUDA graph replay")
    ap.add_argument("--no-single", action="store_true", help="N>1: skip the one-GPU pass of the same workload")
    ap.add_argument("--no-optimizer", action="store_true", help="skip the untimed AdamW / copy-refresh measurement")
    ap.add_argument("--no-others", action="store_true", help="skip the short passes over the other configurations")
    args = ap.parse_args()

    from mgpt_b200 import synth
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # the 64-expert configuration the throughput and scaling targets are stated on, at every N
    # (32768 tokens per GPU: weak scaling; on one GPU all 64 experts are local)
    w = synth.WORKLOADS[args.workload or "c4"]
    if args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()
