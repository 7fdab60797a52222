#!/usr/bin/env python
"""Benchmark of the hot path: one PET-optimised dilated-conv layer executed on the new kernels.

Workload (BASELINE config 2): input [1,512,64,64] fp32 ~ N(0,1), He-normal 3x3 filters [512,512,3,3]; the graph PET's
rewrite produces — space-to-batch (a fused 4-transpose chain) -> dense 3x3 conv on [4,512,32,32] -> batch-to-space
(fused inverse chain) — run as three kernels per step.  One "step" = one image through that graph.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1: launched under torchrun, one rank per GPU, independent replicas (no data-path collective), weak scaling.
Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

X_SHAPE = (1, 512, 64, 64)
W_SHAPE = (512, 512, 3, 3)
S2B = [(2, [0, 1, [-1, 2], 3], 2), (2, [[0, 2], 1, -1, 3], -2), (3, [0, 1, 2, [-1, 3]], 2), (3, [[0, 3], 1, 2, -1], -2)]
B2S = [(0, [0, 1, 2, [-1, 3]], 2), (3, [0, 1, 2, [-1, 3]], -2), (0, [0, 1, [-1, 2], 3], 2), (2, [0, 1, [-1, 2], 3], -2)]
CONV_FLOPS = 2.0 * 4 * 512 * 32 * 32 * 512 * 9          # algorithmic flops of the dense conv per step
CONV_DRAM_TRAFFIC = 27.36e6   # bytes per launch, dram__bytes_read+write of the conv kernel (profiles/conv_tc3xtf32_dilated_layer.md)
RING = 20                                               # distinct buffer sets cycled through: 20 x 8 MiB inputs > 126 MB L2
CONFIG = {"workload": "dilated conv layer 512->512 64x64 d2 p2 fp32 batch 1, PET rewrite: space-to-batch -> dense 3x3 conv -> batch-to-space",
          "kernels_per_step": 3, "l2": f"ring of {RING} input/intermediate/output buffer sets (168 MB of inputs) cycled, larger than L2"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def max_over_ranks(values, world, device=None):
    """Element-wise maximum of `values` over all ranks (the slowest replica defines the job's time)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(values, device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.cpu()]


def replica_throughput(world, steps, ms_total):
    """Whole-job images/s of `world` independent replicas that each ran `steps` images in ms_total (max over ranks)."""
    return world * steps * 1000.0 / ms_total


def synthetic(seed=2000):
    """Seeded stand-ins with the configuration's shapes and distributions: X ~ N(0,1), W He-normal (fan-in 4608)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(X_SHAPE, generator=g)
    w = torch.randn(W_SHAPE, generator=g) * (2.0 / (512 * 9)) ** 0.5
    return x, w


def cpu_reference_sample(filters, threads_note=True):
    """Times the reference's own host operators (oracle/_ref, else the C restatement) on a bounded sample of the
    workload: the full transposes and `filters` of the 512 output channels of the conv.  Returns (images/s scaled
    linearly by channels, dict)."""
    from oracle import petref, pet_oracle
    rng = np.random.default_rng(7)
    x = rng.integers(0, 10000, X_SHAPE).astype(np.uint32)   # the reference evaluates on uint32 (its VType)
    w = rng.integers(0, 10000, (filters,) + W_SHAPE[1:]).astype(np.uint32)
    if petref.available():
        _, secs = petref.dilated_rewrite_u32(x, w)
        kind, cores = "reference", petref.num_threads()
    else:
        t0 = time.perf_counter()
        t = x
        for op in S2B:
            t = pet_oracle.transpose(t, *op)
        t = pet_oracle.conv2d_u32(t, w, pad=(1, 1))
        for op in B2S:
            t = pet_oracle.transpose(t, *op)
        secs = time.perf_counter() - t0
        kind, cores = "port", pet_oracle.lib().oracle_num_threads()
    value = (filters / W_SHAPE[0]) / secs
    return value, {"value": value, "unit": "images/s", "cores": cores, "kind": kind, "secs": secs,
                   "sample": f"whole graph on the host operators (uint32 arithmetic) with {filters} of {W_SHAPE[0]} output channels; "
                             "throughput scaled linearly by channels"}


def config_latencies(ctx):
    """Batch-1 latency (ms) of every benchmark configuration through the graph layer: CUDA-graph replay of the whole
    graph, 20 warm-up + 200 timed passes between two CUDA events (the reference program's protocol; buffers are reused
    between passes, so small graphs run L2-warm exactly as they do in the reference's generated program)."""
    import torch
    from pet_b200 import configs
    from pet_b200.graph import Graph
    out = {}

    def run(name, build, *a, **kw):
        g = Graph(ctx)
        b = configs.GraphBuilder(g)
        g.setOutputs([build(b, *a, **kw)])
        g.compile()
        b.load()
        g.run()
        torch.cuda.synchronize()
        out[name] = {"ms": g.time(rounds=200, warmup=20), "kernels": g.num_launches()}
        # spread of single replays: one event pair per replay (includes the launch gap of a lone replay, so the median sits
        # a few microseconds above the back-to-back mean)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(200)]
        for e0, e1 in evs:
            e0.record()
            g.run()
            e1.record()
        torch.cuda.synchronize()
        lat = sorted(e0.elapsed_time(e1) for e0, e1 in evs)
        out[name].update({"median_ms": lat[len(lat) // 2], "p99_ms": lat[int(len(lat) * 0.99) - 1]})

    x, w = configs.c1_tensors()
    run("c1_conv3x3_original", configs.c1_original, x, w)
    run("c1_conv3x3_h2n_rewrite_corrected", configs.c1_rewrite, x, w)
    run("c1_conv3x3_h2n_rewrite_halo", configs.c1_rewrite_halo, x, w)
    x, w = configs.c2_tensors()
    run("c2_dilated_original", configs.c2_original, x, w)
    run("c2_dilated_space_to_batch_rewrite", configs.c2_rewrite, x, w)
    run("c3_resnet18", configs.resnet18)
    run("c4_bert_base_seq128", configs.bert_encoder)
    run("c5_r3d18", configs.r3d18)
    return out


def model_throughput(ctx, world, dev):
    """Images/s of ResNet-18 (global batch 64) and ResNet3D-18 (global batch 32) with the batch sharded into independent
    replicas, one per GPU, no collective: every rank runs global_batch / world images through its own captured graph;
    the job's time is the slowest rank's (device events, max over ranks)."""
    import torch
    from pet_b200 import configs
    from pet_b200.graph import Graph
    out = {}
    for name, build, gb in (("c3_resnet18", configs.resnet18, 64), ("c5_r3d18", configs.r3d18, 32)):
        per = max(1, gb // world)
        g = Graph(ctx)
        b = configs.GraphBuilder(g)
        g.setOutputs([build(b, batch=per)])
        g.compile()
        b.load()
        g.run()
        torch.cuda.synchronize()
        ms = g.time(rounds=20, warmup=3)
        (ms,) = max_over_ranks([ms], world, dev)
        out[name] = {"global_batch": per * world, "per_gpu_batch": per, "ms": ms, "images_per_s": per * world * 1000.0 / ms,
                     "kernels": g.num_launches(), "scaling": "strong"}
        del g, b
    return out


def run_reference(args, rank, world):
    if rank != 0:
        return
    # rank 0 alone runs the host arm, with all host threads: torchrun presets OMP_NUM_THREADS=1 for its workers
    if world > 1:
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    vals, info = [], None
    for i in range(args.warmup + args.steps):
        v, info = cpu_reference_sample(8)
        if i >= args.warmup:
            vals.append(v)
    value = float(np.mean(vals))
    info["value"] = value
    line = {"impl": "reference", "metric": "images_per_s", "value": value, "unit": "images/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 / value, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u32", "data": "synthetic", "config": CONFIG, "cpu_baseline": info,
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=40)
    ap.add_argument("--impl", default="petb200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-config-latencies", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.steps > 20:
            args.steps, args.warmup = 3, 1   # each step is seconds of host work
        return run_reference(args, rank, world)

    import torch
    import torch.distributed as dist
    from pet_b200.ops import Context

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = Context(local)
    dev = torch.device("cuda", local)
    x, w = synthetic(2000 + rank)
    wd = w.to(dev)

    s2b = ctx.transpose_plan(X_SHAPE, S2B)
    conv = ctx.conv2d_plan(s2b.out_shape, W_SHAPE, 1, 1)
    b2s = ctx.transpose_plan(conv.out_shape, B2S)
    ctx.conv2d_set_weights(conv, wd)   # weight-only preprocessing, outside the timed region as in the reference

    xs = [(x + 0.01 * i).to(dev) for i in range(RING)]
    t1 = [torch.empty(s2b.out_shape, device=dev) for _ in range(RING)]
    t2 = [torch.empty(conv.out_shape, device=dev) for _ in range(RING)]
    ys = [torch.empty(b2s.out_shape, device=dev) for _ in range(RING)]

    def step(i, ev=None):
        j = i % RING
        ctx.layout_run(s2b, xs[j], out=t1[j])
        if ev:
            ev[0].record()
        ctx.conv2d_run(conv, t1[j], out=t2[j])
        if ev:
            ev[1].record()
        ctx.layout_run(b2s, t2[j], out=ys[j])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(3, args.warmup)):
        step(i)
    ctx.sync_check()

    # ---- device-resident throughput (`value`) ----
    conv_events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    l0 = ctx.launches()
    e0.record()
    for i in range(args.steps):
        step(i, conv_events[i])
    e1.record()
    barrier()
    launches = ctx.launches() - l0
    ms_total = e0.elapsed_time(e1)
    conv_ms = float(np.mean([a.elapsed_time(b) for a, b in conv_events]))
    ctx.sync_check()

    # ---- end to end through host buffers (`e2e`): pinned H2D of the input and D2H of the result every step, three
    #      streams so that the copies of neighbouring steps overlap the kernels ----
    NB = 4
    hx = [x.clone().pin_memory() for _ in range(NB)]
    hy = [torch.empty(b2s.out_shape).pin_memory() for _ in range(NB)]
    s_in, s_k, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(NB)]
    ev_k = [torch.cuda.Event() for _ in range(NB)]
    ev_out = [torch.cuda.Event() for _ in range(NB)]

    def e2e_step(i):
        j = i % NB
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_k[j])          # the kernels that last read this slot are done
            xs[j].copy_(hx[j], non_blocking=True)
            ev_in[j].record()
        with torch.cuda.stream(s_k):
            s_k.wait_event(ev_in[j])
            s_k.wait_event(ev_out[j])         # the previous result of this slot has left the device
            ctx.layout_run(s2b, xs[j], out=t1[j])
            ctx.conv2d_run(conv, t1[j], out=t2[j])
            ctx.layout_run(b2s, t2[j], out=ys[j])
            ev_k[j].record()
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_k[j])
            hy[j].copy_(ys[j], non_blocking=True)
            ev_out[j].record()

    for i in range(max(3, args.warmup // 4)):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record(s_in)
    for i in range(args.steps):
        e2e_step(i)
    s_out.synchronize()
    g1.record(s_out)
    barrier()
    e2e_ms = max(g0.elapsed_time(g1), 0.0)
    e2e_wall = (time.perf_counter() - t0) * 1000.0
    e2e_ms = max(e2e_ms, e2e_wall * 0.0)  # device clock is the measure; wall clock kept for the record below
    clocks = sampler.stop() if rank == 0 else None
    ctx.sync_check()

    # ---- max over ranks ----
    ms_total, e2e_ms, conv_ms = max_over_ranks([ms_total, e2e_ms, conv_ms], world, dev)
    models = None if args.no_config_latencies else model_throughput(ctx, world, dev)
    if rank == 0:
        pk, pk_kind = peaks()
        ms_step = ms_total / args.steps
        value = replica_throughput(world, args.steps, ms_total)
        achieved = CONV_FLOPS / (conv_ms * 1e-3) / 1e12
        peak = pk["bf16_tflops_sustained"]
        line = {"metric": "images_per_s", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "tf32x3 (fp32 in/out)",
                "data": "synthetic", "config": dict(CONFIG, parallelism=f"replicas x{world}"),
                "e2e": {"value": replica_throughput(world, args.steps, e2e_ms), "unit": "images/s", "h2d_bytes_per_step": int(np.prod(X_SHAPE)) * 4,
                        "d2h_bytes_per_step": int(np.prod(b2s.out_shape)) * 4, "wall_ms_per_step": e2e_wall / args.steps},
                "gpu_launches": int(launches), "clocks": clocks,
                "roofline": {"bound": "tensor", "kernel": conv.kernel, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                             "frac": achieved / peak, "traffic": CONV_DRAM_TRAFFIC, "peak_source": f"{pk_kind} bf16 sustained",
                             "launch_ms": conv_ms, "issued_tf32_tflops": 3 * achieved, "tf32_peak_est": peak / 2,
                             "frac_of_tf32_issue_peak": 3 * achieved / (peak / 2)}}
        if models is not None:
            line["model_throughput"] = models
        if world == 1 and not args.no_config_latencies:
            line["batch1_latency_ms"] = config_latencies(ctx)
        if not args.no_cpu_baseline:
            try:
                _, line["cpu_baseline"] = cpu_reference_sample(8)
            except Exception as e:  # the checker is optional infrastructure; the GPU numbers stand without it
                line["cpu_baseline"] = {"error": str(e)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    ctx.close()


if __name__ == "__main__":
    main()
