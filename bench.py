#!/usr/bin/env python
"""Benchmark of the hot path: ResNet-18 inference on the new kernels, global batch 64 sharded into one replica per GPU.

Workload (the configuration the throughput metric is quoted on): ResNet-18, fp32, 3x224x224 inputs ~ N(0,1), He-normal
weights, folded BatchNorm, 1000-way FC; seeded synthetic tensors only.  One "step" = one forward pass of the rank's share
(64 / N images) of the global batch through the executed graph.  Strong scaling: the global batch stays 64.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1: launched under torchrun, one rank per GPU, independent replicas, no data-path collective (NCCL only carries the
timing barrier and the max over ranks).  Rank 0 prints ONE JSON line:
  value     images/s, inputs resident in device memory, K steps between two CUDA events, max over ranks
  e2e       the same through host buffers: pinned H2D of the images and D2H of the logits inside the timed region
  roofline  the tensor-core kernel: conv + FC flops of the timed steps / time that kernel was running
  extra     per-config batch-1 latencies, the dilated-conv layer, ResNet3D-18 throughput, the vendor-library baseline
            (cuDNN / cuBLAS through torch, same GPU, same process), the reference's host operators on this box's cores
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

GLOBAL_BATCH = 64
L2_BYTES = 126e6


def resnet18_flops():
    """Algorithmic flops of one image: 2 * outputs * (C * R * S) over the 20 convolutions, plus the FC."""
    total = 2 * 64 * 112 * 112 * 3 * 49
    cin, hw = 64, 56
    for stage, cout in enumerate([64, 128, 256, 512]):
        for i in range(2):
            s = 2 if (stage > 0 and i == 0) else 1
            hw //= s
            total += 2 * cout * hw * hw * cin * 9 + 2 * cout * hw * hw * cout * 9
            if not (s == 1 and cin == cout):
                total += 2 * cout * hw * hw * cin
            cin = cout
    return total, 2 * 512 * 1000


CONV_FLOPS, FC_FLOPS = resnet18_flops()
assert CONV_FLOPS + FC_FLOPS == 3628146688


def config_for(world):
    per = GLOBAL_BATCH // world
    return {"workload": f"ResNet-18 inference fp32 3x224x224, global batch {GLOBAL_BATCH} sharded into {world} replica(s) of {per} images",
            "global_batch": GLOBAL_BATCH, "per_gpu_batch": per, "parallelism": f"replicas x{world}",
            "l2": "every step runs on another of a ring of graph instances (own activations and weights) whose total footprint exceeds the 126 MB L2"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
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


def sum_over_ranks(values, world, device=None):
    import torch
    import torch.distributed as dist
    t = torch.tensor(values, device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [float(v) for v in t.cpu()]


def sharded_throughput(global_batch, steps, ms_total):
    """Whole-job images/s: every step all ranks together process the global batch; ms_total is the slowest rank's time."""
    return global_batch * steps * 1000.0 / ms_total


def build_graph(ctx, build, **kw):
    from pet_b200 import configs
    from pet_b200.graph import Graph
    g = Graph(ctx)
    b = configs.GraphBuilder(g)
    out = build(b, **kw)
    g.setOutputs([out])
    g.compile()
    b.load()
    g.run()
    return g, b, out


# ---- the reference's host operators on this box's cores (cpu_baseline, --impl reference) -----------------------------
class HostReferenceBuilder:
    """Evaluates a configuration with the reference's own host operators where it has them (oracle/_ref: ConvOp::compute
    and MatmulOp::compute, which compute in uint32 — the values are meaningless, the work is the reference's), and with
    the CPU restatement for the operators the reference gives no host body (pooling, activation).  Checker infrastructure,
    used only by the CPU legs of this benchmark."""

    def __init__(self):
        from oracle import pet_oracle, petref
        self.po, self.ref = pet_oracle, petref if petref.available() else None
        self.kind = "reference" if self.ref else "port"
        self.cores = petref.num_threads() if self.ref else pet_oracle.lib().oracle_num_threads()

    def input(self, a):
        return np.asarray(a, np.float32)

    const = input

    def conv(self, x, w, ph, pw, sh=1, sw=1, dh=1, dw=1, bias=None, act="none"):
        xu, wu = (np.abs(x) * 64).astype(np.uint32), (np.abs(w) * 64).astype(np.uint32)
        if self.ref:
            y = self.ref.conv2d_u32(xu, wu, pad=(ph, pw), stride=(sh, sw), dil=(dh, dw))
        else:
            y = self.po.conv2d_u32(xu, wu, pad=(ph, pw), stride=(sh, sw), dil=(dh, dw))
        return (y % 1024).astype(np.float32) / 1024

    def matmul(self, a, b, transA=False, transB=False, bias=None, act="none"):
        au, bu = (np.abs(a) * 64).astype(np.uint32), (np.abs(b) * 64).astype(np.uint32)
        y = self.ref.matmul_u32(au, bu, transA, transB) if self.ref else self.po.matmul(a, b, None, transA, transB)
        return (np.asarray(y) % 1024).astype(np.float32) / 1024

    def add(self, xs):
        return self.po.eltwise("add", xs)

    def relu(self, x):
        return self.po.activation(x, "relu")

    def maxpool(self, x, kh, kw, dh, dw, ph, pw, sh, sw):
        return self.po.maxpool(x, (kh, kw), (ph, pw), (sh, sw))

    def avgpool(self, x, kh=None, kw=None, ph=0, pw=0, sh=1, sw=1):
        if kh is None:
            kh, kw = x.shape[2], x.shape[3]
        return self.po.avgpool(x, (kh, kw), (ph, pw), (sh, sw))

    def reshape(self, x, dims):
        return np.ascontiguousarray(x).reshape(dims)


def cpu_reference_step(images=1):
    """One bounded sample of the workload on the host: `images` images of the batch through ResNet-18 on the reference's
    host operators, all host threads.  Returns (seconds, builder)."""
    from pet_b200 import configs
    hb = HostReferenceBuilder()
    t0 = time.perf_counter()
    configs.resnet18(hb, batch=images)
    return time.perf_counter() - t0, hb


def cpu_baseline_block(images, secs, hb):
    return {"value": images / secs, "unit": "images/s", "cores": hb.cores, "kind": hb.kind, "secs": secs,
            "sample": f"{images} image(s) of the global batch per step through ResNet-18 on the reference's host operators "
                      "(ConvOp::compute / MatmulOp::compute in uint32, OpenMP on all host threads; pooling and ReLU, which the "
                      "reference gives no host body, on the CPU restatement); throughput is per image, nothing is extrapolated"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    # rank 0 alone runs the host arm, with all host threads: torchrun presets OMP_NUM_THREADS=1 for its workers
    if world > 1:
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    images, secs, hb = 1, [], None
    for i in range(args.warmup + args.steps):
        s, hb = cpu_reference_step(images)
        if i >= args.warmup:
            secs.append(s)
    mean = float(np.mean(secs))
    value = images / mean
    info = cpu_baseline_block(images, mean, hb)
    line = {"impl": "reference", "metric": "images_per_s", "value": value, "unit": "images/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 * mean, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u32", "data": "synthetic", "config": config_for(world), "cpu_baseline": info,
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---- vendor-library baseline on the same GPU (N = 1 only) --------------------------------------------------------------
def time_cuda_graph(fn, rounds, warmup=5):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(rounds):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / rounds


def contract_metric(a, b):
    """max |a-b| / max(|b|, 1e-3 max|b|): the parity metric of the floating-point operators."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), max(1e-3 * float(np.max(np.abs(b))), 1e-30))))


def library_baseline(ctx, ours_ms):
    """cuDNN / cuBLAS executing the same configurations on this GPU, through torch's bindings (a stand-in for the
    reference's direct calls; cudnn.benchmark picks the fastest algorithm the way ConvOp::perf's sweep does), replayed as
    CUDA graphs: `default_math` = what the reference's conv calls get on this GPU (TF32 allowed), `fp32` = TF32 off (what
    its cuBLAS calls, issued with fp32 compute, get; and the accuracy class of this backend).  `max_err_vs_fp32` is the
    parity metric between this backend's output and the library's fp32 output on the same seeded tensors;
    `default_math_err_vs_fp32` the same metric for the library's own default-math output.  `bf16x3_*`: this backend with
    its opt-in error-compensated bf16 arithmetic (PETB200_ALGO_TC_BF16X3; every plan of the graph), an accuracy class between
    the library's two."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    from torch_backend import TorchBuilder
    from pet_b200 import configs
    torch.backends.cudnn.benchmark = True
    out = {"how": "torch 2.x bindings of cuDNN/cuBLAS, cudnn.benchmark=True, CUDA-graph replay, same GPU and process"}
    x1, w1 = configs.c1_tensors()
    x2, w2 = configs.c2_tensors()
    cases = [("c1_conv3x3_original", configs.c1_original, (x1, w1), {}, 200), ("c2_dilated_original", configs.c2_original, (x2, w2), {}, 100),
             ("c3_resnet18", configs.resnet18, (), {}, 50), ("c3_resnet18_batch64", configs.resnet18, (), {"batch": 64}, 5),
             ("c4_bert_base_seq128", configs.bert_encoder, (), {}, 30), ("c5_r3d18", configs.r3d18, (), {}, 20)]
    for name, build, a, kw, rounds in cases:
        row = {}
        lib_out = lib_out_default = None
        for mode, tf32 in (("default_math", True), ("fp32", False)):
            tb = TorchBuilder(tf32=tf32)
            consts = []

            class Rec:  # upload constants once, outside the replayed function
                def __getattr__(self, n):
                    return getattr(tb, n)

                def input(self, arr):
                    consts.append(tb.input(arr))
                    return consts[-1]

                const = input

            build(Rec(), *a, **kw)
            it = [0]

            class Replay:
                def __getattr__(self, n):
                    return getattr(tb, n)

                def input(self, arr):
                    it[0] += 1
                    return consts[it[0] - 1]

                const = input

            def fn():
                it[0] = 0
                return build(Replay(), *a, **kw)

            row[mode + "_ms"] = time_cuda_graph(fn, rounds)
            if not tf32:
                lib_out = fn().cpu().numpy()
            else:
                lib_out_default = fn().cpu().numpy()
        row["default_math_err_vs_fp32"] = contract_metric(lib_out_default, lib_out)
        if name in ours_ms:
            row["ours_ms"] = ours_ms[name]["ms"]
            g, _, o = build_graph(ctx, build, **kw) if not a else _build_with_args(ctx, build, a)
            torch.cuda.synchronize()
            row["max_err_vs_fp32"] = contract_metric(g.get_data(o), lib_out)
            del g
        os.environ["PETB200_TC_MATH"] = "bf16x3"  # read when a plan is created
        try:
            g, _, o = build_graph(ctx, build, **kw) if not a else _build_with_args(ctx, build, a)
            torch.cuda.synchronize()
            row["bf16x3_ms"] = g.time(rounds=rounds, warmup=5)
            row["bf16x3_max_err_vs_fp32"] = contract_metric(g.get_data(o), lib_out)
            del g
        finally:
            del os.environ["PETB200_TC_MATH"]
        out[name] = row
    try:
        out["reference_calls"] = reference_calls(ctx)
    except Exception as e:  # (the rows above stand without it)
        out["reference_calls"] = {"error": repr(e)}
    return out


def reference_calls(ctx):
    """The reference's OWN library calls for single operators (baseline/ref_calls.cu: the descriptor set-up and the algorithm
    sweeps of ConvOp::perf and MatmulOp::perf, restated), on the same seeded tensors as this backend: best time of the
    sweep and the parity metric between the two outputs and against an exact (float64) product."""
    import ctypes as C
    import torch
    from pet_b200 import configs
    path = os.path.join(ROOT, "baseline", "libref_calls.so")
    if not os.path.exists(path):
        return {"unavailable": "baseline/libref_calls.so not built (make -C baseline)"}
    try:
        lib = C.CDLL(path)
    except OSError as e:  # (cuDNN / cuBLAS not loadable on this box)
        return {"unavailable": f"baseline/libref_calls.so did not load: {e}"}
    out = {"how": "baseline/ref_calls.cu: cudnnConvolutionForward over the reference's 8 algorithms with default math; "
                  "cublasGemmStridedBatchedEx / cublasGemmEx with fp32 compute over the default and legacy algorithm ids; "
                  "CUDA events over 100 launches after 20 warm-ups"}
    ptr = lambda t: C.c_void_p(t.data_ptr())
    x1, w1 = configs.c1_tensors()
    x2, w2 = configs.c2_tensors()
    for name, x, w, pad, dil in (("c1_conv3x3", x1, w1, 1, 1), ("c2_dilated_conv", x2, w2, 2, 2)):
        xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
        n, c, h, wdt = x.shape
        f, cpg, r, s = w.shape
        y = torch.empty((n, f, h, wdt), device="cuda")
        ms, algo = C.c_float(), C.c_int()
        # ConvOp::perf sets CUDNN_CONVOLUTION mode (the filter is flipped); hand it the flipped filter so that both arms
        # compute the same cross-correlation and the outputs can be compared
        wflip = wd.flip(2, 3).contiguous()
        rc = lib.refcalls_conv2d(ptr(xd), ptr(wflip), ptr(y), n, c, h, wdt, f, cpg, r, s, pad, pad, 1, 1, dil, dil, 100, 20, C.byref(ms), C.byref(algo))
        if rc != 0:
            out[name] = {"unavailable": "no cuDNN algorithm ran"}
            continue
        ours = ctx.conv2d(xd, wd, pad, pad, 1, 1, dil, dil)
        plan = ctx.conv2d_plan(x.shape, w.shape, pad, pad, 1, 1, dil, dil)
        exact = torch.nn.functional.conv2d(xd.double(), wd.double(), padding=pad, dilation=dil).cpu().numpy()
        out[name] = {"library_best_ms": ms.value, "library_algo_index": algo.value, "ours_ms": plan.time(100, 20),
                     "library_err_vs_exact": contract_metric(y.cpu().numpy(), exact), "ours_err_vs_exact": contract_metric(ours.cpu().numpy(), exact)}
    g = torch.Generator(device="cuda").manual_seed(5)
    for name, b, m, n, k in (("bert_qkv_128x768x768", 1, 128, 768, 768), ("bert_ffn1_128x3072x768", 1, 128, 3072, 768),
                             ("bert_ffn2_128x768x3072", 1, 128, 768, 3072), ("bert_scores_12x128x128x64", 12, 128, 128, 64)):
        a = torch.randn((b, m, k), device="cuda", generator=g)
        bm = torch.randn((b, k, n), device="cuda", generator=g) / k ** 0.5
        cm = torch.empty((b, m, n), device="cuda")
        ms, algo = C.c_float(), C.c_int()
        rc = lib.refcalls_matmul(ptr(a), ptr(bm), ptr(cm), b, m, n, k, 0, 0, 100, 20, C.byref(ms), C.byref(algo))
        if rc != 0:
            out[name] = {"unavailable": "no cuBLAS algorithm ran"}
            continue
        plan = ctx.matmul_plan(a.shape, bm.shape)
        ctx.matmul_set_weights(plan, bm)
        ours = ctx.matmul_run(plan, a, None)
        torch.cuda.synchronize()
        exact = (a.double() @ bm.double()).cpu().numpy()
        out[name] = {"library_best_ms": ms.value, "library_algo": algo.value, "ours_ms": time_cuda_graph(lambda: ctx.matmul_run(plan, a, None), 100),
                     "library_err_vs_exact": contract_metric(cm.cpu().numpy(), exact), "ours_err_vs_exact": contract_metric(ours.cpu().numpy(), exact)}
    return out


def _build_with_args(ctx, build, a):
    from pet_b200 import configs
    from pet_b200.graph import Graph
    g = Graph(ctx)
    b = configs.GraphBuilder(g)
    out = build(b, *a)
    g.setOutputs([out])
    g.compile()
    b.load()
    g.run()
    return g, b, out


def config_latencies(ctx):
    """Batch-1 latency (ms) of every benchmark configuration through the graph layer: CUDA-graph replay of the whole
    graph, 20 warm-up + 200 timed passes between two CUDA events (the reference program's protocol; buffers are reused
    between passes, so small graphs run L2-warm exactly as they do in the reference's generated program)."""
    import torch
    from pet_b200 import configs
    out = {}

    def run(name, build, *a, **kw):
        g, _, _ = _build_with_args(ctx, build, a) if a else build_graph(ctx, build, **kw)
        torch.cuda.synchronize()
        out[name] = {"ms": g.time(rounds=200, warmup=20), "kernels": g.num_launches()}
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(200)]
        for e0, e1 in evs:  # spread of single replays (includes the launch gap of a lone replay)
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


def r3d_throughput(ctx, world, dev):
    """Clips/s of ResNet3D-18, global batch 32 sharded into replicas (strong scaling), CUDA-graph replay, max over ranks."""
    import torch
    from pet_b200 import configs
    per = max(1, 32 // world)
    g, _, _ = build_graph(ctx, configs.r3d18, batch=per)
    torch.cuda.synchronize()
    ms = g.time(rounds=10, warmup=3)
    (ms,) = max_over_ranks([ms], world, dev)
    return {"global_batch": per * world, "per_gpu_batch": per, "ms": ms, "clips_per_s": per * world * 1000.0 / ms,
            "kernels": g.num_launches(), "scaling": "strong"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="petb200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip batch-1 latencies, ResNet3D throughput and the library baseline")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.steps > 10:
            args.steps, args.warmup = 5, 1   # each step is about a second of host work
        return run_reference(args, rank, world)

    import torch
    import torch.distributed as dist
    from pet_b200 import configs
    from pet_b200.ops import Context

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = Context(local)
    dev = torch.device("cuda", local)
    per = GLOBAL_BATCH // world
    warmup = max(3, args.warmup)

    # ---- a ring of graph instances (own activations, own weights) so that consecutive steps do not find their data in L2 ----
    graphs = []
    g0, b0, out0 = build_graph(ctx, configs.resnet18, batch=per)
    graphs.append((g0, b0, out0))
    x_shape = b0.data[0][1].shape
    in_bytes, out_bytes = int(np.prod(x_shape)) * 4, per * 1000 * 4
    # per-instance footprint: weights + the larger activations (input, stem output, first stage)
    footprint = 47e6 + per * (3 * 224 * 224 + 64 * 112 * 112 + 4 * 64 * 56 * 56) * 4
    ring = int(min(4, max(2, np.ceil(2.2 * L2_BYTES / footprint))))
    for _ in range(ring - 1):
        graphs.append(build_graph(ctx, configs.resnet18, batch=per))
    torch.cuda.synchronize()
    names = [n for n, _ in g0.steps()]
    kernels = [k for _, k in g0.steps()]
    fc_on_tc = any(n == "matmul" and k.startswith("tc_") for n, k in zip(names, kernels))
    step_flops = per * (CONV_FLOPS + (FC_FLOPS if fc_on_tc else 0))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    slots = (args.steps + ring - 1) // ring
    for i in range(warmup):
        graphs[i % ring][0].run_profiled(0, slots)
    ctx.sync_check()
    for g, _, _ in graphs:
        g.profile_other_ms(slots)   # forget the warm-up passes

    # ---- device-resident throughput (`value`): K steps, step by step with events around the non-tensor-core steps ----
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    l0 = ctx.launches()
    e0.record()
    for i in range(args.steps):
        graphs[i % ring][0].run_profiled(i // ring, slots)
    e1.record()
    barrier()
    launches = ctx.launches() - l0
    ms_total = e0.elapsed_time(e1)
    other_ms = sum(g.profile_other_ms(slots) for g, _, _ in graphs)   # exactly the slots run in the timed region
    tc_ms = ms_total - other_ms
    ctx.sync_check()

    # ---- the same steps as pure CUDA-graph replays (what Graph.run does for a user), for the record ----
    for i in range(warmup):
        graphs[i % ring][0].run()
    barrier()
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for i in range(args.steps):
        graphs[i % ring][0].run()
    r1.record()
    barrier()
    replay_ms = r0.elapsed_time(r1)

    # ---- end to end through host buffers (`e2e`): every step copies the rank's images from pinned host memory, replays
    #      the graph and copies the logits back; three streams, so that the copies of neighbouring steps overlap the kernels ----
    import ctypes as C
    hx = [torch.from_numpy(np.ascontiguousarray(b0.data[0][1])).pin_memory() for _ in range(ring)]
    hy = [torch.empty((per, 1000)).pin_memory() for _ in range(ring)]
    s_in, s_k, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(ring)]
    ev_k = [torch.cuda.Event() for _ in range(ring)]
    ev_out = [torch.cuda.Event() for _ in range(ring)]
    x_dev, y_dev = [None] * ring, [None] * ring
    for j, (g, b, o) in enumerate(graphs):
        x_dev[j] = _device_tensor(g.device_ptr(b.data[0][0]), x_shape, local)
        y_dev[j] = _device_tensor(g.device_ptr(o), (per, 1000), local)

    def e2e_step(i, copy_only=False):
        j = i % ring
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_k[j])          # the kernels that last read this slot are done
            x_dev[j].copy_(hx[j], non_blocking=True)
            ev_in[j].record()
        with torch.cuda.stream(s_k):
            s_k.wait_event(ev_in[j])
            s_k.wait_event(ev_out[j])         # the previous result of this slot has left the device
            if not copy_only:
                graphs[j][0].run(stream=C.c_void_p(s_k.cuda_stream))
            ev_k[j].record()
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_k[j])
            hy[j].copy_(y_dev[j], non_blocking=True)
            ev_out[j].record()

    def e2e_region(copy_only):
        for i in range(max(3, warmup)):
            e2e_step(i, copy_only)
        barrier()
        t0 = time.perf_counter()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(s_in)
        for i in range(args.steps):
            e2e_step(i, copy_only)
        s_out.synchronize()
        a1.record(s_out)
        barrier()
        return a0.elapsed_time(a1), (time.perf_counter() - t0) * 1000.0

    e2e_ms, e2e_wall = e2e_region(False)
    copy_ms, _ = e2e_region(True)   # the host-side ceiling of that path: the same copies with no kernels between them
    clocks = sampler.stop() if rank == 0 else None
    ctx.sync_check()

    # ---- max over ranks ----
    ms_total, e2e_ms, replay_ms, copy_ms = max_over_ranks([ms_total, e2e_ms, replay_ms, copy_ms], world, dev)
    tc_ms_sum, flops_sum = sum_over_ranks([tc_ms, step_flops * args.steps], world, dev)
    (launches_sum,) = sum_over_ranks([launches], world, dev)
    extras = not args.no_extras
    r3d = r3d_throughput(ctx, world, dev) if extras else None
    if rank == 0:
        pk, pk_kind = peaks()
        # all ranks' flops / all ranks' kernel time = the per-GPU rate of the tensor-core kernel
        achieved = flops_sum / (tc_ms_sum * 1e-3) / 1e12
        peak = pk["bf16_tflops_sustained"]
        line = {"metric": "images_per_s", "value": sharded_throughput(GLOBAL_BATCH, args.steps, ms_total), "unit": "images/s",
                "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_total / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "tf32x3 (fp32 in/out)",
                "data": "synthetic", "config": config_for(world),
                "e2e": {"value": sharded_throughput(GLOBAL_BATCH, args.steps, e2e_ms), "unit": "images/s",
                        "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes, "wall_ms_per_step": e2e_wall / args.steps,
                        "copies_only_ms_per_step": copy_ms / args.steps,
                        "copies_only_aggregate_gbs": world * (in_bytes + out_bytes) * args.steps / (copy_ms * 1e-3) / 1e9},
                "gpu_launches": int(launches_sum), "clocks": clocks,
                "graph_replay": {"ms_per_step": replay_ms / args.steps, "images_per_s": sharded_throughput(GLOBAL_BATCH, args.steps, replay_ms),
                                 "note": "the same steps as CUDA-graph replays (Graph.run), no events inside"},
                "roofline": {"bound": "tensor", "kernel": "k_igemm (" + next(k for k in kernels if k.startswith("tc_")) + ")",
                             "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                             "traffic": RN18_B64_DRAM_TRAFFIC if (world == 1 and RN18_B64_DRAM_TRAFFIC) else None,
                             "peak_source": f"{pk_kind} bf16 sustained",
                             "flops_per_step": step_flops, "tc_ms_per_step": tc_ms_sum / world / args.steps,
                             "other_kernels_ms_per_step": (ms_total - tc_ms_sum / world) / args.steps,
                             "how": "fp32-equivalent conv+FC flops of the timed steps / (region time - CUDA-event time of the steps that are not tensor-core launches)"},
                "ring": ring}
        if r3d is not None:
            line["model_throughput"] = {"c5_r3d18": r3d}
        if world == 1 and extras:
            lat = config_latencies(ctx)
            line["batch1_latency_ms"] = lat
            try:
                line["lib_baseline"] = library_baseline(ctx, lat)
            except Exception as e:  # the harness is optional; the product numbers stand without it
                line["lib_baseline"] = {"error": repr(e)}
        if world == 1 and not args.no_cpu_baseline:
            try:
                secs, hb = cpu_reference_step(1)
                secs2, hb = cpu_reference_step(1)
                line["cpu_baseline"] = cpu_baseline_block(1, min(secs, secs2), hb)
            except Exception as e:  # the checker is optional infrastructure; the GPU numbers stand without it
                line["cpu_baseline"] = {"error": str(e)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    ctx.close()


# DRAM traffic of the tensor-core launches of one batch-64 step (dram__bytes_read.sum + dram__bytes_write.sum summed over
# the step's k_igemm launches, one ncu capture of this workload): filled in from the committed profile summary.
RN18_B64_DRAM_TRAFFIC = 1050.3e6


def _device_tensor(ptr, shape, device_index):
    """A torch tensor viewing `ptr` (device memory owned by a graph) without taking ownership."""
    import torch

    class _Arr:
        __cuda_array_interface__ = {"shape": tuple(int(s) for s in shape), "typestr": "<f4", "data": (int(ptr), False), "version": 3,
                                    "strides": None}

    return torch.as_tensor(_Arr(), device=torch.device("cuda", device_index))


if __name__ == "__main__":
    main()
