"""Per-kernel measurements against the roofline that bounds each kernel (python -m pet_b200.perf_report [group ...]).

Groups: `layout` (index-map kernels at sizes far beyond L2: achieved HBM GB/s), `conv` / `matmul` (tensor-core kernels:
achieved fp32-equivalent TFLOP/s and the TF32 issue rate), `convtrans` (transposed convolution), `banded` (G2BMM / GBMML
at the one shape the reference ships kernels for, and a short-sequence one), `rewrite` (config 1's H->N rewrite restored by
the correction kernel and by halo transposes, each route replayed as a CUDA graph).  The `once_*` groups launch every kernel
of a family exactly once (after one warm-up launch) at a size beyond the L2 and print the algorithmic bytes / flops of
each launch: they exist to be run under a profiler, which supplies the durations and the DRAM traffic (`once_ops`: element-wise,
activation, BatchNorm, pooling, softmax, LayerNorm, row mean, small-m matmul, pad / slice / concat; `once_matmul`: the
BERT-base matmul shapes; `once_conv`: the dilated-conv layer, a correction window, a transposed convolution;
`once_attention`: the fused attention launch on BERT-base's heads; `once_bert`: one BERT-base forward pass; `once_rn18 [batch]`: one ResNet-18 forward pass, operator
by operator).  Times come from the C ABI's timing entry point
(CUDA events around repeated launches on plan-owned operands).  Peaks are read from MEASURED_PEAKS.json at the
repository root when present.
"""
import json
import os
import sys

import numpy as np

from .configs import BATCH_TO_SPACE, SPACE_TO_BATCH, H2N, N2H, D2W
from .ops import Context

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


LAYOUT = [
    ("space_to_batch x64", (64, 512, 64, 64), SPACE_TO_BATCH),
    ("batch_to_space x64", (256, 512, 32, 32), BATCH_TO_SPACE),
    ("H2N x256", (256, 64, 56, 56), [H2N]),
    ("N2H x256", (512, 64, 28, 56), [N2H]),
    ("D2W (de-interleave W)", (64, 512, 64, 64), [D2W]),
    ("swap H,W", (64, 64, 128, 256), [(-1, [0, 1, 3, 2], 2)]),
    ("NCHW->NHWC", (64, 256, 56, 56), [(-1, [0, 2, 3, 1], 2)]),
    ("head split [s,h,d]->[h,s,d]", (4096, 12, 64, 16), [(-1, [1, 0, 2, 3], 2)]),
    ("matmul transpose", (64, 1024, 2048), [(-1, [0, 2, 1], 2)]),
]
CONV = [
    ("c1 3x3 64->64 56x56", (1, 64, 56, 56), (64, 64, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("c2 dense 3x3 512->512 [4,32,32]", (4, 512, 32, 32), (512, 512, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("c2 dilated 3x3 512->512 64x64", (1, 512, 64, 64), (512, 512, 3, 3), (2, 2, 1, 1, 2, 2)),
    ("c2 dense batch 16", (64, 512, 32, 32), (512, 512, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("resnet stem 7x7 s2", (1, 3, 224, 224), (64, 3, 7, 7), (3, 3, 2, 2, 1, 1)),
    ("resnet 3x3 512 7x7", (1, 512, 7, 7), (512, 512, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("resnet-18 conv batch 64 (128ch 28x28)", (64, 128, 28, 28), (128, 128, 3, 3), (1, 1, 1, 1, 1, 1)),
]
MATMUL = [("bert qkv 128x768x768", 1, 128, 768, 768, False, False), ("bert scores 12x128x128x64", 12, 128, 128, 64, False, True),
          ("bert ffn1 128x3072x768", 1, 128, 3072, 768, False, False), ("bert ffn2 128x768x3072", 1, 128, 768, 3072, False, False),
          ("square 4096", 1, 4096, 4096, 4096, False, False)]


CONVTRANS = [  # x {n,h,w,f}, w {r,s,f,c}, (ph, pw, sh, sw, oph, opw)
    ("2x upsample 4x4 256->128 8x8 b4", (4, 8, 8, 256), (4, 4, 256, 128), (1, 1, 2, 2, 0, 0)),
    ("2x upsample 4x4 128->64 32x32 b8", (8, 32, 32, 128), (4, 4, 128, 64), (1, 1, 2, 2, 0, 0)),
    ("stride 1 3x3 128->128 32x32 b8", (8, 32, 32, 128), (3, 3, 128, 128), (1, 1, 1, 1, 0, 0)),
]
BANDED = [(1, 10000, 64, 1000, 1), (1, 10000, 64, 1000, 4), (8, 10000, 64, 1000, 1), (12, 4096, 64, 256, 1)]  # b, n, m, w, d


def _graph_time(fn, iters=200):
    """Microseconds per replay of `fn` captured as one CUDA graph (launch overheads of the Python layer excluded)."""
    import torch
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(10):
        g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def rewrite_routes(ctx):
    import torch
    gen = torch.Generator(device="cuda").manual_seed(1)
    x = torch.rand((1, 64, 56, 56), device="cuda", generator=gen) * 2 - 1
    w = torch.rand((64, 64, 3, 3), device="cuda", generator=gen) * 2 - 1
    H2N, N2H_ = (2, [[0, 2], 1, -1, 3], -2), (0, [0, 1, [-1, 2], 3], 2)
    plans = {}
    for shape in ((1, 64, 56, 56), (2, 64, 28, 56), (2, 64, 29, 56)):  # weights are packed once, outside the replayed part
        plans[shape] = ctx.conv2d_plan(shape, w.shape, 1, 1)
        ctx.conv2d_set_weights(plans[shape], w)
    plan = plans[(1, 64, 56, 56)]

    def conv(t):
        return ctx.conv2d_run(plans[tuple(t.shape)], t)

    def original():
        return conv(x)

    def corrected():
        y = ctx.transpose(conv(ctx.transpose(x, *H2N)), *N2H_)
        return ctx.conv2d_correct(plan, x, y, 27, 2)

    def halo():
        return ctx.transpose_halo(conv(ctx.transpose_halo(x, *H2N, "copys", 1)), *N2H_, "dels", 1)

    y0 = original()
    print(f"rewrite max |corrected - original| = {float((corrected() - y0).abs().max()):.3g}, "
          f"max |halo - original| = {float((halo() - y0).abs().max()):.3g}")
    for name, fn in (("original conv", original), ("H2N + conv + N2H + correction of rows 27,28", corrected),
                     ("halo H2N + conv + dropping N2H", halo)):
        print(f"rewrite {name:46s} {_graph_time(fn):8.1f} us per replay")


def once_ops(ctx):
    """One launch of every HBM-bound operator kernel at a size far beyond the L2, each preceded by one warm-up launch."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(3)
    r = lambda *shape: torch.rand(shape, device="cuda", generator=g) - 0.5
    MB = lambda n: f"{n / 1e6:9.1f} MB algorithmic"
    x = r(64, 64, 112, 112)   # 205 MB
    y = r(64, 64, 112, 112)
    runs = [("eltwise add + relu (2 in, 1 out)", lambda: ctx.eltwise("add", [x, y], act="relu"), 12 * x.numel()),
            ("activation gelu", lambda: ctx.activation(x, "gelu"), 8 * x.numel()),
            ("batchnorm", lambda: ctx.batchnorm(x, r(64), r(64), r(64), r(64).abs() + 1), 8 * x.numel()),
            ("maxpool 3x3 s2 p1 (ResNet stem)", lambda: ctx.maxpool(x, 3, 3, 1, 1, 1, 1, 2, 2), 4 * x.numel() * 1.25),
            ("avgpool 7x7 global", lambda: ctx.avgpool(r(2048, 512, 7, 7), 7, 7, 0, 0, 1, 1), 4 * 2048 * 512 * 50),
            ("rowmean 12544 cols", lambda: ctx.rowmean(x.view(64 * 64, 12544), 12544), 4 * x.numel()),
            ("softmax last axis 128 cols", lambda: ctx.softmax(r(12 * 512, 128, 128)), 8 * 12 * 512 * 128 * 128),
            ("softmax last axis 1000 cols", lambda: ctx.softmax(r(65536, 1000)), 8 * 65536 * 1000),
            ("softmax axis 1 of [64,1000,784]", lambda: ctx.softmax(r(64, 1000, 784), 1), 8 * 64 * 1000 * 784),
            ("layernorm 768 cols", lambda: ctx.layernorm(r(65536, 768), r(768), r(768)), 8 * 65536 * 768),
            ("matmul m=1 (classifier head 512 -> 1000)", lambda: ctx.matmul(r(1, 1, 512), r(1, 512, 1000)), 4 * 512 * 1000),
            ("matmul m=8, 4096 x 16384 weights", lambda: ctx.matmul(r(1, 8, 4096), r(1, 4096, 16384)), 4 * 4096 * 16384),
            ("pad [64,64,112,112] by 1", lambda: ctx.pad(x, [0, 0, 1, 1], [0, 0, 1, 1]), 8 * x.numel()),
            ("slice [64,64,112,112] by 1", lambda: ctx.slice(x, [0, 0, 1, 1], [0, 0, 1, 1]), 8 * x.numel() * 0.96),
            ("concat 2 x [64,64,112,112] on C", lambda: ctx.concat([x, y], 1), 16 * x.numel())]
    for name, fn, nbytes in runs:
        fn()
        torch.cuda.synchronize()
        fn()
        torch.cuda.synchronize()
        print(f"once_ops  {name:44s} {MB(nbytes)}")


def once_matmul(ctx):
    import torch
    for name, b, m, n, k, ta, tb in MATMUL[:4]:
        a = torch.rand((b, m, k), device="cuda") - 0.5
        w = torch.rand((b, n, k) if tb else (b, k, n), device="cuda") - 0.5
        plan = ctx.matmul_plan(a.shape, w.shape, ta, tb)
        ctx.matmul_set_weights(plan, w)
        for _ in range(2):
            ctx.matmul_run(plan, a, None)
            torch.cuda.synchronize()
        print(f"once_matmul  {name:30s} {2.0 * b * m * n * k / 1e9:8.3f} GFLOP, {4.0 * b * (m * k + k * n + m * n) / 1e6:7.2f} MB algorithmic")


def once_conv(ctx):
    import torch
    x = torch.randn((4, 512, 32, 32), device="cuda")
    w = torch.randn((512, 512, 3, 3), device="cuda") * 0.02
    plan = ctx.conv2d_plan(x.shape, w.shape, 1, 1)
    ctx.conv2d_set_weights(plan, w)
    for _ in range(2):
        ctx.conv2d_run(plan, x)
        torch.cuda.synchronize()
    print(f"once_conv  dense conv of the dilated layer [4,512,32,32] x [512,512,3,3]: 19.327 GFLOP, 26.21 MB algorithmic")
    xp = torch.randn((16, 64, 56, 56), device="cuda")
    wp = torch.randn((64, 64, 3, 3), device="cuda") * 0.06
    pp = ctx.conv2d_plan(xp.shape, wp.shape, 1, 1)
    ctx.conv2d_set_weights(pp, wp)
    for _ in range(2):
        ctx.conv2d_run(pp, xp)
        torch.cuda.synchronize()
    print(f"once_conv  persistent tiles: 3x3 conv 64 -> 64 channels, 56x56, batch 16 (400 pixel tiles): 3.699 GFLOP, 25.8 MB algorithmic")
    x1, w1 = torch.randn((1, 64, 56, 56), device="cuda"), torch.randn((64, 64, 3, 3), device="cuda")
    p1 = ctx.conv2d_plan(x1.shape, w1.shape, 1, 1)
    ctx.conv2d_set_weights(p1, w1)
    y1 = ctx.conv2d_run(p1, x1)
    for _ in range(2):
        ctx.conv2d_correct(p1, x1, y1, 27, 2)
        torch.cuda.synchronize()
    print("once_conv  correction window rows 27-28 of config 1: 8.26 MFLOP, 0.233 MB algorithmic")
    name, xs, ws, (ph, pw, sh, sw, oph, opw) = CONVTRANS[1]
    pt = ctx.convtrans_plan(xs, ws, ph, pw, sh, sw, 1, 1, oph, opw)
    xt, wt = torch.rand(xs, device="cuda") - 0.5, torch.rand(ws, device="cuda") - 0.5
    ctx.convtrans_run(pt, xt, wt)
    torch.cuda.synchronize()
    ctx.convtrans_run(pt, xt)
    torch.cuda.synchronize()
    print(f"once_conv  transposed conv {name}: {2.0 * np.prod(xs) * ws[0] * ws[1] * ws[3] / 1e9:.3f} GFLOP useful")


def once_banded(ctx):
    """G2BMM and GBMML at the shape the reference ships kernels for, each launched twice (warm-up + one)."""
    import torch
    b, n, m, w, d = BANDED[0]
    q, k = torch.randn((b, n, m), device="cuda"), torch.randn((b, n, m), device="cuda")
    p = torch.randn((b, n, 2 * w + 1), device="cuda")
    for _ in range(2):
        ctx.g2bmm(q, k, w, d)
        torch.cuda.synchronize()
    for _ in range(2):
        ctx.gbmml(p, k, d)
        torch.cuda.synchronize()
    fl, by = 2.0 * b * n * (2 * w + 1) * m, 4.0 * b * n * (2 * m + 2 * w + 1)
    print(f"once_banded  g2bmm / gbmml b{b} n{n} m{m} w{w} d{d}: {fl / 1e9:.3f} GFLOP, {by / 1e6:.1f} MB algorithmic each")


ATTENTION = [(12, 128, 128, 64, 64), (96, 128, 128, 64, 64)]  # BERT-base heads at batch 1 and 8: bs, queries, keys, head widths


def once_attention(ctx):
    """The fused attention launch on BERT-base's heads, twice (warm-up + one)."""
    import torch
    bs, m, n, kd, d = ATTENTION[0]
    q, k, v = (torch.randn(s, device="cuda") for s in ((bs, m, kd), (bs, n, kd), (bs, n, d)))
    for _ in range(2):
        ctx.attention(q, k, v)
        torch.cuda.synchronize()
    print(f"once_attention  bs{bs} m{m} n{n} kd{kd} d{d}: {2.0 * bs * m * n * (kd + d) / 1e6:.1f} MFLOP, "
          f"{4.0 * bs * (m * kd + n * kd + n * d + m * d) / 1e6:.2f} MB algorithmic")


def once_rn18(ctx, batch):
    """One ResNet-18 forward pass at `batch`, operator by operator (no CUDA graph), after one warm-up pass."""
    import torch
    from . import configs
    from .graph import Graph
    g = Graph(ctx)
    b = configs.GraphBuilder(g)
    g.setOutputs([configs.resnet18(b, batch=batch)])
    g.compile(cuda_graph=False)
    b.load()
    for _ in range(2):
        g.run()
        torch.cuda.synchronize()
    print(f"once_rn18  batch {batch}: {g.num_launches()} launches per pass, {batch * 3.628146688:.2f} GFLOP algorithmic (conv + FC)")


def once_bert(ctx):
    """One BERT-base (seq 128) forward pass, operator by operator (no CUDA graph), after one warm-up pass."""
    import torch
    from . import configs
    from .graph import Graph
    g = Graph(ctx)
    b = configs.GraphBuilder(g)
    g.setOutputs([configs.bert_encoder(b)])
    g.compile(cuda_graph=False)
    b.load()
    for _ in range(2):
        g.run()
        torch.cuda.synchronize()
    print(f"once_bert  {g.num_launches()} launches per pass")


def main(argv):
    groups = argv or ["layout", "conv", "matmul"]
    pk, kind = peaks()
    pk_kind = kind
    ctx = Context(0)
    print(f"peaks ({kind}): HBM {pk['hbm_gbs']:.0f} GB/s, bf16 {pk['bf16_tflops']:.0f} TFLOP/s burst")
    if "layout" in groups:
        for name, shape, ops in LAYOUT:
            plan = ctx.transpose_plan(shape, ops)
            ms = plan.time(20, 5)
            gbs = 8.0 * np.prod(shape) / ms / 1e6
            print(f"layout  {name:30s} {plan.kernel:8s} {ms * 1e3:9.1f} us {gbs:8.0f} GB/s  {gbs / pk['hbm_gbs']:.2f} of {kind} HBM peak")
    if "conv" in groups:
        for name, xs, ws, (ph, pw, sh, sw, dh, dw) in CONV:
            plan = ctx.conv2d_plan(xs, ws, ph, pw, sh, sw, dh, dw)
            ms = plan.time(50, 10)
            fl = 2.0 * np.prod(plan.out_shape) * ws[1] * ws[2] * ws[3]
            tf = fl / ms / 1e9
            print(f"conv    {name:38s} {plan.kernel:14s} {ms * 1e3:9.1f} us {tf:7.1f} TFLOP/s fp32-equivalent, "
                  f"{3 * tf:7.1f} TF32 issued = {3 * tf / (pk['bf16_tflops'] / 2):.2f} of bf16/2")
    if "matmul" in groups:
        import torch
        for name, b, m, n, k, ta, tb in MATMUL:
            ashape, bshape = ((b, k, m) if ta else (b, m, k)), ((b, n, k) if tb else (b, k, n))
            plan = ctx.matmul_plan(ashape, bshape, ta, tb)
            ms = plan.time(50, 10)  # both operands activations: B is split on every launch
            a, w = torch.rand(ashape, device="cuda") - 0.5, torch.rand(bshape, device="cuda") - 0.5
            ctx.matmul_set_weights(plan, w)  # B as a weight: split once, outside the replayed part
            us_w = _graph_time(lambda: ctx.matmul_run(plan, a, None))
            tf = 2.0 * b * m * n * k / 1e6
            print(f"matmul  {name:30s} {plan.kernel:14s} {ms * 1e3:9.1f} us {tf / (ms * 1e3):7.1f} TFLOP/s with B an activation; "
                  f"{us_w:8.1f} us {tf / us_w:7.1f} TFLOP/s with B a pre-split weight (graph replay)")
    if "convtrans" in groups:
        import torch
        for name, xs, ws, (ph, pw, sh, sw, oph, opw) in CONVTRANS:
            plan = ctx.convtrans_plan(xs, ws, ph, pw, sh, sw, 1, 1, oph, opw)
            x = torch.rand(xs, device="cuda") - 0.5
            w = torch.rand(ws, device="cuda") - 0.5
            ctx.convtrans_run(plan, x, w)  # weight-only work once, outside the replayed part
            us = _graph_time(lambda: ctx.convtrans_run(plan, x))
            useful = 2.0 * np.prod(xs) * ws[0] * ws[1] * ws[3]  # every input element meets every tap of every output channel
            print(f"convtr  {name:34s} {plan.kernel:14s} {us:9.1f} us per CUDA-graph replay {useful / us / 1e6:7.1f} TFLOP/s useful")
    if "banded" in groups:
        for b, n, m, w, d in BANDED:
            fl = 2.0 * b * n * (2 * w + 1) * m
            by = 4.0 * b * n * (2 * m + 2 * w + 1)
            for kind in ("g2bmm", "gbmml"):
                ms = ctx.banded_time(kind, b, n, m, w, d, rounds=20, warmup=3)
                print(f"banded  {kind} b{b} n{n} m{m} w{w} d{d}: {ms * 1e3:9.1f} us {fl / ms / 1e9:6.1f} TFLOP/s fp32, "
                      f"{by / ms / 1e6:6.0f} GB/s = {by / ms / 1e6 / pk['hbm_gbs']:.2f} of {pk_kind} HBM peak")
    if "attention" in groups:
        import torch
        for bs, m, n, kd, d in ATTENTION:
            q, k, v = (torch.randn(s, device="cuda") for s in ((bs, m, kd), (bs, n, kd), (bs, n, d)))
            us = _graph_time(lambda: ctx.attention(q, k, v))
            us3 = _graph_time(lambda: ctx.matmul(ctx.softmax(ctx.matmul(q, k, transB=True), 2), v))
            print(f"attention  bs{bs} m{m} n{n} kd{kd} d{d}: one launch {us:7.1f} us; matmul -> softmax -> matmul {us3:7.1f} us (graph replays)")
    if "rewrite" in groups:
        rewrite_routes(ctx)
    if "once_ops" in groups:
        once_ops(ctx)
    if "once_matmul" in groups:
        once_matmul(ctx)
    if "once_conv" in groups:
        once_conv(ctx)
    if "once_banded" in groups:
        once_banded(ctx)
    if "once_attention" in groups:
        once_attention(ctx)
    if "once_bert" in groups:
        once_bert(ctx)
    if "once_rn18" in groups:
        i = groups.index("once_rn18")
        once_rn18(ctx, int(groups[i + 1]) if i + 1 < len(groups) and groups[i + 1].isdigit() else 64)
    ctx.sync_check()
    ctx.close()


if __name__ == "__main__":
    main(sys.argv[1:])
