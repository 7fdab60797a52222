"""GPU: the benchmark configurations at FULL size — every layer shape and the whole graphs — against the CPU oracle
(double-accumulated) and against the vendor libraries computing the same graph in true fp32 (cuDNN / cuBLAS with TF32
switched off, through torch; harness only).  The asserted metric is the contract's (conftest.contract_err, bound 1e-3).

The long reductions are the point: K = 4608 (config 2, last ResNet-18 stage), 3072 (BERT FFN), 13824 (last ResNet3D
stage) are where a tensor-core accumulator that truncates after every MMA drifts furthest from the exact sum."""
import numpy as np
import pytest
import torch

from conftest import contract_err, rms_rel_err, scale_err

pytestmark = pytest.mark.gpu
TOL = 1e-3


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def report(name, got, want):
    c, r, s = contract_err(got, want), rms_rel_err(got, want), scale_err(got, want)
    print(f"\n[parity] {name}: contract {c:.2e}  rms-floor {r:.2e}  scale {s:.2e}")
    return c


def lib_fp32():
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False


# ---- config 2 ------------------------------------------------------------------------------------------------------
def test_c2_full_size_all_filters_vs_oracle_and_library(ctx, oracle):
    from pet_b200 import configs
    from test_gpu_layout import S2B, B2S
    x, w = configs.c2_tensors()
    xd, wd = dev(x), dev(w)
    direct = ctx.conv2d(xd, wd, 2, 2, 1, 1, 2, 2)
    rewritten = ctx.transpose_chain(ctx.conv2d(ctx.transpose_chain(xd, S2B), wd, 1, 1), B2S)
    ctx.sync_check()
    assert torch.equal(direct, rewritten)
    got = direct.cpu().numpy()
    want = oracle.conv2d(x, w, pad=(2, 2), dil=(2, 2), wide=True)
    assert report("c2 dilated conv K=4608 vs oracle", got, want) <= TOL
    lib_fp32()
    lib = torch.nn.functional.conv2d(xd, wd, padding=2, dilation=2).cpu().numpy()
    assert report("c2 dilated conv vs cuDNN fp32", got, lib) <= TOL + report("   (cuDNN fp32 itself vs oracle)", lib, want)


# ---- every conv shape of ResNet-18 at 224x224, batch 1 -----------------------------------------------------------------
RN18_LAYERS = [  # (name, cin, cout, hw_in, k, stride, pad)
    ("stem7x7", 3, 64, 224, 7, 2, 3), ("s1_3x3", 64, 64, 56, 3, 1, 1), ("s2_3x3_down", 64, 128, 56, 3, 2, 1),
    ("s2_1x1_down", 64, 128, 56, 1, 2, 0), ("s2_3x3", 128, 128, 28, 3, 1, 1), ("s3_3x3_down", 128, 256, 28, 3, 2, 1),
    ("s3_1x1_down", 128, 256, 28, 1, 2, 0), ("s3_3x3", 256, 256, 14, 3, 1, 1), ("s4_3x3_down", 256, 512, 14, 3, 2, 1),
    ("s4_1x1_down", 256, 512, 14, 1, 2, 0), ("s4_3x3", 512, 512, 7, 3, 1, 1),
]


@pytest.mark.parametrize("layer", RN18_LAYERS, ids=[l[0] for l in RN18_LAYERS])
def test_resnet18_layer_full_size(ctx, oracle, layer):
    name, cin, cout, hw, k, stride, pad = layer
    rng = np.random.default_rng(3000 + cin * 7 + hw + k)
    x = np.maximum(rng.standard_normal((1, cin, hw, hw)), 0 if cin > 3 else -9).astype(np.float32)  # post-ReLU activations
    w = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
    got = ctx.conv2d(dev(x), dev(w), pad, pad, stride, stride, bias=dev(b)).cpu().numpy()
    ctx.sync_check()
    want = oracle.conv2d(x, w, b, pad=(pad, pad), stride=(stride, stride), wide=True)
    assert report(f"resnet18 {name} K={cin * k * k}", got, want) <= TOL
    lib_fp32()
    lib = torch.nn.functional.conv2d(dev(x), dev(w), dev(b), stride, pad).cpu().numpy()
    assert report(f"resnet18 {name} vs cuDNN fp32", got, lib) <= TOL + report("   (cuDNN fp32 itself vs oracle)", lib, want)


# ---- every matmul shape of BERT-base at seq 128 -----------------------------------------------------------------------
BERT_MM = [  # (name, b, m, k, n, transB)
    ("qkv_proj", 1, 128, 768, 768, False), ("qk_t", 12, 128, 64, 128, True), ("pv", 12, 128, 128, 64, False),
    ("ffn_up", 1, 128, 768, 3072, False), ("ffn_down", 1, 128, 3072, 768, False), ("qkv_merged", 1, 128, 768, 2304, False),
]


@pytest.mark.parametrize("case", BERT_MM, ids=[c[0] for c in BERT_MM])
def test_bert_matmul_full_size(ctx, oracle, case):
    name, bs, m, k, n, tb = case
    rng = np.random.default_rng(4000 + k + n)
    a = rng.standard_normal((bs, m, k)).astype(np.float32)
    lim = np.sqrt(6.0 / (k + n))
    b = rng.uniform(-lim, lim, (bs, n, k) if tb else (bs, k, n)).astype(np.float32)
    got = ctx.matmul(dev(a), dev(b), transB=tb).cpu().numpy()
    ctx.sync_check()
    want = oracle.matmul(a, b, None, False, tb, wide=True)
    assert report(f"bert {name} K={k}", got, want) <= TOL
    lib_fp32()
    lib = torch.matmul(dev(a), dev(b).transpose(1, 2) if tb else dev(b)).cpu().numpy()
    assert report(f"bert {name} vs cuBLAS fp32", got, lib) <= TOL + report("   (cuBLAS fp32 itself vs oracle)", lib, want)


# ---- every conv shape of ResNet3D-18 at 16 x 112 x 112, the oracle on a subset of the filters ---------------------------
R3D_LAYERS = [  # (name, cin, cout, d, hw, kernel, stride, pad, filters the oracle computes)
    ("stem3x7x7", 3, 64, 16, 112, (3, 7, 7), (1, 2, 2), (1, 3, 3), 64), ("s1_3x3x3", 64, 64, 16, 56, (3, 3, 3), (1, 1, 1), (1, 1, 1), 8),
    ("s2_down", 64, 128, 16, 56, (3, 3, 3), (2, 2, 2), (1, 1, 1), 16), ("s2_1x1x1", 64, 128, 16, 56, (1, 1, 1), (2, 2, 2), (0, 0, 0), 128),
    ("s2_3x3x3", 128, 128, 8, 28, (3, 3, 3), (1, 1, 1), (1, 1, 1), 16), ("s3_down", 128, 256, 8, 28, (3, 3, 3), (2, 2, 2), (1, 1, 1), 32),
    ("s3_3x3x3", 256, 256, 4, 14, (3, 3, 3), (1, 1, 1), (1, 1, 1), 32), ("s4_down", 256, 512, 4, 14, (3, 3, 3), (2, 2, 2), (1, 1, 1), 64),
    ("s4_3x3x3", 512, 512, 2, 7, (3, 3, 3), (1, 1, 1), (1, 1, 1), 128),
]


@pytest.mark.parametrize("layer", R3D_LAYERS, ids=[l[0] for l in R3D_LAYERS])
def test_r3d18_layer_full_size(ctx, oracle, layer):
    name, cin, cout, d, hw, kern, stride, pad, nf = layer
    rng = np.random.default_rng(5000 + cin + hw)
    x = np.maximum(rng.standard_normal((1, cin, d, hw, hw)), 0 if cin > 3 else -9).astype(np.float32)
    w = (rng.standard_normal((cout, cin) + kern) * np.sqrt(2.0 / (cin * np.prod(kern)))).astype(np.float32)
    y = ctx.conv3d(dev(x), dev(w), pad, stride)
    ctx.sync_check()
    sel = np.sort(rng.choice(cout, nf, replace=False))  # the whole layer runs on the GPU; the oracle checks these filters
    want = oracle.conv3d(x, w[sel], pad=pad, stride=stride, wide=True)
    got = y.cpu().numpy()
    assert report(f"r3d18 {name} K={cin * int(np.prod(kern))} ({nf} of {cout} filters)", got[:, sel], want) <= TOL
    lib_fp32()
    lib = torch.nn.functional.conv3d(dev(x), dev(w), None, stride, pad).cpu().numpy()
    assert report(f"r3d18 {name} vs cuDNN fp32 (all filters)", got, lib) <= TOL + report("   (cuDNN fp32 itself vs oracle)", lib[:, sel], want)


# ---- whole graphs at full size ----------------------------------------------------------------------------------------
def _whole(ctx, build, **kw):
    from test_gpu_graph import run_config, oracle_config
    import os, sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline"))
    from torch_backend import TorchBuilder
    _, _, y = run_config(ctx, build, **kw)
    want = oracle_config(build, **kw)
    lib = build(TorchBuilder(tf32=False), **kw).cpu().numpy()
    return y, want, lib


def _check_whole(name, y, want, lib, depth):
    """A whole graph compounds the rounding of its operators: every conv / matmul meets the contract on its own inputs
    (the tests above and test_bert_layer_operators_in_situ), and independent errors of `depth` such operators in sequence
    add up like a random walk, so the end-to-end bound is 1e-3 * sqrt(depth).  The library's own fp32 execution of the
    same graph is measured beside ours; the two must agree within the sum of their distances from the oracle."""
    lib_own = report(f"   (library fp32 execution of {name} vs oracle)", lib, want)
    ours = report(f"{name} vs oracle", y, want)
    vs_lib = report(f"{name} vs library fp32 execution", y, lib)
    assert ours <= TOL * np.sqrt(depth)
    assert vs_lib <= TOL + lib_own + ours


def test_resnet18_full_size_graph(ctx):
    from pet_b200 import configs
    y, want, lib = _whole(ctx, configs.resnet18)
    assert y.shape == want.shape == (1, 1, 1000)
    _check_whole("resnet18 224x224 logits", y, want, lib, depth=18)


def test_bert_base_full_size_graph(ctx):
    from pet_b200 import configs
    y, want, lib = _whole(ctx, configs.bert_encoder)
    assert y.shape == want.shape == (1, 128, 768)
    _check_whole("bert-base seq128 output", y, want, lib, depth=72)


def test_r3d18_full_size_graph(ctx):
    from pet_b200 import configs
    y, want, lib = _whole(ctx, configs.r3d18)
    assert y.shape == want.shape == (1, 1, 400)
    _check_whole("r3d18 16x112x112 logits", y, want, lib, depth=18)


def test_bert_layer_operators_in_situ(ctx, oracle):
    """One full-size BERT-base layer, operator by operator: each operator runs on the GPU on the outputs of the GPU
    operators before it, and the oracle evaluates the same operator on those same inputs — the per-operator contract,
    measured inside the graph where the inputs have the distributions the model produces."""
    from pet_b200 import configs
    seq, hidden, heads, ffn = 128, 768, 12, 3072
    hd = hidden // heads
    x = configs.rng_for(4, 0).standard_normal((1, seq, hidden)).astype(np.float32)
    W = [configs.xavier_uniform(configs.rng_for(4, i + 1), s)[None] for i, s in
         enumerate([(hidden, hidden)] * 4 + [(hidden, ffn), (ffn, hidden)])]
    ones, zeros = np.ones(hidden, np.float32), np.zeros(hidden, np.float32)

    def mm(a, b, tb=False, act="none"):
        got = ctx.matmul(dev(a), dev(b), transB=tb, act=act).cpu().numpy()
        lin = got if act == "none" else ctx.matmul(dev(a), dev(b), transB=tb).cpu().numpy()
        assert report(f"in situ matmul {a.shape} x {b.shape}", lin, oracle.matmul(a, b, None, False, tb, wide=True)) <= TOL
        return got

    heads_first = lambda v: np.ascontiguousarray(v.reshape(seq, heads, hd).transpose(1, 0, 2))
    q, k, v = (heads_first(mm(x, W[i])) for i in range(3))
    s = mm(q, k, True)
    p = ctx.softmax(dev(s)).cpu().numpy()
    assert contract_err(p, oracle.softmax(s)) <= 1e-5
    c = np.ascontiguousarray(mm(p, v).transpose(1, 0, 2)).reshape(1, seq, hidden)
    r1 = x + mm(c, W[3])
    t1 = ctx.layernorm(dev(r1[0]), dev(ones), dev(zeros)).cpu().numpy()[None]
    assert contract_err(t1[0], oracle.layernorm(r1[0], ones, zeros, 1e-5)) <= 1e-4
    f = mm(mm(t1, W[4], act="gelu"), W[5])
    t2 = ctx.layernorm(dev((t1 + f)[0]), dev(ones), dev(zeros)).cpu().numpy()
    assert contract_err(t2, oracle.layernorm((t1 + f)[0], ones, zeros, 1e-5)) <= 1e-4
    ctx.sync_check()
