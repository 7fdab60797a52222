"""GPU: convolution kernels through the C ABI against the CPU oracle (double-accumulated restatement of the
reference's ConvOp::compute) and the reference-produced integer vectors; correction windows bit-exact."""
import numpy as np
import pytest
import torch

import golden_cases as gc
from conftest import rel_err, rms_rel_err, scale_err

pytestmark = pytest.mark.gpu
TOL = 1e-3        # max relative error the backend has to meet (metric: conftest.rel_err)
TOL_SCALE = 5e-5  # 3xTF32 accuracy statement: max |err| / max |ref|


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("algo", ["tc_3xtf32", "simt_fp32"])
@pytest.mark.parametrize("i", range(len(gc.CONVS)))
def test_conv_on_reference_integer_vectors(ctx, golden, algo, i):
    # small integers: every product and partial sum is exact in fp32 as long as it stays below 2^24, so the float
    # kernels must reproduce the reference's integer outputs exactly
    xs, ws, kw = gc.CONVS[i]
    x, w = gc.small_ints(xs, 100 + i) % 16, gc.small_ints(ws, 200 + i) % 16
    from oracle import pet_oracle as po
    want = po.conv2d_u32(x, w, **kw)
    pad, st, dl = kw["pad"], kw.get("stride", (1, 1)), kw.get("dil", (1, 1))
    y = ctx.conv2d(dev(x.astype(np.float32)), dev(w.astype(np.float32)), pad[0], pad[1], st[0], st[1], dl[0], dl[1], algo=algo)
    ctx.sync_check()
    assert np.array_equal(y.cpu().numpy().astype(np.uint32), want)


CASES = [
    # name, x shape, w shape, (ph,pw,sh,sw,dh,dw)
    ("c1", (1, 64, 56, 56), (64, 64, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("c1_rewrite", (2, 64, 28, 56), (64, 64, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("dilated_small", (1, 32, 16, 16), (48, 32, 3, 3), (2, 2, 1, 1, 2, 2)),
    ("stride2", (2, 16, 28, 28), (32, 16, 3, 3), (1, 1, 2, 2, 1, 1)),
    ("1x1_stride2", (1, 64, 56, 56), (128, 64, 1, 1), (0, 0, 2, 2, 1, 1)),
    ("stem7x7", (1, 3, 224, 224), (64, 3, 7, 7), (3, 3, 2, 2, 1, 1)),
    ("odd_width_14", (1, 256, 14, 14), (256, 256, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("odd_width_7", (3, 64, 7, 7), (96, 64, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("grouped", (1, 32, 12, 12), (64, 8, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("depthwise", (1, 16, 10, 12), (16, 1, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("ragged", (2, 5, 9, 11), (7, 5, 3, 2), (1, 0, 1, 2, 1, 1)),
    ("wide_row", (1, 8, 3, 300), (16, 8, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("tiny_image_batch", (9, 24, 4, 4), (40, 24, 3, 3), (1, 1, 1, 1, 1, 1)),
    ("single_pixel", (1, 8, 1, 4), (8, 8, 1, 1), (0, 0, 1, 1, 1, 1)),
]


@pytest.mark.parametrize("algo", ["auto", "simt_fp32"])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_conv_vs_oracle(ctx, oracle, case, algo):
    name, xs, ws, (ph, pw, sh, sw, dh, dw) = case
    rng = np.random.default_rng(abs(hash(name)) % 2**31)
    x = rng.uniform(-1, 1, xs).astype(np.float32)
    w = (rng.standard_normal(ws) * np.sqrt(2.0 / (ws[1] * ws[2] * ws[3]))).astype(np.float32)
    b = rng.uniform(-1, 1, ws[0]).astype(np.float32)
    want = oracle.conv2d(x, w, b, pad=(ph, pw), stride=(sh, sw), dil=(dh, dw), act="relu", wide=True)
    y = ctx.conv2d(dev(x), dev(w), ph, pw, sh, sw, dh, dw, bias=dev(b), act="relu", algo=algo)
    ctx.sync_check()
    got = y.cpu().numpy()
    assert got.shape == want.shape
    assert rel_err(got, want) <= TOL
    assert scale_err(got, want) <= TOL_SCALE


RES_CASES = [  # tile kinds: split K over a cluster, unsplit, flat whole-plane tiles, CUDA-core fallback
    ("split_k", (1, 128, 28, 28), (128, 128, 3, 3), 1, "auto"), ("unsplit", (8, 64, 56, 56), (64, 64, 3, 3), 1, "auto"),
    ("flat_7", (2, 64, 7, 7), (96, 64, 3, 3), 1, "auto"), ("simt", (1, 8, 9, 11), (12, 8, 3, 3), 1, "simt_fp32"),
]


@pytest.mark.parametrize("case", RES_CASES, ids=[c[0] for c in RES_CASES])
def test_conv_with_residual_equals_conv_then_add(ctx, case):
    _, xs, ws, pad, algo = case
    rng = np.random.default_rng(len(xs) + xs[1])
    x = dev(rng.uniform(-1, 1, xs).astype(np.float32))
    w = dev((rng.standard_normal(ws) / np.sqrt(ws[1] * 9)).astype(np.float32))
    b = dev(rng.uniform(-1, 1, ws[0]).astype(np.float32))
    plain = ctx.conv2d(x, w, pad, pad, bias=b, algo=algo)
    res = dev(rng.uniform(-1, 1, tuple(plain.shape)).astype(np.float32))
    want = ctx.eltwise("add", [plain, res], act="relu")
    got = ctx.conv2d(x, w, pad, pad, bias=b, act="relu", algo=algo, residual=res)
    ctx.sync_check()
    assert torch.equal(got, want)  # same sums in the same order as the two-operator form


def test_auto_picks_the_tensor_core_kernel(ctx):
    plan = ctx.conv2d_plan((1, 64, 56, 56), (64, 64, 3, 3), 1, 1)
    assert plan.kernel.startswith("tc_3xtf32")


def test_dilated_layer_rewrite_equals_direct_conv(ctx, oracle):
    """Config 2 at full size: space-to-batch -> dense conv -> batch-to-space against the dilated conv itself and the
    oracle (on a channel subset, the CPU needs seconds for that)."""
    from test_gpu_layout import S2B, B2S
    g = torch.Generator().manual_seed(2000)
    x = torch.randn((1, 512, 64, 64), generator=g)
    w = torch.randn((512, 512, 3, 3), generator=g) * (2.0 / 4608) ** 0.5
    xd, wd = x.cuda(), w.cuda()
    direct = ctx.conv2d(xd, wd, 2, 2, 1, 1, 2, 2)
    s2b = ctx.transpose_chain(xd, S2B)
    assert tuple(s2b.shape) == (4, 512, 32, 32)
    dense = ctx.conv2d(s2b, wd, 1, 1)
    rewritten = ctx.transpose_chain(dense, B2S)
    ctx.sync_check()
    assert tuple(rewritten.shape) == (1, 512, 64, 64)
    # same kernel, same reduction order per output => the rewrite is bit-identical to the direct dilated conv
    assert torch.equal(rewritten, direct)
    want = oracle.conv2d(x.numpy(), w.numpy()[:32], pad=(2, 2), dil=(2, 2), wide=True)
    got = direct[:, :32].cpu().numpy()
    assert rel_err(got, want) <= TOL and scale_err(got, want) <= TOL_SCALE


@pytest.mark.parametrize("algo", ["auto", "simt_fp32"])
def test_h2n_rewrite_plus_correction_is_bit_identical(ctx, algo):
    """Config 1: split H in two halves stacked on the batch dim, conv, merge back: rows 27 and 28 come out wrong;
    the correction recomputes them from the original input and the result equals the unsplit conv bit for bit."""
    g = torch.Generator().manual_seed(1000)
    x = (torch.rand((1, 64, 56, 56), generator=g) * 2 - 1).cuda()
    w = (torch.rand((64, 64, 3, 3), generator=g) * 2 - 1).cuda()
    plan = ctx.conv2d_plan(x.shape, w.shape, 1, 1, algo=algo)
    ctx.conv2d_set_weights(plan, w)
    whole = ctx.conv2d_run(plan, x)
    h2n = ctx.transpose(x, 2, [[0, 2], 1, -1, 3], -2)
    half_plan = ctx.conv2d_plan(h2n.shape, w.shape, 1, 1, algo=algo)
    ctx.conv2d_set_weights(half_plan, w)
    merged = ctx.transpose(ctx.conv2d_run(half_plan, h2n), 0, [0, 1, [-1, 2], 3], 2)
    diff_rows = torch.unique(torch.nonzero(merged != whole)[:, 2]).tolist()
    assert diff_rows == [27, 28]
    assert int((merged != whole).sum()) <= 2 * 64 * 56
    assert torch.equal(merged[:, :, :27], whole[:, :, :27]) and torch.equal(merged[:, :, 29:], whole[:, :, 29:])
    ctx.conv2d_correct(plan, x, merged, 27, 2)
    ctx.sync_check()
    assert torch.equal(merged, whole)


def test_correction_window_in_both_axes(ctx):
    x = torch.randn((2, 32, 24, 24), device="cuda")
    w = torch.randn((32, 32, 3, 3), device="cuda") * 0.1
    plan = ctx.conv2d_plan(x.shape, w.shape, 1, 1)
    ctx.conv2d_set_weights(plan, w)
    whole = ctx.conv2d_run(plan, x)
    y = whole.clone()
    y[:, :, 11:13, :] = 7.0
    y[:, :, :, 11:13] = -7.0
    ctx.conv2d_correct(plan, x, y, 11, 2)                 # seam rows
    ctx.conv2d_correct(plan, x, y, 0, 24, 11, 2)          # seam columns
    ctx.sync_check()
    assert torch.equal(y, whole)


def test_conv3d_vs_oracle(ctx, oracle):
    rng = np.random.default_rng(33)
    for xs, ws, pad, st in [((1, 8, 6, 12, 12), (16, 8, 3, 3, 3), (1, 1, 1), (1, 1, 1)),
                            ((1, 3, 8, 20, 20), (8, 3, 3, 7, 7), (1, 3, 3), (1, 2, 2)),
                            ((2, 8, 4, 8, 8), (8, 8, 3, 3, 3), (1, 1, 1), (2, 2, 2)),
                            ((1, 16, 4, 6, 8), (8, 16, 1, 1, 1), (0, 0, 0), (2, 2, 2))]:
        x = rng.standard_normal(xs).astype(np.float32)
        w = (rng.standard_normal(ws) * np.sqrt(2.0 / np.prod(ws[1:]))).astype(np.float32)
        want = oracle.conv3d(x, w, pad=pad, stride=st, wide=True)
        for algo in ("auto", "simt_fp32"):
            got = ctx.conv3d(dev(x), dev(w), pad, st, algo=algo).cpu().numpy()
            ctx.sync_check()
            assert got.shape == want.shape
            assert rel_err(got, want) <= TOL and scale_err(got, want) <= TOL_SCALE


MODE_CASES = [
    # raw-tile and reduction modes of the tensor-core kernel: (name, x, w, pad, stride, dil, act)
    ("flat_grouped_7", (2, 64, 7, 7), (64, 32, 3, 3), (1, 1), (1, 1), (1, 1), "tanh"),          # whole-plane tiles, 2 groups
    ("flat_dilated_14", (1, 128, 14, 14), (128, 128, 3, 3), (2, 2), (1, 1), (2, 2), "sigmoid"), # tap mask with dilation
    ("flat_stride2_14", (1, 64, 14, 14), (128, 64, 3, 3), (1, 1), (2, 2), (1, 1), "gelu"),
    ("flat_1x1_7", (4, 256, 7, 7), (512, 256, 1, 1), (0, 0), (1, 1), (1, 1), "relu"),           # chunks of 128 channels
    ("flat_small_chunk", (1, 20, 6, 6), (24, 20, 3, 3), (1, 1), (1, 1), (1, 1), "none"),         # table gather (BC < 32)
    ("cluster_8", (1, 512, 7, 7), (512, 512, 3, 3), (1, 1), (1, 1), (1, 1), "relu"),            # K split over 8 CTAs
    ("cluster_bias_act", (1, 256, 28, 28), (96, 256, 3, 3), (1, 1), (1, 1), (1, 1), "sigmoid"),  # ragged filter count
    ("odd_width_repitch", (1, 8, 30, 150), (16, 8, 3, 3), (1, 1), (1, 1), (1, 1), "none"),       # rows too wide for flat tiles
    ("many_tiles", (6, 32, 56, 56), (96, 32, 3, 3), (1, 1), (1, 1), (1, 1), "relu"),       # 294 tiles on 148 SMs
    ("many_tiles_flat", (40, 64, 14, 14), (64, 64, 3, 3), (1, 1), (1, 1), (1, 1), "none"),        # 80 planes x 2 tiles, flat
    ("many_tiles_odd_k", (5, 24, 40, 40), (32, 24, 3, 3), (1, 1), (1, 1), (1, 1), "tanh"),        # 7 stages per tile (odd)
]


@pytest.mark.parametrize("case", MODE_CASES, ids=[c[0] for c in MODE_CASES])
def test_conv_kernel_modes_vs_oracle(ctx, oracle, case):
    name, xs, ws, pad, st, dil, act = case
    rng = np.random.default_rng(len(name) * 131 + xs[1])
    x = rng.uniform(-1, 1, xs).astype(np.float32)
    w = (rng.standard_normal(ws) * np.sqrt(2.0 / (ws[1] * ws[2] * ws[3]))).astype(np.float32)
    b = rng.uniform(-1, 1, ws[0]).astype(np.float32)
    # The contract metric is asserted on the convolution's own output (+ bias); the fused activation is then checked as
    # what it is, a function applied to that output.  (Judged on tanh/sigmoid values directly, the metric's floor would
    # be a thousandth of 1 while the error comes from sums several times larger.)
    want = oracle.conv2d(x, w, b, pad=pad, stride=st, dil=dil, wide=True)
    lin = ctx.conv2d(dev(x), dev(w), pad[0], pad[1], st[0], st[1], dil[0], dil[1], bias=dev(b))
    got = ctx.conv2d(dev(x), dev(w), pad[0], pad[1], st[0], st[1], dil[0], dil[1], bias=dev(b), act=act).cpu().numpy()
    ctx.sync_check()
    assert got.shape == want.shape
    assert rel_err(lin.cpu().numpy(), want) <= TOL and scale_err(lin.cpu().numpy(), want) <= TOL_SCALE
    assert np.allclose(got, oracle.activation(lin.cpu().numpy(), act), rtol=2e-6, atol=2e-7)
    exact = ctx.conv2d(dev(x), dev(w), pad[0], pad[1], st[0], st[1], dil[0], dil[1], bias=dev(b), algo="simt_fp32")
    # and against the CUDA-core fp32 kernel, whose sequential fp32 sums carry their own rounding error
    assert rel_err(lin.cpu().numpy(), exact.cpu().numpy()) <= TOL + rel_err(exact.cpu().numpy(), want)


def test_conv3d_small_planes_vs_oracle(ctx, oracle):
    """3-D layers whose rows are not 16-byte multiples (the last stages of ResNet3D): flat raw tiles over all depth slices."""
    rng = np.random.default_rng(35)
    for xs, ws, pad, st in [((1, 64, 2, 7, 7), (64, 64, 3, 3, 3), (1, 1, 1), (1, 1, 1)),
                            ((1, 32, 4, 14, 14), (48, 32, 3, 3, 3), (1, 1, 1), (1, 1, 1)),
                            ((2, 32, 4, 14, 14), (64, 32, 1, 1, 1), (0, 0, 0), (2, 2, 2))]:
        x = rng.standard_normal(xs).astype(np.float32)
        w = (rng.standard_normal(ws) * np.sqrt(2.0 / np.prod(ws[1:]))).astype(np.float32)
        want = oracle.conv3d(x, w, pad=pad, stride=st, wide=True)
        got = ctx.conv3d(dev(x), dev(w), pad, st).cpu().numpy()
        ctx.sync_check()
        assert got.shape == want.shape
        assert rel_err(got, want) <= TOL and scale_err(got, want) <= TOL_SCALE


def test_correction_window_on_a_flat_plan_is_bit_identical(ctx):
    x = torch.randn((1, 64, 14, 14), device="cuda")
    w = torch.randn((64, 64, 3, 3), device="cuda") * 0.05
    plan = ctx.conv2d_plan(x.shape, w.shape, 1, 1)
    ctx.conv2d_set_weights(plan, w)
    whole = ctx.conv2d_run(plan, x)
    y = whole.clone()
    y[:, :, 6:8, :] = 3.0
    ctx.conv2d_correct(plan, x, y, 6, 2)
    ctx.sync_check()
    assert torch.equal(y, whole)


def test_invalid_conv_arguments(ctx):
    from pet_b200 import PetError
    with pytest.raises(PetError) as e:
        ctx.conv2d_plan((1, 6, 8, 8), (4, 4, 3, 3), 1, 1)  # 6 channels not divisible by filter channels 4
    assert e.value.status == 1
    with pytest.raises(PetError):
        ctx.conv2d_plan((1, 4, 2, 2), (4, 4, 5, 5), 0, 0)  # empty output
    with pytest.raises(PetError):
        ctx.conv2d_plan((1, 8, 8, 8), (5, 4, 3, 3), 1, 1)  # f % groups != 0 (ConvOp::compute returns nullptr)
    plan = ctx.conv2d_plan((1, 4, 8, 8), (4, 4, 3, 3), 1, 1, bias=True)
    ctx.conv2d_set_weights(plan, torch.zeros((4, 4, 3, 3), device="cuda"))
    with pytest.raises(PetError):
        ctx.conv2d_run(plan, torch.zeros((1, 4, 8, 8), device="cuda"))  # bias promised, none passed


def test_device_status_is_clean_and_timing_entry_point_works(ctx):
    plan = ctx.conv2d_plan((1, 64, 56, 56), (64, 64, 3, 3), 1, 1)
    ms = plan.time(rounds=20, warmup=5)
    assert 0 < ms < 5
    ctx.sync_check()


def test_single_pass_tf32_option(ctx, oracle):
    """PETB200_ALGO_TC_1XTF32: one TF32 pass with round-to-nearest operands, the accuracy class of cuDNN's default
    math mode (what the reference's cudnnConvolutionForward gets on this GPU).  Not the contract's accuracy class: judged
    with the tensor's RMS as the floor of the relative error, bound 5e-3."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 64, 28, 28)).astype(np.float32)
    w = (rng.standard_normal((96, 64, 3, 3)) * np.sqrt(2.0 / 576)).astype(np.float32)
    want = oracle.conv2d(x, w, pad=(1, 1), wide=True)
    plan = ctx.conv2d_plan(x.shape, w.shape, 1, 1, algo="tc_1xtf32")
    assert plan.kernel == "tc_1xtf32_ts"
    ctx.conv2d_set_weights(plan, dev(w))
    got = ctx.conv2d_run(plan, dev(x)).cpu().numpy()
    ctx.sync_check()
    assert rms_rel_err(got, want) <= 5e-3 and scale_err(got, want) <= 1e-3
    a = rng.standard_normal((1, 128, 768)).astype(np.float32)
    b = (rng.standard_normal((1, 768, 256)) / 27.7).astype(np.float32)
    got = ctx.matmul(dev(a), dev(b), algo="tc_1xtf32").cpu().numpy()
    assert rms_rel_err(got, oracle.matmul(a, b)) <= 5e-3


def test_compensated_bf16_option(ctx, oracle):
    """PETB200_ALGO_TC_BF16X3: operands split into two bf16 halves, three products per multiply, fp32 accumulation.  Its
    products carry ~2^-17 relative error, 16x TF32x3's: an accuracy class between the library's fp32 and its default math.
    Stated here: within 5e-3 under the contract's metric (the default algorithm: 1e-3; one TF32 pass: ~2e-1), on every kind
    of operand fetch the kernel has; and exact on small integers, like the other algorithms."""
    rng = np.random.default_rng(11)
    cases = [((2, 64, 28, 28), (96, 64, 3, 3), dict(ph=1, pw=1)),             # 32-channel runs, two per 64-wide stage
             ((2, 64, 28, 28), (64, 16, 3, 3), dict(ph=1, pw=1, groups=4)),   # 16 channels per group: four runs per stage
             ((2, 64, 28, 28), (64, 8, 3, 3), dict(ph=1, pw=1, groups=8)),    # 8 channels per group: eight runs
             ((4, 3, 64, 64), (32, 3, 7, 7), dict(ph=3, pw=3, sh=2, sw=2)),   # offset table
             ((2, 96, 7, 7), (64, 96, 3, 3), dict(ph=1, pw=1)),               # whole-plane tiles with tap masks
             ((1, 256, 32, 32), (128, 256, 3, 3), dict(ph=2, pw=2, dh=2, dw=2))]  # long K: accumulator flush
    for xs, ws, kw in cases:
        x = rng.standard_normal(xs).astype(np.float32)
        w = (rng.standard_normal(ws) * np.sqrt(2.0 / (ws[1] * ws[2] * ws[3]))).astype(np.float32)
        groups = kw.pop("groups", 1)
        want = oracle.conv2d(x, w, pad=(kw["ph"], kw["pw"]), stride=(kw.get("sh", 1), kw.get("sw", 1)),
                             dil=(kw.get("dh", 1), kw.get("dw", 1)), wide=True)
        plan = ctx.conv2d_plan(xs, ws, kw["ph"], kw["pw"], kw.get("sh", 1), kw.get("sw", 1), kw.get("dh", 1), kw.get("dw", 1), algo="tc_bf16x3")
        assert plan.kernel == "tc_bf16x3_ts" and groups == xs[1] // ws[1]
        ctx.conv2d_set_weights(plan, dev(w))
        got = ctx.conv2d_run(plan, dev(x)).cpu().numpy()
        ctx.sync_check()
        assert rel_err(got, want) <= 5e-3 and scale_err(got, want) <= 2e-5, (xs, ws)
    for shape_a, shape_b, ta in (((2, 128, 768), (2, 768, 200), False), ((3, 100, 77), (3, 100, 50), True), ((1, 64, 100), (1, 100, 40), False)):
        a = rng.standard_normal(shape_a).astype(np.float32)
        b = (rng.standard_normal(shape_b) / np.sqrt(shape_b[1])).astype(np.float32)
        got = ctx.matmul(dev(a), dev(b), ta, False, algo="tc_bf16x3").cpu().numpy()
        assert rel_err(got, oracle.matmul(a, b, None, ta, False, wide=True)) <= 5e-3, shape_a
    xi = rng.integers(-3, 4, (2, 40, 13, 17)).astype(np.float32)
    wi = rng.integers(-3, 4, (24, 40, 3, 3)).astype(np.float32)
    assert np.array_equal(ctx.conv2d(dev(xi), dev(wi), 1, 1, algo="tc_bf16x3").cpu().numpy(), oracle.conv2d(xi, wi, pad=(1, 1)))
    ctx.sync_check()


def test_persistent_tiles_equal_one_tile_per_cta(ctx, oracle, monkeypatch):
    """Plans with several pixel tiles per SM and narrow filter tiles run persistent CTAs (the two transform sets take
    alternate tiles, accumulators alternate between two TMEM regions).  Same sums in the same order as one tile per CTA:
    the results are bit-identical, with bias / residual / activation, odd tile counts and a ragged last tile; and they
    meet the contract against the oracle."""
    rng = np.random.default_rng(31)
    for xs, ws, stride, pad in (((16, 64, 56, 56), (64, 64, 3, 3), 1, 1), ((24, 3, 112, 112), (64, 3, 7, 7), 2, 3), ((37, 32, 30, 30), (32, 32, 3, 3), 1, 1)):
        x = dev(rng.standard_normal(xs).astype(np.float32))
        w = dev((rng.standard_normal(ws) * np.sqrt(2.0 / (ws[1] * ws[2] * ws[3]))).astype(np.float32))
        b = dev(rng.uniform(-1, 1, ws[0]).astype(np.float32))
        outs = []
        res = None
        for pp in ("1", "0"):
            monkeypatch.setenv("PETB200_TC_PINGPONG", pp)  # read when the plan is made
            plan = ctx.conv2d_plan(xs, ws, pad, pad, stride, stride, 1, 1, True, "relu")
            ctx.conv2d_set_weights(plan, w)
            y = ctx.conv2d_run(plan, x, b)
            if res is None:
                res = dev(rng.uniform(-1, 1, tuple(y.shape)).astype(np.float32))
            lin_plan = ctx.conv2d_plan(xs, ws, pad, pad, stride, stride, 1, 1, True, "none")
            ctx.conv2d_set_weights(lin_plan, w)
            outs.append((y, ctx.conv2d_run(plan, x, b, residual=res), ctx.conv2d_run(lin_plan, x, b)))
        ctx.sync_check()
        assert all(torch.equal(p1, p0) for p1, p0 in zip(outs[0], outs[1])), xs
        want = oracle.conv2d(x[:2].cpu().numpy(), w.cpu().numpy(), b.cpu().numpy(), pad=(pad, pad), stride=(stride, stride), wide=True)
        assert rel_err(outs[0][2][:2].cpu().numpy(), want) <= TOL, xs


def test_conv_random_shapes_exact(ctx, oracle):
    """Seeded sweep over ragged shapes (groups, strides, dilations, paddings, odd widths, 1..64 channels per group): on
    small integers both the tensor-core and the CUDA-core kernels reproduce the oracle exactly."""
    rng = np.random.default_rng(2024)
    ran = 0
    for _ in range(90):
        g, cpg, fpg = int(rng.choice([1, 1, 1, 2, 4])), int(rng.choice([1, 3, 8, 16, 32, 40, 64])), int(rng.choice([1, 5, 8, 32, 48]))
        n, h, w = int(rng.integers(1, 4)), int(rng.integers(1, 30)), int(rng.integers(1, 30))
        r, s, sh, sw = int(rng.integers(1, 6)), int(rng.integers(1, 6)), int(rng.integers(1, 3)), int(rng.integers(1, 3))
        dh, dw, ph, pw = int(rng.integers(1, 3)), int(rng.integers(1, 3)), int(rng.integers(0, 4)), int(rng.integers(0, 4))
        oh, ow = (h - (r - sh) * dh + 2 * ph) // sh, (w - (s - sw) * dw + 2 * pw) // sw
        if oh <= 0 or ow <= 0 or (r - 1) * dh + 1 > h + 2 * ph or (s - 1) * dw + 1 > w + 2 * pw:
            continue
        x = rng.integers(0, 4, (n, g * cpg, h, w)).astype(np.float32)
        wt = rng.integers(0, 4, (g * fpg, cpg, r, s)).astype(np.float32)
        want = oracle.conv2d(x, wt, None, pad=(ph, pw), stride=(sh, sw), dil=(dh, dw), wide=False)
        for algo in ("tc_3xtf32", "simt_fp32"):
            y = ctx.conv2d(dev(x), dev(wt), ph, pw, sh, sw, dh, dw, algo=algo).cpu().numpy()
            assert y.shape == want.shape and np.array_equal(y, want), (algo, x.shape, wt.shape, ph, pw, sh, sw, dh, dw)
            ran += 1
    ctx.sync_check()
    assert ran >= 100


def test_conv3d_random_shapes_exact(ctx, oracle):
    rng = np.random.default_rng(77)
    ran = 0
    for _ in range(40):
        g, cpg, fpg = int(rng.choice([1, 1, 2])), int(rng.choice([1, 3, 8, 16, 32])), int(rng.choice([1, 5, 8, 32]))
        n, dims = int(rng.integers(1, 3)), [int(rng.integers(1, 8)), int(rng.integers(1, 14)), int(rng.integers(1, 14))]
        k, st = [int(rng.integers(1, 4)) for _ in range(3)], [int(rng.integers(1, 3)) for _ in range(3)]
        dl, pd = [int(rng.integers(1, 3)) for _ in range(3)], [int(rng.integers(0, 3)) for _ in range(3)]
        o = [(dims[i] - (k[i] - st[i]) * dl[i] + 2 * pd[i]) // st[i] for i in range(3)]
        if min(o) <= 0 or any((k[i] - 1) * dl[i] + 1 > dims[i] + 2 * pd[i] for i in range(3)):
            continue
        x = rng.integers(0, 4, (n, g * cpg, *dims)).astype(np.float32)
        wt = rng.integers(0, 4, (g * fpg, cpg, *k)).astype(np.float32)
        want = oracle.conv3d(x, wt, None, pad=tuple(pd), stride=tuple(st), dil=tuple(dl), wide=False)
        for algo in ("tc_3xtf32", "simt_fp32"):
            y = ctx.conv3d(dev(x), dev(wt), pd, st, dl, algo=algo).cpu().numpy()
            assert y.shape == want.shape and np.array_equal(y, want), (algo, x.shape, wt.shape, pd, st, dl)
            ran += 1
    ctx.sync_check()
    assert ran >= 40


def test_correction_windows_random_bit_identical(ctx):
    """Seeded sweep of correction windows (any rows x columns, batches of 1-3 images, odd widths, 1x1 to dilated 5x5 filters):
    the window equals the same region of the full convolution bit for bit and nothing outside it is written.  Small
    windows of multi-image batches used to fail to plan (several images per tile with the full plan's chunk size)."""
    rng = np.random.default_rng(78)
    for _ in range(40):
        cpg, f, n = int(rng.choice([3, 16, 32, 64])), int(rng.choice([8, 32, 48, 128])), int(rng.integers(1, 4))
        h, w, r, dh = int(rng.integers(4, 40)), int(rng.integers(4, 40)), int(rng.choice([1, 3, 5])), int(rng.integers(1, 3))
        ph = (r - 1) * dh // 2
        x = dev(rng.uniform(-1, 1, (n, cpg, h, w)).astype(np.float32))
        wt = dev(rng.uniform(-1, 1, (f, cpg, r, r)).astype(np.float32))
        plan = ctx.conv2d_plan(x.shape, wt.shape, ph, ph, 1, 1, dh, dh)
        ctx.conv2d_set_weights(plan, wt)
        y0 = ctx.conv2d_run(plan, x)
        oh, ow = y0.shape[2], y0.shape[3]
        r0, c0 = int(rng.integers(0, oh)), int(rng.integers(0, ow))
        rn, cn = int(rng.integers(1, oh - r0 + 1)), int(rng.integers(1, ow - c0 + 1))
        y1 = torch.full_like(y0, 7.0)
        ctx.conv2d_correct(plan, x, y1, r0, rn, c0, cn)
        ctx.sync_check()
        case = (tuple(x.shape), tuple(wt.shape), dh, r0, rn, c0, cn)
        assert torch.equal(y1[:, :, r0:r0 + rn, c0:c0 + cn], y0[:, :, r0:r0 + rn, c0:c0 + cn]), case
        y1[:, :, r0:r0 + rn, c0:c0 + cn] = 7.0
        assert bool((y1 == 7.0).all()), case


def test_conv_epilogue_combinations_exact(ctx, oracle):
    """Seeded sweep over bias / ReLU / folded residual on shapes that reach every tiling regime (deep K with few tiles:
    split-K through the cluster; many tiles; stride 2): exact on small integers for both kernel families."""
    rng = np.random.default_rng(5)
    for _ in range(40):
        c, f, n = int(rng.choice([16, 64, 128, 256, 512])), int(rng.choice([8, 32, 64, 100, 256])), int(rng.integers(1, 3))
        hw, r, st = int(rng.choice([4, 7, 8, 14, 28])), int(rng.choice([1, 3])), int(rng.choice([1, 2]))
        p = r // 2
        x = rng.integers(-2, 3, (n, c, hw, hw)).astype(np.float32)
        wt = rng.integers(-2, 3, (f, c, r, r)).astype(np.float32)
        b = rng.integers(-3, 4, f).astype(np.float32)
        act, use_b, use_res = str(rng.choice(["none", "relu"])), bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        want = oracle.conv2d(x, wt, b if use_b else None, pad=(p, p), stride=(st, st), wide=False)
        res = rng.integers(-3, 4, want.shape).astype(np.float32)
        want = want + res if use_res else want
        want = np.maximum(want, 0) if act == "relu" else want
        for algo in ("tc_3xtf32", "simt_fp32"):
            y = ctx.conv2d(dev(x), dev(wt), p, p, st, st, 1, 1, bias=dev(b) if use_b else None, act=act, algo=algo,
                           residual=dev(res) if use_res else None).cpu().numpy()
            assert np.array_equal(y, want), (algo, x.shape, wt.shape, st, act, use_b, use_res)
    ctx.sync_check()


def test_bounded_wait_gives_up_and_reports_instead_of_hanging(ctx):
    """Every wait of the tensor-core kernel has a limit after which the kernel leaves through its abort path and sets a
    status word.  Here the limit is shortened to 5 ms and one plan's filter producer is told to announce more bytes per
    stage than it loads (a completion that never comes): the launch returns, petb200_check_device_status reports
    PETB200_ERR_DEVICE, and the next launches on the same context — the same plan with the hook off — are correct."""
    import ctypes as C
    from pet_b200 import lib as L
    lib = L.load()
    lib.petb200_debug_set_wait_limit.argtypes = [C.c_ulonglong]
    lib.petb200_debug_conv_starve.argtypes = [C.c_void_p, C.c_int]
    x = torch.randn((1, 64, 28, 28), device="cuda")
    w = torch.randn((64, 64, 3, 3), device="cuda") * 0.05
    plan = ctx.conv2d_plan(x.shape, w.shape, 1, 1)
    assert plan.kernel.startswith("tc_")
    ctx.conv2d_set_weights(plan, w)
    good = ctx.conv2d_run(plan, x)
    ctx.sync_check()
    assert lib.petb200_debug_set_wait_limit(5_000_000) == 0
    try:
        assert lib.petb200_debug_conv_starve(plan.h, 1) == 0
        ctx.conv2d_run(plan, x)
        with pytest.raises(L.PetError) as e:
            ctx.sync_check()
        assert e.value.status == L.ERR_DEVICE
    finally:
        lib.petb200_debug_conv_starve(plan.h, 0)
        assert lib.petb200_debug_set_wait_limit(2_000_000_000) == 0
    again = ctx.conv2d_run(plan, x)
    ctx.sync_check()                      # the status word was cleared by the failed check; the context is usable
    assert torch.equal(again, good)
