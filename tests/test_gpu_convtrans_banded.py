"""GPU: transposed convolution and the banded attention products through the C ABI against the CPU oracle
(restatements of ConvTransOp::compute and of the reference's G2BMM / GBMML definitions) and the reference-produced
integer vectors."""
import numpy as np
import pytest
import torch

import golden_cases as gc
from conftest import rel_err, scale_err

pytestmark = pytest.mark.gpu
TOL = 1e-3        # max relative error the backend has to meet (metric: conftest.rel_err)
TOL_SCALE = 5e-5  # 3xTF32 accuracy statement: max |err| / max |ref|


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _ct(ctx, x, w, kw, algo, bias=None, act="none"):
    pad, st, op = kw.get("pad", (0, 0)), kw.get("stride", (1, 1)), kw.get("out_pad", (0, 0))
    return ctx.convtrans(dev(x), dev(w), pad[0], pad[1], st[0], st[1], 1, 1, op[0], op[1],
                         bias=None if bias is None else dev(bias), act=act, algo=algo)


@pytest.mark.parametrize("algo", ["tc_3xtf32", "simt_fp32"])
@pytest.mark.parametrize("i", range(len(gc.CONVTRANS)))
def test_convtrans_on_reference_integer_vectors(ctx, golden, algo, i):
    # small integers: products and partial sums are exact in fp32, so the float kernels must reproduce the integer
    # results of the reference's own host operator
    xs, ws, kw, _ = gc.CONVTRANS[i]
    x, w = gc.small_ints(xs, 300 + i) % 16, gc.small_ints(ws, 400 + i) % 16
    from oracle import pet_oracle as po
    want = po.convtrans_u32(x, w, **kw)
    y = _ct(ctx, x.astype(np.float32), w.astype(np.float32), kw, algo)
    ctx.sync_check()
    assert tuple(y.shape) == want.shape
    assert np.array_equal(y.cpu().numpy().astype(np.uint32), want)


@pytest.mark.parametrize("algo", ["tc_3xtf32", "simt_fp32"])
@pytest.mark.parametrize("phases", ["0", "1"])
def test_convtrans_known_answer_of_the_reference_test(ctx, algo, phases, monkeypatch):
    monkeypatch.setenv("PETB200_CONVTRANS_PHASES", phases)
    x, wt, kw, want = gc.convtrans_kat()
    plan = ctx.convtrans_plan(x.shape, wt.shape, 1, 1, 2, 2, algo=algo)
    y = ctx.convtrans_run(plan, dev(x.astype(np.float32)), dev(wt.astype(np.float32)))
    ctx.sync_check()
    assert np.array_equal(y.cpu().numpy().astype(np.uint32), want)


CT_CASES = [
    # name, x {n,h,w,f}, w {r,s,f,c}, kwargs
    ("upsample2x_k4", (1, 16, 16, 64), (4, 4, 64, 32), dict(pad=(1, 1), stride=(2, 2))),
    ("upsample2x_k3_outpad", (2, 14, 14, 48), (3, 3, 48, 24), dict(pad=(1, 1), stride=(2, 2), out_pad=(1, 1))),
    ("stride1_same", (1, 12, 20, 32), (3, 3, 32, 40), dict(pad=(1, 1))),
    ("stride3_skipped_tap", (1, 6, 5, 16), (4, 3, 16, 12), dict(stride=(3, 3))),
    ("ragged_channels", (2, 5, 7, 5), (3, 2, 5, 7), dict(pad=(0, 1), stride=(2, 1), out_pad=(1, 0))),
    ("dcgan_layer", (4, 8, 8, 256), (4, 4, 256, 128), dict(pad=(1, 1), stride=(2, 2))),
    ("padding_ge_kernel", (1, 6, 6, 8), (2, 2, 8, 8), dict(pad=(3, 3), stride=(2, 2), out_pad=(1, 1))),
]


@pytest.mark.parametrize("algo", ["auto", "simt_fp32"])
@pytest.mark.parametrize("case", CT_CASES, ids=[c[0] for c in CT_CASES])
def test_convtrans_vs_oracle(ctx, oracle, case, algo):
    name, xs, ws, kw = case
    rng = np.random.default_rng(abs(hash(name)) % 2**31)
    x = rng.uniform(-1, 1, xs).astype(np.float32)
    w = (rng.standard_normal(ws) * np.sqrt(2.0 / (ws[0] * ws[1] * ws[2]))).astype(np.float32)
    want = oracle.convtrans(x, w, wide=True, **kw)
    y = _ct(ctx, x, w, kw, algo).cpu().numpy()
    ctx.sync_check()
    assert y.shape == want.shape
    assert rel_err(y, want) <= TOL
    assert scale_err(y, want) <= TOL_SCALE


PHASE_CASES = CT_CASES + [
    ("stride3_k5", (2, 7, 6, 16), (5, 5, 16, 8), dict(pad=(1, 2), stride=(3, 3), out_pad=(2, 1))),
    ("stride2x1", (1, 9, 10, 8), (3, 3, 8, 8), dict(pad=(1, 1), stride=(2, 1))),
    ("odd_width_phases", (1, 7, 7, 24), (4, 4, 24, 20), dict(pad=(1, 1), stride=(2, 2))),
    ("large_batch", (8, 32, 32, 128), (4, 4, 128, 64), dict(pad=(1, 1), stride=(2, 2))),
]


@pytest.mark.parametrize("case", PHASE_CASES, ids=[c[0] for c in PHASE_CASES])
def test_convtrans_phase_decomposition_vs_oracle(ctx, oracle, case, monkeypatch):
    """The sh*sw phase convolutions (forced on, whatever the problem size) against the oracle, with bias and ReLU; where
    the shape does not allow them the plan keeps the zero-insertion path and must agree all the same."""
    name, xs, ws, kw = case
    monkeypatch.setenv("PETB200_CONVTRANS_PHASES", "1")
    rng = np.random.default_rng(len(name) * 7919 + xs[1])
    x = rng.uniform(-1, 1, xs).astype(np.float32)
    w = (rng.standard_normal(ws) * np.sqrt(2.0 / (ws[0] * ws[1] * ws[2]))).astype(np.float32)
    b = rng.uniform(-1, 1, ws[3]).astype(np.float32)
    pad, st, op = kw.get("pad", (0, 0)), kw.get("stride", (1, 1)), kw.get("out_pad", (0, 0))
    plan = ctx.convtrans_plan(xs, ws, pad[0], pad[1], st[0], st[1], 1, 1, op[0], op[1], bias=True, act="relu")
    y = ctx.convtrans_run(plan, dev(x), dev(w), dev(b)).cpu().numpy()
    ctx.sync_check()
    want = np.maximum(oracle.convtrans(x, w, wide=True, **kw) + b, 0)
    assert y.shape == want.shape
    assert rel_err(y, want) <= TOL and scale_err(y, want) <= TOL_SCALE
    # small integers: exact, also against the zero-insertion path
    xi = rng.integers(0, 8, xs).astype(np.float32)
    wi = rng.integers(0, 8, ws).astype(np.float32)
    yi = ctx.convtrans_run(plan, dev(xi), dev(wi), dev(np.zeros(ws[3], np.float32))).cpu().numpy()
    monkeypatch.setenv("PETB200_CONVTRANS_PHASES", "0")
    plan0 = ctx.convtrans_plan(xs, ws, pad[0], pad[1], st[0], st[1], 1, 1, op[0], op[1], bias=True, act="relu")
    y0 = ctx.convtrans_run(plan0, dev(xi), dev(wi), dev(np.zeros(ws[3], np.float32))).cpu().numpy()
    assert np.array_equal(yi, y0)
    assert np.array_equal(yi, oracle.convtrans(xi, wi, wide=False, **kw))


def test_convtrans_bias_activation_and_torch(ctx, oracle):
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, (2, 9, 9, 32)).astype(np.float32)
    w = (rng.standard_normal((3, 3, 32, 16)) * 0.1).astype(np.float32)
    b = rng.uniform(-1, 1, 16).astype(np.float32)
    kw = dict(pad=(1, 1), stride=(2, 2), out_pad=(1, 1))
    want = np.maximum(oracle.convtrans(x, w, wide=True, **kw) + b, 0)
    y = _ct(ctx, x, w, kw, "auto", bias=b, act="relu").cpu().numpy()
    assert rel_err(y, want) <= TOL
    # the same operator as torch states it: weight [f_in, c_out, r, s], NCHW
    tx = torch.from_numpy(x).permute(0, 3, 1, 2).double()
    tw = torch.from_numpy(w).permute(2, 3, 0, 1).double()
    ty = torch.nn.functional.conv_transpose2d(tx, tw, torch.from_numpy(b).double(), stride=2, padding=1, output_padding=1)
    assert rel_err(y, torch.relu(ty).permute(0, 2, 3, 1).numpy()) <= TOL


def test_convtrans_rejects_what_the_reference_rejects(ctx):
    import pet_b200.lib as L
    with pytest.raises(L.PetError):
        ctx.convtrans_plan((1, 4, 4, 8), (3, 3, 8, 8), 1, 1, 1, 1, 2, 2)  # dilation
    with pytest.raises(L.PetError):
        ctx.convtrans_plan((1, 4, 4, 8), (3, 3, 6, 8), 1, 1)  # channel mismatch


def test_convtrans_plan_time(ctx):
    p = ctx.convtrans_plan((1, 16, 16, 64), (4, 4, 64, 64), 1, 1, 2, 2)
    assert p.out_shape == (1, 32, 32, 64)
    assert 0 < p.time(rounds=20, warmup=5) < 5.0


BAND_CASES = [
    # b, n, m, w, d
    (2, 37, 8, 3, 1),
    (1, 300, 64, 40, 1),
    (2, 257, 64, 17, 2),
    (1, 100, 20, 150, 1),   # band wider than the sequence
    (3, 64, 6, 0, 1),       # zero width: the diagonal
    (1, 130, 33, 9, 4),     # m not a multiple of 4
    (1, 50, 16, 7, 64),     # dilation beyond the sequence length
]


@pytest.mark.parametrize("case", BAND_CASES, ids=["b%d_n%d_m%d_w%d_d%d" % c for c in BAND_CASES])
def test_banded_products_vs_oracle(ctx, oracle, case):
    b, n, m, w, d = case
    rng = np.random.default_rng(1000 * n + w)
    q = rng.standard_normal((b, n, m)).astype(np.float32)
    k = rng.standard_normal((b, n, m)).astype(np.float32)
    p = rng.standard_normal((b, n, 2 * w + 1)).astype(np.float32)
    s = ctx.g2bmm(dev(q), dev(k), w, d).cpu().numpy()
    o = ctx.gbmml(dev(p), dev(k), d).cpu().numpy()
    ctx.sync_check()
    want_s, want_o = oracle.g2bmm(q, k, w, d, wide=True), oracle.gbmml(p, k, d, wide=True)
    assert s.shape == want_s.shape and o.shape == want_o.shape
    assert scale_err(s, want_s) <= 1e-5 and scale_err(o, want_o) <= 1e-5
    # positions whose key row is outside the sequence are exact zeros, whatever p holds there
    i = np.arange(n)[:, None] + d * (np.arange(2 * w + 1)[None, :] - w)
    assert np.all(s[:, (i < 0) | (i >= n)] == 0)
    p_bad = p.copy()
    p_bad[:, (i < 0) | (i >= n)] = np.inf
    assert np.array_equal(ctx.gbmml(dev(p_bad), dev(k), d).cpu().numpy(), o)


def test_banded_tensor_core_path_agrees_with_the_cuda_core_kernels(ctx, oracle):
    """Dilation 1 with 16-byte aligned operands runs on the tensor-core kernel (3xTF32); operands that start 4 bytes off an
    aligned address take the exact-fp32 CUDA-core kernels.  Same definition, two implementations: they agree within the
    contract's bound, both meet it against the oracle, and masked positions are exact zeros on both."""
    b, n, m, w = 2, 700, 64, 150
    rng = np.random.default_rng(77)
    q, k = (rng.standard_normal((b, n, m)).astype(np.float32) for _ in range(2))
    p = rng.standard_normal((b, n, 2 * w + 1)).astype(np.float32)

    def shifted(a):  # the same values at an address that is 4 bytes off a 16-byte boundary
        flat = torch.empty(a.size + 1, device="cuda", dtype=torch.float32)
        flat[1:] = torch.from_numpy(a.reshape(-1)).cuda()
        return flat[1:].view(a.shape)

    s_tc, s_cc = ctx.g2bmm(dev(q), dev(k), w, 1).cpu().numpy(), ctx.g2bmm(shifted(q), shifted(k), w, 1).cpu().numpy()
    o_tc, o_cc = ctx.gbmml(dev(p), dev(k), 1).cpu().numpy(), ctx.gbmml(shifted(p), shifted(k), 1).cpu().numpy()
    ctx.sync_check()
    want_s, want_o = oracle.g2bmm(q, k, w, 1, wide=True), oracle.gbmml(p, k, 1, wide=True)
    for got, want in ((s_tc, want_s), (s_cc, want_s), (o_tc, want_o), (o_cc, want_o)):
        assert rel_err(got, want) <= 1e-3
    assert not np.array_equal(s_tc, s_cc) and rel_err(s_tc, s_cc) <= 1e-3 and rel_err(o_tc, o_cc) <= 1e-3
    i = np.arange(n)[:, None] + (np.arange(2 * w + 1)[None, :] - w)
    assert np.all(s_tc[:, (i < 0) | (i >= n)] == 0) and np.all(s_cc[:, (i < 0) | (i >= n)] == 0)


def test_banded_products_small_integers_exact(ctx, oracle):
    rng = np.random.default_rng(8)
    q = rng.integers(0, 16, (2, 90, 24)).astype(np.float32)
    k = rng.integers(0, 16, (2, 90, 24)).astype(np.float32)
    p = rng.integers(0, 16, (2, 90, 23)).astype(np.float32)
    assert np.array_equal(ctx.g2bmm(dev(q), dev(k), 11, 2).cpu().numpy(), oracle.g2bmm(q, k, 11, 2, wide=False))
    assert np.array_equal(ctx.gbmml(dev(p), dev(k), 3).cpu().numpy(), oracle.gbmml(p, k, 3, wide=False))


def test_banded_reference_shape_properties(ctx):
    """The one shape the reference ships kernels for (n=10000, m=64, w=1000, d in {1,4}), checked through properties:
    a sample of entries against a dot product, and GBMML of a one-hot band against a row gather."""
    n, m, w = 10000, 64, 1000
    g = torch.Generator(device="cuda").manual_seed(4)
    q = torch.randn((1, n, m), device="cuda", generator=g)
    k = torch.randn((1, n, m), device="cuda", generator=g)
    for d in (1, 4):
        s = ctx.g2bmm(q, k, w, d)
        ctx.sync_check()
        assert tuple(s.shape) == (1, n, 2 * w + 1)
        ii = torch.randint(0, n, (4096,), device="cuda", generator=g)
        jj = torch.randint(0, 2 * w + 1, (4096,), device="cuda", generator=g)
        rows = ii + d * (jj - w)
        ok = (rows >= 0) & (rows < n)
        want = (q[0, ii].double() * k[0, rows.clamp(0, n - 1)].double()).sum(-1) * ok
        assert float((s[0, ii, jj].double() - want).abs().max()) <= 1e-4
        # one-hot band: column j0 set to 1 selects key row i + d*(j0-w)
        j0 = w + 3
        p = torch.zeros((1, n, 2 * w + 1), device="cuda")
        p[:, :, j0] = 1.0
        o = ctx.gbmml(p, k, d)
        shift = d * (j0 - w)
        # (times 1.0 on the tensor cores: hi + lo of the split value, each kept to TF32's 11 bits -> 2^-21 relative)
        assert bool(((o[0, : n - shift] - k[0, shift:]).abs() <= 1e-6 * k[0, shift:].abs()).all())
        assert float(o[0, n - shift:].abs().max()) == 0.0
    assert 0 < ctx.banded_time("g2bmm", 1, n, m, w, 1, rounds=5, warmup=2) < 50.0
    assert 0 < ctx.banded_time("gbmml", 1, n, m, w, 1, rounds=5, warmup=2) < 50.0


def test_convtrans_random_shapes_exact(ctx, oracle, monkeypatch):
    """Seeded sweep over small ragged shapes, strides up to 3, padding up to the filter extent, output padding: both the
    zero-insertion and the phase path reproduce the oracle exactly on small integers."""
    rng = np.random.default_rng(123)
    ran = 0
    for _ in range(60):
        n, h, w = int(rng.integers(1, 4)), int(rng.integers(1, 12)), int(rng.integers(1, 12))
        f, c = int(rng.choice([1, 3, 8, 16, 33])), int(rng.choice([1, 4, 7, 16, 40]))
        r, s, sh, sw = int(rng.integers(1, 6)), int(rng.integers(1, 6)), int(rng.integers(1, 4)), int(rng.integers(1, 4))
        ph, pw, oph, opw = int(rng.integers(0, r + 1)), int(rng.integers(0, s + 1)), int(rng.integers(0, sh)), int(rng.integers(0, sw))
        if (h - 1) * sh - 2 * ph + r + oph <= 0 or (w - 1) * sw - 2 * pw + s + opw <= 0:
            continue
        x = rng.integers(0, 8, (n, h, w, f)).astype(np.float32)
        wt = rng.integers(0, 8, (r, s, f, c)).astype(np.float32)
        want = oracle.convtrans(x, wt, (ph, pw), (sh, sw), (1, 1), (oph, opw), wide=False)
        for phases in ("0", "1"):
            monkeypatch.setenv("PETB200_CONVTRANS_PHASES", phases)
            plan = ctx.convtrans_plan(x.shape, wt.shape, ph, pw, sh, sw, 1, 1, oph, opw)
            y = ctx.convtrans_run(plan, dev(x), dev(wt)).cpu().numpy()
            assert np.array_equal(y, want), (phases, n, h, w, f, r, s, c, ph, pw, sh, sw, oph, opw)
            ran += 1
    ctx.sync_check()
    assert ran >= 80


def test_banded_random_shapes_exact(ctx, oracle):
    rng = np.random.default_rng(7)
    for _ in range(40):
        b, n, m = int(rng.integers(1, 4)), int(rng.integers(1, 400)), int(rng.choice([1, 3, 8, 20, 64, 100]))
        w, d = int(rng.integers(0, 130)), int(rng.integers(1, 6))
        q = rng.integers(0, 4, (b, n, m)).astype(np.float32)
        k = rng.integers(0, 4, (b, n, m)).astype(np.float32)
        p = rng.integers(0, 4, (b, n, 2 * w + 1)).astype(np.float32)
        assert np.array_equal(ctx.g2bmm(dev(q), dev(k), w, d).cpu().numpy(), oracle.g2bmm(q, k, w, d, wide=False)), (b, n, m, w, d)
        assert np.array_equal(ctx.gbmml(dev(p), dev(k), d).cpu().numpy(), oracle.gbmml(p, k, d, wide=False)), (b, n, m, w, d)
    ctx.sync_check()


def test_captured_gbmml_graph_survives_a_later_larger_gbmml_on_the_same_context(ctx, oracle):
    """The split-band scratch belongs to the context and grows on demand.  A graph captured while a smaller buffer was
    current keeps that buffer's address in its kernel nodes: the buffer must stay valid when a larger product on the same
    context makes the scratch grow."""
    from pet_b200.graph import Graph
    rng = np.random.default_rng(12)

    def build(n, m, w):
        g = Graph(ctx)
        p, v = g.tensor([1, n, 2 * w + 1]), g.tensor([1, n, m])
        y = g.gbmml(p, v, 1)
        g.setOutputs([y])
        g.compile()
        pa = rng.integers(-3, 4, (1, n, 2 * w + 1)).astype(np.float32)   # small integers: exact, whatever the split order
        va = rng.integers(-3, 4, (1, n, m)).astype(np.float32)
        g.set_data(p, pa)
        g.set_data(v, va)
        g.run()
        g.run()  # replay of the captured CUDA graph
        torch.cuda.synchronize()
        return g, y, oracle.gbmml(pa, va, 1, wide=False)

    g1, y1, want1 = build(700, 64, 400)          # a band wide enough to be split over blocks: uses the scratch
    assert np.array_equal(g1.get_data(y1), want1)
    g2, y2, want2 = build(5000, 64, 1200)        # a much larger product on the same context: the scratch grows
    assert np.array_equal(g2.get_data(y2), want2)
    g1.run()                                     # the first graph again, with the buffer address it captured
    torch.cuda.synchronize()
    ctx.sync_check()
    assert np.array_equal(g1.get_data(y1), want1)
