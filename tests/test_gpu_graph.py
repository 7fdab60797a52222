"""GPU: the graph layer (builder, fusion, CUDA-graph replay, per-operator timing) on the benchmark configurations,
checked against the CPU oracle evaluating the same configuration description."""
import numpy as np
import pytest
import torch

from conftest import rel_err, scale_err

pytestmark = pytest.mark.gpu
TOL, TOL_SCALE = 1e-3, 5e-5


def run_config(ctx, build, *args, fuse=True, cuda_graph=True, **kw):
    from pet_b200 import configs
    from pet_b200.graph import Graph
    g = Graph(ctx)
    b = configs.GraphBuilder(g)
    out = build(b, *args, **kw)
    g.setOutputs([out])
    g.compile(fuse=fuse, cuda_graph=cuda_graph)
    b.load()
    g.run()
    g.run()  # second pass replays the captured CUDA graph
    torch.cuda.synchronize()
    ctx.sync_check()
    return g, out, g.get_data(out)


def oracle_config(build, *args, **kw):
    from oracle_backend import OracleBuilder
    return build(OracleBuilder(), *args, **kw)


def test_c1_rewrite_with_correction_is_bit_identical_to_original(ctx):
    from pet_b200 import configs
    x, w = configs.c1_tensors()
    _, _, y0 = run_config(ctx, configs.c1_original, x, w)
    g, _, y1 = run_config(ctx, configs.c1_rewrite, x, w, correct=True)
    assert np.array_equal(y0, y1)
    _, _, y2 = run_config(ctx, configs.c1_rewrite, x, w, correct=False)
    bad = np.unique(np.nonzero(y0 != y2)[2])
    assert list(bad) == [27, 28]
    # The seam transposes fold into the convolution (a 1x3x3 convolution on the [1,64,2,28,56] view of the input), and
    # because the correction window holds every row the split gets wrong, rewrite + correction is recognised as the
    # unsplit convolution: one launch.  With a window that misses one of those rows the correction stays its own launch.
    assert [n for n, _ in g.steps()] == ["conv_seam_healed"] and g.num_launches() == 1

    def partial(b, x, w):
        xi, wi = b.input(x), b.const(w)
        y = b.transpose(b.conv(b.transpose(xi, *configs.H2N), wi, 1, 1), *configs.N2H)
        return b.correction(xi, wi, y, 1, 1, rows=(27, 1))   # row 28 stays wrong
    g4, _, y4 = run_config(ctx, partial, x, w)
    assert [n for n, _ in g4.steps()] == ["conv_seam_folded", "correction"] and g4.num_launches() == 2
    assert list(np.unique(np.nonzero(y0 != y4)[2])) == [28]
    g3, _, y3 = run_config(ctx, configs.c1_rewrite, x, w, correct=True, fuse=False, cuda_graph=False)
    assert [n for n, _ in g3.steps()] == ["transpose", "conv", "transpose", "correction"]
    assert np.array_equal(y1, y3)  # operator by operator: the same bits
    want = oracle_config(configs.c1_original, x, w)
    assert rel_err(y0, want) <= TOL and scale_err(y0, want) <= TOL_SCALE


def test_c1_rewrite_with_halo_transposes_is_bit_identical_to_original(ctx):
    from pet_b200 import configs
    x, w = configs.c1_tensors()
    _, _, y0 = run_config(ctx, configs.c1_original, x, w)
    g, _, y1 = run_config(ctx, configs.c1_rewrite_halo, x, w)
    assert [n for n, _ in g.steps()] == ["transpose_halo", "conv", "transpose_halo"]
    assert np.array_equal(y0, y1)  # same K order per output: the halo route needs no correction
    assert rel_err(y1, oracle_config(configs.c1_rewrite_halo, x, w)) <= TOL


def test_n2h_rewrite_with_zero_gap_transposes_is_bit_identical_to_original(ctx):
    """The other direction: two images stacked along H with one zero row between them (pad = 1), one convolution over the
    taller image, and a split that skips the gap row (extr = 1) — as a captured graph, equal to the batched conv."""
    from pet_b200.graph import Graph
    rng = np.random.default_rng(31)
    x = rng.uniform(-1, 1, (2, 32, 28, 28)).astype(np.float32)
    w = (rng.standard_normal((48, 32, 3, 3)) * 0.06).astype(np.float32)
    outs = []
    for rewrite in (False, True):
        g = Graph(ctx)
        xi, wi = g.tensor(list(x.shape)), g.tensor(list(w.shape), weight=True)
        if rewrite:
            t = g.transpose_halo(xi, 0, [0, 1, [-1, 2], 3], 2, "pad", 1)           # [1,32,57,28]
            y = g.transpose_halo(g.conv(t, wi, 1, 1), 2, [[0, 2], 1, -1, 3], 28, "extr", 1)
        else:
            y = g.conv(xi, wi, 1, 1)
        g.setOutputs([y])
        g.compile()
        g.set_data(xi, x)
        g.set_data(wi, w)
        g.run()
        g.run()
        torch.cuda.synchronize()
        ctx.sync_check()
        assert tuple(y.dims) == (2, 48, 28, 28)
        outs.append(g.get_data(y))
        if rewrite:
            assert [n for n, _ in g.steps()] == ["transpose_halo", "conv", "transpose_halo"]
    assert np.array_equal(outs[0], outs[1])


def test_c2_rewrite_fuses_chains_and_matches_original(ctx):
    from pet_b200 import configs
    x, w = configs.c2_tensors(c=64, hw=32, k=96)
    _, _, y0 = run_config(ctx, configs.c2_original, x, w)
    g, _, y1 = run_config(ctx, configs.c2_rewrite, x, w)
    # space-to-batch, dense conv, batch-to-space: folded back into the dilated convolution on the untouched tensor
    assert [n for n, _ in g.steps()] == ["conv_seam_folded"] and g.num_launches() == 1
    assert np.array_equal(y0, y1)
    g2, _, y2 = run_config(ctx, configs.c2_rewrite, x, w, fuse=False, cuda_graph=False)
    assert g2.num_launches() == 9
    assert np.array_equal(y1, y2)  # 9 kernels op by op give the same bits as the folded one
    want = oracle_config(configs.c2_rewrite, x, w)
    assert rel_err(y1, want) <= TOL and scale_err(y1, want) <= TOL_SCALE


def test_resnet18_reduced(ctx):
    from pet_b200 import configs
    kw = dict(batch=2, size=64, classes=40, width=16)
    g, _, y = run_config(ctx, configs.resnet18, **kw)
    want = oracle_config(configs.resnet18, **kw)
    assert y.shape == want.shape == (1, 2, 40)
    assert rel_err(y, want) <= TOL
    names = [n for n, _ in g.steps()]
    assert "activation" not in names  # every relu was folded into a conv or an add
    assert names.count("conv") == 20
    # a residual Add whose shortcut is computed before the block's second conv is folded into that conv's epilogue
    assert names.count("add") < 8
    g2, _, y2 = run_config(ctx, configs.resnet18, fuse=False, cuda_graph=False, **kw)
    assert [n for n, _ in g2.steps()].count("add") == 8
    assert np.array_equal(y, y2)  # folding changes neither the arithmetic nor its order


def test_bert_reduced(ctx):
    from pet_b200 import configs
    kw = dict(layers=2, seq=32, hidden=64, heads=4, ffn=128)
    g, _, y = run_config(ctx, configs.bert_encoder, **kw)
    want = oracle_config(configs.bert_encoder, **kw)
    assert y.shape == want.shape == (1, 32, 64)
    assert rel_err(y, want) <= TOL
    names = [n for n, _ in g.steps()]
    # head split / merge transposes became operand strides of the attention matmuls, residual adds went into epilogues
    assert "transpose" not in names and "add" not in names
    g2, _, y2 = run_config(ctx, configs.bert_encoder, fuse=False, cuda_graph=False, **kw)
    assert [n for n, _ in g2.steps()].count("transpose") == 8
    # the Q/K/V projections of a layer were merged into one wide matmul, and scores -> softmax -> context became one
    # attention launch per layer (2 layers x (8 - 2 - 2) matmuls)
    assert names.count("matmul") == 8 and names.count("attention") == 2 and "softmax" not in names
    assert [n for n, _ in g2.steps()].count("matmul") == 16
    # the same graph with the attention chain kept as three steps: the fused launch computes the chain in plain fp32
    from pet_b200.graph import Graph
    g3 = Graph(ctx)
    b3 = configs.GraphBuilder(g3)
    o3 = configs.bert_encoder(b3, **kw)
    g3.setOutputs([o3])
    g3.compile(fuse_attention=False)
    b3.load()
    g3.run()
    torch.cuda.synchronize()
    names3 = [n for n, _ in g3.steps()]
    assert names3.count("matmul") == 12 and names3.count("softmax") == 2 and "attention" not in names3
    assert rel_err(g3.get_data(o3), want) <= TOL and rel_err(y, g3.get_data(o3)) <= TOL
    # same products; the wide matmul may split K differently from the three narrow ones, so sums can round differently
    assert rel_err(g3.get_data(o3), y2) <= 1e-5 and rel_err(y, y2) <= TOL


def test_r3d18_reduced(ctx):
    from pet_b200 import configs
    kw = dict(batch=1, frames=4, size=32, classes=10, width=8)
    _, _, y = run_config(ctx, configs.r3d18, **kw)
    want = oracle_config(configs.r3d18, **kw)
    assert y.shape == want.shape == (1, 1, 10)
    assert rel_err(y, want) <= TOL


def test_group_conv_merge_property_of_the_reference_test(ctx):
    """src/Test/group_conv_test_1.cc as a graph: extend + concat + grouped conv + ratio split equals the two separate convs
    (small integers: exact)."""
    import golden_cases as gc
    from pet_b200.graph import Graph
    g = Graph(ctx)
    i0, i1 = g.tensor([1, 2, 4, 4]), g.tensor([1, 2, 4, 4])
    w0, w1 = g.tensor([4, 2, 3, 3], weight=True), g.tensor([6, 2, 3, 3], weight=True)
    merged = g.conv(g.concat([g.extend(i0, 1, 1), g.extend(i1, 1, 2)], 1), g.concat([w0, w1], 0), 1, 1)
    o0, o1 = g.split(merged, 1, [2, 3])
    t0, t1 = g.conv(i0, w0, 1, 1), g.conv(i1, w1, 1, 1)
    g.setOutputs([o0, o1, t0, t1])
    g.compile()
    data = {i0: gc.small_ints((1, 2, 4, 4), 61) % 16, i1: gc.small_ints((1, 2, 4, 4), 62) % 16,
            w0: gc.small_ints((4, 2, 3, 3), 63) % 16, w1: gc.small_ints((6, 2, 3, 3), 64) % 16}
    for t, a in data.items():
        g.set_data(t, a.astype(np.float32))
    g.run()
    torch.cuda.synchronize()
    ctx.sync_check()
    assert tuple(o0.dims) == (1, 4, 4, 4) and tuple(o1.dims) == (1, 6, 4, 4)
    assert np.array_equal(g.get_data(o0), g.get_data(t0)) and np.array_equal(g.get_data(o1), g.get_data(t1))
    from oracle import pet_oracle as po
    assert np.array_equal(g.get_data(t0).astype(np.uint32), po.conv2d_u32(data[i0], data[w0], pad=(1, 1)))


@pytest.mark.parametrize("phases", ["0", "1"])
def test_convtrans_and_banded_attention_in_a_graph(ctx, oracle, phases, monkeypatch):
    """convTrans -> relu, and g2bmm -> softmax -> gbmml (sliding-window attention) built with the reference's method
    names, executed as a captured graph, against the oracle; the transposed convolution through the zero-insertion path
    and through the phase path (whose convolutions run on forked streams inside the capture)."""
    from pet_b200.graph import Graph
    monkeypatch.setenv("PETB200_CONVTRANS_PHASES", phases)
    rng = np.random.default_rng(12)
    g = Graph(ctx)
    x = g.tensor([2, 8, 8, 32])
    w = g.tensor([4, 4, 32, 16], weight=True)
    up = g.relu(g.convTrans(x, w, 1, 1, 2, 2))
    q, k, v = g.tensor([2, 96, 32]), g.tensor([2, 96, 32]), g.tensor([2, 96, 32])
    att = g.gbmml(g.softmax(g.g2bmm(q, k, 8, 2), -1), v, 2)
    g.setOutputs([up, att])
    g.compile()
    assert tuple(up.dims) == (2, 16, 16, 16) and tuple(att.dims) == (2, 96, 32)
    data = {t: rng.standard_normal(t.dims).astype(np.float32) * 0.5 for t in (x, w, q, k, v)}
    for t, a in data.items():
        g.set_data(t, a)
    g.run()
    g.run()
    torch.cuda.synchronize()
    ctx.sync_check()
    names = [n for n, _ in g.steps()]
    assert names.count("convtrans") == 1 and "g2bmm" in names and "gbmml" in names
    want_up = np.maximum(oracle.convtrans(data[x], data[w], pad=(1, 1), stride=(2, 2), wide=True), 0)
    assert rel_err(g.get_data(up), want_up) <= TOL
    sc = oracle.g2bmm(data[q], data[k], 8, 2, wide=True)
    want_att = oracle.gbmml(oracle.softmax(sc), data[v], 2, wide=True)
    assert rel_err(g.get_data(att), want_att) <= TOL
    total, per = g.perf(rounds=10, warmup=3)
    assert len(per) == len(names) and total > 0


def test_perf_and_time_entry_points(ctx):
    from pet_b200 import configs
    x, w = configs.c2_tensors(c=64, hw=32, k=64)
    g, _, _ = run_config(ctx, configs.c2_rewrite, x, w, fuse=False)   # nine operators, one step each
    total, per = g.perf(rounds=20, warmup=5)
    assert len(per) == 9 and all(p > 0 for p in per) and abs(total - sum(per)) < 1e-4
    total2, per2 = g.perf(rounds=20, warmup=5)
    assert per2 == per  # second call is served from the memo table
    ms = g.time(rounds=50, warmup=10)
    assert 0 < ms < 10
    ctx.sync_check()


def test_graph_rejects_invalid_operators(ctx):
    from pet_b200 import PetError
    from pet_b200.graph import Graph
    g = Graph(ctx)
    x = g.tensor([1, 6, 8, 8])
    with pytest.raises(PetError):
        g.conv(x, g.tensor([4, 4, 3, 3]), 1, 1)         # channels not divisible
    with pytest.raises(PetError):
        g.matmul(g.tensor([2, 4, 5]), g.tensor([3, 5, 6]))  # batch mismatch
    with pytest.raises(PetError):
        g.transpose(x, 1, [0, 1, -1, 2, 3], 4)          # 6 % 4 != 0
    with pytest.raises(PetError):
        g.reshape(x, [5, -1])
    with pytest.raises(PetError):
        g.softmax(x, 4)                                  # axis outside the tensor
    with pytest.raises(PetError):
        g.convTrans(x, g.tensor([3, 3, 8, 4]), 1, 1, 1, 1, 2, 2)  # dilated transposed convolution
    with pytest.raises(PetError):
        g.g2bmm(g.tensor([1, 8, 4]), g.tensor([1, 9, 4]), 2)       # operand shapes differ
    with pytest.raises(PetError):
        g.gbmml(g.tensor([1, 8, 4]), g.tensor([1, 8, 4]))          # band extent must be odd
    with pytest.raises(PetError):
        g.run()                                          # not compiled


def test_random_residual_block_graphs_fused_equals_unfused(ctx):
    """Seeded sweep of small residual networks (1-3 basic blocks, identity or 1x1 strided shortcuts, Add operands in either
    order, optional final ReLU): the compiled graph with every rewrite on (activation and residual folding, shortcut on a
    side stream, CUDA-graph capture) gives the same bits as the operator-by-operator execution."""
    from pet_b200.graph import Graph
    rng = np.random.default_rng(11)
    for it in range(20):
        n, c, f = int(rng.integers(1, 3)), int(rng.choice([8, 16, 64])), int(rng.choice([8, 16, 64, 128]))
        hw, st, nblocks = int(rng.choice([7, 8, 14, 28])), int(rng.choice([1, 2])), int(rng.integers(1, 4))
        outs = []
        for fuse in (True, False):
            g = Graph(ctx)
            r2 = np.random.default_rng(1000 + it)
            x = g.tensor([n, c, hw, hw])
            data = {x: r2.integers(-2, 3, (n, c, hw, hw)).astype(np.float32)}

            def weight(shape):
                t = g.tensor(list(shape), weight=True)
                data[t] = r2.integers(-1, 2, shape).astype(np.float32)
                return t

            t, cin = x, c
            for b in range(nblocks):
                cout, s_ = (f, st) if b == 0 else (cin, 1)
                y = g.conv(g.relu(g.conv(t, weight((cout, cin, 3, 3)), 1, 1, s_, s_)), weight((cout, cout, 3, 3)), 1, 1)
                sc = g.conv(t, weight((cout, cin, 1, 1)), 0, 0, s_, s_) if (cout != cin or s_ != 1) else t
                y = g.add([y, sc]) if r2.integers(0, 2) else g.add([sc, y])
                t = g.relu(y) if r2.integers(0, 4) else y
                cin = cout
            g.setOutputs([t])
            g.compile(fuse=fuse, cuda_graph=fuse)
            for k_, v in data.items():
                g.set_data(k_, v)
            g.run()
            g.run()
            torch.cuda.synchronize()
            ctx.sync_check()
            outs.append((g.get_data(t), [nm for nm, _ in g.steps()]))
        assert np.array_equal(outs[0][0], outs[1][0]), (it, n, c, f, hw, st, nblocks, outs[0][1])
        assert len(outs[0][1]) < len(outs[1][1])


def test_random_encoder_graphs_fused_vs_unfused_vs_oracle(ctx):
    """Seeded sweep of small transformer encoders (1-6 heads, head sizes 8-64, ragged sequence lengths): transposes folded
    into matmul strides and merged Q/K/V projections agree with the operator-by-operator graph and with the oracle."""
    from pet_b200 import configs
    rng = np.random.default_rng(3)
    for _ in range(8):
        heads, hd = int(rng.choice([1, 2, 4, 6])), int(rng.choice([8, 16, 32, 64]))
        kw = dict(layers=int(rng.integers(1, 3)), seq=int(rng.choice([8, 20, 32, 77, 128])), hidden=heads * hd, heads=heads,
                  ffn=int(rng.choice([32, 96, 256])))
        _, _, y = run_config(ctx, configs.bert_encoder, **kw)
        _, _, y2 = run_config(ctx, configs.bert_encoder, fuse=False, cuda_graph=False, **kw)
        assert rel_err(y, y2) <= TOL, kw  # two summation orders of the same products, compounded over the layers
        assert rel_err(y, oracle_config(configs.bert_encoder, **kw)) <= TOL, kw


def test_encoder_longer_than_the_attention_launch_serves(ctx):
    """160 keys per head is past what the one-launch attention takes: the chain stays three steps and still matches."""
    from pet_b200 import configs
    kw = dict(layers=1, seq=160, hidden=64, heads=2, ffn=96)
    g, _, y = run_config(ctx, configs.bert_encoder, **kw)
    names = [n for n, _ in g.steps()]
    assert "attention" not in names and names.count("softmax") == 1
    assert rel_err(y, oracle_config(configs.bert_encoder, **kw)) <= TOL


def test_softmax_over_any_axis(ctx, oracle):
    """SoftmaxOp carries an axis (ref: include/operator.h:1887-1938): every axis of a ragged 4-D tensor, through the operator
    entry point and through a graph, against the oracle."""
    from pet_b200.graph import Graph
    rng = np.random.default_rng(8)
    x = (rng.standard_normal((3, 5, 7, 9)) * 3).astype(np.float32)
    for axis in (0, 1, 2, 3, -2):
        want = oracle.softmax(x, axis)
        got = ctx.softmax(torch.from_numpy(x).cuda(), axis).cpu().numpy()
        assert rel_err(got, want) <= 1e-5, axis
        assert np.allclose(got.sum(axis), 1.0, atol=1e-5)
        g = Graph(ctx)
        t = g.tensor(list(x.shape))
        y = g.softmax(t, axis)
        g.setOutputs([y])
        g.compile()
        g.set_data(t, x)
        g.run()
        torch.cuda.synchronize()
        assert np.array_equal(g.get_data(y), got)
    ctx.sync_check()


@pytest.mark.parametrize("case", [("H", (2, 16, 28, 24), (24, 16, 3, 3), dict(ph=1, pw=1)),
                                  ("H", (1, 8, 20, 12), (8, 8, 3, 3), dict(ph=2, pw=2, dh=2, dw=2)),          # dilated
                                  ("H", (1, 8, 24, 16), (16, 4, 3, 3), dict(ph=1, pw=1, sh=2, sw=2)),         # strided, 2 groups
                                  ("W", (2, 16, 12, 40), (24, 16, 3, 3), dict(ph=1, pw=1)),
                                  ("W", (1, 8, 10, 32), (8, 8, 5, 3), dict(ph=2, pw=1, sw=2))],
                         ids=["H", "H_dilated", "H_strided_grouped", "W", "W_5x3_stride_w"])
def test_seam_transpose_pair_folds_into_the_conv_bit_for_bit(ctx, case):
    """Pre transpose -> conv -> Post transpose (the H or the W pair of the reference's generator) as one launch on a view
    of the untouched tensor, against the three operators executed one by one: small integers, so equality is exact
    whatever tile shapes the two plans pick."""
    from pet_b200 import configs
    from pet_b200.graph import Graph
    axis, xs, ws, kw = case
    rng = np.random.default_rng(len(xs) + xs[2])
    x = rng.integers(-4, 5, xs).astype(np.float32)
    w = rng.integers(-3, 4, ws).astype(np.float32)
    pre, post = (configs.H2N, configs.N2H) if axis == "H" else (configs.W2N, configs.N2W)
    outs = []
    for fuse in (True, False):
        g = Graph(ctx)
        xi, wi = g.tensor(list(xs)), g.tensor(list(ws), weight=True)
        y = g.transpose(g.conv(g.transpose(xi, *pre), wi, kw["ph"], kw["pw"], kw.get("sh", 1), kw.get("sw", 1), kw.get("dh", 1), kw.get("dw", 1)), *post)
        g.setOutputs([y])
        g.compile(fuse=fuse, cuda_graph=False)
        g.set_data(xi, x)
        g.set_data(wi, w)
        g.run()
        torch.cuda.synchronize()
        ctx.sync_check()
        names = [n for n, _ in g.steps()]
        assert names == (["conv_seam_folded"] if fuse else ["transpose", "conv", "transpose"])
        outs.append(g.get_data(y))
    assert outs[0].shape == outs[1].shape and np.array_equal(outs[0], outs[1])
