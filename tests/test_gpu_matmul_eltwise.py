"""GPU: matmul, elementwise, activation, pooling, softmax, LayerNorm, batch-norm through the C ABI vs the oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

import golden_cases as gc
from conftest import rel_err, scale_err

pytestmark = pytest.mark.gpu
TOL, TOL_SCALE = 1e-3, 5e-5


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("algo", ["auto", "simt_fp32"])
def test_batch_gemm_known_answer(ctx, golden, algo):
    i0, w0, w1 = gc.batch_gemm_inputs()  # exact in fp32
    f = lambda a: dev(a.astype(np.float32))
    o0 = ctx.matmul(f(i0), f(w0), algo=algo).cpu().numpy().astype(np.uint32)
    o1 = ctx.matmul(f(i0), f(w1), algo=algo).cpu().numpy().astype(np.uint32)
    assert np.array_equal(o0, golden["bgemm_o0"]) and np.array_equal(o1, golden["bgemm_o1"])
    a2 = ctx.concat([f(i0), f(i0)], 0)
    b2 = ctx.concat([f(w0), f(w1)], 0)
    merged = ctx.matmul(a2, b2, algo=algo)
    assert np.array_equal(merged.cpu().numpy().astype(np.uint32), golden["bgemm_merged"])
    parts = ctx.split(merged, 0, [1, 1])
    assert np.array_equal(parts[0].cpu().numpy().astype(np.uint32), golden["bgemm_o0"])
    ctx.sync_check()


MM = [  # b, m, n, k, transA, transB   (BERT-base shapes and ragged ones)
    (1, 128, 768, 768, False, False), (12, 128, 128, 64, False, True), (12, 128, 64, 128, False, False),
    (1, 128, 3072, 768, False, False), (1, 128, 768, 3072, False, False), (1, 1, 1000, 512, False, False),
    (3, 5, 4, 7, False, False), (2, 8, 70, 130, True, True), (1, 3, 100, 257, False, True), (2, 2, 65, 40, True, False),
    (2, 36, 20, 50, True, True), (2, 300, 40, 24, True, False), (1, 64, 33, 100, False, True),
]


@pytest.mark.parametrize("algo", ["auto", "simt_fp32"])
@pytest.mark.parametrize("shape", MM, ids=[str(s) for s in MM])
def test_matmul_vs_oracle(ctx, oracle, shape, algo):
    b, m, n, k, ta, tb = shape
    rng = np.random.default_rng(b * 1000 + m + n + k)
    a = rng.standard_normal((b, k, m) if ta else (b, m, k)).astype(np.float32)
    bm = (rng.standard_normal((b, n, k) if tb else (b, k, n)) / np.sqrt(k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    want = oracle.matmul(a, bm, bias, ta, tb, act="gelu", wide=True)
    got = ctx.matmul(dev(a), dev(bm), ta, tb, bias=dev(bias), act="gelu", algo=algo).cpu().numpy()
    ctx.sync_check()
    assert got.shape == want.shape
    assert rel_err(got, want) <= TOL and scale_err(got, want) <= TOL_SCALE


@pytest.mark.parametrize("shape", [(1, 128, 768, 768), (1, 2, 100, 64), (2, 36, 20, 52)], ids=str)
def test_matmul_with_residual_equals_matmul_then_add(ctx, shape):
    b, m, n, k = shape
    rng = np.random.default_rng(m + n)
    a, bm = dev(rng.standard_normal((b, m, k)).astype(np.float32)), dev((rng.standard_normal((b, k, n)) / np.sqrt(k)).astype(np.float32))
    bias, res = dev(rng.standard_normal(n).astype(np.float32)), dev(rng.standard_normal((b, m, n)).astype(np.float32))
    want = ctx.eltwise("add", [ctx.matmul(a, bm, bias=bias), res])
    got = ctx.matmul(a, bm, bias=bias, residual=res)
    ctx.sync_check()
    assert torch.equal(got, want)


def test_strided_matmul_equals_matmul_on_transposed_copies(ctx):
    """Attention with the head split/merge folded into operand strides: q, k, v stored as [seq, heads, d]."""
    seq, heads, d = 128, 12, 64
    rng = np.random.default_rng(7)
    q, k, v = (dev(rng.standard_normal((seq, heads, d)).astype(np.float32)) for _ in range(3))
    qh, kh, vh = (t.permute(1, 0, 2).contiguous() for t in (q, k, v))                      # [heads, seq, d] copies
    hd = heads * d
    # scores[h] = q[h] . k[h]^T : A and B (stored [n][k]) are strided views, C dense [heads, seq, seq]
    p1 = ctx.matmul_plan((heads, seq, d), (heads, seq, d), transB=True, strides=(d, hd, d, hd, seq * seq, seq))
    s = torch.empty((heads, seq, seq), device="cuda")
    ctx.matmul_run(p1, q, k, out=s)
    assert torch.equal(s, ctx.matmul(qh, kh, transB=True))
    # ctx[h] = s[h] . v[h], written straight into [seq, heads, d]
    p2 = ctx.matmul_plan((heads, seq, seq), (heads, seq, d), strides=(seq * seq, seq, d, hd, d, hd))
    c = torch.empty((seq, heads, d), device="cuda")
    ctx.matmul_run(p2, s, v, out=c)
    assert torch.equal(c, ctx.matmul(s, vh).permute(1, 0, 2).contiguous())
    ctx.sync_check()
    from pet_b200 import PetError
    with pytest.raises(PetError):  # A strides that TMA cannot express: the caller keeps the copy
        ctx.matmul_plan((2, 16, 8), (2, 8, 8), strides=(130, 10, 64, 8, 128, 8))


def test_matmul_rejects_mismatched_operands(ctx):
    from pet_b200 import PetError
    with pytest.raises(PetError):
        ctx.matmul_plan((2, 4, 5), (3, 5, 6))  # batch mismatch (MatmulOp::checkValid)
    with pytest.raises(PetError):
        ctx.matmul_plan((2, 4, 5), (2, 6, 7))  # inner extents differ


def test_eltwise_and_activations(ctx, oracle, golden):
    u, v = gc.small_ints((4, 6, 8, 10), 41), gc.small_ints((8, 10), 42)
    uf, vf = (u % 64).astype(np.float32), (v % 64).astype(np.float32)
    for k in ("add", "sub", "mul"):
        got = ctx.eltwise(k, [dev(uf), dev(vf)]).cpu().numpy()
        assert np.array_equal(got, oracle.eltwise(k, [uf, vf]))  # exact: small integers
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 7, 5, 9)).astype(np.float32)   # odd sizes: scalar path
    x4 = rng.standard_normal((4, 8, 16, 16)).astype(np.float32)  # vector path
    for t in (x, x4):
        assert np.array_equal(ctx.activation(dev(t), "relu").cpu().numpy(), oracle.activation(t, "relu"))
        for act in ("sigmoid", "tanh", "gelu"):
            assert rel_err(ctx.activation(dev(t), act).cpu().numpy(), oracle.activation(t, act)) <= 1e-4
        r = rng.standard_normal(t.shape).astype(np.float32)
        got = ctx.eltwise("add", [dev(t), dev(r)], act="relu").cpu().numpy()  # residual add + relu
        assert np.array_equal(got, np.maximum(t + r, 0))
    ctx.sync_check()


def test_pool_softmax_layernorm_batchnorm(ctx, oracle):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 64, 112, 112)).astype(np.float32)
    assert np.array_equal(ctx.maxpool(dev(x), 3, 3, 1, 1, 1, 1, 2, 2).cpu().numpy(), oracle.maxpool(x, (3, 3), (1, 1), (2, 2)))
    y = rng.standard_normal((2, 512, 7, 7)).astype(np.float32)
    assert rel_err(ctx.avgpool(dev(y), 7, 7, 0, 0, 1, 1).cpu().numpy(), oracle.avgpool(y, (7, 7), (0, 0), (1, 1))) <= 2e-4
    assert rel_err(ctx.avgpool(dev(y), 3, 3, 1, 1, 2, 2).cpu().numpy(), oracle.avgpool(y, (3, 3), (1, 1), (2, 2))) <= 2e-4
    # large windows (one warp per output), with padding and stride
    assert np.array_equal(ctx.maxpool(dev(y), 6, 7, 1, 1, 2, 3, 3, 2).cpu().numpy(), oracle.maxpool(y, (6, 7), (2, 3), (3, 2)))
    assert rel_err(ctx.avgpool(dev(y), 6, 7, 2, 3, 3, 2).cpu().numpy(), oracle.avgpool(y, (6, 7), (2, 3), (3, 2))) <= 2e-4
    assert rel_err(ctx.rowmean(dev(y), 49).cpu().numpy(), y.reshape(-1, 49).mean(1)) <= 2e-4
    s = rng.standard_normal((12, 128, 128)).astype(np.float32) * 4
    assert rel_err(ctx.softmax(dev(s)).cpu().numpy(), oracle.softmax(s)) <= 1e-5
    s2 = rng.standard_normal((5, 1000)).astype(np.float32)
    assert rel_err(ctx.softmax(dev(s2)).cpu().numpy(), oracle.softmax(s2)) <= 1e-5
    h = rng.standard_normal((128, 768)).astype(np.float32)
    g, b = rng.standard_normal(768).astype(np.float32), rng.standard_normal(768).astype(np.float32)
    assert rel_err(ctx.layernorm(dev(h), dev(g), dev(b)).cpu().numpy(), oracle.layernorm(h, g, b)) <= 1e-4
    z = rng.standard_normal((2, 6, 5, 7)).astype(np.float32)
    sc, bi, me = [rng.standard_normal(6).astype(np.float32) for _ in range(3)]
    va = (np.abs(rng.standard_normal(6)) + 0.5).astype(np.float32)
    assert rel_err(ctx.batchnorm(dev(z), dev(sc), dev(bi), dev(me), dev(va)).cpu().numpy(), oracle.batchnorm(z, sc, bi, me, va)) <= 1e-6
    ctx.sync_check()


def test_div_pow_reducemean_gather(ctx):
    rng = np.random.default_rng(17)
    a = rng.uniform(1, 2, (3, 5, 7, 6)).astype(np.float32)
    b = rng.uniform(1, 2, (7, 6)).astype(np.float32)
    ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    # division with the reference's modulo broadcast (operand j read at i % size_j)
    want = (a.reshape(-1) / b.reshape(-1)[np.arange(a.size) % b.size]).reshape(a.shape)
    assert np.array_equal(ctx.div(ta, tb).cpu().numpy(), want)
    # integer power by repeated multiplication, in the order the reference multiplies
    p3 = ctx.pow(ta, 3).cpu().numpy()
    assert np.array_equal(p3, (np.float32(1) * a) * a * a)
    assert np.allclose(ctx.pow(ta, -2).cpu().numpy(), 1.0 / (a * a), rtol=1e-6)
    assert np.array_equal(ctx.pow(ta, 0).cpu().numpy(), np.ones_like(a))
    for axis in range(4):
        y = ctx.reduce_mean(ta, axis).cpu().numpy()
        assert y.shape == tuple(1 if i == axis else d for i, d in enumerate(a.shape))
        assert np.allclose(y, a.astype(np.float64).mean(axis, keepdims=True), rtol=1e-6, atol=1e-7)
    idx = rng.integers(0, 5, (4, 2)).astype(np.int32)
    words = rng.integers(0, 2**32, a.shape, dtype=np.uint64).astype(np.uint32).view(np.float32)  # arbitrary bit patterns
    tw = torch.from_numpy(words).cuda()
    for axis in range(4):
        ii = rng.integers(0, a.shape[axis], (4, 2)).astype(np.int32)
        got = ctx.gather(tw, torch.from_numpy(ii).cuda(), axis).cpu().numpy()
        want = np.moveaxis(np.take(words, ii, axis=axis), [axis, axis + 1], [0, 1])  # index dims first, then the rest
        assert got.shape == want.shape and np.array_equal(got.view(np.uint32), np.ascontiguousarray(want).view(np.uint32))
    bad = torch.tensor([[0, 9], [-1, 2]], dtype=torch.int32).cuda()  # outside [0,5): zeros
    got = ctx.gather(ta, bad, 1).cpu().numpy()
    assert np.all(got[0, 1] == 0) and np.all(got[1, 0] == 0) and np.array_equal(got[0, 0], a[:, 0]) and np.array_equal(got[1, 1], a[:, 2])
    ctx.sync_check()


def test_small_operators_in_a_graph(ctx):
    from pet_b200.graph import Graph
    from pet_b200 import PetError
    rng = np.random.default_rng(18)
    g = Graph(ctx)
    x = g.tensor([4, 6, 8])
    s_ = g.tensor([8])
    table = g.tensor([10, 8])
    ids = g.tensor([4, 6], dtype="INT32")
    g.setInputs([x, s_, table, ids])
    y = g.reduceMean(g.pow(g.div(x, s_), 2), 2)        # mean of (x / s)^2 over the last axis
    e = g.gather(table, ids, 0)                          # embedding lookup [4,6,8]
    z = g.add([x, e])
    g.setOutputs([y, z])
    g.compile()
    assert g.updateConnection()
    xs, ss = rng.uniform(1, 2, (4, 6, 8)).astype(np.float32), rng.uniform(1, 2, 8).astype(np.float32)
    tb, ii = rng.standard_normal((10, 8)).astype(np.float32), rng.integers(0, 10, (4, 6)).astype(np.int32)
    for t, a in ((x, xs), (s_, ss), (table, tb), (ids, ii)):
        g.set_data(t, a)
    g.run()
    g.run()
    torch.cuda.synchronize()
    ctx.sync_check()
    assert tuple(y.dims) == (4, 6, 1) and tuple(e.dims) == (4, 6, 8)
    q = xs / ss
    assert np.allclose(g.get_data(y), (q * q).astype(np.float64).mean(-1, keepdims=True), rtol=1e-6)
    assert np.array_equal(g.get_data(z), xs + tb[ii])
    assert sorted(n for n, _ in g.getOperators()) == ["add", "div", "gather", "pow", "reduce_mean"]
    with pytest.raises(PetError):
        g.resize(x)


def test_matmul_random_shapes_exact(ctx, oracle):
    rng = np.random.default_rng(2025)
    for _ in range(50):
        b, m, n, k = int(rng.integers(1, 5)), int(rng.integers(1, 200)), int(rng.integers(1, 200)), int(rng.integers(1, 200))
        ta, tb = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        a = rng.integers(0, 4, (b, k, m) if ta else (b, m, k)).astype(np.float32)
        bm = rng.integers(0, 4, (b, n, k) if tb else (b, k, n)).astype(np.float32)
        want = oracle.matmul(a, bm, None, ta, tb, wide=False)
        for algo in ("tc_3xtf32", "simt_fp32", "auto"):
            y = ctx.matmul(torch.from_numpy(a).cuda(), torch.from_numpy(bm).cuda(), ta, tb, algo=algo).cpu().numpy()
            assert np.array_equal(y, want), (algo, b, m, n, k, ta, tb)
    ctx.sync_check()


def test_matmul_epilogue_combinations_exact(ctx, oracle):
    rng = np.random.default_rng(6)
    for _ in range(40):
        bs, m = int(rng.choice([1, 1, 2, 12])), int(rng.choice([1, 4, 16, 128, 200]))
        n, k = int(rng.choice([8, 64, 100, 768, 1000])), int(rng.choice([8, 64, 512, 768, 3072]))
        ta, tb = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        a = rng.integers(-2, 3, (bs, k, m) if ta else (bs, m, k)).astype(np.float32)
        bm = rng.integers(-2, 3, (bs, n, k) if tb else (bs, k, n)).astype(np.float32)
        b = rng.integers(-3, 4, n).astype(np.float32)
        act, use_b, use_res = str(rng.choice(["none", "relu"])), bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        want = oracle.matmul(a, bm, b if use_b else None, ta, tb, wide=False)
        res = rng.integers(-3, 4, want.shape).astype(np.float32)
        want = want + res if use_res else want
        want = np.maximum(want, 0) if act == "relu" else want
        for algo in ("auto", "tc_3xtf32", "simt_fp32"):
            y = ctx.matmul(torch.from_numpy(a).cuda(), torch.from_numpy(bm).cuda(), ta, tb, bias=torch.from_numpy(b).cuda() if use_b else None,
                           act=act, algo=algo, residual=torch.from_numpy(res).cuda() if use_res else None).cpu().numpy()
            assert np.array_equal(y, want), (algo, bs, m, n, k, ta, tb, act, use_b, use_res)
    ctx.sync_check()


def test_pool_softmax_layernorm_eltwise_random_shapes(ctx, oracle):
    """Seeded sweep: pooling windows / strides / paddings on ragged planes (max exact, average to rounding), global
    windows, softmax and LayerNorm rows of 1..3000 columns, element-wise operators with the modulo broadcast."""
    rng = np.random.default_rng(41)
    T = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    for _ in range(50):
        n, c, h, w = int(rng.integers(1, 4)), int(rng.integers(1, 9)), int(rng.integers(1, 40)), int(rng.integers(1, 40))
        kh, kw = int(rng.integers(1, min(h, 8) + 1)), int(rng.integers(1, min(w, 8) + 1))
        sh, sw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        ph, pw = int(rng.integers(0, kh // 2 + 1)), int(rng.integers(0, kw // 2 + 1))
        if (h - (kh - sh) + 2 * ph) // sh <= 0 or (w - (kw - sw) + 2 * pw) // sw <= 0:
            continue
        x = rng.integers(-50, 50, (n, c, h, w)).astype(np.float32)
        case = (x.shape, kh, kw, ph, pw, sh, sw)
        assert np.array_equal(ctx.maxpool(T(x), kh, kw, 1, 1, ph, pw, sh, sw).cpu().numpy(), oracle.maxpool(x, (kh, kw), (ph, pw), (sh, sw))), case
        assert np.allclose(ctx.avgpool(T(x), kh, kw, ph, pw, sh, sw).cpu().numpy(), oracle.avgpool(x, (kh, kw), (ph, pw), (sh, sw)),
                           rtol=1e-6, atol=1e-5), case
    for _ in range(6):
        hw = int(rng.integers(6, 30))
        x = rng.standard_normal((2, 5, hw, hw)).astype(np.float32)
        assert np.allclose(ctx.avgpool(T(x), hw, hw, 0, 0, 1, 1).cpu().numpy()[:, :, 0, 0], x.astype(np.float64).mean((2, 3)), rtol=1e-5, atol=1e-6)
    for _ in range(40):
        rows, cols = int(rng.integers(1, 300)), int(rng.choice([1, 2, 7, 32, 64, 100, 128, 257, 768, 1000, 3000]))
        x = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
        g_, b_ = rng.standard_normal(cols).astype(np.float32), rng.standard_normal(cols).astype(np.float32)
        assert np.allclose(ctx.softmax(T(x)).cpu().numpy(), oracle.softmax(x), rtol=2e-5, atol=1e-7), (rows, cols)
        assert np.allclose(ctx.layernorm(T(x), T(g_), T(b_)).cpu().numpy(), oracle.layernorm(x, g_, b_), rtol=1e-4, atol=1e-4), (rows, cols)
    for _ in range(40):
        shape = tuple(int(rng.integers(1, 12)) for _ in range(int(rng.integers(1, 5))))
        a = rng.integers(-9, 10, shape).astype(np.float32)
        b = rng.integers(-9, 10, shape[int(rng.integers(0, len(shape))):]).astype(np.float32)
        for kind in ("add", "sub", "mul"):
            assert np.array_equal(ctx.eltwise(kind, [T(a), T(b)]).cpu().numpy(), oracle.eltwise(kind, [a, b])), (kind, shape, b.shape)
    ctx.sync_check()


def test_strided_matmul_random_views_exact(ctx):
    """Seeded sweep of operands and results that are strided views of larger buffers (row pitches and batch strides with
    gaps, B stored either way): exact on small integers, and nothing outside the result view is written."""
    rng = np.random.default_rng(61)
    as_view = np.lib.stride_tricks.as_strided
    for _ in range(40):
        bs, m, n = int(rng.integers(1, 5)), int(rng.integers(1, 150)), int(rng.integers(1, 150))
        k, tb = int(rng.choice([4, 8, 32, 64, 100, 128])), bool(rng.integers(0, 2))
        a_row = k + 4 * int(rng.integers(0, 4))
        a_batch = m * a_row + 4 * int(rng.integers(0, 5))
        brows, blen = (n, k) if tb else (k, n)
        b_row = blen + int(rng.integers(0, 5))
        b_batch = brows * b_row + int(rng.integers(0, 7))
        c_row = n + int(rng.integers(0, 5))
        c_batch = m * c_row + int(rng.integers(0, 9))
        A = rng.integers(-2, 3, bs * a_batch + 8).astype(np.float32)
        B = rng.integers(-2, 3, bs * b_batch + 8).astype(np.float32)
        av = as_view(A, (bs, m, k), (4 * a_batch, 4 * a_row, 4))
        bv = as_view(B, (bs, brows, blen), (4 * b_batch, 4 * b_row, 4))
        want = np.einsum("bmk,bnk->bmn" if tb else "bmk,bkn->bmn", av.astype(np.float64), bv.astype(np.float64)).astype(np.float32)
        plan = ctx.matmul_plan((bs, m, k), (bs, n, k) if tb else (bs, k, n), False, tb,
                               strides=(a_batch, a_row, b_batch, b_row, c_batch, c_row))
        ta, tbm = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()  # kept alive until the result has been read
        tc = torch.full((bs * c_batch + 8,), 7.0, device="cuda")
        ctx.check(ctx.lib.petb200_matmul_run(plan.h, ta.data_ptr(), tbm.data_ptr(), None, tc.data_ptr(), None))
        torch.cuda.synchronize()
        out = tc.cpu().numpy()
        case = (bs, m, n, k, tb, a_batch, a_row, b_batch, b_row, c_batch, c_row)
        assert np.array_equal(as_view(out, (bs, m, n), (4 * c_batch, 4 * c_row, 4)), want), case
        as_view(out, (bs, m, n), (4 * c_batch, 4 * c_row, 4))[...] = 7.0
        assert (out == 7.0).all(), case
    ctx.sync_check()


@pytest.mark.parametrize("shape", [(12, 128, 128, 64, 64),   # BERT-base: heads, queries, keys, head width (q/k), head width (v)
                                   (3, 50, 100, 40, 72),     # ragged everywhere
                                   (1, 7, 1, 1, 1), (2, 33, 128, 128, 128), (5, 200, 31, 8, 33), (40, 16, 64, 32, 96),
                                   (40, 60, 64, 32, 96), (160, 16, 128, 64, 64)])  # enough CTAs for the 16-row variant
def test_attention_rows_against_oracle(ctx, oracle, shape):
    """One launch for MatmulOp(transB) -> SoftmaxOp -> MatmulOp: against the oracle evaluating the three operators, and
    against this backend's own three operators (the fused kernel is plain fp32, so it sits closer to the oracle)."""
    bs, m, n, kd, d = shape
    rng = np.random.default_rng(sum(shape))
    q = (rng.standard_normal((bs, m, kd)) / np.sqrt(kd)).astype(np.float32)  # the 1/sqrt(d) of attention, folded into q
    k = rng.standard_normal((bs, n, kd)).astype(np.float32)
    v = rng.standard_normal((bs, n, d)).astype(np.float32)
    want = oracle.matmul(oracle.softmax(oracle.matmul(q, k, transB=True), 2), v)
    got = ctx.attention(dev(q), dev(k), dev(v)).cpu().numpy()
    assert got.shape == want.shape == (bs, m, d)
    # (the metric judges outputs that cancel to ~0 against a thousandth of the largest one, so fp32 rounding of the scores
    # alone shows up at 1e-4)
    assert rel_err(got, want) <= TOL and scale_err(got, want) <= 2e-6, shape
    three = ctx.matmul(ctx.softmax(ctx.matmul(dev(q), dev(k), transB=True), 2), dev(v)).cpu().numpy()
    assert rel_err(three, want) <= TOL and rel_err(got, three) <= TOL
    # operands off the 16-byte grid take the generic kernel, aligned ones the tiled kernel: same sums in the same order
    shifted = []
    for t in (q, k, v):
        buf = torch.zeros(t.size + 1, device="cuda")
        buf[1:].copy_(dev(t).reshape(-1))
        shifted.append(buf[1:].view(*t.shape))
    assert shifted[0].data_ptr() % 16 == 4
    assert np.array_equal(ctx.attention(*shifted).cpu().numpy(), got)
    # rows of a wider matrix as operands (the head split of a merged Q/K/V projection): same result bit for bit
    if kd == d:
        wide = torch.zeros((max(m, n), bs, 3, kd + 4), device="cuda")
        wide[:m, :, 0, :kd] = dev(q).transpose(0, 1)
        wide[:n, :, 1, :kd] = dev(k).transpose(0, 1)
        wide[:n, :, 2, :kd] = dev(v).transpose(0, 1)
        out = torch.zeros((m, bs, d), device="cuda")
        row, bat = wide.stride(0), wide.stride(1)
        st = (C.c_longlong * 8)(bat, row, bat, row, bat, row, out.stride(1), out.stride(0))
        ctx.check(ctx.lib.petb200_attention_run(ctx.h, wide[:, :, 0].data_ptr(), wide[:, :, 1].data_ptr(), wide[:, :, 2].data_ptr(), out.data_ptr(),
                                                bs, m, n, kd, d, st, None))
        torch.cuda.synchronize()
        assert np.array_equal(out.transpose(0, 1).cpu().numpy(), got)
    ctx.sync_check()


def test_attention_rows_limits(ctx):
    from pet_b200 import lib as L
    z = lambda *s: torch.zeros(s, device="cuda")
    with pytest.raises(L.PetError) as e:
        ctx.attention(z(1, 8, 16), z(1, 129, 16), z(1, 129, 16))  # 129 keys
    assert e.value.status == L.ERR_UNSUPPORTED
    with pytest.raises(L.PetError):
        ctx.attention(z(1, 8, 16), z(1, 16, 8), z(1, 16, 8))            # head widths of q and k differ
    bad = (C.c_longlong * 8)(64, 8, 64, 16, 64, 16, 64, 16)  # q rows 8 apart but 16 long
    t = z(1, 4, 16)
    assert ctx.lib.petb200_attention_run(ctx.h, t.data_ptr(), t.data_ptr(), t.data_ptr(), z(1, 4, 16).data_ptr(), 1, 4, 4, 16, 16, bad, None) == L.ERR_INVALID
    assert ctx.lib.petb200_attention_supported(128, 128, 64, 64) == 1
    assert ctx.lib.petb200_attention_supported(128, 256, 64, 64) == 0
