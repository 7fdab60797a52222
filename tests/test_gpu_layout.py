"""GPU: layout / index kernels through the C ABI, bit-exact against the reference-produced vectors and the oracle."""
import numpy as np
import pytest
import torch

import golden_cases as gc

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).cuda()


def host(t):
    return t.cpu().numpy().view(np.uint32)


@pytest.mark.parametrize("name", sorted(gc.TRANSPOSES))
def test_transpose_bit_exact_vs_reference_vectors(ctx, golden, name):
    shape, split, after, factor = gc.TRANSPOSES[name]
    got = host(ctx.transpose(dev(gc.words(shape, 11)), split, after, factor))
    want = golden["tr_" + name]
    assert got.shape == want.shape and np.array_equal(got, want)


def test_copy_ops_bit_exact_vs_reference_vectors(ctx, golden):
    t = gc.words((4, 6, 8, 10), 12)
    assert np.array_equal(host(ctx.pad(dev(t), *gc.PAD)), golden["pad"])
    assert np.array_equal(host(ctx.slice(dev(t), *gc.SLICE)), golden["slice"])
    for d in range(4):
        assert np.array_equal(host(ctx.extend(dev(t), d, 2)), golden[f"extend_{d}"])
        assert np.array_equal(host(ctx.concat([dev(t)] * 3, d)), golden[f"concat_{d}"])
        for j, o in enumerate(ctx.split(dev(t), d, [1, 1])):
            assert np.array_equal(host(o), golden[f"split_{d}_{j}"])
    for j, o in enumerate(ctx.split(dev(t), 1, [1, 2])):
        assert np.array_equal(host(o), golden[f"split_ratio_{j}"])


def test_n2h_kernel_reproduces_the_reference_fixture_digest(ctx):
    """The reference's committed transpose fixture (src/Test/dat/transpose_test/input.dat, packed into tests/golden)
    through the CUDA N2H kernel: the result must hash to the SHA-256 of the output file the reference's own
    transpose_test_1 writes."""
    import hashlib
    import os
    from test_oracle import PACKED_FIXTURE, REF_FIXTURE_OUT_SHA
    x = np.load(PACKED_FIXTURE)["digits"].astype(np.uint32)
    y = host(ctx.transpose(dev(x), 0, [0, 1, [-1, 2], 3], 2))
    assert y.shape == (8, 16, 64, 32)
    assert hashlib.sha256(gc.tpm_text(y)).hexdigest() == REF_FIXTURE_OUT_SHA


S2B = [(2, [0, 1, [-1, 2], 3], 2), (2, [[0, 2], 1, -1, 3], -2), (3, [0, 1, 2, [-1, 3]], 2), (3, [[0, 3], 1, 2, -1], -2)]
B2S = [(0, [0, 1, 2, [-1, 3]], 2), (3, [0, 1, 2, [-1, 3]], -2), (0, [0, 1, [-1, 2], 3], 2), (2, [0, 1, [-1, 2], 3], -2)]


@pytest.mark.parametrize("shape", [(1, 8, 16, 16), (2, 5, 12, 20), (1, 512, 64, 64)])
def test_fused_space_to_batch_chain_equals_op_by_op(ctx, oracle, shape):
    x = gc.words(shape, 3)
    want = x
    for op in S2B:
        want = oracle.transpose(want, *op)
    fused = ctx.transpose_chain(dev(x), S2B)
    assert tuple(fused.shape) == want.shape and np.array_equal(host(fused), want)
    step = dev(x)
    for op in S2B:
        step = ctx.transpose(step, *op)
    assert torch.equal(step, fused)
    back = ctx.transpose_chain(fused, B2S)  # the inverse chain restores the tensor
    assert np.array_equal(host(back), x)


@pytest.mark.parametrize("shape,split,after,factor", [
    ((3, 7, 5), -1, [2, 1, 0], 2),           # ragged extents, no 32-multiple anywhere
    ((1, 33, 65), -1, [0, 2, 1], 2),         # the reference's transpose kernel drops these remainders
    ((6, 10, 3, 9), 1, [0, [2, -1], 1, 3], 5),
    ((2, 1, 1, 4), -1, [3, 0, 1, 2], 2),
    ((1,), -1, [0], 2),
    ((128, 12, 64), -1, [1, 0, 2], 2),       # BERT head split
    ((12, 128, 64), -1, [0, 2, 1], 2),       # K^T
])
def test_transpose_edge_shapes(ctx, oracle, shape, split, after, factor):
    x = gc.words(shape, 21)
    want = oracle.transpose(x, split, after, factor)
    got = ctx.transpose(dev(x), split, after, factor)
    assert tuple(got.shape) == want.shape and np.array_equal(host(got), want)


def test_large_layout_round_trip_and_checksum(ctx):
    # size-independent properties at a size far beyond L2: a permutation preserves the multiset (sum) and the
    # inverse restores the tensor exactly
    x = torch.randint(-2**31, 2**31 - 1, (64, 64, 128, 128), dtype=torch.int32, device="cuda")  # 256 MiB
    y = ctx.transpose(x, 2, [[0, 2], 1, -1, 3], -2)   # H2N
    assert int(y.to(torch.int64).sum()) == int(x.to(torch.int64).sum())
    z = ctx.transpose(y, 0, [0, 1, [-1, 2], 3], 2)    # N2H
    assert torch.equal(z, x)
    t = ctx.transpose(x, -1, [0, 1, 3, 2], 2)
    assert torch.equal(t, x.transpose(2, 3).contiguous())


def test_invalid_layout_requests_are_rejected(ctx):
    from pet_b200 import PetError
    x = torch.zeros((3, 5), dtype=torch.int32, device="cuda")
    with pytest.raises(PetError) as e:
        ctx.transpose(x, 1, [0, 1, -1], 2)  # 5 % 2 != 0: the reference marks the output invalid
    assert e.value.status == 1
    with pytest.raises(PetError):
        ctx.transpose(x, -1, [0, 0], 2)  # not a permutation
    with pytest.raises(PetError):
        ctx.slice(x, [0, 0], [3, 0])  # empty result
    with pytest.raises(PetError):
        ctx.split(x, 1, [1, 1])  # 5 not divisible by the ratio sum


@pytest.mark.parametrize("i", range(len(gc.HALO_TRANSPOSES)))
def test_halo_transpose_bit_exact_vs_reference_vectors(ctx, golden, i):
    shape, split, after, factor, mode, amount = gc.HALO_TRANSPOSES[i]
    x = gc.words(shape, 500 + i)
    y = ctx.transpose_halo(dev(x.view(np.int32)), split, after, factor, mode, amount)
    ctx.sync_check()
    want = golden[f"halo_{i}"]
    assert tuple(y.shape) == want.shape
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want)


HALO_BIG = [
    # config-1 sized: H split with a one-row halo and its inverse merge; stacked images with a zero row and its inverse split
    ((1, 64, 56, 56), 2, [[0, 2], 1, -1, 3], -2, "copys", 1),
    ((2, 64, 29, 56), 0, [0, 1, [-1, 2], 3], 2, "dels", 1),
    ((2, 64, 28, 56), 0, [0, 1, [-1, 2], 3], 2, "pad", 1),
    ((1, 64, 57, 56), 2, [[0, 2], 1, -1, 3], 28, "extr", 1),
    ((8, 32, 30, 33), 0, [0, 1, 2, [-1, 3]], 2, "pad", 3),    # odd row length: word kernels
    ((4, 16, 9, 130), 3, [[0, 3], 1, 2, -1], -2, "copys", 2),
]


@pytest.mark.parametrize("case", HALO_BIG, ids=[f"{c[4]}{c[5]}_{'x'.join(map(str, c[0]))}" for c in HALO_BIG])
def test_halo_transpose_vs_oracle(ctx, oracle, case):
    shape, split, after, factor, mode, amount = case
    x = gc.words(shape, 77)
    want = oracle.transpose_halo(x, split, after, factor, mode, amount)
    y = ctx.transpose_halo(dev(x.view(np.int32)), split, after, factor, mode, amount)
    ctx.sync_check()
    assert tuple(y.shape) == want.shape
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want)


def test_halo_rewrite_equals_unsplit_conv_and_correction_route(ctx):
    """Config 1 (3x3, 64 channels, 56x56): the H->N rewrite restored three ways — halo split + dropping merge, the
    correction kernel on the seam rows, and the unsplit conv — agree (small integers: every route is exact)."""
    x = torch.from_numpy((gc.small_ints((1, 64, 56, 56), 91) % 8).astype(np.float32)).cuda()
    w = torch.from_numpy((gc.small_ints((64, 64, 3, 3), 92) % 8).astype(np.float32)).cuda()
    y0 = ctx.conv2d(x, w, 1, 1)
    xs = ctx.transpose_halo(x, 2, [[0, 2], 1, -1, 3], -2, "copys", 1)
    assert tuple(xs.shape) == (2, 64, 29, 56)
    y1 = ctx.transpose_halo(ctx.conv2d(xs, w, 1, 1), 0, [0, 1, [-1, 2], 3], 2, "dels", 1)
    assert torch.equal(y1, y0)
    xm = ctx.transpose(x, 2, [[0, 2], 1, -1, 3], -2)                    # plain H2N: seam rows 27/28 come out wrong ...
    y2 = ctx.transpose(ctx.conv2d(xm, w, 1, 1), 0, [0, 1, [-1, 2], 3], 2)
    assert not torch.equal(y2, y0)
    plan = ctx.conv2d_plan(x.shape, w.shape, 1, 1)
    ctx.conv2d_set_weights(plan, w)
    ctx.conv2d_correct(plan, x, y2, 27, 2)                              # ... until the correction recomputes them
    ctx.sync_check()
    assert torch.equal(y2, y0)


def test_halo_transpose_rejects_bad_requests(ctx):
    from pet_b200 import PetError
    with pytest.raises(PetError):
        ctx.transpose_halo_plan((1, 4, 9, 8), 2, [[0, 2], 1, -1, 3], -2, "copys", 1)       # 9 is not 2 x n
    with pytest.raises(PetError):
        ctx.transpose_halo_plan((6, 4, 8, 8), 0, [0, 1, [-1, 2], 3], 3, "dels", 1)         # dels needs a pair [2][n]
    with pytest.raises(PetError):
        ctx.transpose_halo_plan((2, 4, 8, 8), -1, [0, 1, 3, 2], 2, "pad", 1)               # no merged pair


def test_transposes_match_the_reference_tests_reshape_definitions(ctx):
    for name, x, (split, after, factor), want in gc.reshape_transpose_definitions():
        got = host(ctx.transpose(dev(x), split, after, factor))
        assert got.shape == want.shape and np.array_equal(got, want), name


def test_halo_transpose_random_shapes(ctx, oracle):
    """Seeded sweep: the four parameters on H and on W, amounts 1-3, ragged extents, two or three merged blocks."""
    rng = np.random.default_rng(7)
    for _ in range(60):
        mode, amt = str(rng.choice(["copys", "dels", "pad", "extr"])), int(rng.integers(1, 4))
        n_, c_, on_h = int(rng.integers(1, 4)), int(rng.integers(1, 5)), bool(rng.integers(0, 2))
        half, other, blocks = int(rng.integers(amt + 1, 20)), int(rng.integers(1, 40)), int(rng.integers(2, 4))
        split_hw = (2, [[0, 2], 1, -1, 3]) if on_h else (3, [[0, 3], 1, 2, -1])
        merge_hw = (0, [0, 1, [-1, 2], 3]) if on_h else (0, [0, 1, 2, [-1, 3]])
        place = (lambda e: (e, other)) if on_h else (lambda e: (other, e))
        if mode == "copys":
            shape, args = (n_, c_) + place(2 * half), split_hw + (-2,)
        elif mode == "dels":
            shape, args = (2 * n_, c_) + place(half), merge_hw + (2,)
        elif mode == "pad":
            shape, args = (blocks * n_, c_) + place(half), merge_hw + (blocks,)
        else:
            shape, args = (n_, c_) + place(blocks * (half + amt) - amt), split_hw + (half,)
        x = gc.words(shape, 900 + amt)
        want = oracle.transpose_halo(x, *args, mode, amt)
        got = host(ctx.transpose_halo(dev(x), *args, mode, amt))
        assert got.shape == want.shape and np.array_equal(got, want), (mode, amt, shape)
    ctx.sync_check()


def _random_transpose(rng, shape):
    """A random valid TransposeOp on `shape`: optional split by a divisor (either sign convention), a random permutation
    of the resulting dims, one merged group of up to three neighbours."""
    nd = len(shape)
    split, factor = int(rng.integers(-1, nd)), 2
    if split >= 0:
        f = int(rng.choice([d for d in range(1, shape[split] + 1) if shape[split] % d == 0]))
        factor = f if rng.integers(0, 2) else -f
    items = list(range(nd)) + ([-1] if split >= 0 else [])
    perm = [items[i] for i in rng.permutation(len(items))]
    gsz = int(rng.integers(1, min(3, len(perm)) + 1))
    gpos = int(rng.integers(0, len(perm) - gsz + 1))
    after = perm[:gpos] + ([perm[gpos:gpos + gsz]] if gsz > 1 else perm[gpos:gpos + 1]) + perm[gpos + gsz:]
    return split, after, factor


def test_random_transposes_and_fused_pairs_bit_exact(ctx, oracle):
    from pet_b200 import PetError
    rng = np.random.default_rng(99)
    singles = pairs = 0
    for _ in range(120):
        shape = tuple(int(rng.choice([1, 2, 3, 4, 6, 8, 12, 16, 33])) for _ in range(int(rng.integers(2, 6))))
        x = gc.words(shape, 1234)
        t1 = _random_transpose(rng, shape)
        want = oracle.transpose(x, *t1)
        got = host(ctx.transpose(dev(x), *t1))
        assert got.shape == want.shape and np.array_equal(got, want), (shape, t1)
        singles += 1
        t2 = _random_transpose(rng, want.shape)
        want2 = oracle.transpose(want, *t2)
        try:
            got2 = host(ctx.transpose_chain(dev(x), [t1, t2]))
        except PetError as e:  # a pair that is not one index map stays two steps in the graph layer
            assert "not expressible" in str(e), (shape, t1, t2, str(e))
            continue
        assert got2.shape == want2.shape and np.array_equal(got2, want2), (shape, t1, t2)
        pairs += 1
    ctx.sync_check()
    assert singles == 120 and pairs >= 60
