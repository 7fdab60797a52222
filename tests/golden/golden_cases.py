"""Recipes of the inputs behind tests/golden/ref_vectors.npz (shared by the generator and the tests)."""
import numpy as np

TRANSPOSES = {  # name: (input shape, split, after, factor) — constructor arguments of the reference's TransposeOp
    "N2H": ((4, 6, 8, 10), 0, [0, 1, [-1, 2], 3], 2),
    "H2N": ((4, 6, 8, 10), 2, [[0, 2], 1, -1, 3], -2),
    "N2W": ((4, 6, 8, 10), 0, [0, 1, 2, [-1, 3]], 2),
    "W2N": ((4, 6, 8, 10), 3, [[0, 3], 1, 2, -1], -2),
    "C2H": ((4, 6, 8, 10), 1, [0, 1, [2, -1], 3], 2),
    "C2W": ((4, 6, 8, 10), 1, [0, 1, 2, [3, -1]], 2),
    "D2H": ((4, 6, 8, 10), 2, [0, 1, [-1, 2], 3], 2),
    "D2H_inv": ((4, 6, 8, 10), 2, [0, 1, [-1, 2], 3], -2),
    "D2W": ((4, 6, 8, 10), 3, [0, 1, 2, [-1, 3]], 2),
    "D2W_inv": ((4, 6, 8, 10), 3, [0, 1, 2, [-1, 3]], -2),
    "swap_hw": ((4, 6, 8, 10), -1, [0, 1, 3, 2], 2),
    "flatten1": ((4, 6, 8, 10), -1, [0, [1, 2, 3]], 2),
    "perm2031": ((4, 6, 8, 10), -1, [2, 0, 3, 1], 2),
    "mm_swap": ((3, 40, 24), -1, [0, 2, 1], 2),
    "promote": ((12, 20), 0, [-1, 0, 1], 1),
    "heads": ((16, 4, 8), -1, [1, 0, 2], 2),
}
HALO_TRANSPOSES = [  # (input shape, split, after, factor, mode, amount): TransposeOp with pad / extr / copys / dels
    ((2, 3, 8, 4), 2, [[0, 2], 1, -1, 3], -2, "copys", 1),    # H2N before a 3x3 conv: two halves with one halo row
    ((2, 3, 8, 4), 2, [[0, 2], 1, -1, 3], -2, "copys", 2),
    ((2, 2, 4, 12), 3, [[0, 3], 1, 2, -1], -2, "copys", 1),   # W2N
    ((4, 3, 5, 4), 0, [0, 1, [-1, 2], 3], 2, "dels", 1),      # N2H after it: drops the rows computed from the halo
    ((4, 3, 6, 4), 0, [0, 1, [-1, 2], 3], 2, "dels", 2),
    ((4, 2, 3, 7), 0, [0, 1, 2, [-1, 3]], 2, "dels", 1),      # N2W
    ((4, 3, 5, 4), 0, [0, 1, [-1, 2], 3], 2, "pad", 1),       # N2H before a conv: zero rows between the images
    ((4, 2, 3, 5), 0, [0, 1, 2, [-1, 3]], 2, "pad", 2),
    ((6, 2, 3, 4), 0, [0, 1, [-1, 2], 3], 3, "pad", 1),       # three images stacked
    ((2, 3, 11, 4), 2, [[0, 2], 1, -1, 3], -2, "extr", 1),    # H2N after it: skips the gap rows
    ((2, 2, 4, 12), 3, [[0, 3], 1, 2, -1], 5, "extr", 2),
]
CONVS = [  # (x shape, w shape, kwargs)
    ((2, 8, 12, 10), (6, 4, 3, 3), dict(pad=(1, 1))),
    ((2, 8, 12, 10), (6, 4, 3, 3), dict(pad=(2, 2), dil=(2, 2))),
    ((2, 8, 12, 10), (6, 4, 3, 3), dict(pad=(1, 0), stride=(2, 2))),
    ((1, 6, 9, 11), (4, 6, 1, 1), dict(pad=(0, 0))),
    ((1, 3, 15, 15), (5, 3, 7, 7), dict(pad=(3, 3), stride=(2, 2))),
]
CONVTRANS = [  # (x shape {n,h,w,f}, w shape {r,s,f,c}, kwargs, whole) — ConvTransOp; `whole` picks the reference's
    # whole-tensor body (complete only when oh == ow == c), otherwise its one-position body fills the tensor
    ((1, 4, 4, 3), (4, 4, 3, 8), dict(pad=(1, 1), stride=(2, 2)), True),
    ((2, 5, 4, 3), (3, 3, 3, 5), dict(pad=(1, 0), stride=(2, 1), out_pad=(1, 0)), False),
    ((1, 4, 5, 2), (3, 2, 2, 3), dict(pad=(0, 1), stride=(3, 2), out_pad=(2, 1)), False),
    ((1, 6, 5, 2), (4, 3, 2, 3), dict(stride=(3, 3)), False),  # (h+2ph-r) % sh = 2: the reference skips tap rr = 3
    ((1, 3, 3, 2), (2, 2, 2, 2), dict(pad=(3, 3), stride=(2, 2), out_pad=(1, 1)), False),  # padding >= kernel
]
PAD = ([0, 1, 2, 0], [1, 0, 3, 2])
SLICE = ([0, 1, 2, 0], [1, 0, 3, 2])


def words(shape, seed):
    """Arbitrary 32-bit patterns (copy-type operators must move them untouched)."""
    return np.random.default_rng(seed).integers(0, 2**32, shape, dtype=np.uint64).astype(np.uint32)


def small_ints(shape, seed):
    """Values in [0, 10000), the range the reference's own dataRand uses (include/tensor.h:171-186)."""
    return np.random.default_rng(seed).integers(0, 10000, shape, dtype=np.int64).astype(np.uint32)


def digits(shape, seed):
    return np.random.default_rng(seed).integers(0, 10, shape, dtype=np.int64).astype(np.uint32)


def batch_gemm_inputs():
    m, n, k = 8, 8, 4
    i0 = np.arange(m * k, dtype=np.uint32).reshape(1, m, k)
    w0 = (np.arange(k * n, dtype=np.uint32) * 3).reshape(1, k, n)
    w1 = (np.arange(k * n, dtype=np.uint32) * 7).reshape(1, k, n)
    return i0, w0, w1


def pad_slice_inputs():
    return np.arange(49, dtype=np.uint32).reshape(1, 1, 7, 7), np.arange(25, dtype=np.uint32).reshape(1, 1, 5, 5)


def tpm_text(arr):
    """The text format the reference's transpose test writes: '%u ' per element, newline after every 32."""
    flat = np.asarray(arr, dtype=np.uint32).ravel()
    lines = [" ".join(map(str, flat[i:i + 32])) + " \n" for i in range(0, flat.size, 32)]
    return "".join(lines).encode()


def convtrans_kat():
    """Inputs and expected output of the reference's own ConvTransOp test (src/Test/convtrans_test_1.cc:14-76): x = its own
    offset, weight[r,s,f,c] = ((f*R + r)*S + s)*C + c, 4x4 filter, stride 2, padding 1; the expected values are the ones
    that test lists (as [c][oh][ow])."""
    n, c, h, w, f, r, s = 1, 2, 2, 2, 3, 4, 4
    x = np.arange(n * h * w * f, dtype=np.uint32).reshape(n, h, w, f)
    rr, ss, ff, cc = np.meshgrid(np.arange(r), np.arange(s), np.arange(f), np.arange(c), indexing="ij")
    wt = (((ff * r + rr) * s + ss) * c + cc).astype(np.uint32)
    want = np.array([[[190, 740, 770, 592], [992, 2704, 2836, 1832], [1184, 3232, 3364, 2168], [1114, 2660, 2762, 1624]],
                     [[193, 755, 785, 604], [1016, 2770, 2902, 1874], [1208, 3298, 3430, 2210], [1135, 2711, 2813, 1654]]],
                    np.uint32)
    return x, wt, dict(pad=(1, 1), stride=(2, 2)), np.ascontiguousarray(want.transpose(1, 2, 0))[None]


def reshape_transpose_definitions():
    """The reshape/transpose statements of D2H, its inverse, N2H and H2N that the reference's transpose_test_2.py gives
    (src/Test/transpose_test_2.py:4-33), as (name, input, TransposeOp arguments, expected) on that file's shapes."""
    i0 = np.arange(64, dtype=np.uint32).reshape(1, 1, 8, 8)
    d2h = i0.reshape(1, 1, 4, 2, 8).transpose(0, 1, 3, 2, 4).reshape(1, 1, 8, 8)           # h_d2_d1
    d2h_inv = d2h.reshape(1, 1, 2, 4, 8).transpose(0, 1, 3, 2, 4).reshape(1, 1, 8, 8)      # h_d1_d2
    j0 = np.arange(32, dtype=np.uint32).reshape(2, 1, 4, 4)
    n2h = j0.reshape(1, 2, 1, 4, 4).transpose(0, 2, 1, 3, 4).reshape(1, 1, 8, 4)           # nd2_hm2
    h2n = n2h.reshape(1, 1, 2, 4, 4).transpose(0, 2, 1, 3, 4).reshape(2, 1, 4, 4)          # nm2_hd2
    return [("D2H", i0, TRANSPOSES["D2H"][1:], np.ascontiguousarray(d2h)),
            ("D2H_inv", np.ascontiguousarray(d2h), TRANSPOSES["D2H_inv"][1:], np.ascontiguousarray(d2h_inv)),
            ("N2H", j0, TRANSPOSES["N2H"][1:], np.ascontiguousarray(n2h)),
            ("H2N", np.ascontiguousarray(n2h), TRANSPOSES["H2N"][1:], np.ascontiguousarray(h2n))]
