"""Generates tests/golden/ref_vectors.npz by running the REFERENCE's own host operators (oracle/_ref/libpetref.so,
built from the reference checkout by oracle/Makefile) on small deterministic inputs.  Run it where the reference
checkout exists:   python tests/golden/make_golden.py
The tests then check the CPU oracle (and, on a GPU, the CUDA kernels) against these stored outputs; nothing at
test time needs the reference.  Inputs are not stored: they are rebuilt from the recipes in golden_cases.py.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
sys.path.insert(0, HERE)

import golden_cases as gc  # noqa: E402
from oracle import petref as pr  # noqa: E402


def main():
    if not pr.available():
        raise SystemExit("oracle/_ref/libpetref.so missing: run `make -C oracle ref` with the reference checkout present")
    out = {}
    for name, (shape, split, after, factor) in gc.TRANSPOSES.items():
        out["tr_" + name] = pr.transpose(gc.words(shape, 11), split, after, factor)
    for i, (xs, ws, kw) in enumerate(gc.CONVS):
        out[f"conv_{i}"] = pr.conv2d_u32(gc.small_ints(xs, 100 + i), gc.small_ints(ws, 200 + i), **kw)
    for i, (xs, ws, kw, whole) in enumerate(gc.CONVTRANS):
        out[f"convtrans_{i}"] = pr.convtrans_u32(gc.small_ints(xs, 300 + i), gc.small_ints(ws, 400 + i), whole=whole, **kw)
    # the reference's own generated index expression (TransposeEngine::getLambda), evaluated at every output position
    for i, (shape, split, after, factor, mode, amount) in enumerate(gc.HALO_TRANSPOSES):
        out[f"halo_{i}"] = pr.transpose_halo(gc.words(shape, 500 + i), split, after, factor, mode, amount)
    # src/Test/batch_gemm_test.cc: inputs i, 3i, 7i; two matmuls and the merged batch matmul
    i0, w0, w1 = gc.batch_gemm_inputs()
    out["bgemm_o0"] = pr.matmul_u32(i0, w0)
    out["bgemm_o1"] = pr.matmul_u32(i0, w1)
    out["bgemm_merged"] = pr.matmul_u32(pr.concat([i0, i0], 0), pr.concat([w0, w1], 0))
    a, b = gc.small_ints((3, 5, 7), 31), gc.small_ints((3, 7, 4), 32)
    out["mm_nn"] = pr.matmul_u32(a, b)
    out["mm_tt"] = pr.matmul_u32(np.ascontiguousarray(a.transpose(0, 2, 1)), np.ascontiguousarray(b.transpose(0, 2, 1)), True, True)
    # src/Test/pad_slice_test.cc: 7x7 input, 5x5 kernel, pad 2, inputs = index; direct vs pad->conv->slice
    x, w = gc.pad_slice_inputs()
    out["padslice_o1"] = pr.conv2d_u32(x, w, pad=(2, 2))
    padded = pr.pad(x, [0, 0, 0, 0], [0, 0, 1, 1])
    out["padslice_o2"] = pr.slice_(pr.conv2d_u32(padded, w, pad=(2, 2)), [0, 0, 0, 0], [0, 0, 1, 1])
    t = gc.words((4, 6, 8, 10), 12)
    out["pad"] = pr.pad(t, *gc.PAD)
    out["slice"] = pr.slice_(t, *gc.SLICE)
    for d in range(4):
        out[f"extend_{d}"] = pr.extend(t, d, 2)
        out[f"concat_{d}"] = pr.concat([t, t, t], d)
        for j, o in enumerate(pr.split(t, d, [1, 1])):
            out[f"split_{d}_{j}"] = o
    for j, o in enumerate(pr.split(t, 1, [1, 2])):
        out[f"split_ratio_{j}"] = o
    u, v = gc.small_ints((4, 6, 8, 10), 41), gc.small_ints((8, 10), 42)
    for k in ("add", "sub", "mul"):
        out["elt_" + k] = pr.eltwise_u32(k, [u, v])
    # the H->N rewrite of a 3x3 conv (config 1 at reduced channel count): which outputs differ from the original
    x, w = gc.small_ints((1, 8, 56, 56), 51), gc.small_ints((8, 8, 3, 3), 52)
    y0 = pr.conv2d_u32(x, w, pad=(1, 1))
    h2n = pr.transpose(x, 2, [[0, 2], 1, -1, 3], -2)
    y1 = pr.transpose(pr.conv2d_u32(h2n, w, pad=(1, 1)), 0, [0, 1, [-1, 2], 3], 2)
    bad_rows = np.unique(np.nonzero(y0 != y1)[2])
    out["h2n_bad_rows"] = bad_rows.astype(np.int32)
    out["h2n_bad_count"] = np.array([int((y0 != y1).sum())], np.int64)
    # the dilated rewrite (space-to-batch, dense conv, batch-to-space) equals the dilated conv exactly
    x, w = gc.small_ints((1, 4, 16, 16), 61), gc.small_ints((6, 4, 3, 3), 62)
    yd, _ = pr.dilated_rewrite_u32(x, w)
    out["dilated_rewrite"] = yd
    out["dilated_direct"] = pr.conv2d_u32(x, w, pad=(2, 2), dil=(2, 2))
    # N2H on the shape of the reference's committed fixture (src/Test/dat/transpose_test): digest of the
    # reference's text format ("%u " per element, newline every 32) for a seeded digit tensor
    dig = gc.digits((16, 16, 32, 32), 71)
    y = pr.transpose(dig, 0, [0, 1, [-1, 2], 3], 2)
    out["n2h_digits_sha256"] = np.frombuffer(hashlib.sha256(gc.tpm_text(y)).digest(), np.uint8)
    np.savez_compressed(os.path.join(HERE, "ref_vectors.npz"), **out)
    print("wrote", len(out), "arrays,", os.path.getsize(os.path.join(HERE, "ref_vectors.npz")), "bytes")


if __name__ == "__main__":
    main()
