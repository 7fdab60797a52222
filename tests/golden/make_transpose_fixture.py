"""Packs the reference's committed transpose fixture (src/Test/dat/transpose_test/input.dat: 16*16*32*32 decimal digits,
the input of its transpose_test_1) into tests/golden/transpose_fixture_input.npz, so that the known answer it pins — the
SHA-256 of the output file the reference's own test writes — can be checked where the reference checkout is absent.

    python tests/golden/make_transpose_fixture.py <reference checkout>
"""
import os
import sys

import numpy as np

if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("PET_REFERENCE_DIR", "")
    src = os.path.join(ref, "src", "Test", "dat", "transpose_test", "input.dat")
    x = np.array(open(src).read().split(), dtype=np.uint8)
    assert x.size == 16 * 16 * 32 * 32 and x.max() <= 9
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "transpose_fixture_input.npz")
    np.savez_compressed(out, digits=x.reshape(16, 16, 32, 32))
    print(out, os.path.getsize(out), "bytes")
