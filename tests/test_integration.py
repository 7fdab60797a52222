"""The reference-side binding (integration/): the reference's own host code — graph API, mutation generator, SearchEngine —
compiled where it lies and linked against libpetb200, with every Operator::perf answered by the backend and the chosen
graph executed through it.

CPU: the library links and the virtual perf() calls of the reference's operator classes land in the binding's bodies.
GPU: the reference's unchanged SearchEngine::run optimises the single-convolution graphs of its own rule tests on measured
costs, the graph it chooses runs on the GPU and equals the oracle; the H->N mutant built with the reference's Graph API
runs on the GPU and equals the reference's own host evaluation of the same graph."""
import ctypes as C
import math
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "integration", "_build", "libpet_on_petb200.so")
REF_DIR = os.environ.get("PET_REFERENCE_DIR", os.path.join(ROOT, "..", "reference"))  # a checkout beside this repository


def load():
    """Builds the library when the reference checkout and its objects are here; otherwise uses the prebuilt one."""
    if os.path.exists(os.path.join(REF_DIR, "src", "Graph", "operator.cc")) and os.path.isdir(os.path.join(ROOT, "oracle", "_ref", "obj")):
        from pet_b200 import build
        build.build()
        subprocess.run(["make", "-C", os.path.join(ROOT, "integration"), f"REF={REF_DIR}"], check=True, stdout=subprocess.DEVNULL)
    if not os.path.exists(LIB):
        pytest.skip("integration/_build/libpet_on_petb200.so not built (needs the reference checkout)")
    return C.CDLL(LIB)


def test_perf_calls_of_the_reference_classes_resolve_to_the_binding():
    lib = load()
    out = (C.c_double * 4)()
    assert lib.petb200_pet_perf_probe(out) == 4   # ConvOp, MatmulOp, TransposeOp, MaxPoolOp: all four landed in the binding
    import torch
    if not torch.cuda.is_available():
        assert all(math.isinf(v) for v in out)    # no device: "unsupported", as the reference reports a failed library call
    else:
        assert all(0 < v < 5 for v in out)


def _search(lib, conv):
    n, c, h, w, f, r, s, ph, pw, dh, dw = conv
    rng = np.random.default_rng(sum(conv))
    x = rng.integers(-4, 5, (n, c, h, w)).astype(np.float32)   # small integers: every sum is exact in fp32
    wt = rng.integers(-3, 4, (f, c, r, s)).astype(np.float32)
    oh, ow = h - (r - 1) * dh + 2 * ph, w - (s - 1) * dw + 2 * pw
    y, yd = np.zeros((n, f, oh, ow), np.float32), np.zeros((n, f, oh, ow), np.float32)
    rep = C.create_string_buffer(1 << 16)
    perf = (C.c_double * 2)()
    rc = lib.petb200_pet_search_conv((C.c_int * 11)(*conv), x.ctypes.data_as(C.c_void_p), wt.ctypes.data_as(C.c_void_p),
                                     y.ctypes.data_as(C.c_void_p), yd.ctypes.data_as(C.c_void_p), rep, len(rep), perf)
    return rc, x, wt, y, yd, rep.value.decode(), list(perf)


@pytest.mark.gpu
@pytest.mark.parametrize("conv", [(1, 64, 56, 56, 64, 3, 3, 1, 1, 1, 1),      # config 1 (ref: src/Test/single_rule_test_1_n2h.cc)
                                  (1, 64, 32, 32, 64, 3, 3, 2, 2, 2, 2)],     # a dilated conv (ref: src/Test/single_op_test_5.cc)
                         ids=["c1_conv3x3", "dilated_d2"])
def test_search_engine_runs_on_backend_costs_and_its_choice_executes(oracle, conv):
    lib = load()
    before = lib.petb200_shim_perf_calls()
    rc, x, wt, y, yd, report, perf = _search(lib, conv)
    assert rc == 0, report
    assert lib.petb200_shim_perf_calls() - before >= 3     # the search costed its candidates through the binding
    assert 0 < perf[1] <= perf[0] < 1                       # measured milliseconds; the chosen graph is no slower than the original
    print("\n[search] original %.4f ms, chosen %.4f ms:\n%s" % (perf[0], perf[1], report))
    want = oracle.conv2d(x, wt, pad=(conv[7], conv[8]), dil=(conv[9], conv[10]), wide=True)
    assert np.array_equal(yd, want)                          # the original operator through the walker
    # The chosen graph: equal to the original operator, except — if the search picked a partially equivalent mutant — on
    # the rows next to the seam the mutant introduces (the reference accepts those and only costs their correction).
    rows = np.unique(np.nonzero(y != want)[2])
    assert len(rows) <= 2 * (conv[5] - 1) * conv[9], rows


@pytest.mark.gpu
def test_h2n_mutant_on_gpu_equals_the_reference_host_evaluation():
    lib = load()
    conv = (1, 32, 28, 28, 48, 3, 3, 1, 1, 1, 1)
    n, c, h, w, f, r, s = conv[:7]
    rng = np.random.default_rng(5)
    x = rng.integers(-4, 5, (n, c, h, w)).astype(np.float32)
    wt = rng.integers(-3, 4, (f, c, r, s)).astype(np.float32)
    yg, yh = np.zeros((n, f, h, w), np.float32), np.zeros((n, f, h, w), np.uint32)
    rep = C.create_string_buffer(1 << 14)
    rc = lib.petb200_pet_run_h2n_rewrite((C.c_int * 11)(*conv), x.ctypes.data_as(C.c_void_p), wt.ctypes.data_as(C.c_void_p),
                                         yg.ctypes.data_as(C.c_void_p), yh.ctypes.data_as(C.c_void_p), rep, len(rep))
    assert rc == 0, rep.value.decode()
    assert rep.value.decode().count("Transpose") == 2 and "Conv" in rep.value.decode()
    assert np.array_equal(yg.astype(np.int64) % (1 << 32), yh.astype(np.int64))   # bit for bit what the reference computes
