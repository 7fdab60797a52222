"""GPU: the allocation-free matmul entry point, for callers that may not allocate device memory (no context, no plan;
its only scratch is a fixed array inside the library).  Checked through the C ABI against the plan-based entry point
and against the CPU oracle on two calls in a row — the second with other shapes and data, so anything left in the shared array by the first call
would show.  Collected last on purpose: a failure here leaves every other test already run."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import rel_err, scale_err

pytestmark = pytest.mark.gpu
TOL, TOL_SCALE = 1e-3, 5e-5   # the same bounds the other floating-point tests use


def call(lib, a, b, bias, transA, transB, bs, m, n, k, ksplit, act):
    c = torch.empty((bs, m, n), device="cuda", dtype=torch.float32)
    err = C.create_string_buffer(256)
    rc = lib.petb200_matmul_splitk_noalloc(int(transA), int(transB), bs, m, n, k, ksplit, C.c_void_p(a.data_ptr()),
                                           C.c_void_p(b.data_ptr()), C.c_void_p(bias.data_ptr()) if bias is not None else None,
                                           C.c_void_p(c.data_ptr()), act, C.c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
    return rc, err.value.decode(), c


def test_two_calls_in_a_row_match_the_plan_based_entry_point(ctx, oracle):
    from pet_b200 import lib as L
    lib = L.load()
    g = torch.Generator().manual_seed(77)
    cases = [  # (b, m, n, k, transA, transB, ksplit, act)
        (1, 128, 768, 3072, False, False, 16, "gelu"),   # 1.5 Mi partial sums: most of the fixed array
        (3, 37, 29, 101, True, True, 7, "none"),         # ragged, transposed operands, a smaller footprint
    ]
    for b, m, n, k, ta, tb, ks, act in cases:
        a = torch.randn((b, k, m) if ta else (b, m, k), generator=g).cuda()
        bm = (torch.randn((b, n, k) if tb else (b, k, n), generator=g) / k ** 0.5).cuda()
        bias = torch.randn(n, generator=g).cuda()
        rc, msg, got = call(lib, a, bm, bias, ta, tb, b, m, n, k, ks, L.ACT[act])
        assert rc == 0, msg
        want = ctx.matmul(a, bm, ta, tb, bias=bias, act=act)   # existing entry point (petb200_matmul_plan/run)
        torch.cuda.synchronize()
        assert rel_err(got.cpu().numpy(), want.cpu().numpy()) <= TOL
        assert scale_err(got.cpu().numpy(), want.cpu().numpy()) <= TOL_SCALE
        # and against the oracle: the sums themselves (no activation) under the contract metric, then the activation as a
        # function of those sums
        rc, msg, lin = call(lib, a, bm, bias, ta, tb, b, m, n, k, ks, L.ACT["none"])
        assert rc == 0, msg
        ref = oracle.matmul(a.cpu().numpy(), bm.cpu().numpy(), bias.cpu().numpy(), ta, tb, wide=True)
        assert rel_err(lin.cpu().numpy(), ref) <= TOL
        assert np.allclose(got.cpu().numpy(), oracle.activation(lin.cpu().numpy(), act), rtol=2e-6, atol=2e-7)


def test_sizes_beyond_the_fixed_array_are_rejected():
    from pet_b200 import lib as L
    lib = L.load()
    a = torch.zeros((1, 2048, 64), device="cuda")
    b = torch.zeros((1, 64, 2048), device="cuda")
    rc, msg, _ = call(lib, a, b, None, False, False, 1, 2048, 2048, 64, 1, 0)   # 4 Mi partial sums > 2 Mi
    assert rc == L.ERR_UNSUPPORTED and "exceed the fixed scratch" in msg
    rc, msg, _ = call(lib, a, b, None, False, False, 1, 2048, 2048, 64, 0, 0)
    assert rc == L.ERR_INVALID
