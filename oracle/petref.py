"""TEST INFRASTRUCTURE ONLY — ctypes front-end of oracle/_ref/libpetref.so, i.e. the reference's own host
operators (tpm::Graph / Operator::compute) compiled from the reference sources by oracle/Makefile.

Used to pin the restatement in pet_oracle.c, to generate tests/golden/, and as the `reference` CPU arm of
bench.py.  `available()` is False when the library was never built (no reference checkout at build time).
"""
import ctypes as C
import os

import numpy as np

from .pet_oracle import perm_spec

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "_ref", "libpetref.so")
_LIB = None


def available():
    return os.path.exists(_PATH)


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(_PATH)
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _ia(v):
    return (C.c_int * len(v))(*[int(x) for x in v])


def _u32(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype != np.uint32 else a


def num_threads():
    return lib().petref_num_threads()


def _ok(rc, what):
    if rc != 0:
        raise RuntimeError(f"reference rejected {what} (rc={rc})")


def transpose(x, split, after, factor=2):
    xin = _u32(x)
    sizes, flat = perm_spec(after)
    nd = C.c_int()
    od = (C.c_int * 16)()
    out = np.empty(xin.size, np.uint32)
    _ok(lib().petref_transpose(_p(xin), xin.ndim, _ia(xin.shape), split, len(sizes), _ia(sizes), _ia(flat), factor,
                               _p(out), C.byref(nd), od), "transpose")
    return out.reshape([od[i] for i in range(nd.value)]).view(x.dtype)


_TT = {"N2H": 1, "N2W": 2, "H2N": 3, "W2N": 4, "D2H": 7, "D2W": 8}
# which (type, position) makes TransposeOp::getTTParam hand out each parameter (src/Graph/operator.cc:2406-2438)
HALO_MODES = {"pad": ("N2H", 1), "extr": ("N2H", 2), "copys": ("H2N", 1), "dels": ("H2N", 2)}


def transpose_lambda(shape, split, after, factor, mode, amount):
    """(lambda source, output dims) the reference generates for a TransposeOp carrying `amount` of pad/extr/copys/dels."""
    sizes, flat = perm_spec(after)
    ttype, pos = HALO_MODES[mode]
    buf = C.create_string_buffer(4096)
    nd = C.c_int()
    od = (C.c_int * 16)()
    _ok(lib().petref_transpose_lambda(len(shape), _ia(shape), split, len(sizes), _ia(sizes), _ia(flat), factor, _TT[ttype],
                                      pos, amount, amount, buf, 4096, C.byref(nd), od), "transpose lambda")
    return buf.value.decode(), tuple(od[i] for i in range(nd.value))


class _Lenient:
    """I[0][a,b,...] of the generated lambda: reads outside the tensor give 0 (TVM evaluates only the taken branch)."""

    def __init__(self, a):
        self.a = a

    def __getitem__(self, idx):
        if any(i < 0 or i >= n for i, n in zip(idx, self.a.shape)):
            return 0
        return self.a[idx]


class _Tir:
    @staticmethod
    def if_then_else(c, x, y):
        return x if c else y

    @staticmethod
    def const(v, t):
        return 0


class _Tvm:
    tir = _Tir


def transpose_halo(x, split, after, factor, mode, amount):
    """Evaluates the reference's own generated index expression at every output position (small tensors only)."""
    src, od = transpose_lambda(x.shape, split, after, factor, mode, amount)
    fn = eval(src, {"tvm": _Tvm, "I": [_Lenient(np.ascontiguousarray(x))]})
    out = np.zeros(od, x.dtype)
    for idx in np.ndindex(*od):
        out[idx] = fn(*idx)
    return out


def conv2d_u32(x, w, pad=(0, 0), stride=(1, 1), dil=(1, 1), return_secs=False):
    x, w = _u32(x), _u32(w)
    n, c, h, ww = x.shape
    f, cpg, r, s = w.shape
    oh = (h - (r - stride[0]) * dil[0] + 2 * pad[0]) // stride[0]
    ow = (ww - (s - stride[1]) * dil[1] + 2 * pad[1]) // stride[1]
    y = np.empty((n, f, oh, ow), np.uint32)
    yd = (C.c_int * 4)()
    secs = C.c_double()
    _ok(lib().petref_conv(_p(x), _ia(x.shape), _p(w), _ia(w.shape), pad[0], pad[1], stride[0], stride[1], dil[0],
                          dil[1], _p(y), yd, C.byref(secs)), "conv")
    assert tuple(yd) == y.shape, (tuple(yd), y.shape)
    return (y, secs.value) if return_secs else y


def convtrans_u32(x, w, pad=(0, 0), stride=(1, 1), dil=(1, 1), out_pad=(0, 0), whole=False):
    """ConvTransOp of the reference: whole=True runs its whole-tensor body (only complete when oh == ow == c),
    whole=False its one-position body at every output position."""
    x, w = _u32(x), _u32(w)
    n, h, ww, f = x.shape
    r, s, _, c = w.shape
    oh = (h - 1) * stride[0] - 2 * pad[0] + dil[0] * (r - 1) + out_pad[0] + 1
    ow = (ww - 1) * stride[1] - 2 * pad[1] + dil[1] * (s - 1) + out_pad[1] + 1
    y = np.empty((n, oh, ow, c), np.uint32)
    yd = (C.c_int * 4)()
    _ok(lib().petref_convtrans(_p(x), _ia(x.shape), _p(w), _ia(w.shape), pad[0], pad[1], stride[0], stride[1], dil[0],
                               dil[1], out_pad[0], out_pad[1], int(whole), _p(y), yd), "convtrans")
    assert tuple(yd) == y.shape, (tuple(yd), y.shape)
    return y


def matmul_u32(a, b, transA=False, transB=False):
    a, b = _u32(a), _u32(b)
    bs = a.shape[0]
    m = a.shape[2] if transA else a.shape[1]
    n = b.shape[1] if transB else b.shape[2]
    c = np.empty((bs, m, n), np.uint32)
    cd = (C.c_int * 3)()
    _ok(lib().petref_matmul(_p(a), _ia(a.shape), _p(b), _ia(b.shape), int(transA), int(transB), _p(c), cd, None),
        "matmul")
    assert tuple(cd) == c.shape
    return c


def pad(x, begin, end):
    xin = _u32(x)
    out = np.empty([d + b + e for d, b, e in zip(xin.shape, begin, end)], np.uint32)
    od = (C.c_int * 16)()
    _ok(lib().petref_pad(_p(xin), xin.ndim, _ia(xin.shape), _ia(begin), _ia(end), _p(out), od), "pad")
    return out.view(x.dtype)


def slice_(x, begin, end):
    xin = _u32(x)
    out = np.empty([d - b - e for d, b, e in zip(xin.shape, begin, end)], np.uint32)
    od = (C.c_int * 16)()
    _ok(lib().petref_slice(_p(xin), xin.ndim, _ia(xin.shape), _ia(begin), _ia(end), _p(out), od), "slice")
    return out.view(x.dtype)


def extend(x, dim, num):
    xin = _u32(x)
    shp = list(xin.shape)
    shp[dim] *= num + 1
    out = np.empty(shp, np.uint32)
    od = (C.c_int * 16)()
    _ok(lib().petref_extend(_p(xin), xin.ndim, _ia(xin.shape), dim, num, _p(out), od), "extend")
    return out.view(x.dtype)


def concat(xs, dim):
    ins = [_u32(x) for x in xs]
    nd = ins[0].ndim
    shp = list(ins[0].shape)
    shp[dim] = sum(a.shape[dim] for a in ins)
    out = np.empty(shp, np.uint32)
    ptrs = (C.c_void_p * len(ins))(*[a.ctypes.data for a in ins])
    dims = _ia([d for a in ins for d in a.shape])
    od = (C.c_int * 16)()
    _ok(lib().petref_concat(len(ins), ptrs, nd, dims, dim, _p(out), od), "concat")
    return out.view(xs[0].dtype)


def split(x, dim, sizes):
    xin = _u32(x)
    nd = xin.ndim
    od = (C.c_int * (nd * len(sizes)))()
    _ok(lib().petref_split(_p(xin), nd, _ia(xin.shape), dim, len(sizes), _ia(sizes), None, od), "split")
    outs = [np.empty([od[i * nd + j] for j in range(nd)], np.uint32) for i in range(len(sizes))]
    ptrs = (C.c_void_p * len(outs))(*[o.ctypes.data for o in outs])
    _ok(lib().petref_split(_p(xin), nd, _ia(xin.shape), dim, len(sizes), _ia(sizes), ptrs, od), "split")
    return [o.view(x.dtype) for o in outs]


def eltwise_u32(kind, xs):
    k = {"add": 0, "sub": 1, "mul": 2}[kind]
    ins = [_u32(x) for x in xs]
    out = np.empty(ins[0].shape, np.uint32)
    ptrs = (C.c_void_p * len(ins))(*[a.ctypes.data for a in ins])
    _ok(lib().petref_eltwise(k, len(ins), ptrs, _ia([a.ndim for a in ins]), _ia([d for a in ins for d in a.shape]),
                             _p(out)), kind)
    return out


def dilated_rewrite_u32(x, w):
    """space-to-batch -> dense 3x3 conv -> batch-to-space on the reference's host operators; returns (y, secs)."""
    x, w = _u32(x), _u32(w)
    n, c, h, ww = x.shape
    y = np.empty((n, w.shape[0], h, ww), np.uint32)
    yd = (C.c_int * 4)()
    secs = C.c_double()
    _ok(lib().petref_dilated_rewrite(_p(x), _ia(x.shape), _p(w), _ia(w.shape), _p(y), yd, C.byref(secs)),
        "dilated rewrite")
    assert tuple(yd) == y.shape, (tuple(yd), y.shape)
    return y, secs.value
