"""TEST INFRASTRUCTURE ONLY — numpy front-end of the CPU restatement in pet_oracle.c.

Only tests/, the smoke check and bench.py's cpu_baseline leg may import this module; the product never does.
Each wrapper names the reference operator it restates (paths inside the reference project).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

ACT = {"none": 0, "relu": 1, "sigmoid": 2, "tanh": 3, "gelu": 4}


def build():
    """Compile pet_oracle.c into libpet_oracle.so (gcc, a second or two)."""
    subprocess.run(["make", "-C", _HERE, "oracle"], check=True, stdout=subprocess.DEVNULL)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libpet_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = C.CDLL(path)
        _LIB.oracle_transpose_u32.restype = C.c_int
        _LIB.oracle_conv_out.restype = C.c_int
        _LIB.oracle_convtrans_out.restype = C.c_int
        _LIB.oracle_num_threads.restype = C.c_int
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _ia(v):
    return (C.c_int * len(v))(*[int(x) for x in v])


def _u32(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype != np.uint32 else a


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def conv_out(size, k, pad, stride, dil):
    return lib().oracle_conv_out(size, k, pad, stride, dil)


def conv2d(x, w, bias=None, pad=(0, 0), stride=(1, 1), dil=(1, 1), act="none", wide=True, rows=None):
    """ConvOp::compute (src/Graph/operator.cc:94-158) in float; wide=True accumulates in double."""
    x, w, bias = _f32(x), _f32(w), _f32(bias)
    n, c, h, ww = x.shape
    f, cpg, r, s = w.shape
    oh = conv_out(h, r, pad[0], stride[0], dil[0])
    ow = conv_out(ww, s, pad[1], stride[1], dil[1])
    y = np.zeros((n, f, oh, ow), np.float32)
    r0, r1 = (0, oh) if rows is None else rows
    lib().oracle_conv2d_rows_f32(_p(x), _p(w), _p(bias), _p(y), n, c, h, ww, f, cpg, r, s, pad[0], pad[1],
                                 stride[0], stride[1], dil[0], dil[1], ACT[act], int(wide), r0, r1)
    return y


def conv2d_u32(x, w, pad=(0, 0), stride=(1, 1), dil=(1, 1)):
    """ConvOp::compute on the reference's own value type (uint32, wrap-around)."""
    x, w = _u32(x), _u32(w)
    n, c, h, ww = x.shape
    f, cpg, r, s = w.shape
    oh = conv_out(h, r, pad[0], stride[0], dil[0])
    ow = conv_out(ww, s, pad[1], stride[1], dil[1])
    y = np.zeros((n, f, oh, ow), np.uint32)
    lib().oracle_conv2d_u32(_p(x), _p(w), _p(y), n, c, h, ww, f, cpg, r, s, pad[0], pad[1], stride[0], stride[1],
                            dil[0], dil[1])
    return y


def conv3d(x, w, bias=None, pad=(0, 0, 0), stride=(1, 1, 1), dil=(1, 1, 1), act="none", wide=True):
    x, w, bias = _f32(x), _f32(w), _f32(bias)
    n, c, d, h, ww = x.shape
    f, cpg, t, r, s = w.shape
    od = conv_out(d, t, pad[0], stride[0], dil[0])
    oh = conv_out(h, r, pad[1], stride[1], dil[1])
    ow = conv_out(ww, s, pad[2], stride[2], dil[2])
    y = np.zeros((n, f, od, oh, ow), np.float32)
    lib().oracle_conv3d_f32(_p(x), _p(w), _p(bias), _p(y), n, c, d, h, ww, f, cpg, t, r, s, *pad, *stride, *dil,
                            ACT[act], int(wide))
    return y


def matmul(a, b, bias=None, transA=False, transB=False, act="none", wide=True):
    """MatmulOp::compute (src/Graph/operator.cc:620-654) in float."""
    a, b, bias = _f32(a), _f32(b), _f32(bias)
    bs = a.shape[0]
    m, k = (a.shape[2], a.shape[1]) if transA else (a.shape[1], a.shape[2])
    n = b.shape[1] if transB else b.shape[2]
    c = np.zeros((bs, m, n), np.float32)
    lib().oracle_matmul_f32(_p(a), _p(b), _p(bias), _p(c), bs, m, n, k, int(transA), int(transB), ACT[act],
                            int(wide))
    return c


def matmul_u32(a, b, transA=False, transB=False):
    a, b = _u32(a), _u32(b)
    bs = a.shape[0]
    m, k = (a.shape[2], a.shape[1]) if transA else (a.shape[1], a.shape[2])
    n = b.shape[1] if transB else b.shape[2]
    c = np.zeros((bs, m, n), np.uint32)
    lib().oracle_matmul_u32(_p(a), _p(b), _p(c), bs, m, n, k, int(transA), int(transB))
    return c


def perm_spec(after):
    """after = list whose items are ints or lists of ints (TransposeOp's Perm, include/operator.h:1032-1098)."""
    groups = [list(g) if isinstance(g, (list, tuple)) else [g] for g in after]
    return [len(g) for g in groups], [i for g in groups for i in g]


def transpose(x, split, after, factor=2):
    """TransposeOp::compute (src/Graph/operator.cc:2172-2210); bit-exact on 32-bit words."""
    xin = _u32(x)
    sizes, flat = perm_spec(after)
    od = (C.c_int * 16)()
    nd = lib().oracle_transpose_u32(None, xin.ndim, _ia(xin.shape), split, len(sizes), _ia(sizes), _ia(flat),
                                    factor, None, od)
    if nd < 0:
        raise ValueError("split does not divide the dimension")
    out = np.empty([od[i] for i in range(nd)], np.uint32)
    lib().oracle_transpose_u32(_p(xin), xin.ndim, _ia(xin.shape), split, len(sizes), _ia(sizes), _ia(flat), factor,
                               _p(out), od)
    return out.view(x.dtype) if x.dtype.itemsize == 4 else out


def transpose_halo(x, split, after, factor, mode, amount):
    """A TransposeOp whose split or merge carries one of the reference's padding / halo parameters
    (TransposeOp::getTTParam, src/Graph/operator.cc:2403-2441; TransSplit / TransFuse::putTranspose,
    src/Transpose/transpose.cc:22-42,70-106).  With `n` the inner extent of the split or merged pair:
      extr   split   out[a][b] = in[a*(n+extr) + b]
      copys  split   out[a][b] = in[a*n + b - a*copys], b < n + copys   (dim == 2n)
      pad    merge   out[i] = in[i // (n+pad)][i % (n+pad)] if i % (n+pad) < n else 0, extent A*(n+pad) - pad
      dels   merge   out[i] = in[i // (n-dels)][i % (n-dels) + (i // (n-dels)) * dels]   (A == 2)
    Word-exact (numpy indexing only)."""
    x = np.ascontiguousarray(x)
    groups = [list(g) if isinstance(g, (list, tuple)) else [g] for g in after]
    extr = amount if mode == "extr" else 0
    copys = amount if mode == "copys" else 0
    pad_ = amount if mode == "pad" else 0
    dels = amount if mode == "dels" else 0
    t = x
    if split >= 0:
        d = x.shape[split]
        n = factor if factor > 0 else d // (-factor)
        if copys:
            assert d == 2 * n
            idx = np.array([[a * n + b - a * copys for b in range(n + copys)] for a in range(2)])
        else:
            parts = (d - 1) // (n + extr) + 1 if extr else d // n
            idx = np.array([[a * (n + extr) + b for b in range(n)] for a in range(parts)])
        t = np.take(x, idx.reshape(-1), axis=split)
        t = t.reshape(x.shape[:split] + idx.shape + x.shape[split + 1:])

    def item(i):  # constructor numbering -> axis after the split (include/operator.h:1133-1143)
        if split < 0:
            return i
        return split + 1 if i == -1 else (i + 1 if i > split else i)

    order = [item(i) for g in groups for i in g]
    t = np.transpose(t, order)
    out_shape, pos, merged_axis = [], 0, None
    for gi, g in enumerate(groups):
        if len(g) > 1 and (pad_ or dels):
            assert len(g) == 2
            merged_axis = gi
            out_shape += [t.shape[pos], t.shape[pos + 1]]
        else:
            out_shape.append(int(np.prod(t.shape[pos:pos + len(g)])))
        pos += len(g)
    t = np.ascontiguousarray(t).reshape(out_shape)
    if merged_axis is None:
        return t
    a_ext, n = t.shape[merged_axis], t.shape[merged_axis + 1]
    lead = t.shape[:merged_axis]
    tail = t.shape[merged_axis + 2:]
    if pad_:
        out = np.zeros(lead + (a_ext * (n + pad_) - pad_,) + tail, x.dtype)
        for a in range(a_ext):
            sl = [slice(None)] * merged_axis
            out[tuple(sl + [slice(a * (n + pad_), a * (n + pad_) + n)])] = t[tuple(sl + [a])]
        return out
    assert a_ext == 2 and dels < n
    sl = [slice(None)] * merged_axis
    return np.concatenate([t[tuple(sl + [0, slice(0, n - dels)])], t[tuple(sl + [1, slice(dels, n)])]], axis=merged_axis)


def pad(x, begin, end):
    """PadOp::compute (src/Graph/operator.cc:1640-1662)."""
    xin = _u32(x)
    out = np.empty([d + b + e for d, b, e in zip(xin.shape, begin, end)], np.uint32)
    lib().oracle_pad_u32(_p(xin), xin.ndim, _ia(xin.shape), _ia(begin), _ia(end), _p(out))
    return out.view(x.dtype)


def slice_(x, begin, end):
    """SliceOp::compute (src/Graph/operator.cc:1741-1773)."""
    xin = _u32(x)
    out = np.empty([d - b - e for d, b, e in zip(xin.shape, begin, end)], np.uint32)
    lib().oracle_slice_u32(_p(xin), xin.ndim, _ia(xin.shape), _ia(begin), _ia(end), _p(out))
    return out.view(x.dtype)


def extend(x, dim, num):
    """ExtendOp::compute (src/Graph/operator.cc:2577-2597)."""
    xin = _u32(x)
    shp = list(xin.shape)
    shp[dim] *= num + 1
    out = np.empty(shp, np.uint32)
    lib().oracle_extend_u32(_p(xin), xin.ndim, _ia(xin.shape), dim, num, _p(out))
    return out.view(x.dtype)


def concat(xs, dim):
    """ConcatOp::compute (src/Graph/operator.cc:1813-1850)."""
    ins = [_u32(x) for x in xs]
    shp = list(ins[0].shape)
    shp[dim] = sum(a.shape[dim] for a in ins)
    out = np.empty(shp, np.uint32)
    outer = int(np.prod(shp[:dim], dtype=np.int64))
    inner = int(np.prod(shp[dim + 1:], dtype=np.int64))
    off = 0
    for a in ins:
        lib().oracle_axis_block_u32(_p(a), _p(out), C.c_size_t(outer), C.c_size_t(inner), a.shape[dim], shp[dim],
                                    off, 1)
        off += a.shape[dim]
    return out.view(xs[0].dtype)


def split(x, dim, sizes):
    """SplitOp::computeV with ratio sizes (src/Graph/operator.cc:1978-2020, shapes :2074-2101)."""
    xin = _u32(x)
    total = sum(sizes)
    if xin.shape[dim] % total:
        raise ValueError("ratios do not divide the dimension")
    unit = xin.shape[dim] // total
    outer = int(np.prod(xin.shape[:dim], dtype=np.int64))
    inner = int(np.prod(xin.shape[dim + 1:], dtype=np.int64))
    outs, off = [], 0
    for s in sizes:
        shp = list(xin.shape)
        shp[dim] = unit * s
        o = np.empty(shp, np.uint32)
        lib().oracle_axis_block_u32(_p(xin), _p(o), C.c_size_t(outer), C.c_size_t(inner), shp[dim], xin.shape[dim],
                                    off, 0)
        off += shp[dim]
        outs.append(o.view(x.dtype))
    return outs


def eltwise(kind, xs, out_shape=None):
    """AddOp/SubOp/MulOp with the reference's `i % size` operand indexing (src/Graph/operator.cc:2983-3002)."""
    k = {"add": 0, "sub": 1, "mul": 2}[kind]
    u32 = xs[0].dtype == np.uint32
    ins = [(_u32(x) if u32 else _f32(x)) for x in xs]
    out_shape = out_shape or ins[0].shape
    out = np.empty(out_shape, np.uint32 if u32 else np.float32)
    ptrs = (C.c_void_p * len(ins))(*[a.ctypes.data for a in ins])
    sizes = (C.c_size_t * len(ins))(*[a.size for a in ins])
    fn = lib().oracle_eltwise_u32 if u32 else lib().oracle_eltwise_f32
    fn(k, len(ins), ptrs, sizes, _p(out), C.c_size_t(out.size))
    return out


def batchnorm(x, scale, bias, mean, var, eps=1e-5):
    """BatchNormOp::compute (src/Graph/operator.cc:2660-2681)."""
    x = _f32(x)
    y = np.empty_like(x)
    inner = int(np.prod(x.shape[2:], dtype=np.int64))
    lib().oracle_batchnorm_f32(_p(x), _p(_f32(scale)), _p(_f32(bias)), _p(_f32(mean)), _p(_f32(var)), _p(y),
                               C.c_size_t(x.shape[0]), x.shape[1], C.c_size_t(inner), C.c_float(eps))
    return y


def activation(x, act):
    x = _f32(x)
    y = np.empty_like(x)
    lib().oracle_activation_f32(_p(x), _p(y), C.c_size_t(x.size), ACT[act])
    return y


def _pool(fn, x, k, pad, stride):
    x = _f32(x)
    n, c, h, w = x.shape
    oh = (h - (k[0] - stride[0]) + 2 * pad[0]) // stride[0]
    ow = (w - (k[1] - stride[1]) + 2 * pad[1]) // stride[1]
    y = np.empty((n, c, oh, ow), np.float32)
    fn(_p(x), _p(y), n, c, h, w, k[0], k[1], pad[0], pad[1], stride[0], stride[1])
    return y


def maxpool(x, k, pad, stride):
    """cuDNN MAX pooling as the reference configures it (src/Graph/code_engine.cc:1281-1311)."""
    return _pool(lib().oracle_maxpool_f32, x, k, pad, stride)


def avgpool(x, k, pad, stride):
    """cuDNN AVERAGE_COUNT_EXCLUDE_PADDING pooling (src/Graph/code_engine.cc:1281-1311)."""
    return _pool(lib().oracle_avgpool_f32, x, k, pad, stride)


def softmax(x, axis=-1):
    """Softmax as the reference's online_softmax kernel defines it for the last axis (src/Graph/code_engine.cc:424-486);
    any other axis is the same computation on the tensor with that axis moved last (SoftmaxOp carries an axis,
    include/operator.h:1887-1938)."""
    x = _f32(x)
    axis = axis + x.ndim if axis < 0 else axis
    if axis != x.ndim - 1:
        return np.ascontiguousarray(np.moveaxis(softmax(np.ascontiguousarray(np.moveaxis(x, axis, -1))), -1, axis))
    y = np.empty_like(x)
    lib().oracle_softmax_f32(_p(x), _p(y), C.c_size_t(x.size // x.shape[-1]), x.shape[-1])
    return y


def layernorm(x, gamma, beta, eps=1e-5):
    x = _f32(x)
    y = np.empty_like(x)
    lib().oracle_layernorm_f32(_p(x), _p(_f32(gamma)), _p(_f32(beta)), _p(y), C.c_size_t(x.size // x.shape[-1]),
                               x.shape[-1], C.c_float(eps))
    return y


def convtrans_out(size, k, pad, stride, dil, out_pad):
    return lib().oracle_convtrans_out(size, k, pad, stride, dil, out_pad)


def _convtrans_shapes(x, w, pad, stride, dil, out_pad):
    n, h, ww, f = x.shape
    r, s, f2, c = w.shape
    assert f == f2, (x.shape, w.shape)
    oh = (h - 1) * stride[0] - 2 * pad[0] + dil[0] * (r - 1) + out_pad[0] + 1
    ow = (ww - 1) * stride[1] - 2 * pad[1] + dil[1] * (s - 1) + out_pad[1] + 1
    return n, h, ww, f, r, s, c, oh, ow


def convtrans(x, w, pad=(0, 0), stride=(1, 1), dil=(1, 1), out_pad=(0, 0), wide=True):
    """ConvTransOp in float: x [n,h,w,f], w [r,s,f,c] -> [n,oh,ow,c]."""
    x, w = _f32(x), _f32(w)
    n, h, ww, f, r, s, c, oh, ow = _convtrans_shapes(x, w, pad, stride, dil, out_pad)
    y = np.zeros((n, oh, ow, c), np.float32)
    lib().oracle_convtrans_f32(_p(x), _p(w), _p(y), n, h, ww, f, r, s, c, pad[0], pad[1], stride[0], stride[1], dil[0],
                               dil[1], out_pad[0], out_pad[1], int(wide))
    return y


def convtrans_u32(x, w, pad=(0, 0), stride=(1, 1), dil=(1, 1), out_pad=(0, 0)):
    """ConvTransOp on the reference's own value type (uint32, wrap-around)."""
    x, w = _u32(x), _u32(w)
    n, h, ww, f, r, s, c, oh, ow = _convtrans_shapes(x, w, pad, stride, dil, out_pad)
    y = np.zeros((n, oh, ow, c), np.uint32)
    lib().oracle_convtrans_u32(_p(x), _p(w), _p(y), n, h, ww, f, r, s, c, pad[0], pad[1], stride[0], stride[1], dil[0],
                               dil[1], out_pad[0], out_pad[1])
    return y


def g2bmm(q, k, width, dilation=1, wide=True):
    """Banded Q.K^T: q, k [b,n,m] -> [b,n,2*width+1]."""
    q, k = _f32(q), _f32(k)
    b, n, m = q.shape
    y = np.zeros((b, n, 2 * width + 1), np.float32)
    lib().oracle_g2bmm_f32(_p(q), _p(k), _p(y), b, n, m, width, dilation, int(wide))
    return y


def gbmml(p, v, dilation=1, wide=True):
    """Banded P.V: p [b,n,2w+1], v [b,n,m] -> [b,n,m]."""
    p, v = _f32(p), _f32(v)
    b, n, bw = p.shape
    m = v.shape[2]
    y = np.zeros((b, n, m), np.float32)
    lib().oracle_gbmml_f32(_p(p), _p(v), _p(y), b, n, m, (bw - 1) // 2, dilation, int(wide))
    return y


def div(a, b):
    """DivOp as a division with the element-wise operators' modulo broadcast (operand j read at i % size_j,
    src/Graph/operator.cc:2996-2998).  The reference's own host body subtracts (operator.cc:3258-3259)."""
    a, b = _f32(a), _f32(b)
    i = np.arange(a.size)
    return (a.reshape(-1)[i % a.size] / b.reshape(-1)[i % b.size]).reshape(a.shape)


def pow_(x, p):
    """PowOp::compute: repeated multiplication starting from 1 (powVType, include/common.h:157-162)."""
    x = _f32(x)
    r = np.ones_like(x)
    for _ in range(abs(int(p))):
        r = r * x
    return (np.float32(1) / r) if p < 0 else r


def reduce_mean(x, axis):
    """ReduceMeanOp: the axis stays with extent 1 (src/Graph/operator.cc:3454-3458)."""
    return _f32(x).astype(np.float64).mean(axis, keepdims=True).astype(np.float32)


def gather(data, indices, axis):
    """GatherOp: output dims = indices dims + data dims without the axis (src/Graph/operator.cc:3420-3428; index
    expression src/Graph/code_engine.cc:1465-1487)."""
    t = np.take(np.ascontiguousarray(data), np.asarray(indices), axis=axis)
    k = np.asarray(indices).ndim
    return np.ascontiguousarray(np.moveaxis(t, list(range(axis, axis + k)), list(range(k))))


def rel_err(a, b):
    """The parity metric for floating-point operators: max |a-b| / max(|b|, 1e-3*max|b|)."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    floor = 1e-3 * max(float(np.max(np.abs(b))), 1e-30)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), floor)))
