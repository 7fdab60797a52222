"""Evaluates a configuration from pet_b200.configs with the CPU oracle: same builder methods, numpy arrays as tensors."""
import numpy as np

from oracle import pet_oracle as po


class OracleBuilder:
    def input(self, a):
        return np.asarray(a, np.float32)

    const = input

    def conv(self, x, w, ph, pw, sh=1, sw=1, dh=1, dw=1, bias=None, act="none"):
        return po.conv2d(x, w, bias, pad=(ph, pw), stride=(sh, sw), dil=(dh, dw), act=act, wide=True)

    def conv3d(self, x, w, pad, stride=(1, 1, 1), dil=(1, 1, 1), bias=None, act="none"):
        return po.conv3d(x, w, bias, pad=tuple(pad), stride=tuple(stride), dil=tuple(dil), act=act, wide=True)

    def matmul(self, a, b, transA=False, transB=False, bias=None, act="none"):
        a = a[None] if a.ndim == 2 else a
        b = b[None] if b.ndim == 2 else b
        return po.matmul(a, b, bias, transA, transB, act=act, wide=True)

    def transpose(self, x, split, after, factor=2):
        return po.transpose(x, split, after, factor)

    def transpose_halo(self, x, split, after, factor, mode, amount):
        return po.transpose_halo(x, split, after, factor, mode, amount)

    def pad(self, x, begin, end):
        return po.pad(x, begin, end)

    def slice(self, x, begin, end):
        return po.slice_(x, begin, end)

    def extend(self, x, dim, num):
        return po.extend(x, dim, num)

    def concat(self, xs, dim):
        return po.concat(xs, dim)

    def split(self, x, dim, sizes):
        return po.split(x, dim, [1] * sizes if isinstance(sizes, int) else sizes)

    def add(self, xs):
        return po.eltwise("add", xs)

    def sub(self, a, b):
        return po.eltwise("sub", [a, b])

    def mul(self, xs):
        return po.eltwise("mul", xs)

    def relu(self, x):
        return po.activation(x, "relu")

    def sigmoid(self, x):
        return po.activation(x, "sigmoid")

    def tanh(self, x):
        return po.activation(x, "tanh")

    def gelu(self, x):
        return po.activation(x, "gelu")

    def maxpool(self, x, kh, kw, dh, dw, ph, pw, sh, sw):
        return po.maxpool(x, (kh, kw), (ph, pw), (sh, sw))

    def avgpool(self, x, kh=None, kw=None, ph=0, pw=0, sh=1, sw=1):
        if kh is None:
            kh, kw = x.shape[2], x.shape[3]
        return po.avgpool(x, (kh, kw), (ph, pw), (sh, sw))

    def softmax(self, x, axis):
        return po.softmax(x, axis)

    def layernorm(self, x, gamma=None, beta=None, eps=1e-5):
        return po.layernorm(x, gamma, beta, eps)

    def batchnorm(self, x, scale, bias, mean, var, epsilon=1e-5, momentum=0.9):
        return po.batchnorm(x, scale, bias, mean, var, epsilon)

    def reshape(self, x, dims):
        return np.ascontiguousarray(x).reshape(dims)

    def identity(self, x):
        return x

    def correction(self, x, w, y, ph, pw, sh=1, sw=1, dh=1, dw=1, rows=None, cols=None, bias=None, act="none"):
        full = po.conv2d(x, w, bias, pad=(ph, pw), stride=(sh, sw), dil=(dh, dw), act=act, wide=True)
        r0, rn = rows if rows is not None else (0, y.shape[2])
        c0, cn = cols if cols is not None else (0, y.shape[3])
        out = y.copy()
        out[:, :, r0:r0 + rn, c0:c0 + cn] = full[:, :, r0:r0 + rn, c0:c0 + cn]
        return out
