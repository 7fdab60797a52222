"""Operator-level host API over the C ABI.  torch is used for device memory and streams only.

Method names and argument meaning follow the reference's operators (include/operator.h in the reference project):
conv(ph,pw,sh,sw,dh,dw), matmul(transA,transB), transpose(split, after, factor), pad/slice(begin,end),
extend(dim,num), concat/split(dim), maxpool/avgpool(kh,kw,...,ph,pw,sh,sw), softmax, batchnorm.
Unsupported or invalid operators raise PetError carrying the C-ABI status.
"""
import ctypes as C

import numpy as np
import torch

from . import lib as L


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _f32(t):
    assert t.is_cuda and t.dtype == torch.float32, "device fp32 tensors only"
    return t.contiguous()


def perm_spec(after):
    groups = [list(g) if isinstance(g, (list, tuple)) else [g] for g in after]
    return [len(g) for g in groups], [i for g in groups for i in g]


class Plan:
    def __init__(self, ctx, handle):
        self.ctx, self.h = ctx, handle

    def __del__(self):
        if getattr(self, "h", None) and self.ctx.h:
            self.ctx.lib.petb200_plan_destroy(self.h)
            self.h = None

    @property
    def kernel(self):
        return self.ctx.lib.petb200_plan_kernel(self.h).decode()

    @property
    def device_bytes(self):
        return self.ctx.lib.petb200_plan_device_bytes(self.h)

    def time(self, rounds=200, warmup=200):
        """Milliseconds per launch on plan-owned operands (the perf_engine measurement)."""
        ms = C.c_float()
        self.ctx.check(self.ctx.lib.petb200_plan_time(self.h, rounds, warmup, C.byref(ms), _stream()))
        return ms.value


class Context:
    def __init__(self, device=0):
        self.lib = L.load()
        self.h = C.c_void_p()
        rc = self.lib.petb200_ctx_create(int(device), C.byref(self.h))
        if rc:
            raise L.PetError(rc, self.lib.petb200_last_error(None).decode())
        self.device = torch.device("cuda", int(device))
        self._plans = {}

    def close(self):
        if self.h:
            self._plans.clear()
            self.lib.petb200_ctx_destroy(self.h)
            self.h = None

    def check(self, rc):
        if rc:
            raise L.PetError(rc, self.lib.petb200_last_error(self.h).decode())

    def launches(self):
        return int(self.lib.petb200_launch_count(self.h))

    def sync_check(self):
        """Synchronise the current stream and raise if a kernel reported a device-side error."""
        self.check(self.lib.petb200_check_device_status(self.h, _stream()))

    # ---- convolution ---------------------------------------------------------------------------------------
    def conv2d_plan(self, xshape, wshape, ph, pw, sh=1, sw=1, dh=1, dw=1, bias=False, act="none", algo="auto"):
        n, c, h, w = xshape
        f, cpg, r, s = wshape
        if cpg <= 0 or c % cpg:
            raise L.PetError(L.ERR_INVALID, "input channels not divisible by filter channels")
        args = [n, c, h, w, f, r, s, ph, pw, sh, sw, dh, dw, c // cpg, int(bool(bias)), L.ACT[act]]
        h_ = C.c_void_p()
        self.check(self.lib.petb200_conv2d_plan(self.h, L.ints(args), L.ALGO[algo], C.byref(h_)))
        p = Plan(self, h_)
        od = (C.c_int * 4)()
        self.check(self.lib.petb200_conv2d_out_dims(h_, od))
        p.out_shape = tuple(od)
        return p

    def conv2d_set_weights(self, plan, w):
        plan._w = _f32(w)  # keep alive: the CUDA-core path reads the caller's tensor
        self.check(self.lib.petb200_conv2d_set_weights(plan.h, _ptr(plan._w), _stream()))

    def conv2d_run(self, plan, x, bias=None, out=None, residual=None):
        """y = act(conv(x) + bias [+ residual]); residual (shaped like y) folds a following Add into the epilogue."""
        x = _f32(x)
        y = out if out is not None else torch.empty(plan.out_shape, device=x.device, dtype=torch.float32)
        b = _ptr(_f32(bias) if bias is not None else None)
        if residual is not None:
            if tuple(residual.shape) != tuple(plan.out_shape):
                raise L.PetError(L.ERR_INVALID, "residual must have the shape of the output")
            self.check(self.lib.petb200_conv_run_residual(plan.h, _ptr(x), b, _ptr(_f32(residual)), _ptr(y), _stream()))
        else:
            self.check(self.lib.petb200_conv2d_run(plan.h, _ptr(x), b, _ptr(y), _stream()))
        return y

    def conv2d_correct(self, plan, x, y, oh0, ohn, ow0=0, own=None, bias=None):
        """Recompute rows [oh0,oh0+ohn) x cols [ow0,ow0+own) of y from the ORIGINAL input x."""
        own = plan.out_shape[3] - ow0 if own is None else own
        self.check(self.lib.petb200_conv2d_correct(plan.h, _ptr(_f32(x)), _ptr(bias), _ptr(y), oh0, ohn, ow0, own,
                                                   _stream()))
        return y

    def conv2d(self, x, w, ph, pw, sh=1, sw=1, dh=1, dw=1, bias=None, act="none", algo="auto", residual=None):
        key = ("conv2d", tuple(x.shape), tuple(w.shape), ph, pw, sh, sw, dh, dw, bias is not None, act, algo)
        plan = self._plans.get(key)
        if plan is None:
            plan = self._plans[key] = self.conv2d_plan(x.shape, w.shape, ph, pw, sh, sw, dh, dw, bias is not None, act, algo)
        self.conv2d_set_weights(plan, w)
        return self.conv2d_run(plan, x, bias, residual=residual)

    def conv3d_plan(self, xshape, wshape, pad, stride=(1, 1, 1), dil=(1, 1, 1), bias=False, act="none", algo="auto"):
        n, c, d, h, w = xshape
        f, cpg, t, r, s = wshape
        if cpg <= 0 or c % cpg:
            raise L.PetError(L.ERR_INVALID, "input channels not divisible by filter channels")
        args = [n, c, d, h, w, f, t, r, s, *pad, *stride, *dil, c // cpg, int(bool(bias)), L.ACT[act]]
        h_ = C.c_void_p()
        self.check(self.lib.petb200_conv3d_plan(self.h, L.ints(args), L.ALGO[algo], C.byref(h_)))
        p = Plan(self, h_)
        o = lambda i, k, pd, st, dl: (i - (k - st) * dl + 2 * pd) // st
        p.out_shape = (n, f, o(d, t, pad[0], stride[0], dil[0]), o(h, r, pad[1], stride[1], dil[1]),
                       o(w, s, pad[2], stride[2], dil[2]))
        return p

    def conv3d(self, x, w, pad, stride=(1, 1, 1), dil=(1, 1, 1), bias=None, act="none", algo="auto", residual=None):
        key = ("conv3d", tuple(x.shape), tuple(w.shape), tuple(pad), tuple(stride), tuple(dil), bias is not None, act, algo)
        plan = self._plans.get(key)
        if plan is None:
            plan = self._plans[key] = self.conv3d_plan(x.shape, w.shape, pad, stride, dil, bias is not None, act, algo)
        plan._w = _f32(w)
        self.check(self.lib.petb200_conv3d_set_weights(plan.h, _ptr(plan._w), _stream()))
        y = torch.empty(plan.out_shape, device=x.device, dtype=torch.float32)
        if residual is not None:
            self.check(self.lib.petb200_conv_run_residual(plan.h, _ptr(_f32(x)), _ptr(bias), _ptr(_f32(residual)), _ptr(y), _stream()))
        else:
            self.check(self.lib.petb200_conv3d_run(plan.h, _ptr(_f32(x)), _ptr(bias), _ptr(y), _stream()))
        return y

    # ---- transposed convolution, banded attention products -------------------------------------------------
    def convtrans_plan(self, xshape, wshape, ph, pw, sh=1, sw=1, dh=1, dw=1, oph=0, opw=0, bias=False, act="none",
                       algo="auto"):
        """ConvTransOp: x {n,h,w,f}, weight {r,s,f,c} -> {n,oh,ow,c} (channels last, as the reference defines it)."""
        n, h, w, f = xshape
        r, s, f2, c = wshape
        if f != f2:
            raise L.PetError(L.ERR_INVALID, "input channels differ from the filter's")
        args = [n, c, h, w, f, r, s, ph, pw, sh, sw, dh, dw, 1, int(bool(bias)), L.ACT[act], oph, opw]
        h_ = C.c_void_p()
        self.check(self.lib.petb200_convtrans_plan(self.h, L.ints(args), L.ALGO[algo], C.byref(h_)))
        p = Plan(self, h_)
        od = (C.c_int * 4)()
        self.check(self.lib.petb200_convtrans_out_dims(h_, od))
        p.out_shape = tuple(od)
        return p

    def convtrans_run(self, plan, x, w=None, bias=None):
        """w given: (re)do the weight-only work first; w None: reuse the weights of the previous call."""
        if w is not None:
            plan._w = _f32(w)
            self.check(self.lib.petb200_convtrans_set_weights(plan.h, _ptr(plan._w), _stream()))
        y = torch.empty(plan.out_shape, device=x.device, dtype=torch.float32)
        self.check(self.lib.petb200_convtrans_run(plan.h, _ptr(_f32(x)), _ptr(_f32(bias) if bias is not None else None),
                                                  _ptr(y), _stream()))
        return y

    def convtrans(self, x, w, ph, pw, sh=1, sw=1, dh=1, dw=1, oph=0, opw=0, bias=None, act="none", algo="auto"):
        key = ("convtrans", tuple(x.shape), tuple(w.shape), ph, pw, sh, sw, dh, dw, oph, opw, bias is not None, act, algo)
        plan = self._plans.get(key)
        if plan is None:
            plan = self._plans[key] = self.convtrans_plan(x.shape, w.shape, ph, pw, sh, sw, dh, dw, oph, opw,
                                                          bias is not None, act, algo)
        return self.convtrans_run(plan, x, w, bias)

    def g2bmm(self, q, k, width, dilation=1):
        """Banded Q.K^T: q, k [b,n,m] -> [b,n,2*width+1]; key row i + dilation*(j-width), zero outside [0,n)."""
        q, k = _f32(q), _f32(k)
        if q.dim() != 3 or tuple(q.shape) != tuple(k.shape):
            raise L.PetError(L.ERR_INVALID, "g2bmm operands must be 3-D and of equal shape")
        b, n, m = q.shape
        y = torch.empty((b, n, 2 * width + 1), device=q.device, dtype=torch.float32)
        self.check(self.lib.petb200_g2bmm_run(self.h, _ptr(q), _ptr(k), _ptr(y), b, n, m, width, dilation, _stream()))
        return y

    def gbmml(self, p, v, dilation=1):
        """Banded P.V: p [b,n,2w+1], v [b,n,m] -> [b,n,m]."""
        p, v = _f32(p), _f32(v)
        if p.dim() != 3 or v.dim() != 3 or p.shape[:2] != v.shape[:2] or p.shape[2] % 2 != 1:
            raise L.PetError(L.ERR_INVALID, "gbmml operands must be [b,n,2w+1] and [b,n,m]")
        b, n, bw = p.shape
        m = v.shape[2]
        y = torch.empty((b, n, m), device=p.device, dtype=torch.float32)
        self.check(self.lib.petb200_gbmml_run(self.h, _ptr(p), _ptr(v), _ptr(y), b, n, m, (bw - 1) // 2, dilation, _stream()))
        return y

    def banded_time(self, kind, b, n, m, width, dilation=1, rounds=100, warmup=10):
        ms = C.c_float()
        self.check(self.lib.petb200_banded_time(self.h, {"g2bmm": 0, "gbmml": 1}[kind], b, n, m, width, dilation, rounds,
                                                warmup, C.byref(ms), _stream()))
        return ms.value

    # ---- matmul --------------------------------------------------------------------------------------------
    def matmul_plan(self, ashape, bshape, transA=False, transB=False, bias=False, act="none", algo="auto", strides=None):
        """strides: optional (A batch, A row, B batch, B row, C batch, C row) in elements for operands that are strided
        views (the logical shapes stay ashape/bshape); the result then has to be passed in through `out`."""
        if len(ashape) != 3 or len(bshape) != 3 or ashape[0] != bshape[0]:
            raise L.PetError(L.ERR_INVALID, "matmul operands must be 3-D with equal batch")  # MatmulOp::checkValid
        b = ashape[0]
        m, k = (ashape[2], ashape[1]) if transA else (ashape[1], ashape[2])
        n, k2 = (bshape[1], bshape[2]) if transB else (bshape[2], bshape[1])
        if k != k2:
            raise L.PetError(L.ERR_INVALID, "matmul inner extents differ")
        h_ = C.c_void_p()
        if strides is not None:
            st = (C.c_longlong * 6)(*[int(v) for v in strides])
            self.check(self.lib.petb200_matmul_plan_strided(self.h, int(transA), int(transB), b, m, n, k, int(bool(bias)),
                                                            L.ACT[act], L.ALGO[algo], st, C.byref(h_)))
        else:
            self.check(self.lib.petb200_matmul_plan(self.h, int(transA), int(transB), b, m, n, k, int(bool(bias)), L.ACT[act],
                                                    L.ALGO[algo], C.byref(h_)))
        p = Plan(self, h_)
        p.out_shape = (b, m, n)
        return p

    def matmul_set_weights(self, plan, b):
        """B is a weight: do its preprocessing once (ref: the weight-only operators hoisted by src/Graph/code_engine.cc:187-193);
        matmul_run then takes b=None."""
        plan._b = _f32(b)
        self.check(self.lib.petb200_matmul_set_weights(plan.h, _ptr(plan._b), _stream()))

    def matmul_run(self, plan, a, b, bias=None, out=None, residual=None):
        c = out if out is not None else torch.empty(plan.out_shape, device=a.device, dtype=torch.float32)
        if residual is not None:
            if tuple(residual.shape) != tuple(plan.out_shape):
                raise L.PetError(L.ERR_INVALID, "residual must have the shape of the output")
            self.check(self.lib.petb200_matmul_run_residual(plan.h, _ptr(_f32(a)), _ptr(_f32(b) if b is not None else None), _ptr(bias),
                                                            _ptr(_f32(residual)),
                                                            _ptr(c), _stream()))
        else:
            self.check(self.lib.petb200_matmul_run(plan.h, _ptr(_f32(a)), _ptr(_f32(b) if b is not None else None), _ptr(bias), _ptr(c),
                                                   _stream()))
        return c

    def matmul(self, a, b, transA=False, transB=False, bias=None, act="none", algo="auto", residual=None):
        key = ("matmul", tuple(a.shape), tuple(b.shape), transA, transB, bias is not None, act, algo)
        plan = self._plans.get(key)
        if plan is None:
            plan = self._plans[key] = self.matmul_plan(a.shape, b.shape, transA, transB, bias is not None, act, algo)
        return self.matmul_run(plan, a, b, bias, residual=residual)

    # ---- layout --------------------------------------------------------------------------------------------
    def transpose_plan(self, shape, ops):
        """ops: list of (split, after, factor) applied left to right and fused into one kernel."""
        descs = (L.TransposeDesc * len(ops))()
        for d, (split, after, factor) in zip(descs, ops):
            sizes, flat = perm_spec(after)
            d.split, d.factor, d.ngroups = split, factor, len(sizes)
            for i, v in enumerate(sizes):
                d.group_sizes[i] = v
            for i, v in enumerate(flat):
                d.flat[i] = v
        h_ = C.c_void_p()
        self.check(self.lib.petb200_transpose_plan(self.h, len(shape), L.ints(shape), len(ops), descs, C.byref(h_)))
        return self._layout_plan(h_)

    def transpose_halo_plan(self, shape, split, after, factor, mode, amount):
        """One TransposeOp with `amount` of the reference's pad / extr / copys / dels (TransposeOp::getTTParam)."""
        d = L.TransposeDesc()
        sizes, flat = perm_spec(after)
        d.split, d.factor, d.ngroups = split, factor, len(sizes)
        for i, v in enumerate(sizes):
            d.group_sizes[i] = v
        for i, v in enumerate(flat):
            d.flat[i] = v
        amt = {m: (amount if m == mode else 0) for m in ("pad", "extr", "copys", "dels")}
        if mode not in amt:
            raise L.PetError(L.ERR_INVALID, "mode must be pad, extr, copys or dels")
        h_ = C.c_void_p()
        self.check(self.lib.petb200_transpose_halo_plan(self.h, len(shape), L.ints(shape), C.byref(d), amt["pad"], amt["extr"],
                                                        amt["copys"], amt["dels"], C.byref(h_)))
        return self._layout_plan(h_)

    def transpose_halo(self, x, split, after, factor, mode, amount):
        key = ("halo", tuple(x.shape), split, repr(after), factor, mode, amount)
        return self.layout_run(self._cached_layout(key, lambda: self.transpose_halo_plan(x.shape, split, after, factor, mode, amount)), x)

    def _layout_plan(self, h_):
        p = Plan(self, h_)
        od = (C.c_int * 16)()
        nd = self.lib.petb200_layout_out_dims(h_, od)
        p.out_shape = tuple(od[i] for i in range(nd))
        return p

    def layout_run(self, plan, x, out=None):
        assert x.is_cuda and x.element_size() == 4
        x = x.contiguous()
        y = out if out is not None else torch.empty(plan.out_shape, device=x.device, dtype=x.dtype)
        self.check(self.lib.petb200_layout_run(plan.h, _ptr(x), _ptr(y), _stream()))
        return y

    def _cached_layout(self, key, make):
        plan = self._plans.get(key)
        if plan is None:
            plan = self._plans[key] = make()
        return plan

    def transpose(self, x, split, after, factor=2):
        return self.transpose_chain(x, [(split, after, factor)])

    def transpose_chain(self, x, ops):
        key = ("tr", tuple(x.shape), repr(ops))
        return self.layout_run(self._cached_layout(key, lambda: self.transpose_plan(tuple(x.shape), ops)), x)

    def pad(self, x, begin, end):
        def make():
            h_ = C.c_void_p()
            self.check(self.lib.petb200_pad_plan(self.h, x.dim(), L.ints(x.shape), L.ints(begin), L.ints(end), C.byref(h_)))
            return self._layout_plan(h_)
        return self.layout_run(self._cached_layout(("pad", tuple(x.shape), tuple(begin), tuple(end)), make), x)

    def slice(self, x, begin, end):
        def make():
            h_ = C.c_void_p()
            self.check(self.lib.petb200_slice_plan(self.h, x.dim(), L.ints(x.shape), L.ints(begin), L.ints(end), C.byref(h_)))
            return self._layout_plan(h_)
        return self.layout_run(self._cached_layout(("slice", tuple(x.shape), tuple(begin), tuple(end)), make), x)

    def extend(self, x, dim, num):
        def make():
            h_ = C.c_void_p()
            self.check(self.lib.petb200_extend_plan(self.h, x.dim(), L.ints(x.shape), dim, num, C.byref(h_)))
            return self._layout_plan(h_)
        return self.layout_run(self._cached_layout(("extend", tuple(x.shape), dim, num), make), x)

    def concat(self, xs, dim):
        xs = [t.contiguous() for t in xs]
        shp = list(xs[0].shape)
        shp[dim] = sum(t.shape[dim] for t in xs)
        out = torch.empty(shp, device=xs[0].device, dtype=xs[0].dtype)
        ptrs = (C.c_void_p * len(xs))(*[t.data_ptr() for t in xs])
        self.check(self.lib.petb200_concat_run(self.h, len(shp), L.ints(shp), dim, len(xs), L.ints([t.shape[dim] for t in xs]),
                                               ptrs, _ptr(out), _stream()))
        return out

    def split(self, x, dim, sizes):
        """sizes are RATIOS, scaled by dim / sum(sizes) as SplitOp::computeShapeV does."""
        x = x.contiguous()
        total = sum(sizes)
        if total <= 0 or x.shape[dim] % total:
            raise L.PetError(L.ERR_INVALID, "split ratios do not divide the dimension")
        unit = x.shape[dim] // total
        outs = []
        for s in sizes:
            shp = list(x.shape)
            shp[dim] = unit * s
            outs.append(torch.empty(shp, device=x.device, dtype=x.dtype))
        ptrs = (C.c_void_p * len(outs))(*[t.data_ptr() for t in outs])
        self.check(self.lib.petb200_split_run(self.h, x.dim(), L.ints(x.shape), dim, len(outs),
                                              L.ints([t.shape[dim] for t in outs]), _ptr(x), ptrs, _stream()))
        return outs

    # ---- elementwise & friends -----------------------------------------------------------------------------
    def eltwise(self, kind, xs, act="none", out=None):
        xs = [_f32(t) for t in xs]
        y = out if out is not None else torch.empty_like(xs[0])
        ptrs = (C.c_void_p * len(xs))(*[t.data_ptr() for t in xs])
        sizes = (C.c_size_t * len(xs))(*[t.numel() for t in xs])
        self.check(self.lib.petb200_eltwise_run(self.h, {"add": 0, "sub": 1, "mul": 2}[kind], len(xs), ptrs, sizes, _ptr(y),
                                                y.numel(), L.ACT[act], _stream()))
        return y

    def activation(self, x, act, out=None):
        x = _f32(x)
        y = out if out is not None else torch.empty_like(x)
        self.check(self.lib.petb200_activation_run(self.h, _ptr(x), _ptr(y), x.numel(), L.ACT[act], _stream()))
        return y

    def batchnorm(self, x, scale, bias, mean, var, eps=1e-5):
        x = _f32(x)
        y = torch.empty_like(x)
        inner = x[0, 0].numel()
        self.check(self.lib.petb200_batchnorm_run(self.h, _ptr(x), _ptr(_f32(scale)), _ptr(_f32(bias)), _ptr(_f32(mean)),
                                                  _ptr(_f32(var)), _ptr(y), x.shape[0], x.shape[1], inner, C.c_float(eps),
                                                  _stream()))
        return y

    def _pool(self, kind, x, kh, kw, ph, pw, sh, sw):
        x = _f32(x)
        n, c, h, w = x.shape
        oh, ow = (h - (kh - sh) + 2 * ph) // sh, (w - (kw - sw) + 2 * pw) // sw
        y = torch.empty((n, c, oh, ow), device=x.device, dtype=torch.float32)
        self.check(self.lib.petb200_pool2d_run(self.h, kind, _ptr(x), _ptr(y), n, c, h, w, kh, kw, ph, pw, sh, sw, _stream()))
        return y

    def maxpool(self, x, kh, kw, dh, dw, ph, pw, sh, sw):
        if dh != 1 or dw != 1:  # the reference asserts dilation 1 for pooling (src/Graph/operator.cc:2774-2844)
            raise L.PetError(L.ERR_UNSUPPORTED, "dilated pooling")
        return self._pool(0, x, kh, kw, ph, pw, sh, sw)

    def avgpool(self, x, kh, kw, ph, pw, sh, sw):
        return self._pool(1, x, kh, kw, ph, pw, sh, sw)

    def div(self, a, b):
        a, b = _f32(a), _f32(b)
        out = torch.empty(a.shape if a.numel() >= b.numel() else b.shape, device=a.device, dtype=torch.float32)
        self.check(self.lib.petb200_div_run(self.h, _ptr(a), a.numel(), _ptr(b), b.numel(), _ptr(out), out.numel(), _stream()))
        return out

    def pow(self, x, p):
        x = _f32(x)
        y = torch.empty_like(x)
        self.check(self.lib.petb200_pow_run(self.h, _ptr(x), _ptr(y), x.numel(), int(p), _stream()))
        return y

    @staticmethod
    def _around(shape, axis):
        outer = int(np.prod(shape[:axis], dtype=np.int64))
        inner = int(np.prod(shape[axis + 1:], dtype=np.int64))
        return outer, int(shape[axis]), inner

    def reduce_mean(self, x, axis):
        x = _f32(x)
        outer, ln, inner = self._around(x.shape, axis)
        shape = list(x.shape)
        shape[axis] = 1
        y = torch.empty(shape, device=x.device, dtype=torch.float32)
        self.check(self.lib.petb200_reducemean_run(self.h, _ptr(x), _ptr(y), outer, ln, inner, _stream()))
        return y

    def gather(self, data, indices, axis):
        """GatherOp: output dims = indices dims + data dims without `axis`."""
        data = data.contiguous()
        idx = indices.to(torch.int32).contiguous()
        outer, ln, inner = self._around(data.shape, axis)
        shape = list(idx.shape) + [d for i, d in enumerate(data.shape) if i != axis]
        out = torch.empty(shape, device=data.device, dtype=data.dtype)
        self.check(self.lib.petb200_gather_run(self.h, _ptr(data), _ptr(idx), _ptr(out), idx.numel(), outer, ln, inner, _stream()))
        return out

    def rowmean(self, x, cols):
        x = _f32(x)
        rows = x.numel() // cols
        y = torch.empty(rows, device=x.device, dtype=torch.float32)
        self.check(self.lib.petb200_rowmean_run(self.h, _ptr(x), _ptr(y), rows, cols, _stream()))
        return y

    def softmax(self, x, axis=-1):
        """SoftmaxOp over `axis` (ref: include/operator.h:1887-1938)."""
        x = _f32(x)
        y = torch.empty_like(x)
        axis = axis + x.dim() if axis < 0 else axis
        if not 0 <= axis < x.dim():
            raise L.PetError(L.ERR_INVALID, "softmax axis out of range")
        outer = int(np.prod(x.shape[:axis], dtype=np.int64))
        inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
        self.check(self.lib.petb200_softmax_axis_run(self.h, _ptr(x), _ptr(y), outer, x.shape[axis], inner, _stream()))
        return y

    def attention(self, q, k, v):
        """softmax_rows(q k^T) v per batch entry in one launch: q [bs, m, kd], k [bs, n, kd], v [bs, n, d] -> [bs, m, d]
        (the reference's MatmulOp(transB) -> SoftmaxOp -> MatmulOp chain; n, kd, d <= 128)."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        if q.dim() != 3 or k.dim() != 3 or v.dim() != 3 or k.shape[0] != q.shape[0] or v.shape[0] != q.shape[0] or \
                k.shape[2] != q.shape[2] or v.shape[1] != k.shape[1]:
            raise L.PetError(L.ERR_INVALID, "attention: q [bs,m,kd], k [bs,n,kd], v [bs,n,d] expected")
        y = torch.empty((q.shape[0], q.shape[1], v.shape[2]), device=q.device, dtype=torch.float32)
        self.check(self.lib.petb200_attention_run(self.h, _ptr(q), _ptr(k), _ptr(v), _ptr(y), q.shape[0], q.shape[1], k.shape[1],
                                                   q.shape[2], v.shape[2], None, _stream()))
        return y

    def layernorm(self, x, gamma=None, beta=None, eps=1e-5):
        x = _f32(x)
        y = torch.empty_like(x)
        self.check(self.lib.petb200_layernorm_run(self.h, _ptr(x), _ptr(gamma), _ptr(beta), _ptr(y),
                                                  x.numel() // x.shape[-1], x.shape[-1], C.c_float(eps), _stream()))
        return y
