"""Graph-level host API: the counterpart of the reference's Python module (`cpp_module.Graph`, src/ffi/ffi_pet.cc:32-175)
for building an operator graph, plus the execution and timing entry points that replace CodeEngine / SearchEngine.getPerf.

Method names and argument order follow the reference FFI: tensor, conv, matmul, transpose, pad, slice, concat, split,
extend, add, sub, mul, relu, sigmoid, tanh, maxpool, avgpool, softmax, batchnorm, reshape, flatten, identity,
setOutputs.  Additions the reference lacks: conv3d, gelu, layernorm, correction, compile, run, perf, time.
Tensors are small handle objects (`Tensor.id`, `Tensor.dims`).
"""
import ctypes as C
import os

import numpy as np

from . import lib as L

_i, _vp, _fp, _sz = C.c_int, C.c_void_p, C.c_float, C.c_size_t
_ip = C.POINTER(C.c_int)

GRAPH_SYMBOLS = {
    "petb200_graph_create": (_i, [_vp, C.POINTER(_vp)]),
    "petb200_graph_destroy": (None, [_vp]),
    "petb200_graph_last_error": (C.c_char_p, [_vp]),
    "petb200_graph_tensor": (_i, [_vp, _i, _ip, _i, _ip]),
    "petb200_graph_tensor_dims": (_i, [_vp, _i, _ip]),
    "petb200_graph_conv": (_i, [_vp] + [_i] * 10 + [_ip]),
    "petb200_graph_conv3d": (_i, [_vp, _i, _i, _i, _ip, _ip, _ip, _i, _ip]),
    "petb200_graph_convtrans": (_i, [_vp] + [_i] * 12 + [_ip]),
    "petb200_graph_g2bmm": (_i, [_vp, _i, _i, _i, _i, _ip]),
    "petb200_graph_gbmml": (_i, [_vp, _i, _i, _i, _ip]),
    "petb200_graph_matmul": (_i, [_vp, _i, _i, _i, _i, _i, _i, _ip]),
    "petb200_graph_transpose": (_i, [_vp, _i, C.POINTER(L.TransposeDesc), _ip]),
    "petb200_graph_transpose_halo": (_i, [_vp, _i, C.POINTER(L.TransposeDesc), _i, _i, _i, _i, _ip]),
    "petb200_graph_pad": (_i, [_vp, _i, _ip, _ip, _ip]),
    "petb200_graph_slice": (_i, [_vp, _i, _ip, _ip, _ip]),
    "petb200_graph_extend": (_i, [_vp, _i, _i, _i, _ip]),
    "petb200_graph_concat": (_i, [_vp, _i, _ip, _i, _ip]),
    "petb200_graph_split": (_i, [_vp, _i, _i, _i, _ip, _ip]),
    "petb200_graph_eltwise": (_i, [_vp, _i, _i, _ip, _ip]),
    "petb200_graph_activation": (_i, [_vp, _i, _i, _ip]),
    "petb200_graph_pool": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _ip]),
    "petb200_graph_softmax": (_i, [_vp, _i, _i, _ip]),
    "petb200_graph_div": (_i, [_vp, _i, _i, _ip]),
    "petb200_graph_pow": (_i, [_vp, _i, _i, _ip]),
    "petb200_graph_reducemean": (_i, [_vp, _i, _i, _ip]),
    "petb200_graph_gather": (_i, [_vp, _i, _i, _i, _ip]),
    "petb200_graph_layernorm": (_i, [_vp, _i, _i, _i, _fp, _ip]),
    "petb200_graph_batchnorm": (_i, [_vp, _i, _i, _i, _i, _i, _fp, _ip]),
    "petb200_graph_reshape": (_i, [_vp, _i, _i, _ip, _ip]),
    "petb200_graph_correction": (_i, [_vp] + [_i] * 15 + [_ip]),
    "petb200_graph_set_outputs": (_i, [_vp, _i, _ip]),
    "petb200_graph_compile": (_i, [_vp, _i]),
    "petb200_graph_set_data": (_i, [_vp, _i, _vp, _sz, _vp]),
    "petb200_graph_get_data": (_i, [_vp, _i, _vp, _sz, _vp]),
    "petb200_graph_device_ptr": (_vp, [_vp, _i]),
    "petb200_graph_run": (_i, [_vp, _vp]),
    "petb200_graph_num_launches": (_i, [_vp]),
    "petb200_graph_num_steps": (_i, [_vp]),
    "petb200_graph_step_name": (C.c_char_p, [_vp, _i]),
    "petb200_graph_step_kernel": (C.c_char_p, [_vp, _i]),
    "petb200_graph_perf": (_i, [_vp, _i, _i, C.POINTER(_fp), C.POINTER(_fp)]),
    "petb200_graph_time": (_i, [_vp, _i, _i, C.POINTER(_fp), _vp]),
    "petb200_graph_run_profiled": (_i, [_vp, _vp, _i, _i]),
    "petb200_graph_profile_other_ms": (_i, [_vp, _i, C.POINTER(_fp)]),
}

_bound = False


def _lib():
    global _bound
    lib = L.load()
    if not _bound:
        for name, (res, args) in GRAPH_SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _bound = True
    return lib


class Tensor:
    def __init__(self, graph, tid):
        self.graph, self.id = graph, tid

    @property
    def dims(self):
        buf = (C.c_int * 8)()
        nd = self.graph.lib.petb200_graph_tensor_dims(self.graph.h, self.id, buf)
        return tuple(buf[i] for i in range(nd))

    def __repr__(self):
        return f"Tensor#{self.id}{list(self.dims)}"


def _tid(t):
    return -1 if t is None else t.id


class Graph:
    """Builds, compiles and runs an operator graph on one GPU through the C ABI."""

    def __init__(self, ctx):
        self.lib = _lib()
        self.ctx = ctx
        self.h = C.c_void_p()
        rc = self.lib.petb200_graph_create(ctx.h, C.byref(self.h))
        if rc:
            raise L.PetError(rc, "graph_create failed")

    def __del__(self):
        if getattr(self, "h", None) and self.ctx.h:
            self.lib.petb200_graph_destroy(self.h)
            self.h = None

    def _check(self, rc):
        if rc:
            raise L.PetError(rc, self.lib.petb200_graph_last_error(self.h).decode())

    def _out(self, fn, *args):
        out = C.c_int()
        self._check(fn(self.h, *args, C.byref(out)))
        return Tensor(self, out.value)

    # ---- builders (reference names) ----
    def tensor(self, dims, dtype="FLOAT", weight=False):
        # ref: Tensor::Float32, and Tensor::Int32 for gather indices only (include/tensor.h:11-14)
        if dtype not in ("FLOAT", "Float32", "float32", "INT32", "Int32", "int32"):
            raise L.PetError(L.ERR_UNSUPPORTED, "tensors are fp32, or int32 for gather indices")
        out = C.c_int()
        self._check(self.lib.petb200_graph_tensor(self.h, len(dims), L.ints(dims), int(weight), C.byref(out)))
        return Tensor(self, out.value)

    def conv(self, input, weight, ph, pw, sh=1, sw=1, dh=1, dw=1, bias=None, act="none"):
        return self._out(self.lib.petb200_graph_conv, input.id, weight.id, _tid(bias), ph, pw, sh, sw, dh, dw, L.ACT[act])

    def conv3d(self, input, weight, pad, stride=(1, 1, 1), dil=(1, 1, 1), bias=None, act="none"):
        return self._out(self.lib.petb200_graph_conv3d, input.id, weight.id, _tid(bias), L.ints(pad), L.ints(stride), L.ints(dil), L.ACT[act])

    def convTrans(self, input, weight, ph, pw, sh=1, sw=1, dh=1, dw=1, oph=0, opw=0, bias=None, act="none"):
        """ConvTransOp: input {n,h,w,f}, weight {r,s,f,c} -> {n,oh,ow,c} (ref: Graph::convTrans, src/ffi/ffi_pet.cc:45-48)."""
        return self._out(self.lib.petb200_graph_convtrans, input.id, weight.id, _tid(bias), ph, pw, sh, sw, dh, dw, oph, opw,
                         L.ACT[act])

    def g2bmm(self, A, B, width, dilation=1):
        return self._out(self.lib.petb200_graph_g2bmm, A.id, B.id, width, dilation)

    def gbmml(self, A, B, dilation=1):
        return self._out(self.lib.petb200_graph_gbmml, A.id, B.id, dilation)

    def matmul(self, A, B, transA=False, transB=False, bias=None, act="none"):
        return self._out(self.lib.petb200_graph_matmul, A.id, B.id, _tid(bias), int(transA), int(transB), L.ACT[act])

    @staticmethod
    def _desc(split, after, factor):
        groups = [list(g) if isinstance(g, (list, tuple)) else [g] for g in after]
        d = L.TransposeDesc()
        d.split, d.factor, d.ngroups = split, factor, len(groups)
        flat = [i for g in groups for i in g]
        for i, g in enumerate(groups):
            d.group_sizes[i] = len(g)
        for i, v in enumerate(flat):
            d.flat[i] = v
        return d

    def transpose(self, input, split, after, factor=2):
        return self._out(self.lib.petb200_graph_transpose, input.id, C.byref(self._desc(split, after, factor)))

    def transpose_halo(self, input, split, after, factor, mode, amount):
        """TransposeOp with `amount` of pad / extr / copys / dels (what setPaddingSize + Pre/Post select in the reference)."""
        if mode not in ("pad", "extr", "copys", "dels"):
            raise L.PetError(L.ERR_INVALID, "mode must be pad, extr, copys or dels")
        a = [amount if m == mode else 0 for m in ("pad", "extr", "copys", "dels")]
        return self._out(self.lib.petb200_graph_transpose_halo, input.id, C.byref(self._desc(split, after, factor)), *a)

    def flatten(self, input, axis):
        nd = len(input.dims)  # Graph::flatten, src/Graph/graph.cc:342-358
        return self.transpose(input, -1, [list(range(axis)), list(range(axis, nd))])

    def pad(self, input, begin, end):
        return self._out(self.lib.petb200_graph_pad, input.id, L.ints(begin), L.ints(end))

    def slice(self, input, begin, end):
        return self._out(self.lib.petb200_graph_slice, input.id, L.ints(begin), L.ints(end))

    def extend(self, input, dim, num):
        return self._out(self.lib.petb200_graph_extend, input.id, dim, num)

    def concat(self, inputs, dim):
        return self._out(self.lib.petb200_graph_concat, len(inputs), L.ints([t.id for t in inputs]), dim)

    def split(self, input, dim, sizes):
        if isinstance(sizes, int):
            sizes = [1] * sizes  # split(input, dim, num): equal parts
        outs = (C.c_int * len(sizes))()
        self._check(self.lib.petb200_graph_split(self.h, input.id, dim, len(sizes), L.ints(sizes), outs))
        return [Tensor(self, o) for o in outs]

    def _elt(self, kind, inputs):
        return self._out(self.lib.petb200_graph_eltwise, kind, len(inputs), L.ints([t.id for t in inputs]))

    def add(self, inputs):
        return self._elt(0, inputs)

    def sub(self, input0, input1):
        return self._elt(1, [input0, input1])

    def mul(self, inputs):
        return self._elt(2, inputs)

    def _act(self, input, act):
        return self._out(self.lib.petb200_graph_activation, input.id, L.ACT[act])

    def relu(self, input):
        return self._act(input, "relu")

    def sigmoid(self, input):
        return self._act(input, "sigmoid")

    def tanh(self, input):
        return self._act(input, "tanh")

    def gelu(self, input):
        return self._act(input, "gelu")

    def maxpool(self, input, kh, kw, dh, dw, ph, pw, sh, sw):
        if dh != 1 or dw != 1:
            raise L.PetError(L.ERR_UNSUPPORTED, "dilated pooling")
        return self._out(self.lib.petb200_graph_pool, 0, input.id, kh, kw, ph, pw, sh, sw)

    def avgpool(self, input, kh=None, kw=None, ph=0, pw=0, sh=1, sw=1):
        if kh is None:  # global average pool: Graph::avgpool(input, output)
            kh, kw = input.dims[2], input.dims[3]
        return self._out(self.lib.petb200_graph_pool, 1, input.id, kh, kw, ph, pw, sh, sw)

    def softmax(self, input, axis):
        return self._out(self.lib.petb200_graph_softmax, input.id, axis)

    def layernorm(self, input, gamma=None, beta=None, eps=1e-5):
        return self._out(self.lib.petb200_graph_layernorm, input.id, _tid(gamma), _tid(beta), C.c_float(eps))

    def batchnorm(self, input, scale, bias, mean, var, epsilon=1e-5, momentum=0.9):
        return self._out(self.lib.petb200_graph_batchnorm, input.id, scale.id, bias.id, mean.id, var.id, C.c_float(epsilon))

    def reshape(self, input, dims):
        return self._out(self.lib.petb200_graph_reshape, input.id, len(dims), L.ints(dims))

    def identity(self, input):
        return self.reshape(input, input.dims)

    def div(self, input0, input1):
        return self._out(self.lib.petb200_graph_div, input0.id, input1.id)

    def pow(self, input, pow):
        return self._out(self.lib.petb200_graph_pow, input.id, int(pow))

    def reduceMean(self, input, axis):
        return self._out(self.lib.petb200_graph_reducemean, input.id, axis)

    def gather(self, data, indices, axis):
        """indices: a tensor whose 32-bit words are int32 values (set_data with an int32 array)."""
        return self._out(self.lib.petb200_graph_gather, data.id, indices.id, axis)

    def resize(self, input, sizes=None):
        # ref: ResizeOp has neither a host body nor generated code (src/Graph/operator.cc:3696-3699 asserts)
        raise L.PetError(L.ERR_UNSUPPORTED, "resize: the reference defines only its shape; nothing to execute")

    def setInputs(self, inputs):
        """Kept for the reference's call sequence (Graph::setInputs): inputs are the tensors no operator produces."""
        self._declared_inputs = list(inputs)

    def getOperators(self):
        """(name, kernel) of every executable step after compile(), the closest counterpart of Graph::getOperators."""
        return self.steps()

    def updateConnection(self):
        """Connections are maintained as operators are added; kept for the reference's call sequence."""
        return True

    def correction(self, input, weight, y, ph, pw, sh=1, sw=1, dh=1, dw=1, rows=None, cols=None, bias=None, act="none"):
        """Recompute rows=(first, count) and cols=(first, count) of y — the rewritten sub-graph's output in the original
        layout — from the original conv operands."""
        oh, ow = y.dims[2], y.dims[3]
        r0, rn = rows if rows is not None else (0, oh)
        c0, cn = cols if cols is not None else (0, ow)
        return self._out(self.lib.petb200_graph_correction, input.id, weight.id, _tid(bias), y.id, ph, pw, sh, sw, dh, dw,
                         L.ACT[act], r0, rn, c0, cn)

    def setOutputs(self, outputs):
        self._check(self.lib.petb200_graph_set_outputs(self.h, len(outputs), L.ints([t.id for t in outputs])))

    # ---- execution (replaces CodeEngine.genCode + the emitted program) ----
    def compile(self, fuse=True, cuda_graph=True, fuse_attention=True):
        self._check(self.lib.petb200_graph_compile(self.h, (0 if fuse else 1) | (0 if cuda_graph else 2) | (0 if fuse_attention else 8)))
        return self

    def set_data(self, tensor, array, stream=None):
        if np.issubdtype(np.asarray(array).dtype, np.integer):  # index tensors: the int32 words go in untouched
            a = np.ascontiguousarray(array, dtype=np.int32).view(np.float32)
        else:
            a = np.ascontiguousarray(array, dtype=np.float32)
        self._check(self.lib.petb200_graph_set_data(self.h, tensor.id, a.ctypes.data_as(C.c_void_p), a.size, stream))
        if stream is None:
            import torch
            torch.cuda.synchronize()

    def get_data(self, tensor, stream=None):
        out = np.empty(tensor.dims, np.float32)
        self._check(self.lib.petb200_graph_get_data(self.h, tensor.id, out.ctypes.data_as(C.c_void_p), out.size, stream))
        return out

    def device_ptr(self, tensor):
        return self.lib.petb200_graph_device_ptr(self.h, tensor.id)

    def run(self, stream=None):
        self._check(self.lib.petb200_graph_run(self.h, stream))

    def run_profiled(self, slot, nslots, stream=None):
        """One pass issued step by step with CUDA events around every step that is not a tensor-core launch (slot of nslots
        event sets); see profile_other_ms."""
        self._check(self.lib.petb200_graph_run_profiled(self.h, stream, slot, nslots))

    def profile_other_ms(self, nslots):
        """Summed duration (ms) of the non-tensor-core steps over the `nslots` profiled passes."""
        ms = C.c_float()
        self._check(self.lib.petb200_graph_profile_other_ms(self.h, nslots, C.byref(ms)))
        return ms.value

    def steps(self):
        n = self.lib.petb200_graph_num_steps(self.h)
        return [(self.lib.petb200_graph_step_name(self.h, i).decode(), self.lib.petb200_graph_step_kernel(self.h, i).decode())
                for i in range(n)]

    def num_launches(self):
        return self.lib.petb200_graph_num_launches(self.h)

    def perf(self, rounds=200, warmup=200):
        """Sum of per-operator measured times in ms and the per-step list (SearchEngine::getPerf over Operator::perf)."""
        n = self.lib.petb200_graph_num_steps(self.h)
        per = (C.c_float * max(n, 1))()
        tot = C.c_float()
        self._check(self.lib.petb200_graph_perf(self.h, rounds, warmup, C.byref(tot), per))
        return tot.value, [per[i] for i in range(n)]

    def time(self, rounds=1000, warmup=100, stream=None):
        """ms per whole-graph pass: warm-up, then `rounds` replays between two CUDA events (the reference's protocol)."""
        ms = C.c_float()
        self._check(self.lib.petb200_graph_time(self.h, rounds, warmup, C.byref(ms), stream))
        return ms.value
