"""Evaluates a configuration from pet_b200.configs with the vendor libraries through torch (cuDNN / cuBLAS on the GPU,
TF32 switched off: true fp32 math; or on: the libraries' default math mode on this GPU) — the library execution of the
same graph that the parity contract names, and the timing baseline of the benchmark.  torch's bindings stand in for the
reference's direct calls (cudnnConvolutionForward, ref: src/Graph/operator.cc:296-515; cublasGemmStridedBatchedEx,
ref: :728-832).  Harness only, never on the product path; layout operators other than plain permutations go through the
CPU oracle (bit-exact copies either way; parity tests only).  The product (pet_b200/) must not import this."""
import numpy as np
import torch
import torch.nn.functional as F



def _t(a):
    return a if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def _act(y, act):
    return {"none": lambda v: v, "relu": F.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh,
            "gelu": lambda v: F.gelu(v, approximate="none")}[act](y)


class TorchBuilder:
    def __init__(self, tf32=False, dtype=torch.float32):
        self.tf32, self.dtype = tf32, dtype

    def _lib(self):
        torch.backends.cuda.matmul.allow_tf32 = self.tf32
        torch.backends.cudnn.allow_tf32 = self.tf32

    def input(self, a):
        return _t(a).to(self.dtype)

    const = input

    def conv(self, x, w, ph, pw, sh=1, sw=1, dh=1, dw=1, bias=None, act="none"):
        self._lib()
        return _act(F.conv2d(x, w, bias, (sh, sw), (ph, pw), (dh, dw), x.shape[1] // w.shape[1]), act)

    def conv3d(self, x, w, pad, stride=(1, 1, 1), dil=(1, 1, 1), bias=None, act="none"):
        self._lib()
        return _act(F.conv3d(x, w, bias, tuple(stride), tuple(pad), tuple(dil), x.shape[1] // w.shape[1]), act)

    def matmul(self, a, b, transA=False, transB=False, bias=None, act="none"):
        self._lib()
        a = a[None] if a.dim() == 2 else a
        b = b[None] if b.dim() == 2 else b
        y = torch.matmul(a.transpose(1, 2) if transA else a, b.transpose(1, 2) if transB else b)
        return _act(y if bias is None else y + bias, act)

    def _np(self, name, x, *args):
        from oracle import pet_oracle as po  # only the parity tests reach this
        return _t(getattr(po, name)(x.cpu().numpy(), *args))

    def transpose(self, x, split, after, factor=2):
        if split == -1 and all(not isinstance(g, (list, tuple)) for g in after):
            return x.permute(*after).contiguous()
        return self._np("transpose", x, split, after, factor)

    def add(self, xs):
        y = xs[0]
        for t in xs[1:]:
            y = y + t
        return y

    def relu(self, x):
        return F.relu(x)

    def gelu(self, x):
        return F.gelu(x, approximate="none")

    def maxpool(self, x, kh, kw, dh, dw, ph, pw, sh, sw):
        return F.max_pool2d(x, (kh, kw), (sh, sw), (ph, pw))

    def avgpool(self, x, kh=None, kw=None, ph=0, pw=0, sh=1, sw=1):
        if kh is None:
            kh, kw = x.shape[2], x.shape[3]
        return F.avg_pool2d(x, (kh, kw), (sh, sw), (ph, pw), count_include_pad=False)

    def softmax(self, x, axis):
        return torch.softmax(x, axis)

    def layernorm(self, x, gamma=None, beta=None, eps=1e-5):
        return F.layer_norm(x, (x.shape[-1],), gamma, beta, eps)

    def reshape(self, x, dims):
        return x.contiguous().reshape(list(dims))

    def identity(self, x):
        return x
