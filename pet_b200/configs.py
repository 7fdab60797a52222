"""The benchmark configurations as operator graphs, written once against a small builder interface so that the same
description can be lowered onto the GPU graph (GraphBuilder below) or evaluated by any other backend that offers the
same methods (the tests evaluate it with the CPU oracle).

Shapes and value distributions follow the configuration list: seeded synthetic tensors only, no dataset items and
no pretrained weights.  Topologies: the PET rewrites of a 3x3 conv (H split onto the batch + correction) and of a
dilated conv (space-to-batch), ResNet-18 with folded BatchNorm, a post-LN BERT-base encoder, ResNet3D-18.
"""
import numpy as np

# TransposeOp constructor arguments of the named rewrites (reference: src/Mutant/generator.cc:1027-1046,1085-1092)
H2N = (2, [[0, 2], 1, -1, 3], -2)
N2H = (0, [0, 1, [-1, 2], 3], 2)
W2N = (3, [[0, 3], 1, 2, -1], -2)
N2W = (0, [0, 1, 2, [-1, 3]], 2)
D2H = (2, [0, 1, [-1, 2], 3], 2)
D2H_INV = (2, [0, 1, [-1, 2], 3], -2)
D2W = (3, [0, 1, 2, [-1, 3]], 2)
D2W_INV = (3, [0, 1, 2, [-1, 3]], -2)
SPACE_TO_BATCH = [D2H, H2N, D2W, W2N]
BATCH_TO_SPACE = [N2W, D2W_INV, N2H, D2H_INV]


class GraphBuilder:
    """Lowers a configuration onto pet_b200.graph.Graph and remembers the data of every constant."""

    def __init__(self, graph):
        self.g = graph
        self.data = []  # (tensor, ndarray)

    def input(self, array):
        t = self.g.tensor(array.shape)
        self.data.append((t, array))
        return t

    def const(self, array):
        t = self.g.tensor(array.shape, weight=True)
        self.data.append((t, array))
        return t

    def load(self):
        """After graph.compile(): copy every remembered array to the device."""
        for t, a in self.data:
            self.g.set_data(t, a)

    def __getattr__(self, name):  # every operator method is the Graph's own
        return getattr(self.g, name)


def rng_for(config, index):
    return np.random.default_rng(1000 * config + index)


def he_normal(rng, shape):
    fan_in = int(np.prod(shape[1:]))
    return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)


def xavier_uniform(rng, shape):
    lim = np.sqrt(6.0 / (shape[0] + shape[1]))
    return rng.uniform(-lim, lim, shape).astype(np.float32)


# ---- config 1: 3x3 conv, original and the H->N partially equivalent rewrite with correction ----------------------
def c1_tensors(c=64, hw=56, k=64):
    return (rng_for(1, 0).uniform(-1, 1, (1, c, hw, hw)).astype(np.float32),
            rng_for(1, 1).uniform(-1, 1, (k, c, 3, 3)).astype(np.float32))


def c1_original(b, x, w):
    return b.conv(b.input(x), b.const(w), 1, 1)


def c1_rewrite(b, x, w, correct=True):
    xi, wi = b.input(x), b.const(w)
    y = b.transpose(b.conv(b.transpose(xi, *H2N), wi, 1, 1), *N2H)
    if correct:
        half = x.shape[2] // 2
        y = b.correction(xi, wi, y, 1, 1, rows=(half - 1, 2))  # the two rows whose windows cross the seam
    return y


def c1_rewrite_halo(b, x, w):
    """The same H->N rewrite made exact without a correction: the halves overlap by one halo row (copys = 1) and the merge
    drops the row each half computed from the other's territory (dels = 1)."""
    xi, wi = b.input(x), b.const(w)
    return b.transpose_halo(b.conv(b.transpose_halo(xi, *H2N, "copys", 1), wi, 1, 1), *N2H, "dels", 1)


# ---- config 2: dilated conv, original and the space-to-batch rewrite -------------------------------------------
def c2_tensors(c=512, hw=64, k=512):
    return (rng_for(2, 0).standard_normal((1, c, hw, hw)).astype(np.float32), he_normal(rng_for(2, 1), (k, c, 3, 3)))


def c2_original(b, x, w):
    return b.conv(b.input(x), b.const(w), 2, 2, 1, 1, 2, 2)


def c2_rewrite(b, x, w):
    t = b.input(x)
    for op in SPACE_TO_BATCH:
        t = b.transpose(t, *op)
    t = b.conv(t, b.const(w), 1, 1)
    for op in BATCH_TO_SPACE:
        t = b.transpose(t, *op)
    return t


# ---- config 3: ResNet-18, BatchNorm folded (gamma 1, beta 0, mean 0, var 1 => scale 1/sqrt(1+eps), bias 0) --------
def resnet18(b, batch=1, size=224, classes=1000, width=64):
    r = rng_for(3, 0)
    fold = np.float32(1.0 / np.sqrt(1.0 + 1e-5))
    idx = [0]

    def conv_bn(t, cin, cout, k, stride, pad, act):
        idx[0] += 1
        w = he_normal(rng_for(3, idx[0]), (cout, cin, k, k)) * fold
        bias = np.zeros(cout, np.float32)
        return b.conv(t, b.const(w), pad, pad, stride, stride, 1, 1, bias=b.const(bias), act=act)

    def block(t, cin, cout, stride):
        y = conv_bn(t, cin, cout, 3, stride, 1, "relu")
        y = conv_bn(y, cout, cout, 3, 1, 1, "none")
        sc = t if (stride == 1 and cin == cout) else conv_bn(t, cin, cout, 1, stride, 0, "none")
        return b.relu(b.add([y, sc]))

    x = r.standard_normal((batch, 3, size, size)).astype(np.float32)
    t = conv_bn(b.input(x), 3, width, 7, 2, 3, "relu")
    t = b.maxpool(t, 3, 3, 1, 1, 1, 1, 2, 2)
    cin = width
    for stage, cout in enumerate([width, 2 * width, 4 * width, 8 * width]):
        for i in range(2):
            t = block(t, cin, cout, 2 if (stage > 0 and i == 0) else 1)
            cin = cout
    t = b.avgpool(t)                                  # global average pool
    t = b.reshape(t, [1, batch, cin])                 # flatten -> [1, N, 512]
    wf = he_normal(rng_for(3, 99), (classes, cin)).T.copy()  # stored [512, classes]
    return b.matmul(t, b.const(wf.reshape(1, cin, classes)), bias=b.const(np.zeros(classes, np.float32)))


# ---- config 4: BERT-base encoder stack (post-LN, GELU in the erf form) -----------------------------------------
def bert_encoder(b, layers=12, seq=128, hidden=768, heads=12, ffn=3072, eps=1e-5):
    hd = hidden // heads
    x = rng_for(4, 0).standard_normal((seq, hidden)).astype(np.float32)
    t = b.reshape(b.input(x), [1, seq, hidden])
    idx = [0]

    def dense(t, cin, cout, act="none", scale=1.0):
        idx[0] += 1
        w = xavier_uniform(rng_for(4, idx[0]), (cin, cout)) * np.float32(scale)
        return b.matmul(t, b.const(w.reshape(1, cin, cout)), bias=b.const(np.zeros(cout, np.float32)), act=act)

    def split_heads(t):  # [1, seq, hidden] -> [heads, seq, hd]
        return b.transpose(b.reshape(t, [seq, heads, hd]), -1, [1, 0, 2])

    ones, zeros = np.ones(hidden, np.float32), np.zeros(hidden, np.float32)
    for _ in range(layers):
        q = split_heads(dense(t, hidden, hidden, scale=1.0 / np.sqrt(hd)))  # 1/sqrt(d) folded into Wq
        k = split_heads(dense(t, hidden, hidden))
        v = split_heads(dense(t, hidden, hidden))
        p = b.softmax(b.matmul(q, k, transB=True), 2)                        # [heads, seq, seq]
        c = b.transpose(b.matmul(p, v), -1, [1, 0, 2])                       # [seq, heads, hd]
        a = dense(b.reshape(c, [1, seq, hidden]), hidden, hidden)
        t = b.layernorm(b.add([t, a]), b.const(ones), b.const(zeros), eps)
        f = dense(dense(t, hidden, ffn, act="gelu"), ffn, hidden)
        t = b.layernorm(b.add([t, f]), b.const(ones), b.const(zeros), eps)
    return t


# ---- config 5: ResNet3D-18 ------------------------------------------------------------------------------------
def r3d18(b, batch=1, frames=16, size=112, classes=400, width=64):
    fold = np.float32(1.0 / np.sqrt(1.0 + 1e-5))
    idx = [0]

    def conv_bn(t, cin, cout, k, stride, pad, act):
        idx[0] += 1
        w = he_normal(rng_for(5, idx[0]), (cout, cin) + tuple(k)) * fold
        return b.conv3d(t, b.const(w), pad, stride, (1, 1, 1), bias=b.const(np.zeros(cout, np.float32)), act=act)

    def block(t, cin, cout, stride):
        s3 = (stride,) * 3
        y = conv_bn(t, cin, cout, (3, 3, 3), s3, (1, 1, 1), "relu")
        y = conv_bn(y, cout, cout, (3, 3, 3), (1, 1, 1), (1, 1, 1), "none")
        sc = t if (stride == 1 and cin == cout) else conv_bn(t, cin, cout, (1, 1, 1), s3, (0, 0, 0), "none")
        return b.relu(b.add([y, sc]))

    x = rng_for(5, 0).standard_normal((batch, 3, frames, size, size)).astype(np.float32)
    t = conv_bn(b.input(x), 3, width, (3, 7, 7), (1, 2, 2), (1, 3, 3), "relu")
    cin = width
    for stage, cout in enumerate([width, 2 * width, 4 * width, 8 * width]):
        for i in range(2):
            t = block(t, cin, cout, 2 if (stage > 0 and i == 0) else 1)
            cin = cout
    d = t.dims if hasattr(t, "dims") else t.shape
    t = b.avgpool(b.reshape(t, [d[0], d[1], d[2] * d[3], d[4]]))   # global average over (D, H, W)
    t = b.reshape(t, [1, batch, cin])
    wf = he_normal(rng_for(5, 99), (classes, cin)).T.copy()
    return b.matmul(t, b.const(wf.reshape(1, cin, classes)), bias=b.const(np.zeros(classes, np.float32)))
