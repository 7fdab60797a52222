"""Library baseline on the same GPU: what the reference's backend would get from cuDNN / cuBLAS for the benchmark
configurations (reference call sites: cudnnConvolutionForward best-of-8 algorithms, src/Graph/operator.cc:296-515;
cublasGemmStridedBatchedEx, :728-832).  torch's cuDNN/cuBLAS bindings stand in for the reference's direct calls:
`cudnn.benchmark` picks the fastest algorithm the way ConvOp::perf's sweep does.  Two math modes are reported:
  default : CUDNN_DEFAULT_MATH / cublas default — TF32 tensor cores allowed (what the reference's calls get on B200)
  fp32    : TF32 disabled (the accuracy class this repository's 3xTF32 kernels match)
This is a measurement harness, not part of the product; run:  python baseline/lib_baseline.py
"""
import json
import sys

import torch
import torch.nn.functional as F


def time_fn(fn, warmup=20, rounds=200):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(rounds):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / rounds


def resnet18(x, ws):
    it = iter(ws)

    def cb(t, stride, pad, relu):
        t = F.conv2d(t, next(it), None, stride, pad)
        return F.relu(t) if relu else t

    t = F.max_pool2d(cb(x, 2, 3, True), 3, 2, 1)
    cin = 64
    for stage, cout in enumerate([64, 128, 256, 512]):
        for i in range(2):
            s = 2 if (stage > 0 and i == 0) else 1
            y = cb(cb(t, s, 1, True), 1, 1, False)
            sc = t if (s == 1 and cin == cout) else cb(t, s, 0, False)
            t = F.relu(y + sc)
            cin = cout
    return F.adaptive_avg_pool2d(t, 1).flatten(1) @ next(it)


def resnet18_weights(dev):
    ws = [torch.randn(64, 3, 7, 7, device=dev)]
    cin = 64
    for stage, cout in enumerate([64, 128, 256, 512]):
        for i in range(2):
            s = 2 if (stage > 0 and i == 0) else 1
            ws += [torch.randn(cout, cin, 3, 3, device=dev) * 0.05, torch.randn(cout, cout, 3, 3, device=dev) * 0.05]
            if not (s == 1 and cin == cout):
                ws.append(torch.randn(cout, cin, 1, 1, device=dev) * 0.05)
            cin = cout
    ws.append(torch.randn(512, 1000, device=dev) * 0.05)
    return ws


def bert(x, ws, heads=12):
    seq, hid = x.shape
    hd = hid // heads
    it = iter(ws)
    t = x
    for _ in range(12):
        q, k, v = [(t @ next(it)).view(seq, heads, hd).transpose(0, 1) for _ in range(3)]
        p = torch.softmax(q @ k.transpose(1, 2) / hd ** 0.5, -1)
        a = (p @ v).transpose(0, 1).reshape(seq, hid) @ next(it)
        t = F.layer_norm(t + a, (hid,))
        f = F.gelu(t @ next(it)) @ next(it)
        t = F.layer_norm(t + f, (hid,))
    return t


def main():
    dev = torch.device("cuda", 0)
    torch.backends.cudnn.benchmark = True
    out = {}
    for mode, tf32 in (("default_math_tf32", True), ("fp32", False)):
        torch.backends.cudnn.allow_tf32 = tf32
        torch.backends.cuda.matmul.allow_tf32 = tf32
        r = {}
        x, w = torch.randn(1, 64, 56, 56, device=dev), torch.randn(64, 64, 3, 3, device=dev)
        r["c1_conv3x3_original"] = time_fn(lambda: F.conv2d(x, w, None, 1, 1))
        x2, w2 = torch.randn(1, 512, 64, 64, device=dev), torch.randn(512, 512, 3, 3, device=dev) * 0.02
        r["c2_dilated_original"] = time_fn(lambda: F.conv2d(x2, w2, None, 1, 2, 2))
        x3 = torch.randn(4, 512, 32, 32, device=dev)
        r["c2_dense_conv_of_rewrite"] = time_fn(lambda: F.conv2d(x3, w2, None, 1, 1))
        xr, wr = torch.randn(1, 3, 224, 224, device=dev), resnet18_weights(dev)
        r["c3_resnet18"] = time_fn(lambda: resnet18(xr, wr))
        xb = torch.randn(128, 768, device=dev)
        wb = []
        for _ in range(12):
            wb += [torch.randn(768, 768, device=dev) * 0.03 for _ in range(4)] + [torch.randn(768, 3072, device=dev) * 0.03,
                                                                                 torch.randn(3072, 768, device=dev) * 0.03]
        r["c4_bert_base_seq128"] = time_fn(lambda: bert(xb, wb))
        x5, w5 = torch.randn(1, 64, 16, 56, 56, device=dev), torch.randn(64, 64, 3, 3, 3, device=dev) * 0.02
        r["c5_r3d18_conv3d_64ch_16x56x56"] = time_fn(lambda: F.conv3d(x5, w5, None, 1, 1))
        out[mode] = r
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    sys.exit(main())
