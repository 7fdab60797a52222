// TEST INFRASTRUCTURE ONLY.  C-ABI wrapper around the reference's own host operators (namespace tpm),
// compiled against the reference headers and linked with the reference's unmodified sources into
// oracle/_ref/libpetref.so.  It lets the Python tests and the fixture generator drive
//   tpm::Graph::{conv,matmul,transpose,pad,slice,concat,split,extend,add,sub,mul,batchnorm}  (include/graph.h:38-190)
// and read back what  Operator::compute()  (src/Graph/operator.cc) produced.  The reference evaluates on
// VType = uint32_t (include/common.h:137); copy-type operators only move words, so float tensors are passed
// through as their bit patterns and come back bit-exact.
//
// Every function returns 0 on success, a negative value when the reference rejected the operator.
#include "graph.h"
#include "operator.h"
#include "tensor.h"
#include "transpose.h"
#include <chrono>
#include <cstring>
#include <omp.h>

namespace tpm {
// The banded-attention launchers live in src/custom_ops.cu (TVM output, GPU only).  They are referenced from
// the timing bodies in operator.cc but never reached from host evaluation; stubs keep the link closed
// without compiling 5.8k lines of generated kernels.
void _sg2bmm(float *, float *, float *, int, int, int, int, int) {}
void _sgbmml(float *, float *, float *, int, int, int, int, int) {}
} // namespace tpm

using namespace tpm;

namespace {
Dim mkdim(const int *d, int n) { return Dim(d, d + n); }

Tensor *feed(Graph &g, const uint32_t *data, const int *dims, int nd, bool weight = false) {
    Tensor *t = g.tensor(mkdim(dims, nd));
    if (weight)
        t->setType(Tensor::Weight);
    t->dataMalloc();
    t->setData(const_cast<uint32_t *>(data));
    return t;
}

int fetch(Tensor *t, uint32_t *out, int *out_nd, int *out_dims) {
    if (t == nullptr || t->getDataPtr() == nullptr)
        return -2;
    const Dim &d = t->getDims();
    if (out_nd)
        *out_nd = (int)d.size();
    if (out_dims)
        for (size_t i = 0; i < d.size(); ++i)
            out_dims[i] = d[i];
    if (out)
        std::memcpy(out, t->getDataPtr(), t->size() * sizeof(uint32_t));
    return 0;
}

Perm mkperm(int ngroups, const int *group_sizes, const int *flat) {
    std::vector<PermItem> items;
    int p = 0;
    for (int i = 0; i < ngroups; ++i) {
        std::vector<int> v(flat + p, flat + p + group_sizes[i]);
        p += group_sizes[i];
        items.emplace_back(PermItem(v));
    }
    return Perm(items);
}
} // namespace

extern "C" {

int petref_num_threads() { return omp_get_max_threads(); }

// TransposeOp(input, split, after, factor)  — include/operator.h:1154-1159, host body operator.cc:2172-2210.
// `flat`/`group_sizes` describe `after`: group i holds group_sizes[i] indices (index -1 = second half of the split dim).
int petref_transpose(const uint32_t *in, int nd, const int *dims, int split, int ngroups,
                     const int *group_sizes, const int *flat, int factor, uint32_t *out, int *out_nd,
                     int *out_dims) {
    Graph g;
    Tensor *x = feed(g, in, dims, nd);
    Operator *op = g.transpose(x, split, mkperm(ngroups, group_sizes, flat), factor);
    Tensor *y = op->getOutputs()[0];
    if (!y->isValid())
        return -1;
    if (op->compute() == nullptr)
        return -1;
    return fetch(y, out, out_nd, out_dims);
}

// ConvOp — include/operator.h:264-372, host body operator.cc:94-158, shape :208-237.  Returns seconds spent in
// compute() through *secs when it is not null.
int petref_conv(const uint32_t *x, const int *xd, const uint32_t *w, const int *wd, int ph, int pw, int sh,
                int sw, int dh, int dw, uint32_t *y, int *yd, double *secs) {
    Graph g;
    Tensor *tx = feed(g, x, xd, 4);
    Tensor *tw = feed(g, w, wd, 4, true);
    Operator *op = g.conv(tx, tw, ph, pw, sh, sw, dh, dw);
    auto t0 = std::chrono::steady_clock::now();
    if (op->compute() == nullptr)
        return -1;
    auto t1 = std::chrono::steady_clock::now();
    if (secs)
        *secs = std::chrono::duration<double>(t1 - t0).count();
    int nd;
    return fetch(op->getOutputs()[0], y, &nd, yd);
}

// MatmulOp — include/operator.h:374-464, host body operator.cc:620-654.  3-D operands [b,m,k] x [b,k,n].
int petref_matmul(const uint32_t *a, const int *ad, const uint32_t *b, const int *bd, int transA, int transB,
                  uint32_t *c, int *cd, double *secs) {
    Graph g;
    Tensor *ta = feed(g, a, ad, 3);
    Tensor *tb = feed(g, b, bd, 3);
    Operator *op = g.matmul(ta, tb, (bool)transA, (bool)transB);
    auto t0 = std::chrono::steady_clock::now();
    if (op->compute() == nullptr)
        return -1;
    auto t1 = std::chrono::steady_clock::now();
    if (secs)
        *secs = std::chrono::duration<double>(t1 - t0).count();
    int nd;
    return fetch(op->getOutputs()[0], c, &nd, cd);
}

// PadOp — operator.h:781-816, operator.cc:1640-1662.
int petref_pad(const uint32_t *in, int nd, const int *dims, const int *begin, const int *end, uint32_t *out,
               int *out_dims) {
    Graph g;
    Tensor *x = feed(g, in, dims, nd);
    Operator *op = g.pad(x, mkdim(begin, nd), mkdim(end, nd));
    op->getOutputs()[0]->dataMalloc();
    if (op->compute() == nullptr)
        return -1;
    int n;
    return fetch(op->getOutputs()[0], out, &n, out_dims);
}

// SliceOp — operator.h:819-854, operator.cc:1741-1773.
int petref_slice(const uint32_t *in, int nd, const int *dims, const int *begin, const int *end, uint32_t *out,
                 int *out_dims) {
    Graph g;
    Tensor *x = feed(g, in, dims, nd);
    Operator *op = g.slice(x, mkdim(begin, nd), mkdim(end, nd));
    op->getOutputs()[0]->dataMalloc();
    if (op->compute() == nullptr)
        return -1;
    int n;
    return fetch(op->getOutputs()[0], out, &n, out_dims);
}

// ExtendOp — operator.h:1204-1255, operator.cc:2577-2597.
int petref_extend(const uint32_t *in, int nd, const int *dims, int dim, int num, uint32_t *out, int *out_dims) {
    Graph g;
    Tensor *x = feed(g, in, dims, nd);
    Operator *op = g.extend(x, dim, num);
    if (op->compute() == nullptr)
        return -1;
    int n;
    return fetch(op->getOutputs()[0], out, &n, out_dims);
}

// ConcatOp — operator.h:856-934, operator.cc:1813-1850.  dims is [n_in][nd] row-major.
int petref_concat(int n_in, const uint32_t *const *ins, int nd, const int *dims, int dim, uint32_t *out,
                  int *out_dims) {
    Graph g;
    TensorVec tv;
    for (int i = 0; i < n_in; ++i)
        tv.emplace_back(feed(g, ins[i], dims + i * nd, nd));
    Operator *op = g.concat(tv, dim);
    if (op->compute() == nullptr)
        return -1;
    int n;
    return fetch(op->getOutputs()[0], out, &n, out_dims);
}

// SplitOp with ratio sizes — operator.h:936-1030, operator.cc:1978-2020, shapes :2074-2101.
// out_dims is [n_out][nd] row-major; outs[i] may be null to query shapes only.
int petref_split(const uint32_t *in, int nd, const int *dims, int dim, int n_out, const int *sizes,
                 uint32_t *const *outs, int *out_dims) {
    Graph g;
    Tensor *x = feed(g, in, dims, nd);
    Operator *op = g.split(x, dim, std::vector<int>(sizes, sizes + n_out));
    for (auto t : op->getOutputs())
        if (!t->isValid())
            return -1;
    auto res = static_cast<SplitOp *>(op)->computeV();
    if ((int)res.size() != n_out)
        return -1;
    for (int i = 0; i < n_out; ++i) {
        int n;
        if (fetch(res[i], outs ? outs[i] : nullptr, &n, out_dims + i * nd))
            return -2;
    }
    return 0;
}

// AddOp / SubOp / MulOp with the reference's `i % size` broadcast — operator.cc:2983-3002 and neighbours.
// kind: 0 add, 1 sub, 2 mul.
int petref_eltwise(int kind, int n_in, const uint32_t *const *ins, const int *nds, const int *dims_flat,
                   uint32_t *out) {
    Graph g;
    TensorVec tv;
    int p = 0;
    for (int i = 0; i < n_in; ++i) {
        tv.emplace_back(feed(g, ins[i], dims_flat + p, nds[i]));
        p += nds[i];
    }
    Operator *op = nullptr;
    if (kind == 0)
        op = g.add(tv);
    else if (kind == 1)
        op = g.sub(tv[0], tv[1]);
    else if (kind == 2)
        op = g.mul(tv);
    else
        return -3;
    if (op->compute() == nullptr)
        return -1;
    int n;
    int od[8];
    return fetch(op->getOutputs()[0], out, &n, od);
}

// Whole-graph host evaluation of the dilated-conv rewrite the throughput benchmark times:
//   D2H -> H2N -> D2W -> W2N -> conv(pad 1, dilation 1) -> N2W -> D2W^-1 -> N2H -> D2H^-1
// built with the reference's graph API and evaluated operator by operator exactly as SubGraph::compute does
// (src/Graph/graph.cc:1355-1386).  `f_sample` output channels are evaluated (the weight tensor passed in has
// f_sample filters); seconds for the whole chain are returned through *secs.
int petref_dilated_rewrite(const uint32_t *x, const int *xd, const uint32_t *w, const int *wd, uint32_t *y,
                           int *yd, double *secs) {
    Graph g;
    Tensor *t = feed(g, x, xd, 4);
    Tensor *tw = feed(g, w, wd, 4, true);
    auto t0 = std::chrono::steady_clock::now();
    auto step = [&](Operator *op) -> Tensor * {
        if (op->compute() == nullptr)
            return nullptr;
        return op->getOutputs()[0];
    };
    // forward space-to-batch (generator.cc:1027-1046 and :1085-1092 give these constructor arguments)
    if (!(t = step(g.transpose(t, 2, Perm({0, 1, PermItem({-1, 2}), 3}), 2))))
        return -1; // D2H
    if (!(t = step(g.transpose(t, 2, Perm({PermItem({0, 2}), 1, -1, 3}), -2))))
        return -1; // H2N
    if (!(t = step(g.transpose(t, 3, Perm({0, 1, 2, PermItem({-1, 3})}), 2))))
        return -1; // D2W
    if (!(t = step(g.transpose(t, 3, Perm({PermItem({0, 3}), 1, 2, -1}), -2))))
        return -1; // W2N
    if (!(t = step(g.conv(t, tw, 1, 1, 1, 1, 1, 1))))
        return -1;
    if (!(t = step(g.transpose(t, 0, Perm({0, 1, 2, PermItem({-1, 3})}), 2))))
        return -1; // N2W
    if (!(t = step(g.transpose(t, 3, Perm({0, 1, 2, PermItem({-1, 3})}), -2))))
        return -1; // D2W inverse
    if (!(t = step(g.transpose(t, 0, Perm({0, 1, PermItem({-1, 2}), 3}), 2))))
        return -1; // N2H
    if (!(t = step(g.transpose(t, 2, Perm({0, 1, PermItem({-1, 2}), 3}), -2))))
        return -1; // D2H inverse
    auto t1 = std::chrono::steady_clock::now();
    if (secs)
        *secs = std::chrono::duration<double>(t1 - t0).count();
    int nd;
    return fetch(t, y, &nd, yd);
}

// ConvTransOp — include/operator.h:466-614.  x {n,h,w,f}, w {r,s,f,c}, y {n,oh,ow,c}.  whole = 1 runs the reference's
// whole-tensor body (operator.cc:931-983; it takes its row/column loop bounds from output dims 2 and 3, so it only
// fills the tensor when oh == ow == c); whole = 0 runs the reference's one-position body (operator.cc:1006-1040)
// at every output position.
int petref_convtrans(const uint32_t *x, const int *xd, const uint32_t *w, const int *wd, int ph, int pw, int sh, int sw,
                     int dh, int dw, int oph, int opw, int whole, uint32_t *y, int *yd) {
    Graph g;
    Tensor *tx = feed(g, x, xd, 4);
    Tensor *tw = feed(g, w, wd, 4, true);
    auto *op = new ConvTransOp(tx, tw, ph, pw, sh, sw, dh, dw, oph, opw);
    Tensor *out = op->getOutputs()[0];
    if (whole) {
        if (op->compute() == nullptr)
            return -1;
    } else {
        const Dim od = out->getDims();
        for (int a = 0; a < od[0]; ++a)
            for (int b = 0; b < od[1]; ++b)
                for (int c = 0; c < od[2]; ++c)
                    for (int d = 0; d < od[3]; ++d) {
                        auto pr = op->compute(DimRange(Dim{a, b, c, d}));
                        if (!pr.second || !pr.second())
                            return -1;
                    }
    }
    int nd;
    return fetch(out, y, &nd, yd);
}

// The index expression the reference generates for a TransposeOp with padding / halo parameters: builds the operator,
// marks it the way markTransType would (type, Pre/Post position, padding sizes — include/operator.h:1180-1190), takes
// its micro-operations from TransposeOp::getTTParam (src/Graph/operator.cc:2403-2441) and asks TransposeEngine::getLambda
// (src/Transpose/transpose.cc:185-214) for the Python lambda that CodeEngine hands to TVM (src/Graph/code_engine.cc:27-84).
// Also returns the output dims the micro-operations produce.  type: 1 N2H, 2 N2W, 3 H2N, 4 W2N, 7 D2H, 8 D2W; pos: 1 Pre, 2 Post.
int petref_transpose_lambda(int nd, const int *dims, int split, int ngroups, const int *group_sizes, const int *flat,
                            int factor, int type, int pos, int pad_h, int pad_w, char *buf, int buflen, int *out_nd,
                            int *out_dims) {
    Graph g;
    Tensor *x = g.tensor(mkdim(dims, nd));
    auto *op = dynamic_cast<TransposeOp *>(g.transpose(x, split, mkperm(ngroups, group_sizes, flat), factor));
    if (op == nullptr)
        return -1;
    op->setType((TransposeOp::TransType)type);
    op->setPos((TransposeOp::TransPos)pos);
    op->setPaddingSize(pad_h, pad_w);
    auto micro = op->getTTParam();
    std::vector<TransBasic *> raw;
    for (auto &m : micro)
        raw.push_back(m.get());
    std::vector<int> in(dims, dims + nd);
    std::string lam = TransposeEngine::getInstance().getLambda(raw, in);
    if ((int)lam.size() + 1 > buflen)
        return -3;
    std::memcpy(buf, lam.c_str(), lam.size() + 1);
    std::vector<std::string> vars;
    for (int i = 0; i < nd; ++i)
        vars.push_back(std::string(1, (char)('a' + i)));
    DecisionTree *tree = new DecisionTree(vars);
    std::vector<int> od = in;
    for (auto *m : raw)
        tree = m->putTranspose(tree, od);
    *out_nd = (int)od.size();
    for (size_t i = 0; i < od.size(); ++i)
        out_dims[i] = od[i];
    return 0;
}

} // extern "C"
