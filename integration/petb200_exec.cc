// Reference-side binding, execution half: a tpm::SubGraph walked into petb200_graph and run on the GPU — what
// CodeEngine::genCode + the emitted program do in the reference (ref: src/Graph/code_engine.cc:91-256) — plus the C entry
// points the tests drive (petb200_shim.h).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <iostream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <unordered_set>
#include <vector>
#include <cuda_runtime.h>

// every system header the reference's headers pull in comes first, so that the access hack below only touches the reference
#include <algorithm>
#include <cassert>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <ctime>
#include <cublas_v2.h>
#include <cuda.h>
#include <cudnn.h>
#include <curand.h>
#include <functional>
#include <functional> // hash
#include <initializer_list>
#include <iomanip>
#include <ios>
#include <iostream>
#include <iterator>
#include <list>
#include <map>
#include <memory>
#include <numeric>
#include <optional>
#include <pybind11/embed.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <set>
#include <sstream>
#include <stdlib.h>
#include <string>
#include <time.h>
#include <tuple>
#include <type_traits>
#include <unistd.h>
#include <unordered_map>
#include <unordered_set>
#include <variant>
#include <vector>
#define private public
#define protected public
#include "generator.h"
#include "graph.h"
#include "operator.h"
#include "perf_engine.h"
#include "search_engine.h"
#include "tensor.h"
#undef private
#undef protected

#include "petb200.h"
#include "petb200_graph.h"
#include "petb200_shim.h"

namespace {

using tpm::Operator;
using tpm::Tensor;

// Operators in the order CodeEngine::genCode emits them: reversed DFS post-order over the successor lists
// (ref: src/Graph/code_engine.cc:151-167).
std::vector<Operator *> gencode_order(tpm::SubGraph &sg) {
    std::unordered_set<const Operator *> seen;
    std::vector<Operator *> rev;
    std::function<void(Operator *)> dfs = [&](Operator *op) {
        if (seen.count(op))
            return;
        seen.insert(op);
        for (auto &&next : op->getSuccessors())
            dfs(next);
        rev.emplace_back(op);
    };
    for (auto &&op : sg.getOperators())
        dfs(op);
    return std::vector<Operator *>(rev.rbegin(), rev.rend());
}

struct Walk {
    petb200_graph *g = nullptr;
    std::map<const Tensor *, int> id;
    std::string err;
    ~Walk() {
        if (g)
            petb200_graph_destroy(g);
    }
    int fail(const std::string &m) {
        err = m;
        return PETB200_ERR_UNSUPPORTED;
    }
    int in(const Tensor *t) {
        auto it = id.find(t);
        if (it != id.end())
            return it->second;
        int tid = -1;
        const tpm::Dim &d = t->getDims();
        if (petb200_graph_tensor(g, (int)d.size(), d.data(), t->getType() == Tensor::Weight, &tid) != PETB200_OK)
            return -1;
        id[t] = tid;
        return tid;
    }
    int bias_of(Tensor *b) { return b ? in(b) : -1; }

    int add(Operator *op) {
        const auto &I = op->getInputs();
        const auto &O = op->getOutputs();
        int out = -1, rc = PETB200_OK;
        switch (op->getType()) {
        case Operator::Conv: {
            auto *c = static_cast<tpm::ConvOp *>(op);
            rc = petb200_graph_conv(g, in(I[0]), in(I[1]), bias_of(c->getBias()), c->getPh(), c->getPw(), c->getSh(), c->getSw(), c->getDh(),
                                    c->getDw(), (int)c->getAct(), &out);
            break;
        }
        case Operator::Matmul: {
            auto *m = static_cast<tpm::MatmulOp *>(op);
            rc = petb200_graph_matmul(g, in(I[0]), in(I[1]), bias_of(m->getBias()), m->getTransA(), m->getTransB(), (int)m->getAct(), &out);
            break;
        }
        case Operator::Transpose: {
            petb200_transpose_desc d;
            if (!petb200_shim_fill_transpose_desc(op, &d))
                return fail("transpose with more than 8 flat dims");
            rc = petb200_graph_transpose(g, in(I[0]), &d, &out);
            break;
        }
        case Operator::Add:
        case Operator::Sub:
        case Operator::Mul: {
            std::vector<int> xs;
            for (auto *t : I)
                xs.push_back(in(t));
            rc = petb200_graph_eltwise(g, op->getType() == Operator::Add ? 0 : (op->getType() == Operator::Sub ? 1 : 2), (int)xs.size(), xs.data(), &out);
            break;
        }
        case Operator::Activation:
            rc = petb200_graph_activation(g, in(I[0]), (int)static_cast<tpm::ActivationOp *>(op)->getActType(), &out);
            break;
        case Operator::Pad: {
            auto *p = static_cast<tpm::PadOp *>(op);
            rc = petb200_graph_pad(g, in(I[0]), p->getBegin().data(), p->getEnd().data(), &out);
            break;
        }
        case Operator::Slice: {
            auto *s = static_cast<tpm::SliceOp *>(op);
            rc = petb200_graph_slice(g, in(I[0]), s->begin.data(), s->end.data(), &out);
            break;
        }
        case Operator::Extend: {
            auto *e = static_cast<tpm::ExtendOp *>(op);
            rc = petb200_graph_extend(g, in(I[0]), e->dim, e->num, &out);
            break;
        }
        case Operator::Concat: {
            std::vector<int> xs;
            for (auto *t : I)
                xs.push_back(in(t));
            rc = petb200_graph_concat(g, (int)xs.size(), xs.data(), static_cast<tpm::ConcatOp *>(op)->getDim(), &out);
            break;
        }
        case Operator::Split: {
            auto *s = static_cast<tpm::SplitOp *>(op);
            std::vector<int> outs(O.size(), -1);
            rc = petb200_graph_split(g, in(I[0]), s->getDim(), (int)s->sizes.size(), s->sizes.data(), outs.data());
            if (rc == PETB200_OK)
                for (size_t i = 0; i < O.size(); ++i)
                    id[O[i]] = outs[i];
            return rc;
        }
        case Operator::MaxPool: {
            auto *p = static_cast<tpm::MaxPoolOp *>(op);
            rc = petb200_graph_pool(g, 0, in(I[0]), p->kh, p->kw, p->ph, p->pw, p->sh, p->sw, &out);
            break;
        }
        case Operator::AvgPool: {
            auto *p = static_cast<tpm::AvgPoolOp *>(op);
            rc = petb200_graph_pool(g, 1, in(I[0]), p->kh, p->kw, p->ph, p->pw, p->sh, p->sw, &out);
            break;
        }
        case Operator::Softmax:
            rc = petb200_graph_softmax(g, in(I[0]), static_cast<tpm::SoftmaxOp *>(op)->getAxis(), &out);
            break;
        case Operator::Reshape:
        case Operator::Identity: {
            const tpm::Dim &d = O[0]->getDims();
            rc = petb200_graph_reshape(g, in(I[0]), (int)d.size(), d.data(), &out);
            break;
        }
        default:
            return fail("operator " + Operator::getOpName(op->getType()) + " has no lowering in this walker");
        }
        if (rc != PETB200_OK) {
            err = petb200_graph_last_error(g);
            return rc;
        }
        id[O[0]] = out;
        return PETB200_OK;
    }
};

// Lowers `sg`, loads `data` (reference tensor hash -> host floats) into the tensors nothing in the graph produces, runs
// one pass and reads tensor `result` back.
int run_subgraph(tpm::SubGraph &sg, const std::map<uint64_t, const float *> &data, const Tensor *result, float *y, std::string &err) {
    petb200_ctx *ctx = petb200_shim_ctx();
    if (!ctx) {
        err = "no backend context";
        return PETB200_ERR_CUDA;
    }
    Walk w;
    int rc = petb200_graph_create(ctx, &w.g);
    if (rc)
        return rc;
    for (Operator *op : gencode_order(sg))
        if ((rc = w.add(op)) != PETB200_OK) {
            err = w.err;
            return rc;
        }
    const int out_id = w.id.at(result);
    if ((rc = petb200_graph_set_outputs(w.g, 1, &out_id)) != PETB200_OK || (rc = petb200_graph_compile(w.g, 0)) != PETB200_OK) {
        err = petb200_graph_last_error(w.g);
        return rc;
    }
    for (auto &kv : w.id) {
        const Tensor *t = kv.first;
        if (const_cast<Tensor *>(t)->getOutputOf() != nullptr && data.find(t->getHash()) == data.end())
            continue;
        auto it = data.find(t->getHash());
        if (it == data.end())
            continue;
        if ((rc = petb200_graph_set_data(w.g, kv.second, it->second, t->size(), nullptr)) != PETB200_OK) {
            err = petb200_graph_last_error(w.g);
            return rc;
        }
    }
    cudaDeviceSynchronize();
    if ((rc = petb200_graph_run(w.g, nullptr)) != PETB200_OK || (rc = petb200_graph_get_data(w.g, out_id, y, result->size(), nullptr)) != PETB200_OK) {
        err = petb200_graph_last_error(w.g);
        return rc;
    }
    cudaDeviceSynchronize();
    return petb200_check_device_status(ctx, nullptr);
}

} // namespace

extern "C" int petb200_pet_perf_probe(double out_ms[4]) {
    const long before = petb200_shim_perf_calls();
    auto g = std::make_unique<tpm::Graph>();
    auto x = g->tensor({1, 8, 8, 8});
    auto w = g->tensor({8, 8, 3, 3});
    std::vector<Operator *> ops;
    ops.push_back(g->conv(x, w, 1, 1));
    auto a = g->tensor({1, 16, 32}), b = g->tensor({1, 32, 16});
    ops.push_back(g->matmul(a, b));
    ops.push_back(g->transpose(x, 2, {{0, 2}, 1, -1, 3}, -2));
    ops.push_back(g->maxpool(x, 2, 2, 1, 1, 0, 0, 2, 2));
    for (size_t i = 0; i < ops.size(); ++i)
        out_ms[i] = ops[i]->perf(nullptr, 1, 0); // through the vtable of the reference's classes
    return (int)(petb200_shim_perf_calls() - before);
}

extern "C" int petb200_pet_search_conv(const int conv[11], const float *x, const float *w, float *y, float *y_direct, char *report,
                                       size_t report_len, double perf_ms[2]) {
    const int n = conv[0], c = conv[1], h = conv[2], wd = conv[3], f = conv[4], r = conv[5], s = conv[6];
    auto g = std::make_unique<tpm::Graph>();
    auto i0 = g->tensor({n, c, h, wd});
    auto w0 = g->tensor({f, c, r, s});
    g->conv(i0, w0, conv[7], conv[8], 1, 1, conv[9], conv[10]);
    g->updateConnection();
    std::shared_ptr<tpm::SubGraph> graph = std::make_shared<tpm::SubGraph>(g->getOperators()), best;
    // SubGraph clones tensors but keeps their hashes (ref: src/Graph/graph.cc:692-734): data is keyed by hash
    std::map<uint64_t, const float *> data;
    data[i0->getHash()] = x;
    data[w0->getHash()] = w;
    std::string err;
    int rc;
    if (y_direct) {
        const Tensor *out = graph->getOutputs()[0];
        if ((rc = run_subgraph(*graph, data, out, y_direct, err)) != PETB200_OK) {
            snprintf(report, report_len, "original graph failed: %s", err.c_str());
            return rc;
        }
    }
    tpm::SearchEngine engine(std::make_shared<tpm::Generator>());
    if (engine.run(graph, best) != 0 || !best) {
        snprintf(report, report_len, "SearchEngine::run failed");
        return PETB200_ERR_INVALID;
    }
    perf_ms[0] = engine.getPerf(graph, false, false);
    perf_ms[1] = engine.getPerf(best, false, false);
    std::ostringstream os;
    for (Operator *op : gencode_order(*best))
        os << op->toString() << "\n";
    snprintf(report, report_len, "%s", os.str().c_str());
    if (best->getOutputs().size() != 1) {
        snprintf(report, report_len, "chosen graph has %zu outputs", best->getOutputs().size());
        return PETB200_ERR_INVALID;
    }
    if ((rc = run_subgraph(*best, data, best->getOutputs()[0], y, err)) != PETB200_OK) {
        std::string text = os.str() + "execution failed: " + err;
        snprintf(report, report_len, "%s", text.c_str());
    }
    return rc;
}

extern "C" int petb200_pet_run_h2n_rewrite(const int conv[11], const float *x, const float *w, float *y_gpu, unsigned *y_host, char *report,
                                           size_t report_len) {
    const int n = conv[0], c = conv[1], h = conv[2], wd = conv[3], f = conv[4], r = conv[5], s = conv[6];
    auto g = std::make_unique<tpm::Graph>();
    auto i0 = g->tensor({n, c, h, wd});
    auto w0 = g->tensor({f, c, r, s});
    // the mutant PET's generator derives for this operator (ref: src/Mutant/generator.cc:1027-1046): H -> N, conv, N -> H
    auto t1 = g->transpose(i0, 2, {{0, 2}, 1, -1, 3}, -2)->getOutputs()[0];
    auto t2 = g->conv(t1, w0, conv[7], conv[8], 1, 1, conv[9], conv[10])->getOutputs()[0];
    g->transpose(t2, 0, {0, 1, {-1, 2}, 3}, 2);
    g->updateConnection();
    auto sg = std::make_shared<tpm::SubGraph>(g->getOperators());
    if (sg->getOutputs().size() != 1) {
        snprintf(report, report_len, "rewrite graph has %zu outputs", sg->getOutputs().size());
        return PETB200_ERR_INVALID;
    }
    std::ostringstream os;
    for (Operator *op : gencode_order(*sg))
        os << op->toString() << "\n";
    snprintf(report, report_len, "%s", os.str().c_str());
    // the reference's own host evaluation of the same graph (uint32 arithmetic; ref: src/Graph/graph.cc:1353-1386)
    for (auto t : sg->getTensors())
        t->dataMalloc();
    for (auto t : sg->getInputs()) {
        const float *src = t->getHash() == i0->getHash() ? x : (t->getHash() == w0->getHash() ? w : nullptr);
        if (!src)
            return PETB200_ERR_INVALID;
        for (size_t i = 0; i < t->size(); ++i)
            t->setData(i, (tpm::VType)(long long)src[i]);
    }
    if (!sg->compute())
        return PETB200_ERR_INVALID;
    Tensor *out = sg->getOutputs()[0];
    for (size_t i = 0; i < out->size(); ++i)
        y_host[i] = out->getData(i);
    std::map<uint64_t, const float *> data;
    data[i0->getHash()] = x;
    data[w0->getHash()] = w;
    std::string err;
    const int rc = run_subgraph(*sg, data, out, y_gpu, err);
    if (rc != PETB200_OK) {
        std::string text = os.str() + "execution failed: " + err;
        snprintf(report, report_len, "%s", text.c_str());
    }
    return rc;
}
