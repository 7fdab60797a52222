// Host side above the operator C ABI: a graph of tensors and operators built with the reference's builder
// vocabulary, an executor that plays the role of CodeEngine (order, fuse, plan, replay under a CUDA graph) and a
// timing table that plays the role of PerfEngine (memoised per-operator milliseconds).  Everything here goes
// through the functions declared in include/petb200.h; there is no other way into the kernels.
#include "../../include/petb200_graph.h"
#include <algorithm>
#include <cstdarg>
#include <cstring>
#include <cuda_runtime.h>
#include <map>
#include <memory>
#include <string>
#include <tuple>
#include <vector>

namespace {

using Dim = std::vector<int>;

// OpType values follow the reference's enum names (ref: include/operator.h:19-51) for the operators that exist there.
enum OpType { Conv, Matmul, Transpose, Pad, Slice, Concat, Split, Extend, Add, Sub, Mul, Activation, MaxPool, AvgPool,
              Softmax, BatchNorm, Reshape, Conv3d, LayerNorm, Correction, ConvTrans, G2BMM, GBMML, Div, Pow, ReduceMean, Gather,
              Attention /* a step only: Matmul(transB) -> Softmax -> Matmul fused by the executor */ };

struct Tensor {
    Dim dims;
    bool weight = false;
    int outputOf = -1;           // operator id, -1 for graph inputs
    std::vector<int> inputOf;    // consumers
    int alias = -1;              // tensor whose storage this one shares (reshape, correction, merged matmul outputs)
    long long view_off = 0;      // element offset inside the aliased tensor
    int pitch = 0;               // > 0: rows of `inner` contiguous elements, `pitch` elements apart (a column slice of a
    int inner = 0;               //      wider matrix); only operand-stride folding understands such tensors
    float *dev = nullptr;
    bool owns = false;
    bool has_data = false;
    size_t size() const {
        size_t n = 1;
        for (int d : dims)
            n *= (size_t)d;
        return n;
    }
};

struct Operator {
    OpType type;
    std::vector<int> inputs, outputs;
    // attributes (a flat bag; which are used depends on type)
    int ph = 0, pw = 0, sh = 1, sw = 1, dh = 1, dw = 1, act = 0, bias = -1;
    int pad3[3] = {0, 0, 0}, stride3[3] = {1, 1, 1}, dil3[3] = {1, 1, 1};
    int transA = 0, transB = 0;
    petb200_transpose_desc tr{};
    Dim begin, end;
    int dim = 0, num = 0, axis = 0;
    Dim sizes;
    int kh = 0, kw = 0;
    float eps = 1e-5f;
    int win[4] = {0, 0, 0, 0};
    int oph = 0, opw = 0;         // ConvTrans output padding
    int halo[4] = {0, 0, 0, 0};   // Transpose: pad, extr, copys, dels (TransposeOp::getTTParam), all 0 for a plain transpose
    int width = 0, dilation = 1;  // G2BMM / GBMML band half-width and key step
    bool fused_away = false; // absorbed into another step
    // Matmul whose operands/result are strided views of other tensors (folded batch-swap transposes):
    bool mm_strided = false;
    long long mm_strides[6] = {0, 0, 0, 0, 0, 0};
    int mm_in[2] = {-1, -1}; // tensor read in place of inputs[i], or -1
    int mm_out_op = -1;      // transpose after the matmul whose output the matmul writes directly, or -1
    // Leader of a group of matmuls that share their A operand and were merged into one (weights side by side along N):
    std::vector<int> merged_w, merged_b; // the members' weight / bias tensors, in column order
    int merged_out = -1, merged_wt = -1, merged_bias = -1; // the wide result, weight and bias tensors of the merged matmul
    // Conv between a Pre/Post pair of seam transposes (H->N before, N->H after; or the W pair), folded into the conv itself:
    // the conv reads `seam_in` (the pair's input, in the original layout) and writes the output of operator `seam_out_op`
    // (the second transpose), both through reshaped views; 'H' or 'W', 0 = not folded.
    char seam_axis = 0;
    int seam_in = -1, seam_out_op = -1;
};

// One executable step after fusion.
struct Step {
    std::string name;
    std::vector<int> ops;      // operator ids it covers
    petb200_plan *plan = nullptr;
    const char *kernel = "";
    OpType type;
    int launches = 1;
    bool weight_only = false;  // consumes only weights: hoisted out of the replayed sequence
    int residual = -1;         // conv/matmul: tensor added in the epilogue (a folded residual Add), or -1
    // A step whose result is read only as another step's residual (the shortcut convolution of a ResNet block) runs on a
    // second stream beside the steps between it and that reader:
    bool side = false;
    int join_from = -1;        // index of the side step this step has to wait for, or -1
    // Attention step: extents {bs, m, n, kd, d}, the tensors read as q, k, v and written, their batch / row strides
    int att_dims[5] = {0, 0, 0, 0, 0}, att_t[4] = {-1, -1, -1, -1};
    long long att_st[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
};

// PerfEngine's memo tables (ref: include/perf_engine.h:15-21): argument tuple -> milliseconds.
struct PerfEngine {
    std::map<std::vector<int>, float> table;
    bool check(const std::vector<int> &k) const { return table.count(k) != 0; }
    float get(const std::vector<int> &k) const { return table.at(k); }
    void save(const std::vector<int> &k, float ms) { table[k] = ms; }
};

} // namespace

struct petb200_graph {
    petb200_ctx *ctx = nullptr;
    std::vector<Tensor> tensors;
    std::vector<Operator> ops;
    std::vector<int> outputs;
    std::vector<Step> steps;
    std::vector<int> hoisted; // indices of weight-only steps
    bool compiled = false;
    cudaGraphExec_t exec = nullptr;
    cudaStream_t cap_stream = nullptr;
    cudaStream_t side_stream = nullptr; // side-branch steps (see Step::side)
    bool use_graph = true;
    bool hoisted_done = false;
    PerfEngine perf;
    std::string err;
    // petb200_graph_run_profiled: per slot, one event pair around every replayed step that is not a tensor-core launch
    std::vector<cudaEvent_t> prof_events;
    std::vector<char> prof_recorded; // per slot: run since the last read
    int prof_slots = 0, prof_pairs = 0;

    int fail(int status, const char *fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        err = buf;
        return status;
    }
    int pass(int rc) { // propagate an operator-ABI error text
        if (rc)
            err = petb200_last_error(ctx);
        return rc;
    }
    bool valid_tensor(int t) const { return t >= 0 && t < (int)tensors.size(); }
    int root(int t) const {
        while (tensors[t].alias >= 0)
            t = tensors[t].alias;
        return t;
    }
    int new_tensor(const Dim &d, bool weight = false) {
        Tensor t;
        t.dims = d;
        t.weight = weight;
        tensors.push_back(t);
        return (int)tensors.size() - 1;
    }
    int add_op(Operator &&op) {
        int id = (int)ops.size();
        for (int t : op.inputs)
            tensors[t].inputOf.push_back(id);
        for (int t : op.outputs)
            tensors[t].outputOf = id;
        ops.push_back(std::move(op));
        compiled = false;
        return id;
    }
    ~petb200_graph() {
        for (cudaEvent_t e : prof_events)
            cudaEventDestroy(e);
        for (auto &s : steps)
            if (s.plan)
                petb200_plan_destroy(s.plan);
        for (auto &t : tensors)
            if (t.owns && t.dev)
                cudaFree(t.dev);
        if (exec)
            cudaGraphExecDestroy(exec);
        if (cap_stream)
            cudaStreamDestroy(cap_stream);
        if (side_stream)
            cudaStreamDestroy(side_stream);
        for (auto &s : steps) {
            if (s.ev_fork)
                cudaEventDestroy(s.ev_fork);
            if (s.ev_join)
                cudaEventDestroy(s.ev_join);
        }
    }

    int run_step(Step &s, cudaStream_t st);
    int run_all(cudaStream_t st, bool include_hoisted, int prof_slot = -1);
    int compile(int flags);
    int capture();
};

static float *dev_of(petb200_graph *g, int t) {
    if (t < 0)
        return nullptr;
    long long off = 0;
    while (g->tensors[t].alias >= 0) {
        off += g->tensors[t].view_off;
        t = g->tensors[t].alias;
    }
    return g->tensors[t].dev ? g->tensors[t].dev + off : nullptr;
}

int petb200_graph::run_step(Step &s, cudaStream_t st) {
    Operator &op = ops[s.ops.front()];
    switch (s.type) {
    case Conv:
    case Conv3d:
        return pass(petb200_conv_run_residual(s.plan, dev_of(this, op.seam_axis ? op.seam_in : op.inputs[0]), dev_of(this, op.bias),
                                              dev_of(this, s.residual), dev_of(this, ops[s.ops.back()].outputs[0]), st));
    case ConvTrans:
        return pass(petb200_convtrans_run(s.plan, dev_of(this, op.inputs[0]), dev_of(this, op.bias), dev_of(this, op.outputs[0]), st));
    case G2BMM:
    case GBMML: {
        const Dim &b = tensors[op.inputs[1]].dims; // [bs, n, m]
        auto fn = s.type == G2BMM ? petb200_g2bmm_run : petb200_gbmml_run;
        return pass(fn(ctx, dev_of(this, op.inputs[0]), dev_of(this, op.inputs[1]), dev_of(this, op.outputs[0]), b[0], b[1], b[2], op.width,
                       op.dilation, st));
    }
    case Div:
        return pass(petb200_div_run(ctx, dev_of(this, op.inputs[0]), tensors[op.inputs[0]].size(), dev_of(this, op.inputs[1]),
                                    tensors[op.inputs[1]].size(), dev_of(this, op.outputs[0]), tensors[op.outputs[0]].size(), st));
    case Pow:
        return pass(petb200_pow_run(ctx, dev_of(this, op.inputs[0]), dev_of(this, op.outputs[0]), tensors[op.outputs[0]].size(), op.num, st));
    case ReduceMean:
    case Gather: {
        const Dim &d = tensors[op.inputs[0]].dims;
        size_t outer = 1, inner = 1;
        for (int i = 0; i < op.axis; ++i)
            outer *= (size_t)d[i];
        for (size_t i = op.axis + 1; i < d.size(); ++i)
            inner *= (size_t)d[i];
        if (s.type == ReduceMean)
            return pass(petb200_reducemean_run(ctx, dev_of(this, op.inputs[0]), dev_of(this, op.outputs[0]), outer, d[op.axis], inner, st));
        return pass(petb200_gather_run(ctx, dev_of(this, op.inputs[0]), reinterpret_cast<const int *>(dev_of(this, op.inputs[1])),
                                       dev_of(this, op.outputs[0]), tensors[op.inputs[1]].size(), outer, d[op.axis], inner, st));
    }
    case Correction:
        return pass(petb200_conv2d_correct(s.plan, dev_of(this, op.inputs[0]), dev_of(this, op.bias), dev_of(this, op.outputs[0]),
                                           op.win[0], op.win[1], op.win[2], op.win[3], st));
    case Matmul: {
        const bool wb = tensors[op.inputs[1]].weight;
        const int ta = op.mm_in[0] >= 0 ? op.mm_in[0] : op.inputs[0], tb = op.mm_in[1] >= 0 ? op.mm_in[1] : op.inputs[1];
        if (op.merged_out >= 0) // merged siblings: one wide matmul on the side-by-side weights
            return pass(petb200_matmul_run_residual(s.plan, dev_of(this, ta), nullptr, dev_of(this, op.merged_bias), nullptr,
                                                    dev_of(this, op.merged_out), st));
        return pass(petb200_matmul_run_residual(s.plan, dev_of(this, ta), wb ? nullptr : dev_of(this, tb),
                                                dev_of(this, op.bias), dev_of(this, s.residual), dev_of(this, ops[s.ops.back()].outputs[0]), st));
    }
    case Transpose:
    case Pad:
    case Slice:
    case Extend:
        return pass(petb200_layout_run(s.plan, dev_of(this, op.inputs[0]), dev_of(this, ops[s.ops.back()].outputs[0]), st));
    case Concat: {
        const Tensor &o = tensors[op.outputs[0]];
        std::vector<const void *> parts;
        std::vector<int> ext;
        for (int t : op.inputs) {
            parts.push_back(dev_of(this, t));
            ext.push_back(tensors[t].dims[op.dim]);
        }
        return pass(petb200_concat_run(ctx, (int)o.dims.size(), o.dims.data(), op.dim, (int)parts.size(), ext.data(), parts.data(),
                                       dev_of(this, op.outputs[0]), st));
    }
    case Split: {
        const Tensor &in = tensors[op.inputs[0]];
        std::vector<void *> parts;
        std::vector<int> ext;
        for (int t : op.outputs) {
            parts.push_back(dev_of(this, t));
            ext.push_back(tensors[t].dims[op.dim]);
        }
        return pass(petb200_split_run(ctx, (int)in.dims.size(), in.dims.data(), op.dim, (int)parts.size(), ext.data(),
                                      dev_of(this, op.inputs[0]), parts.data(), st));
    }
    case Add:
    case Sub:
    case Mul: {
        std::vector<const float *> ins;
        std::vector<size_t> sz;
        for (int t : op.inputs) {
            ins.push_back(dev_of(this, t));
            sz.push_back(tensors[t].size());
        }
        const int out = ops[s.ops.back()].outputs[0];
        const int act = s.ops.size() > 1 ? ops[s.ops.back()].act : 0;
        return pass(petb200_eltwise_run(ctx, s.type == Add ? 0 : (s.type == Sub ? 1 : 2), (int)ins.size(), ins.data(), sz.data(),
                                        dev_of(this, out), tensors[out].size(), act, st));
    }
    case Activation:
        return pass(petb200_activation_run(ctx, dev_of(this, op.inputs[0]), dev_of(this, op.outputs[0]), tensors[op.outputs[0]].size(), op.act, st));
    case MaxPool:
    case AvgPool: {
        const Dim &d = tensors[op.inputs[0]].dims;
        return pass(petb200_pool2d_run(ctx, s.type == MaxPool ? 0 : 1, dev_of(this, op.inputs[0]), dev_of(this, op.outputs[0]), d[0], d[1], d[2],
                                       d[3], op.kh, op.kw, op.ph, op.pw, op.sh, op.sw, st));
    }
    case Softmax: {
        const Dim &d = tensors[op.inputs[0]].dims;
        size_t outer = 1, inner = 1;
        for (int i = 0; i < op.axis; ++i)
            outer *= (size_t)d[i];
        for (size_t i = (size_t)op.axis + 1; i < d.size(); ++i)
            inner *= (size_t)d[i];
        return pass(petb200_softmax_axis_run(ctx, dev_of(this, op.inputs[0]), dev_of(this, op.outputs[0]), outer, d[op.axis], inner, st));
    }
    case LayerNorm: {
        const Dim &d = tensors[op.inputs[0]].dims;
        return pass(petb200_layernorm_run(ctx, dev_of(this, op.inputs[0]), dev_of(this, op.inputs.size() > 1 ? op.inputs[1] : -1),
                                          dev_of(this, op.inputs.size() > 2 ? op.inputs[2] : -1), dev_of(this, op.outputs[0]),
                                          tensors[op.inputs[0]].size() / d.back(), d.back(), op.eps, st));
    }
    case BatchNorm: {
        const Dim &d = tensors[op.inputs[0]].dims;
        size_t inner = 1;
        for (size_t i = 2; i < d.size(); ++i)
            inner *= (size_t)d[i];
        return pass(petb200_batchnorm_run(ctx, dev_of(this, op.inputs[0]), dev_of(this, op.inputs[1]), dev_of(this, op.inputs[2]),
                                          dev_of(this, op.inputs[3]), dev_of(this, op.inputs[4]), dev_of(this, op.outputs[0]), (size_t)d[0], d[1],
                                          inner, op.eps, st));
    }
    case Attention:
        return pass(petb200_attention_run(ctx, dev_of(this, s.att_t[0]), dev_of(this, s.att_t[1]), dev_of(this, s.att_t[2]), dev_of(this, s.att_t[3]),
                                          s.att_dims[0], s.att_dims[1], s.att_dims[2], s.att_dims[3], s.att_dims[4], s.att_st, st));
    case Reshape:
        return PETB200_OK;
    }
    return PETB200_ERR_UNSUPPORTED;
}

int petb200_graph::run_all(cudaStream_t st, bool include_hoisted, int prof_slot) {
    int pair = 0;
    for (auto &s : steps) {
        if (s.weight_only && !include_hoisted)
            continue;
        const bool timed = prof_slot >= 0 && !s.side && strncmp(s.kernel, "tc_", 3) != 0;
        if (timed && cudaEventRecord(prof_events[((size_t)prof_slot * prof_pairs + pair) * 2], st) != cudaSuccess)
            return fail(PETB200_ERR_CUDA, "profile event record failed");
        const unsigned long long before = petb200_launch_count(ctx);
        cudaStream_t where = st;
        if (s.side && side_stream) { // fork: everything issued so far precedes the side step
            if (cudaEventRecord(s.ev_fork, st) != cudaSuccess || cudaStreamWaitEvent(side_stream, s.ev_fork, 0) != cudaSuccess)
                return fail(PETB200_ERR_CUDA, "side-branch fork failed");
            where = side_stream;
        }
        if (s.join_from >= 0 && side_stream && cudaStreamWaitEvent(st, steps[s.join_from].ev_join, 0) != cudaSuccess)
            return fail(PETB200_ERR_CUDA, "side-branch join failed");
        int rc = run_step(s, where);
        if (rc)
            return rc;
        if (where != st && cudaEventRecord(s.ev_join, side_stream) != cudaSuccess)
            return fail(PETB200_ERR_CUDA, "side-branch join record failed");
        if (timed && cudaEventRecord(prof_events[((size_t)prof_slot * prof_pairs + pair++) * 2 + 1], st) != cudaSuccess)
            return fail(PETB200_ERR_CUDA, "profile event record failed");
        s.launches = (int)(petb200_launch_count(ctx) - before); // what the step really launches (plans decide, e.g. a per-call operand pack)
    }
    return PETB200_OK;
}

int petb200_graph::compile(int flags) {
    const bool fuse = !(flags & 1);
    use_graph = !(flags & 2);
    for (auto &s : steps) {
        if (s.plan)
            petb200_plan_destroy(s.plan);
        if (s.ev_fork)
            cudaEventDestroy(s.ev_fork);
        if (s.ev_join)
            cudaEventDestroy(s.ev_join);
    }
    steps.clear();
    if (exec) {
        cudaGraphExecDestroy(exec);
        exec = nullptr;
    }
    for (auto &op : ops) {
        op.fused_away = false;
        if (op.merged_out >= 0) // views created by an earlier compile
            for (int t = 0; t < (int)tensors.size(); ++t)
                if (tensors[t].alias == op.merged_out && tensors[t].pitch > 0)
                    tensors[t].alias = -1, tensors[t].view_off = 0, tensors[t].pitch = tensors[t].inner = 0;
        op.merged_w.clear();
        op.merged_b.clear();
        op.merged_out = op.merged_wt = op.merged_bias = -1;
    }
    hoisted_done = false;
    // ---- topological order (Kahn, like SubGraph::compute) ----
    const int n = (int)ops.size();
    std::vector<int> cnt(n, 0), order;
    for (int i = 0; i < n; ++i) {
        std::vector<int> preds;
        for (int t : ops[i].inputs)
            if (tensors[t].outputOf >= 0)
                preds.push_back(tensors[t].outputOf);
        if (ops[i].bias >= 0 && tensors[ops[i].bias].outputOf >= 0)
            preds.push_back(tensors[ops[i].bias].outputOf);
        std::sort(preds.begin(), preds.end());
        preds.erase(std::unique(preds.begin(), preds.end()), preds.end());
        cnt[i] = (int)preds.size();
        if (!cnt[i])
            order.push_back(i);
    }
    for (size_t st = 0; st < order.size(); ++st) {
        std::vector<int> succ;
        for (int t : ops[order[st]].outputs)
            for (int c : tensors[t].inputOf)
                succ.push_back(c);
        std::sort(succ.begin(), succ.end());
        succ.erase(std::unique(succ.begin(), succ.end()), succ.end());
        for (int c : succ)
            if (--cnt[c] == 0)
                order.push_back(c);
    }
    if ((int)order.size() != n)
        return fail(PETB200_ERR_INVALID, "graph has a cycle");
    if (outputs.empty())
        for (int t = 0; t < (int)tensors.size(); ++t)
            if (tensors[t].outputOf >= 0 && tensors[t].inputOf.empty())
                outputs.push_back(t);
    auto is_output = [&](int t) { return std::find(outputs.begin(), outputs.end(), t) != outputs.end(); };
    auto sole_consumer = [&](int t) -> int { return (tensors[t].inputOf.size() == 1 && !is_output(t)) ? tensors[t].inputOf[0] : -1; };

    // ---- fold [X,Y,Z] -> [Y,X,Z] transposes around matmuls into operand strides (BERT's head split / merge) ----
    auto batch_swap = [&](const Operator &t) {
        const petb200_transpose_desc &d = t.tr;
        return t.type == Transpose && !t.fused_away && d.split < 0 && d.ngroups == 3 && d.group_sizes[0] == 1 &&
               d.group_sizes[1] == 1 && d.group_sizes[2] == 1 && d.flat[0] == 1 && d.flat[1] == 0 && d.flat[2] == 2 &&
               tensors[t.inputs[0]].dims.size() == 3;
    };
    for (int id = 0; id < n && fuse; ++id) {
        Operator &op = ops[id];
        op.mm_strided = false;
        op.mm_in[0] = op.mm_in[1] = op.mm_out_op = -1;
        if (op.type != Matmul)
            continue;
        const Dim &o = tensors[op.outputs[0]].dims, &x = tensors[op.inputs[0]].dims;
        const int bsz = o[0], m = o[1], nn = o[2], k = op.transA ? x[1] : x[2];
        long long st[6] = {(long long)m * k, op.transA ? m : k, (long long)k * nn, op.transB ? k : nn, (long long)m * nn, nn};
        int in_t[2] = {-1, -1}, out_op = -1;
        for (int i = 0; i < 2; ++i) {
            const int t = op.inputs[i], prod = tensors[t].outputOf;
            if (tensors[t].weight || prod < 0 || !batch_swap(ops[prod]) || sole_consumer(t) != id)
                continue;
            const Dim &src = tensors[ops[prod].inputs[0]].dims; // stored [X, Y, Z], read as [Y, X, Z]
            st[2 * i] = src[2];
            st[2 * i + 1] = (long long)src[1] * src[2];
            in_t[i] = ops[prod].inputs[0];
        }
        const int c = sole_consumer(op.outputs[0]);
        if (c >= 0 && batch_swap(ops[c])) { // written as [m, b, n]
            st[4] = nn;
            st[5] = (long long)bsz * nn;
            out_op = c;
        }
        if (in_t[0] < 0 && in_t[1] < 0 && out_op < 0)
            continue;
        petb200_plan *trial = nullptr; // does the tensor-core kernel take these strides?
        if (petb200_matmul_plan_strided(ctx, op.transA, op.transB, bsz, m, nn, k, op.bias >= 0, 0, PETB200_ALGO_AUTO, st, &trial) !=
            PETB200_OK)
            continue;
        petb200_plan_destroy(trial);
        op.mm_strided = true;
        for (int i = 0; i < 6; ++i)
            op.mm_strides[i] = st[i];
        for (int i = 0; i < 2; ++i)
            if (in_t[i] >= 0) {
                op.mm_in[i] = in_t[i];
                ops[tensors[op.inputs[i]].outputOf].fused_away = true;
            }
        if (out_op >= 0) {
            op.mm_out_op = out_op;
            ops[out_op].fused_away = true;
        }
    }

    // ---- merge matmuls that share their A operand (BERT's Q/K/V projections) into one wide matmul ----
    // PET's own optimiser rewrites such siblings into one operator (ref: src/Mutant/generator.cc:1495-1552); here the
    // weights are laid side by side along N and every member's result becomes a column slice of the wide result.  Only done
    // when all readers of those results are operands already folded into strides above (nothing else understands a
    // pitched tensor).
    for (int xt = 0; xt < (int)tensors.size() && fuse; ++xt) {
        std::vector<int> grp;
        for (int c : tensors[xt].inputOf) {
            const Operator &o = ops[c];
            if (o.type != Matmul || o.fused_away || o.mm_strided || o.inputs[0] != xt || o.transA || o.transB || o.act != 0 ||
                !tensors[o.inputs[1]].weight || (o.bias >= 0 && !tensors[o.bias].weight) || is_output(o.outputs[0]))
                continue;
            // one weight matrix shared by the whole batch (the wide weight is laid out as [1, k, ntot])
            if (tensors[o.inputs[1]].dims.size() != 3 || tensors[o.inputs[1]].dims[0] != 1)
                continue;
            const Dim &od = tensors[o.outputs[0]].dims; // [bs, m, ni]
            bool ok_out = !tensors[o.outputs[0]].inputOf.empty();
            for (int rc_ : tensors[o.outputs[0]].inputOf) { // every reader: Reshape -> folded transpose -> strided matmul operand
                const Operator &r = ops[rc_];
                if (r.type != Reshape) {
                    ok_out = false;
                    break;
                }
                const int R = r.outputs[0];
                // The reshape must keep the rows of the result intact — [bs*m rows] x [row split in two] — because the
                // readers are re-addressed by giving exactly those rows the pitch of the wide result.
                const Dim &rd = tensors[R].dims;
                ok_out = ok_out && rd.size() == 3 && rd[1] * rd[2] == od[2] && rd[0] == od[0] * od[1];
                ok_out = ok_out && !is_output(R) && !tensors[R].inputOf.empty();
                for (int tc : tensors[R].inputOf) {
                    const Operator &tr = ops[tc];
                    const int user = tr.type == Transpose && tr.fused_away ? sole_consumer(tr.outputs[0]) : -1;
                    ok_out = ok_out && user >= 0 && ops[user].mm_strided && (ops[user].mm_in[0] == R || ops[user].mm_in[1] == R);
                }
            }
            if (ok_out && (grp.empty() || ((ops[grp[0]].bias >= 0) == (o.bias >= 0) &&
                                           tensors[ops[grp[0]].inputs[1]].dims[1] == tensors[o.inputs[1]].dims[1])))
                grp.push_back(c);
        }
        if (grp.size() < 2)
            continue;
        std::sort(grp.begin(), grp.end());
        const Dim o0 = tensors[ops[grp[0]].outputs[0]].dims;
        const int kdim = tensors[ops[grp[0]].inputs[1]].dims[1];
        int ntot = 0;
        for (int c : grp)
            ntot += tensors[ops[c].outputs[0]].dims[2];
        const int M = new_tensor({o0[0], o0[1], ntot}), Wm = new_tensor({1, kdim, ntot}, true);
        const int Bm = ops[grp[0]].bias >= 0 ? new_tensor({ntot}, true) : -1;
        Operator &lead = ops[grp[0]];
        lead.merged_out = M, lead.merged_wt = Wm, lead.merged_bias = Bm;
        int off = 0;
        for (int c : grp) {
            Operator &o = ops[c];
            const int O = o.outputs[0], ni = tensors[O].dims[2];
            lead.merged_w.push_back(o.inputs[1]);
            if (Bm >= 0)
                lead.merged_b.push_back(o.bias);
            tensors[O].alias = M, tensors[O].view_off = off, tensors[O].pitch = ntot, tensors[O].inner = ni;
            for (int rc_ : tensors[O].inputOf) // readers address rows `ntot` apart instead of `ni`
                for (int tc : tensors[ops[rc_].outputs[0]].inputOf) {
                    Operator &user = ops[sole_consumer(ops[tc].outputs[0])];
                    for (int j = 0; j < 2; ++j)
                        if (user.mm_in[j] == ops[rc_].outputs[0])
                            user.mm_strides[2 * j + 1] = ntot;
                }
            if (c != grp[0])
                o.fused_away = true;
            off += ni;
        }
    }

    // ---- fold a seam-transpose pair into the convolution between them ----
    // PET's H->N rewrite is  TransposeOp(2, {{0,2},1,-1,3}, -2) -> Conv -> TransposeOp(0, {0,1,{-1,2},3}, 2)  (ref:
    // src/Mutant/generator.cc:1027-1046; the pair is what markTransType labels Pre/Post, :1889-1958).  Both transposes are
    // pure re-indexings of N and H: the contiguous [N,C,H,W] input IS the 5-D tensor [N,C,2,H/2,W], the two halves being
    // two depth slices, so "H->N, conv2d, N->H" is one 3-D convolution with a 1 x R x S filter on that view, whose
    // [N,F,2,OH/2,OW] result is the [N,F,OH,OW] tensor the second transpose would have produced.  The W pair
    // (TransposeOp(3, {{0,3},1,2,-1}, -2) ... TransposeOp(0, {0,1,2,{-1,3}}, 2)) views [N,C,H,W] as [N,C,2H,W/2] — row
    // 2h+p holds half p of row h — and becomes a 2-D convolution with the row dilation and row padding doubled (row
    // stride 1 only).  Same products in the same order as the three-operator form; no copy, one launch.
    auto is_tr = [&](const Operator &t, int split, int factor, std::initializer_list<int> sizes, std::initializer_list<int> flat) {
        if (t.type != Transpose || t.fused_away || t.halo[0] || t.halo[1] || t.halo[2] || t.halo[3] || t.tr.split != split ||
            t.tr.factor != factor || t.tr.ngroups != (int)sizes.size())
            return false;
        int i = 0;
        for (int v : sizes)
            if (t.tr.group_sizes[i++] != v)
                return false;
        i = 0;
        for (int v : flat)
            if (t.tr.flat[i++] != v)
                return false;
        return true;
    };
    for (int id = 0; id < n && fuse; ++id) {
        Operator &op = ops[id];
        if (op.type != Conv || op.fused_away || tensors[op.inputs[0]].dims.size() != 4)
            continue;
        const int pre = tensors[op.inputs[0]].outputOf, post = sole_consumer(op.outputs[0]);
        if (pre < 0 || post < 0 || sole_consumer(op.inputs[0]) != id || tensors[ops[pre].inputs[0]].dims.size() != 4)
            continue;
        // Space-to-batch: D2H, H2N, D2W, W2N -> dense conv -> N2W, D2W^-1, N2H, D2H^-1 (the rewrite of a dilated conv, ref:
        // src/Mutant/generator.cc:1085-1092) is the convolution with dilation and padding doubled on the untouched tensor:
        // phase (p_h, p_w) of the input only ever meets phase (p_h, p_w) of the output.  Stride 1 only.
        int pre4[4], post4[4];
        bool ok = op.sh == 1 && op.sw == 1;
        int t = op.inputs[0];
        for (int i = 3; i >= 0 && ok; --i) { // walk up: W2N, D2W, H2N, D2H
            pre4[i] = tensors[t].outputOf;
            ok = pre4[i] >= 0 && sole_consumer(t) == (i == 3 ? id : pre4[i + 1]) && tensors[ops[pre4[i]].inputs[0]].dims.size() == 4;
            if (ok)
                t = ops[pre4[i]].inputs[0];
        }
        ok = ok && is_tr(ops[pre4[0]], 2, 2, {1, 1, 2, 1}, {0, 1, -1, 2, 3}) && is_tr(ops[pre4[1]], 2, -2, {2, 1, 1, 1}, {0, 2, 1, -1, 3}) &&
             is_tr(ops[pre4[2]], 3, 2, {1, 1, 1, 2}, {0, 1, 2, -1, 3}) && is_tr(ops[pre4[3]], 3, -2, {2, 1, 1, 1}, {0, 3, 1, 2, -1});
        t = op.outputs[0];
        for (int i = 0; i < 4 && ok; ++i) { // walk down: N2W, D2W^-1, N2H, D2H^-1
            post4[i] = sole_consumer(t);
            ok = post4[i] >= 0;
            if (ok)
                t = ops[post4[i]].outputs[0];
        }
        ok = ok && is_tr(ops[post4[0]], 0, 2, {1, 1, 1, 2}, {0, 1, 2, -1, 3}) && is_tr(ops[post4[1]], 3, -2, {1, 1, 1, 2}, {0, 1, 2, -1, 3}) &&
             is_tr(ops[post4[2]], 0, 2, {1, 1, 2, 1}, {0, 1, -1, 2, 3}) && is_tr(ops[post4[3]], 2, -2, {1, 1, 2, 1}, {0, 1, -1, 2, 3});
        if (ok) {
            op.seam_axis = 'S';
            op.seam_in = ops[pre4[0]].inputs[0];
            op.seam_out_op = post4[3];
            for (int i = 0; i < 4; ++i)
                ops[pre4[i]].fused_away = ops[post4[i]].fused_away = true;
            continue;
        }
        char axis = 0;
        if (is_tr(ops[pre], 2, -2, {2, 1, 1, 1}, {0, 2, 1, -1, 3}) && is_tr(ops[post], 0, 2, {1, 1, 2, 1}, {0, 1, -1, 2, 3}))
            axis = 'H';
        else if (is_tr(ops[pre], 3, -2, {2, 1, 1, 1}, {0, 3, 1, 2, -1}) && is_tr(ops[post], 0, 2, {1, 1, 1, 2}, {0, 1, 2, -1, 3}) && op.sh == 1)
            axis = 'W';
        if (axis) {
            op.seam_axis = axis;
            op.seam_in = ops[pre].inputs[0];
            op.seam_out_op = post;
            ops[pre].fused_away = ops[post].fused_away = true;
        }
        // H pair followed by the correction of its seam: when the correction window holds every output row the split got
        // wrong (rows of the upper half whose filter reaches into the lower half, rows of the lower half whose filter
        // reaches back up), rewrite + correction IS the unsplit convolution on the untouched tensor — one launch.
        const int cor = axis == 'H' ? sole_consumer(ops[post].outputs[0]) : -1;
        if (cor >= 0 && ops[cor].type == Correction && !ops[cor].fused_away) {
            const Operator &c = ops[cor];
            const Dim &x0 = tensors[op.seam_in].dims, &wd = tensors[op.inputs[1]].dims, &od = tensors[c.outputs[0]].dims;
            const int half = x0[2] / 2, ohh = od[2] / 2, r = wd[2];
            const int top_first = std::max(0, (half + op.ph - (r - 1) * op.dh + op.sh - 1) / op.sh);
            const int bottom_end = ohh + (op.ph + op.sh - 1) / op.sh;
            if (c.inputs[0] == op.seam_in && c.inputs[1] == op.inputs[1] && c.inputs[2] == ops[post].outputs[0] && c.bias == op.bias &&
                c.ph == op.ph && c.pw == op.pw && c.sh == op.sh && c.sw == op.sw && c.dh == op.dh && c.dw == op.dw && c.act == op.act &&
                ohh * op.sh == half && c.win[2] == 0 && c.win[3] == od[3] && c.win[0] <= top_first && c.win[0] + c.win[1] >= bottom_end) {
                op.seam_axis = 'X';
                op.seam_out_op = cor;
                ops[cor].fused_away = true;
            }
        }
    }

    // ---- build steps with fusion ----
    std::vector<char> emitted(n, 0); // operators already covered by a step
    // An attention head, Matmul(q, k^T) -> Softmax(last axis) -> Matmul(p, v) with no other reader of the scores or of the
    // probabilities, becomes one launch.  The step is emitted at the position of the SECOND product (by then v exists too);
    // the first product and the softmax are remembered here, keyed by the second product's id.
    static const bool fuse_attention = [] { const char *e = getenv("PETB200_FUSE_ATTENTION"); return !e || atoi(e) != 0; }();
    std::map<int, int> attn_first; // second matmul -> first matmul
    auto attention_tail = [&](const Operator &m1) -> int { // id of the second product if m1 starts such a chain, else -1
        if (m1.type != Matmul || m1.transA || !m1.transB || m1.bias >= 0 || m1.act != 0 || m1.merged_out >= 0 || m1.mm_out_op >= 0 ||
            tensors[m1.inputs[0]].weight || tensors[m1.inputs[1]].weight)
            return -1;
        const int sm = sole_consumer(m1.outputs[0]);
        if (sm < 0 || ops[sm].type != Softmax || ops[sm].fused_away || tensors[ops[sm].inputs[0]].dims.size() != 3 || ops[sm].axis != 2)
            return -1;
        const int c2 = sole_consumer(ops[sm].outputs[0]);
        if (c2 < 0)
            return -1;
        const Operator &m2 = ops[c2];
        if (m2.type != Matmul || m2.fused_away || m2.inputs[0] != ops[sm].outputs[0] || m2.transA || m2.transB || m2.bias >= 0 || m2.act != 0 ||
            m2.merged_out >= 0 || m2.mm_in[0] >= 0 || tensors[m2.inputs[1]].weight)
            return -1;
        const Dim &sd = tensors[m1.outputs[0]].dims, &qd = tensors[m1.inputs[0]].dims, &od = tensors[m2.outputs[0]].dims; // [bs,m,n] [bs,m,kd] [bs,m,d]
        if (od[0] != sd[0] || !petb200_attention_supported(sd[1], sd[2], qd[2], od[2]))
            return -1;
        return c2;
    };
    for (int id : order) {
        Operator &op = ops[id];
        if (op.fused_away)
            continue;
        if (fuse && fuse_attention && !(flags & 8) && op.type == Matmul) {
            const int tail = attention_tail(op);
            if (tail >= 0) { // deferred to the second product
                attn_first[tail] = id;
                op.fused_away = true;
                ops[sole_consumer(op.outputs[0])].fused_away = true;
                continue;
            }
        }
        if (op.type == Matmul && attn_first.count(id)) {
            const Operator &m1 = ops[attn_first[id]];
            const int sm = tensors[m1.outputs[0]].inputOf[0];
            const Dim &sd = tensors[m1.outputs[0]].dims, &qd = tensors[m1.inputs[0]].dims, &od = tensors[op.outputs[0]].dims;
            Step a;
            a.type = Attention;
            a.name = "attention";
            a.kernel = "k_attention";
            a.ops = {attn_first[id], sm, id};
            if (op.mm_out_op >= 0)
                a.ops.push_back(op.mm_out_op); // the step's result is the transposed tensor
            const int dims5[5] = {sd[0], sd[1], sd[2], qd[2], od[2]};
            std::copy(dims5, dims5 + 5, a.att_dims);
            const long long m = sd[1], nk = sd[2], kd = qd[2], d = od[2];
            const long long dense1[6] = {m * kd, kd, nk * kd, kd, 0, 0}, dense2[6] = {0, 0, nk * d, d, m * d, d};
            const long long *s1 = m1.mm_strided ? m1.mm_strides : dense1, *s2 = op.mm_strided ? op.mm_strides : dense2;
            const long long st8[8] = {s1[0], s1[1], s1[2], s1[3], s2[2], s2[3], s2[4], s2[5]};
            std::copy(st8, st8 + 8, a.att_st);
            a.att_t[0] = m1.mm_in[0] >= 0 ? m1.mm_in[0] : m1.inputs[0];
            a.att_t[1] = m1.mm_in[1] >= 0 ? m1.mm_in[1] : m1.inputs[1];
            a.att_t[2] = op.mm_in[1] >= 0 ? op.mm_in[1] : op.inputs[1];
            a.att_t[3] = ops[a.ops.back()].outputs[0];
            for (int o : a.ops)
                emitted[o] = 1;
            steps.push_back(a);
            continue;
        }
        Step s;
        s.type = op.type;
        s.ops.push_back(id);
        s.weight_only = true;
        for (int t : op.inputs)
            s.weight_only = s.weight_only && tensors[t].weight;
        int rc = PETB200_OK;
        switch (op.type) {
        case Conv:
        case Conv3d:
        case Matmul: {
            int act = op.act;
            if (fuse && act == 0) { // fold a sole-consumer activation into the epilogue
                int c = sole_consumer(op.outputs[0]);
                if (c >= 0 && ops[c].type == Activation) {
                    act = ops[c].act;
                    ops[c].fused_away = true;
                    s.ops.push_back(c);
                } else if (c >= 0 && ops[c].type == Add && ops[c].inputs.size() == 2 && !ops[c].fused_away) {
                    // ... or a residual Add (and the activation after it), when the other summand already exists at
                    // this point of the order: y = act(conv + bias + residual), the Add's own arithmetic in its own order
                    const int other = ops[c].inputs[0] == op.outputs[0] ? ops[c].inputs[1] : ops[c].inputs[0];
                    const int prod = tensors[other].outputOf;
                    if (other != op.outputs[0] && tensors[other].dims == tensors[op.outputs[0]].dims && (prod < 0 || emitted[prod])) {
                        s.residual = other;
                        ops[c].fused_away = true;
                        s.ops.push_back(c);
                        const int c2 = sole_consumer(ops[c].outputs[0]);
                        if (c2 >= 0 && ops[c2].type == Activation) {
                            act = ops[c2].act;
                            ops[c2].fused_away = true;
                            s.ops.push_back(c2);
                        }
                    }
                }
            }
            const Dim &x = tensors[op.inputs[0]].dims, &w = tensors[op.inputs[1]].dims;
            if (op.type == Conv && op.seam_axis) {
                const Dim &x0 = tensors[op.seam_in].dims; // the original layout [N, C, H, W]
                if (op.seam_axis == 'H') {
                    int a[21] = {x0[0], x0[1], 2, x0[2] / 2, x0[3], w[0], 1, w[2], w[3], 0, op.ph, op.pw, 1, op.sh, op.sw, 1, op.dh, op.dw,
                                 x[1] / w[1], op.bias >= 0, act};
                    rc = petb200_conv3d_plan(ctx, a, PETB200_ALGO_AUTO, &s.plan);
                } else if (op.seam_axis == 'W') {
                    int a[16] = {x0[0], x0[1], 2 * x0[2], x0[3] / 2, w[0], w[2], w[3], 2 * op.ph, op.pw, 1, op.sw, 2 * op.dh, op.dw, x[1] / w[1],
                                 op.bias >= 0, act};
                    rc = petb200_conv2d_plan(ctx, a, PETB200_ALGO_AUTO, &s.plan);
                } else if (op.seam_axis == 'X') { // H pair + its correction: the unsplit convolution
                    int a[16] = {x0[0], x0[1], x0[2], x0[3], w[0], w[2], w[3], op.ph, op.pw, op.sh, op.sw, op.dh, op.dw, x[1] / w[1], op.bias >= 0,
                                 act};
                    rc = petb200_conv2d_plan(ctx, a, PETB200_ALGO_AUTO, &s.plan);
                } else { // space-to-batch pair: the dilated convolution itself
                    int a[16] = {x0[0], x0[1], x0[2], x0[3], w[0], w[2], w[3], 2 * op.ph, 2 * op.pw, 1, 1, 2 * op.dh, 2 * op.dw, x[1] / w[1],
                                 op.bias >= 0, act};
                    rc = petb200_conv2d_plan(ctx, a, PETB200_ALGO_AUTO, &s.plan);
                }
                s.name = op.seam_axis == 'X' ? "conv_seam_healed" : "conv_seam_folded";
                // the step covers the transposes too (fused_away): the ones before the conv, then the ones after it, the last
                // of which names the step's result
                for (int t = op.inputs[0]; tensors[t].outputOf >= 0 && ops[tensors[t].outputOf].fused_away && t != op.seam_in;
                     t = ops[tensors[t].outputOf].inputs[0])
                    s.ops.insert(s.ops.begin() + 1, tensors[t].outputOf);
                for (int t = op.outputs[0];;) {
                    const int c = tensors[t].inputOf[0];
                    s.ops.push_back(c);
                    if (c == op.seam_out_op)
                        break;
                    t = ops[c].outputs[0];
                }
            } else if (op.type == Conv) {
                int a[16] = {x[0], x[1], x[2], x[3], w[0], w[2], w[3], op.ph, op.pw, op.sh, op.sw, op.dh, op.dw, x[1] / w[1], op.bias >= 0, act};
                rc = petb200_conv2d_plan(ctx, a, PETB200_ALGO_AUTO, &s.plan);
                s.name = "conv";
            } else if (op.type == Conv3d) {
                int a[21] = {x[0], x[1], x[2], x[3], x[4], w[0], w[2], w[3], w[4], op.pad3[0], op.pad3[1], op.pad3[2], op.stride3[0], op.stride3[1],
                             op.stride3[2], op.dil3[0], op.dil3[1], op.dil3[2], x[1] / w[1], op.bias >= 0, act};
                rc = petb200_conv3d_plan(ctx, a, PETB200_ALGO_AUTO, &s.plan);
                s.name = "conv3d";
            } else {
                const Dim &o = tensors[op.merged_out >= 0 ? op.merged_out : op.outputs[0]].dims;
                const int k = op.transA ? x[1] : x[2];
                if (op.merged_out >= 0) {
                    rc = petb200_matmul_plan(ctx, 0, 0, o[0], o[1], o[2], k, op.merged_bias >= 0, act, PETB200_ALGO_AUTO, &s.plan);
                } else if (op.mm_strided) {
                    rc = petb200_matmul_plan_strided(ctx, op.transA, op.transB, o[0], o[1], o[2], k, op.bias >= 0, act, PETB200_ALGO_AUTO,
                                                     op.mm_strides, &s.plan);
                    if (op.mm_out_op >= 0)
                        s.ops.push_back(op.mm_out_op); // the step's result is the transposed tensor
                } else {
                    rc = petb200_matmul_plan(ctx, op.transA, op.transB, o[0], o[1], o[2], k, op.bias >= 0, act, PETB200_ALGO_AUTO, &s.plan);
                }
                s.name = "matmul";
                s.launches = 1 + (op.transA ? 0 : 1) + (tensors[op.inputs[1]].weight ? 0 : 1);
            }
            s.weight_only = false;
            break;
        }
        case Correction: {
            const Dim &x = tensors[op.inputs[0]].dims, &w = tensors[op.inputs[1]].dims;
            int a[16] = {x[0], x[1], x[2], x[3], w[0], w[2], w[3], op.ph, op.pw, op.sh, op.sw, op.dh, op.dw, x[1] / w[1], op.bias >= 0, op.act};
            rc = petb200_conv2d_plan(ctx, a, PETB200_ALGO_AUTO, &s.plan);
            s.name = "correction";
            s.weight_only = false;
            break;
        }
        case Transpose: {
            auto has_halo = [](const Operator &o) { return o.halo[0] || o.halo[1] || o.halo[2] || o.halo[3]; };
            if (has_halo(op)) { // carries padding / halo parameters: its own index map, not part of a fused chain
                const Dim &d0 = tensors[op.inputs[0]].dims;
                rc = petb200_transpose_halo_plan(ctx, (int)d0.size(), d0.data(), &op.tr, op.halo[0], op.halo[1], op.halo[2], op.halo[3], &s.plan);
                s.name = "transpose_halo";
                s.launches = op.halo[0] ? 2 : 1;
                break;
            }
            std::vector<petb200_transpose_desc> chain = {op.tr};
            int last = id;
            while (fuse) { // extend the chain while the intermediate has a single consumer that is a transpose
                int c = sole_consumer(ops[last].outputs[0]);
                if (c < 0 || ops[c].type != Transpose || has_halo(ops[c]))
                    break;
                chain.push_back(ops[c].tr);
                petb200_plan *trial = nullptr;
                const Dim &d0 = tensors[op.inputs[0]].dims;
                if (petb200_transpose_plan(ctx, (int)d0.size(), d0.data(), (int)chain.size(), chain.data(), &trial) != PETB200_OK) {
                    chain.pop_back(); // not expressible as one index map: leave the rest for its own step
                    break;
                }
                petb200_plan_destroy(trial);
                ops[c].fused_away = true;
                s.ops.push_back(c);
                last = c;
            }
            const Dim &d0 = tensors[op.inputs[0]].dims;
            rc = petb200_transpose_plan(ctx, (int)d0.size(), d0.data(), (int)chain.size(), chain.data(), &s.plan);
            s.name = chain.size() > 1 ? "transpose_chain" : "transpose";
            break;
        }
        case Pad: {
            const Dim &d = tensors[op.inputs[0]].dims;
            rc = petb200_pad_plan(ctx, (int)d.size(), d.data(), op.begin.data(), op.end.data(), &s.plan);
            s.name = "pad";
            break;
        }
        case Slice: {
            const Dim &d = tensors[op.inputs[0]].dims;
            rc = petb200_slice_plan(ctx, (int)d.size(), d.data(), op.begin.data(), op.end.data(), &s.plan);
            s.name = "slice";
            break;
        }
        case Extend: {
            const Dim &d = tensors[op.inputs[0]].dims;
            rc = petb200_extend_plan(ctx, (int)d.size(), d.data(), op.dim, op.num, &s.plan);
            s.name = "extend";
            break;
        }
        case Concat:
            s.name = "concat";
            s.launches = (int)op.inputs.size();
            break;
        case Split:
            s.name = "split";
            s.launches = (int)op.outputs.size();
            break;
        case Add:
        case Sub:
        case Mul:
            s.name = op.type == Add ? "add" : (op.type == Sub ? "sub" : "mul");
            if (fuse) {
                int c = sole_consumer(op.outputs[0]);
                if (c >= 0 && ops[c].type == Activation) {
                    ops[c].fused_away = true;
                    s.ops.push_back(c);
                }
            }
            break;
        case ConvTrans: {
            const Dim &x = tensors[op.inputs[0]].dims, &w = tensors[op.inputs[1]].dims; // {n,h,w,f}, {r,s,f,c}
            int a[18] = {x[0], w[3], x[1], x[2], x[3], w[0], w[1], op.ph, op.pw, op.sh, op.sw, op.dh, op.dw, 1, op.bias >= 0, op.act, op.oph, op.opw};
            rc = petb200_convtrans_plan(ctx, a, PETB200_ALGO_AUTO, &s.plan);
            s.name = "convtrans";
            s.launches = 2;
            s.weight_only = false;
            break;
        }
        case G2BMM:
            s.name = "g2bmm";
            break;
        case Div:
            s.name = "div";
            break;
        case Pow:
            s.name = "pow";
            break;
        case ReduceMean:
            s.name = "reduce_mean";
            break;
        case Gather:
            s.name = "gather";
            break;
        case GBMML:
            s.name = "gbmml";
            break;
        case Activation:
            s.name = "activation";
            break;
        case MaxPool:
            s.name = "maxpool";
            break;
        case AvgPool:
            s.name = "avgpool";
            break;
        case Softmax:
            s.name = "softmax";
            break;
        case LayerNorm:
            s.name = "layernorm";
            break;
        case BatchNorm:
            s.name = "batchnorm";
            break;
        case Reshape:
            s.name = "reshape";
            s.launches = 0;
            break;
        }
        if (rc)
            return pass(rc);
        s.kernel = s.plan ? petb200_plan_kernel(s.plan) : (s.type == G2BMM ? "k_g2bmm" : (s.type == GBMML ? "k_gbmml" : (s.launches ? "eltwise" : "alias")));
        for (int o : s.ops)
            emitted[o] = 1;
        steps.push_back(s);
    }
    // ---- side branches: a conv/matmul step read only as a later step's residual runs beside the main chain ----
    // (the shortcut convolution of a ResNet block: it is moved up to right after the step that produces its input and put on
    // a second stream, so that it overlaps the block's first convolution)
    if (fuse && !(flags & 4)) {
        auto residual_reader = [&](size_t i) -> int { // the one later step that reads step i's result, as its residual only
            const int out = ops[steps[i].ops.back()].outputs[0];
            if (is_output(out) || tensors[out].inputOf.empty())
                return -1;
            int reader = -1;
            for (int c : tensors[out].inputOf) {
                int owner = -1;
                for (size_t j = i + 1; j < steps.size() && owner < 0; ++j)
                    if (steps[j].residual == out && std::find(steps[j].ops.begin(), steps[j].ops.end(), c) != steps[j].ops.end())
                        owner = (int)j;
                if (owner < 0 || (reader >= 0 && reader != owner))
                    return -1;
                reader = owner;
            }
            return reader;
        };
        for (size_t i = 0; i < steps.size(); ++i) {
            if (steps[i].weight_only || steps[i].side || (steps[i].type != Conv && steps[i].type != Conv3d && steps[i].type != Matmul))
                continue;
            if (residual_reader(i) < 0)
                continue;
            // earliest slot: right after the last step that produces one of its (non-weight) inputs
            const Operator &op = ops[steps[i].ops.front()];
            size_t earliest = 0;
            for (int t : op.inputs) {
                if (tensors[t].weight)
                    continue;
                const int prod = tensors[root(t)].outputOf;
                for (size_t j = 0; j < i; ++j)
                    if (prod >= 0 && std::find(steps[j].ops.begin(), steps[j].ops.end(), prod) != steps[j].ops.end())
                        earliest = std::max(earliest, j + 1);
            }
            if (earliest < i)
                std::rotate(steps.begin() + earliest, steps.begin() + i, steps.begin() + i + 1);
            const size_t at = std::min(earliest, i);
            const int reader = residual_reader(at);
            if (reader < 0 || reader == (int)at + 1 || steps[reader].join_from >= 0)
                continue; // nothing to overlap with
            if (!side_stream && cudaStreamCreateWithFlags(&side_stream, cudaStreamNonBlocking) != cudaSuccess)
                return fail(PETB200_ERR_CUDA, "side stream creation failed");
            if (cudaEventCreateWithFlags(&steps[at].ev_fork, cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&steps[at].ev_join, cudaEventDisableTiming) != cudaSuccess)
                return fail(PETB200_ERR_CUDA, "event creation failed");
            steps[at].side = true;
        }
        for (size_t i = 0; i < steps.size(); ++i) // (indices are final only now)
            if (steps[i].side)
                steps[residual_reader(i)].join_from = (int)i;
    }
    // ---- storage: one buffer per non-aliased tensor (kept across recompiles) ----
    for (auto &t : tensors) {
        if (t.alias >= 0 || t.dev)
            continue;
        if (cudaMalloc((void **)&t.dev, std::max<size_t>(t.size(), 1) * sizeof(float)) != cudaSuccess)
            return fail(PETB200_ERR_NOMEM, "tensor allocation of %zu floats failed", t.size());
        t.owns = true;
    }
    compiled = true;
    return PETB200_OK;
}

// Work that depends on weights only, done once per set of weights and kept out of the replayed sequence (the
// reference hoists the same operators, src/Graph/code_engine.cc:187-193): weight-only steps first, then the
// packing of conv filters and constant matmul operands.
static int prepare_weights(petb200_graph *g, cudaStream_t st) {
    for (auto &s : g->steps)
        if (s.weight_only) {
            int rc = g->run_step(s, st);
            if (rc)
                return rc;
            for (int o : s.ops)
                for (int t : g->ops[o].outputs)
                    g->tensors[t].has_data = true;
        }
    for (auto &s : g->steps) {
        Operator &op = g->ops[s.ops.front()];
        if (s.weight_only || op.inputs.size() < 2)
            continue;
        const Tensor &w = g->tensors[op.inputs[1]];
        const bool ready = w.has_data || g->tensors[g->root(op.inputs[1])].has_data;
        int rc = PETB200_OK;
        if (s.type == Matmul && op.merged_out >= 0) {
            // lay the members' weights (and biases) side by side, then preprocess the wide matrix once
            bool all = true;
            for (int wt : op.merged_w)
                all = all && g->tensors[wt].has_data;
            for (int bt : op.merged_b)
                all = all && g->tensors[bt].has_data;
            if (!all)
                continue;
            const Dim &wd = g->tensors[op.merged_wt].dims; // [1, k, ntot]
            size_t off = 0;
            for (size_t i = 0; i < op.merged_w.size(); ++i) {
                const int ni = g->tensors[op.merged_w[i]].dims[2];
                if (cudaMemcpy2DAsync(dev_of(g, op.merged_wt) + off, (size_t)wd[2] * 4, dev_of(g, op.merged_w[i]), (size_t)ni * 4,
                                      (size_t)ni * 4, (size_t)wd[1], cudaMemcpyDeviceToDevice, st) != cudaSuccess)
                    return g->fail(PETB200_ERR_CUDA, "merged weight copy failed");
                if (!op.merged_b.empty() &&
                    cudaMemcpyAsync(dev_of(g, op.merged_bias) + off, dev_of(g, op.merged_b[i]), (size_t)ni * 4, cudaMemcpyDeviceToDevice, st) !=
                        cudaSuccess)
                    return g->fail(PETB200_ERR_CUDA, "merged bias copy failed");
                off += (size_t)ni;
            }
            g->tensors[op.merged_wt].has_data = true;
            rc = petb200_matmul_set_weights(s.plan, dev_of(g, op.merged_wt), st);
            if (rc)
                return g->pass(rc);
            continue;
        }
        if ((s.type == Conv || s.type == Correction) && ready)
            rc = petb200_conv2d_set_weights(s.plan, dev_of(g, op.inputs[1]), st);
        else if (s.type == Conv3d && ready)
            rc = petb200_conv3d_set_weights(s.plan, dev_of(g, op.inputs[1]), st);
        else if (s.type == ConvTrans && ready)
            rc = petb200_convtrans_set_weights(s.plan, dev_of(g, op.inputs[1]), st);
        else if (s.type == Matmul && w.weight && ready)
            rc = petb200_matmul_set_weights(s.plan, dev_of(g, op.inputs[1]), st);
        if (rc)
            return g->pass(rc);
    }
    return PETB200_OK;
}

int petb200_graph::capture() {
    if (!cap_stream && cudaStreamCreateWithFlags(&cap_stream, cudaStreamNonBlocking) != cudaSuccess)
        return fail(PETB200_ERR_CUDA, "stream creation failed");
    // weight-only steps and weight packing run once, eagerly; one eager pass also warms every lazily built plan
    int rc = prepare_weights(this, cap_stream);
    if (rc)
        return rc;
    rc = run_all(cap_stream, false);
    if (rc)
        return rc;
    if (cudaStreamSynchronize(cap_stream) != cudaSuccess)
        return fail(PETB200_ERR_CUDA, "warm-up pass failed: %s", cudaGetErrorString(cudaGetLastError()));
    cudaGraph_t graph = nullptr;
    if (cudaStreamBeginCapture(cap_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
        return fail(PETB200_ERR_CUDA, "begin capture failed");
    rc = run_all(cap_stream, false);
    cudaError_t e = cudaStreamEndCapture(cap_stream, &graph);
    if (rc || e != cudaSuccess) {
        if (graph)
            cudaGraphDestroy(graph);
        cudaGetLastError();
        return rc ? rc : fail(PETB200_ERR_CUDA, "end capture failed: %s", cudaGetErrorString(e));
    }
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess)
        return fail(PETB200_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
    return PETB200_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------------------------
#define G_CHECK_T(g, t)                                                                                      \
    if (!(g)->valid_tensor(t))                                                                               \
    return (g)->fail(PETB200_ERR_INVALID, "tensor id %d does not exist", (t))

extern "C" int petb200_graph_create(petb200_ctx *ctx, petb200_graph **out) {
    if (!ctx || !out)
        return PETB200_ERR_INVALID;
    *out = new petb200_graph();
    (*out)->ctx = ctx;
    return PETB200_OK;
}
extern "C" void petb200_graph_destroy(petb200_graph *g) { delete g; }
extern "C" const char *petb200_graph_last_error(const petb200_graph *g) { return g ? g->err.c_str() : "null graph"; }

extern "C" int petb200_graph_tensor(petb200_graph *g, int nd, const int *dims, int is_weight, int *tensor) {
    if (!g || !dims || !tensor || nd < 0 || nd > 8)
        return PETB200_ERR_INVALID;
    for (int i = 0; i < nd; ++i)
        if (dims[i] <= 0)
            return g->fail(PETB200_ERR_INVALID, "tensor dim %d is %d", i, dims[i]);
    *tensor = g->new_tensor(Dim(dims, dims + nd), is_weight != 0);
    return PETB200_OK;
}
extern "C" int petb200_graph_tensor_dims(const petb200_graph *g, int tensor, int *dims) {
    if (!g || !g->valid_tensor(tensor))
        return -1;
    const Dim &d = g->tensors[tensor].dims;
    if (dims)
        std::copy(d.begin(), d.end(), dims);
    return (int)d.size();
}

static int conv_extent(int in, int k, int p, int s, int d) { return (in - (k - s) * d + 2 * p) / s; }

extern "C" int petb200_graph_conv(petb200_graph *g, int x, int w, int bias, int ph, int pw, int sh, int sw, int dh, int dw,
                                  int act, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    G_CHECK_T(g, w);
    const Dim &xd = g->tensors[x].dims, &wd = g->tensors[w].dims;
    // ref: ConvOp::checkValid / compute: 4-D operands, c divisible by filter channels, f divisible by groups
    if (xd.size() != 4 || wd.size() != 4 || wd[1] <= 0 || xd[1] % wd[1] || wd[0] % (xd[1] / wd[1]) || sh <= 0 || sw <= 0 || dh <= 0 || dw <= 0)
        return g->fail(PETB200_ERR_INVALID, "conv: operand shapes do not form a valid convolution");
    if (bias >= 0 && (!g->valid_tensor(bias) || (int)g->tensors[bias].size() != wd[0]))
        return g->fail(PETB200_ERR_INVALID, "conv: bias must have one value per filter");
    Dim od = {xd[0], wd[0], conv_extent(xd[2], wd[2], ph, sh, dh), conv_extent(xd[3], wd[3], pw, sw, dw)};
    if (od[2] <= 0 || od[3] <= 0)
        return g->fail(PETB200_ERR_INVALID, "conv: empty output");
    Operator op;
    op.type = Conv;
    op.inputs = {x, w};
    op.bias = bias;
    op.ph = ph, op.pw = pw, op.sh = sh, op.sw = sw, op.dh = dh, op.dw = dw, op.act = act;
    // ref: ConvOp::checkAndSetTensorTypeForConstructor marks the filter as a weight
    g->tensors[w].weight = true;
    *out = g->new_tensor(od);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_conv3d(petb200_graph *g, int x, int w, int bias, const int pad[3], const int stride[3],
                                    const int dil[3], int act, int *out) {
    if (!g || !out || !pad || !stride || !dil)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    G_CHECK_T(g, w);
    const Dim &xd = g->tensors[x].dims, &wd = g->tensors[w].dims;
    if (xd.size() != 5 || wd.size() != 5 || wd[1] <= 0 || xd[1] % wd[1] || wd[0] % (xd[1] / wd[1]))
        return g->fail(PETB200_ERR_INVALID, "conv3d: operand shapes do not form a valid convolution");
    Dim od = {xd[0], wd[0]};
    for (int i = 0; i < 3; ++i) {
        if (stride[i] <= 0 || dil[i] <= 0 || pad[i] < 0)
            return g->fail(PETB200_ERR_INVALID, "conv3d: bad stride/dilation/pad");
        od.push_back(conv_extent(xd[2 + i], wd[2 + i], pad[i], stride[i], dil[i]));
        if (od.back() <= 0)
            return g->fail(PETB200_ERR_INVALID, "conv3d: empty output");
    }
    Operator op;
    op.type = Conv3d;
    op.inputs = {x, w};
    op.bias = bias;
    op.act = act;
    for (int i = 0; i < 3; ++i)
        op.pad3[i] = pad[i], op.stride3[i] = stride[i], op.dil3[i] = dil[i];
    g->tensors[w].weight = true;
    *out = g->new_tensor(od);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

// ref: Graph::convTrans, src/Graph/graph.cc:120-131; shape ConvTransOp::computeShape, src/Graph/operator.cc:1043-1063.
extern "C" int petb200_graph_convtrans(petb200_graph *g, int x, int w, int bias, int ph, int pw, int sh, int sw, int dh, int dw, int oph,
                                       int opw, int act, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    G_CHECK_T(g, w);
    const Dim &xd = g->tensors[x].dims, &wd = g->tensors[w].dims; // {n,h,w,f}, {r,s,f,c}
    if (xd.size() != 4 || wd.size() != 4 || xd[3] != wd[2])
        return g->fail(PETB200_ERR_INVALID, "convTrans: operands must be {n,h,w,f} and {r,s,f,c}");
    if (dh != 1 || dw != 1) // ref: ConvTransOp::checkValid, src/Graph/operator.cc:1103-1104
        return g->fail(PETB200_ERR_UNSUPPORTED, "convTrans: dilation must be 1");
    if (sh <= 0 || sw <= 0 || ph < 0 || pw < 0 || oph < 0 || opw < 0)
        return g->fail(PETB200_ERR_INVALID, "convTrans: bad stride/pad");
    const int oh = (xd[1] - 1) * sh - 2 * ph + (wd[0] - 1) + oph + 1, ow = (xd[2] - 1) * sw - 2 * pw + (wd[1] - 1) + opw + 1;
    if (oh <= 0 || ow <= 0)
        return g->fail(PETB200_ERR_INVALID, "convTrans: empty output");
    Operator op;
    op.type = ConvTrans;
    op.inputs = {x, w};
    op.bias = bias;
    op.act = act;
    op.ph = ph, op.pw = pw, op.sh = sh, op.sw = sw, op.dh = dh, op.dw = dw, op.oph = oph, op.opw = opw;
    g->tensors[w].weight = true;
    *out = g->new_tensor(Dim{xd[0], oh, ow, wd[3]});
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

// ref: Graph::g2bmm / Graph::gbmml, include/graph.h:80-90; shapes G2BMMOp::computeShape / GBMMLOp::computeShape,
// src/Graph/operator.cc:1414-1422,1552-1560; validity :1390-1412,1528-1550.
extern "C" int petb200_graph_g2bmm(petb200_graph *g, int a, int b, int width, int dilation, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, a);
    G_CHECK_T(g, b);
    const Dim &ad = g->tensors[a].dims, &bd = g->tensors[b].dims;
    if (ad.size() != 3 || ad != bd || width < 0 || dilation <= 0)
        return g->fail(PETB200_ERR_INVALID, "g2bmm: operands must be 3-D and of equal shape, width >= 0, dilation > 0");
    Operator op;
    op.type = G2BMM;
    op.inputs = {a, b};
    op.width = width, op.dilation = dilation;
    *out = g->new_tensor(Dim{ad[0], ad[1], 2 * width + 1});
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_gbmml(petb200_graph *g, int a, int b, int dilation, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, a);
    G_CHECK_T(g, b);
    const Dim &ad = g->tensors[a].dims, &bd = g->tensors[b].dims;
    if (ad.size() != 3 || bd.size() != 3 || ad[0] != bd[0] || ad[1] != bd[1] || ad[2] % 2 != 1 || dilation <= 0)
        return g->fail(PETB200_ERR_INVALID, "gbmml: operands must be [b,n,2w+1] and [b,n,m], dilation > 0");
    Operator op;
    op.type = GBMML;
    op.inputs = {a, b};
    op.width = (ad[2] - 1) / 2, op.dilation = dilation;
    *out = g->new_tensor(Dim{ad[0], ad[1], bd[2]});
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_matmul(petb200_graph *g, int a, int b, int bias, int transA, int transB, int act, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, a);
    G_CHECK_T(g, b);
    // ref: MatmulOp::dimExtend promotes 2-D operands to batch 1 (src/Graph/operator.cc:656-662)
    for (int t : {a, b})
        if (g->tensors[t].dims.size() == 2)
            g->tensors[t].dims.insert(g->tensors[t].dims.begin(), 1);
    const Dim &ad = g->tensors[a].dims, &bd = g->tensors[b].dims;
    // ref: MatmulOp::checkValid (src/Graph/operator.cc:697-715)
    if (ad.size() != 3 || bd.size() != 3 || ad[0] != bd[0] || (transA ? ad[1] : ad[2]) != (transB ? bd[2] : bd[1]))
        return g->fail(PETB200_ERR_INVALID, "matmul: operands must be 3-D with equal batch and inner extents");
    if (g->tensors[a].weight && g->tensors[b].weight)
        return g->fail(PETB200_ERR_INVALID, "matmul: both operands are weights");
    Operator op;
    op.type = Matmul;
    op.inputs = {a, b};
    op.bias = bias;
    op.transA = transA != 0, op.transB = transB != 0, op.act = act;
    *out = g->new_tensor({ad[0], transA ? ad[2] : ad[1], transB ? bd[1] : bd[2]});
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_transpose(petb200_graph *g, int x, const petb200_transpose_desc *desc, int *out) {
    if (!g || !desc || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    const Dim &d = g->tensors[x].dims;
    petb200_plan *trial = nullptr; // shape inference and validation are the lowering's
    int rc = petb200_transpose_plan(g->ctx, (int)d.size(), d.data(), 1, desc, &trial);
    if (rc)
        return g->pass(rc);
    int od[16];
    int nd = petb200_layout_out_dims(trial, od);
    petb200_plan_destroy(trial);
    Operator op;
    op.type = Transpose;
    op.inputs = {x};
    op.tr = *desc;
    *out = g->new_tensor(Dim(od, od + nd), g->tensors[x].weight); // ref: Graph::transpose keeps the Weight type
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

// A TransposeOp with the reference's padding / halo parameters (ref: TransposeOp::setPaddingSize + getTTParam,
// include/operator.h:1187-1190, src/Graph/operator.cc:2403-2441); see petb200_transpose_halo_plan.
extern "C" int petb200_graph_transpose_halo(petb200_graph *g, int x, const petb200_transpose_desc *desc, int pad, int extr, int copys,
                                            int dels, int *out) {
    if (!g || !desc || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    const Dim &d = g->tensors[x].dims;
    petb200_plan *trial = nullptr; // shape inference and validation are the lowering's
    int rc = petb200_transpose_halo_plan(g->ctx, (int)d.size(), d.data(), desc, pad, extr, copys, dels, &trial);
    if (rc)
        return g->pass(rc);
    int od[16];
    int nd = petb200_layout_out_dims(trial, od);
    petb200_plan_destroy(trial);
    Operator op;
    op.type = Transpose;
    op.inputs = {x};
    op.tr = *desc;
    op.halo[0] = pad, op.halo[1] = extr, op.halo[2] = copys, op.halo[3] = dels;
    *out = g->new_tensor(Dim(od, od + nd), g->tensors[x].weight);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

static int pad_slice(petb200_graph *g, OpType type, int x, const int *begin, const int *end, int *out) {
    if (!g || !begin || !end || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    const Dim &d = g->tensors[x].dims;
    Dim od(d.size());
    for (size_t i = 0; i < d.size(); ++i) {
        od[i] = type == Pad ? d[i] + begin[i] + end[i] : d[i] - begin[i] - end[i];
        if (begin[i] < 0 || end[i] < 0 || od[i] <= 0)
            return g->fail(PETB200_ERR_INVALID, "%s: window outside the tensor", type == Pad ? "pad" : "slice");
    }
    Operator op;
    op.type = type;
    op.inputs = {x};
    op.begin.assign(begin, begin + d.size());
    op.end.assign(end, end + d.size());
    *out = g->new_tensor(od, g->tensors[x].weight);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}
extern "C" int petb200_graph_pad(petb200_graph *g, int x, const int *begin, const int *end, int *out) { return pad_slice(g, Pad, x, begin, end, out); }
extern "C" int petb200_graph_slice(petb200_graph *g, int x, const int *begin, const int *end, int *out) { return pad_slice(g, Slice, x, begin, end, out); }

extern "C" int petb200_graph_extend(petb200_graph *g, int x, int dim, int num, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    Dim d = g->tensors[x].dims;
    if (dim < 0 || dim >= (int)d.size() || num < 0)
        return g->fail(PETB200_ERR_INVALID, "extend: bad dim/num");
    d[dim] *= num + 1;
    Operator op;
    op.type = Extend;
    op.inputs = {x};
    op.dim = dim, op.num = num;
    *out = g->new_tensor(d, g->tensors[x].weight);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_concat(petb200_graph *g, int n, const int *xs, int dim, int *out) {
    if (!g || !xs || !out || n < 1)
        return PETB200_ERR_INVALID;
    for (int i = 0; i < n; ++i)
        G_CHECK_T(g, xs[i]);
    Dim d = g->tensors[xs[0]].dims;
    if (dim < 0 || dim >= (int)d.size())
        return g->fail(PETB200_ERR_INVALID, "concat: bad dim");
    bool weight = true;
    d[dim] = 0;
    for (int i = 0; i < n; ++i) {
        const Dim &e = g->tensors[xs[i]].dims;
        if (e.size() != d.size())
            return g->fail(PETB200_ERR_INVALID, "concat: rank mismatch");
        for (size_t j = 0; j < e.size(); ++j)
            if ((int)j != dim && e[j] != g->tensors[xs[0]].dims[j])
                return g->fail(PETB200_ERR_INVALID, "concat: extents differ outside the concat dim");
        d[dim] += e[dim];
        weight = weight && g->tensors[xs[i]].weight;
    }
    Operator op;
    op.type = Concat;
    op.inputs.assign(xs, xs + n);
    op.dim = dim;
    *out = g->new_tensor(d, weight);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_split(petb200_graph *g, int x, int dim, int n, const int *sizes, int *outs) {
    if (!g || !sizes || !outs || n < 1)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    const Dim d = g->tensors[x].dims;
    if (dim < 0 || dim >= (int)d.size())
        return g->fail(PETB200_ERR_INVALID, "split: bad dim");
    int total = 0;
    for (int i = 0; i < n; ++i)
        total += sizes[i];
    // ref: SplitOp::computeShapeV — sizes are ratios scaled by dim / sum (src/Graph/operator.cc:2074-2101)
    if (total <= 0 || d[dim] % total)
        return g->fail(PETB200_ERR_INVALID, "split: ratios do not divide the dimension");
    Operator op;
    op.type = Split;
    op.inputs = {x};
    op.dim = dim;
    op.sizes.assign(sizes, sizes + n);
    for (int i = 0; i < n; ++i) {
        Dim od = d;
        od[dim] = d[dim] / total * sizes[i];
        if (od[dim] <= 0)
            return g->fail(PETB200_ERR_INVALID, "split: empty part");
        outs[i] = g->new_tensor(od, g->tensors[x].weight);
        op.outputs.push_back(outs[i]);
    }
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_eltwise(petb200_graph *g, int kind, int n, const int *xs, int *out) {
    if (!g || !xs || !out || kind < 0 || kind > 2 || n < 1 || n > 4 || (kind == 1 && n != 2))
        return PETB200_ERR_INVALID;
    for (int i = 0; i < n; ++i)
        G_CHECK_T(g, xs[i]);
    Operator op;
    op.type = kind == 0 ? Add : (kind == 1 ? Sub : Mul);
    op.inputs.assign(xs, xs + n);
    *out = g->new_tensor(g->tensors[xs[0]].dims); // ref: the output takes the first operand's shape; others are read modulo their size
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_activation(petb200_graph *g, int x, int act, int *out) {
    if (!g || !out || act < 1 || act > PETB200_ACT_GELU)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    Operator op;
    op.type = Activation;
    op.inputs = {x};
    op.act = act;
    *out = g->new_tensor(g->tensors[x].dims);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_pool(petb200_graph *g, int kind, int x, int kh, int kw, int ph, int pw, int sh, int sw, int *out) {
    if (!g || !out || kind < 0 || kind > 1 || kh <= 0 || kw <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    const Dim &d = g->tensors[x].dims;
    if (d.size() != 4)
        return g->fail(PETB200_ERR_INVALID, "pool: input must be 4-D");
    Dim od = {d[0], d[1], (d[2] - (kh - sh) + 2 * ph) / sh, (d[3] - (kw - sw) + 2 * pw) / sw};
    if (od[2] <= 0 || od[3] <= 0)
        return g->fail(PETB200_ERR_INVALID, "pool: empty output");
    Operator op;
    op.type = kind == 0 ? MaxPool : AvgPool;
    op.inputs = {x};
    op.kh = kh, op.kw = kw, op.ph = ph, op.pw = pw, op.sh = sh, op.sw = sw;
    *out = g->new_tensor(od);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_softmax(petb200_graph *g, int x, int axis, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    const int nd = (int)g->tensors[x].dims.size();
    if (axis < 0)
        axis += nd;
    if (axis < 0 || axis >= nd) // ref: SoftmaxOp::checkValid, include/operator.h:1890-1892
        return g->fail(PETB200_ERR_INVALID, "softmax over axis %d of a %d-D tensor", axis, nd);
    Operator op;
    op.type = Softmax;
    op.inputs = {x};
    op.axis = axis;
    *out = g->new_tensor(g->tensors[x].dims);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

// ref: Graph::div / pow / reduceMean / gather (include/graph.h; src/ffi/ffi_pet.cc:110-125).
extern "C" int petb200_graph_div(petb200_graph *g, int a, int b, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, a);
    G_CHECK_T(g, b);
    Operator op;
    op.type = Div;
    op.inputs = {a, b};
    // ref: the element-wise operators take the first input's shape; the second is read modulo its size (operator.cc:2983-3002)
    *out = g->new_tensor(g->tensors[a].dims);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_pow(petb200_graph *g, int x, int p, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    Operator op;
    op.type = Pow;
    op.inputs = {x};
    op.num = p;
    *out = g->new_tensor(g->tensors[x].dims);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_reducemean(petb200_graph *g, int x, int axis, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    Dim d = g->tensors[x].dims;
    if (axis < 0)
        axis += (int)d.size();
    if (axis < 0 || axis >= (int)d.size())
        return g->fail(PETB200_ERR_INVALID, "reduceMean: axis out of range");
    Operator op;
    op.type = ReduceMean;
    op.inputs = {x};
    op.axis = axis;
    d[axis] = 1; // ref: ReduceMeanOp::computeShape, src/Graph/operator.cc:3454-3458
    *out = g->new_tensor(d);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_gather(petb200_graph *g, int data, int indices, int axis, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, data);
    G_CHECK_T(g, indices);
    const Dim &a = g->tensors[data].dims;
    if (axis < 0)
        axis += (int)a.size();
    if (axis < 0 || axis >= (int)a.size())
        return g->fail(PETB200_ERR_INVALID, "gather: axis out of range");
    Dim d = g->tensors[indices].dims; // ref: GatherOp::computeShape, src/Graph/operator.cc:3420-3428
    for (int i = 0; i < (int)a.size(); ++i)
        if (i != axis)
            d.push_back(a[i]);
    if (d.size() > 8)
        return g->fail(PETB200_ERR_UNSUPPORTED, "gather: result has more than 8 dims");
    Operator op;
    op.type = Gather;
    op.inputs = {data, indices};
    op.axis = axis;
    *out = g->new_tensor(d);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_layernorm(petb200_graph *g, int x, int gamma, int beta, float eps, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    const int cols = g->tensors[x].dims.back();
    for (int t : {gamma, beta})
        if (t >= 0 && (!g->valid_tensor(t) || (int)g->tensors[t].size() != cols))
            return g->fail(PETB200_ERR_INVALID, "layernorm: gamma/beta must match the last axis");
    if ((gamma < 0) != (beta < 0))
        return g->fail(PETB200_ERR_INVALID, "layernorm: pass both gamma and beta or neither");
    Operator op;
    op.type = LayerNorm;
    op.inputs = {x};
    if (gamma >= 0) {
        op.inputs.push_back(gamma);
        op.inputs.push_back(beta);
    }
    op.eps = eps;
    *out = g->new_tensor(g->tensors[x].dims);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_batchnorm(petb200_graph *g, int x, int scale, int bias, int mean, int var, float eps, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    if (g->tensors[x].dims.size() < 2)
        return g->fail(PETB200_ERR_INVALID, "batchnorm: input needs a channel dim");
    const int c = g->tensors[x].dims[1];
    for (int t : {scale, bias, mean, var})
        if (!g->valid_tensor(t) || (int)g->tensors[t].size() != c)
            return g->fail(PETB200_ERR_INVALID, "batchnorm: parameter tensors must have one value per channel");
    Operator op;
    op.type = BatchNorm;
    op.inputs = {x, scale, bias, mean, var};
    op.eps = eps;
    *out = g->new_tensor(g->tensors[x].dims);
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_reshape(petb200_graph *g, int x, int nd, const int *dims, int *out) {
    if (!g || !dims || !out || nd < 1 || nd > 8)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    Dim d(dims, dims + nd);
    long long known = 1;
    int infer = -1;
    for (int i = 0; i < nd; ++i) {
        if (d[i] == -1) {
            if (infer >= 0)
                return g->fail(PETB200_ERR_INVALID, "reshape: more than one inferred dim");
            infer = i;
        } else if (d[i] <= 0) {
            return g->fail(PETB200_ERR_INVALID, "reshape: bad dim");
        } else {
            known *= d[i];
        }
    }
    const long long total = (long long)g->tensors[x].size();
    if (infer >= 0) {
        if (total % known)
            return g->fail(PETB200_ERR_INVALID, "reshape: sizes do not match");
        d[infer] = (int)(total / known);
    } else if (known != total) {
        return g->fail(PETB200_ERR_INVALID, "reshape: sizes do not match");
    }
    Operator op;
    op.type = Reshape;
    op.inputs = {x};
    *out = g->new_tensor(d, g->tensors[x].weight);
    g->tensors[*out].alias = x; // ref: reshape is pointer aliasing in the emitted program (code_engine.cc:1681-1690)
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_correction(petb200_graph *g, int x, int w, int bias, int y, int ph, int pw, int sh, int sw, int dh,
                                        int dw, int act, int oh0, int ohn, int ow0, int own, int *out) {
    if (!g || !out)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, x);
    G_CHECK_T(g, w);
    G_CHECK_T(g, y);
    const Dim &xd = g->tensors[x].dims, &wd = g->tensors[w].dims, &yd = g->tensors[y].dims;
    if (xd.size() != 4 || wd.size() != 4 || yd.size() != 4 || wd[1] <= 0 || xd[1] % wd[1])
        return g->fail(PETB200_ERR_INVALID, "correction: operands must be 4-D conv operands");
    Dim od = {xd[0], wd[0], conv_extent(xd[2], wd[2], ph, sh, dh), conv_extent(xd[3], wd[3], pw, sw, dw)};
    if (od != yd)
        return g->fail(PETB200_ERR_INVALID, "correction: y does not have the shape of the original convolution's output");
    if (oh0 < 0 || ohn <= 0 || oh0 + ohn > od[2] || ow0 < 0 || own <= 0 || ow0 + own > od[3])
        return g->fail(PETB200_ERR_INVALID, "correction: window outside the output");
    Operator op;
    op.type = Correction;
    op.inputs = {x, w, y};
    op.bias = bias;
    op.ph = ph, op.pw = pw, op.sh = sh, op.sw = sw, op.dh = dh, op.dw = dw, op.act = act;
    op.win[0] = oh0, op.win[1] = ohn, op.win[2] = ow0, op.win[3] = own;
    g->tensors[w].weight = true;
    *out = g->new_tensor(od);
    g->tensors[*out].alias = y; // corrected in place
    op.outputs = {*out};
    g->add_op(std::move(op));
    return PETB200_OK;
}

extern "C" int petb200_graph_set_outputs(petb200_graph *g, int n, const int *tensors) {
    if (!g || (n > 0 && !tensors))
        return PETB200_ERR_INVALID;
    for (int i = 0; i < n; ++i)
        G_CHECK_T(g, tensors[i]);
    g->outputs.assign(tensors, tensors + n);
    g->compiled = false;
    return PETB200_OK;
}

extern "C" int petb200_graph_compile(petb200_graph *g, int flags) {
    if (!g)
        return PETB200_ERR_INVALID;
    return g->compile(flags);
}

extern "C" int petb200_graph_set_data(petb200_graph *g, int tensor, const float *host, size_t n, petb200_stream stream) {
    if (!g || !host)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, tensor);
    if (!g->compiled)
        return g->fail(PETB200_ERR_INVALID, "set_data before compile");
    Tensor &t = g->tensors[tensor];
    if (n != t.size())
        return g->fail(PETB200_ERR_INVALID, "set_data: tensor holds %zu floats, %zu given", t.size(), n);
    if (cudaMemcpyAsync(dev_of(g, tensor), host, n * sizeof(float), cudaMemcpyHostToDevice, (cudaStream_t)stream) != cudaSuccess)
        return g->fail(PETB200_ERR_CUDA, "set_data: copy failed");
    t.has_data = true;
    if (t.weight) { // packed copies of this weight are stale: redo the hoisted work on next run
        if (g->exec)
            cudaGraphExecDestroy(g->exec);
        g->exec = nullptr;
        g->hoisted_done = false;
    }
    return PETB200_OK;
}

extern "C" int petb200_graph_get_data(petb200_graph *g, int tensor, float *host, size_t n, petb200_stream stream) {
    if (!g || !host)
        return PETB200_ERR_INVALID;
    G_CHECK_T(g, tensor);
    if (!g->compiled || n != g->tensors[tensor].size())
        return g->fail(PETB200_ERR_INVALID, "get_data: not compiled or size mismatch");
    if (cudaMemcpyAsync(host, dev_of(g, tensor), n * sizeof(float), cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess ||
        cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess)
        return g->fail(PETB200_ERR_CUDA, "get_data: copy failed");
    return PETB200_OK;
}

extern "C" void *petb200_graph_device_ptr(petb200_graph *g, int tensor) {
    return (g && g->valid_tensor(tensor) && g->compiled) ? dev_of(g, tensor) : nullptr;
}

extern "C" int petb200_graph_run(petb200_graph *g, petb200_stream stream) {
    if (!g)
        return PETB200_ERR_INVALID;
    if (!g->compiled)
        return g->fail(PETB200_ERR_INVALID, "run before compile");
    cudaStream_t st = (cudaStream_t)stream;
    if (!g->use_graph) {
        if (!g->hoisted_done) { // first run after (re)loading weights: hoisted work
            int rc = prepare_weights(g, st);
            if (rc)
                return rc;
            rc = g->run_all(st, false);
            g->hoisted_done = true;
            return rc;
        }
        return g->run_all(st, false);
    }
    if (!g->exec) {
        cudaStreamSynchronize(st); // inputs copied on the caller's stream must have landed before the capture pass
        int rc = g->capture();
        if (rc)
            return rc;
        return PETB200_OK; // the eager pass inside capture() already produced this run's outputs
    }
    if (cudaGraphLaunch(g->exec, st) != cudaSuccess)
        return g->fail(PETB200_ERR_CUDA, "graph launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return PETB200_OK;
}

extern "C" int petb200_graph_run_profiled(petb200_graph *g, petb200_stream stream, int slot, int nslots) {
    if (!g || slot < 0 || nslots <= 0 || slot >= nslots)
        return PETB200_ERR_INVALID;
    if (!g->compiled)
        return g->fail(PETB200_ERR_INVALID, "run before compile");
    cudaStream_t st = (cudaStream_t)stream;
    if (!g->hoisted_done) {
        int rc = prepare_weights(g, st);
        if (rc)
            return rc;
        g->hoisted_done = true;
    }
    int pairs = 0;
    for (auto &s : g->steps)
        if (!s.weight_only && !s.side && strncmp(s.kernel, "tc_", 3) != 0)
            ++pairs;
    if (nslots != g->prof_slots || pairs != g->prof_pairs) {
        for (cudaEvent_t e : g->prof_events)
            cudaEventDestroy(e);
        g->prof_events.assign((size_t)nslots * pairs * 2, nullptr);
        for (auto &e : g->prof_events)
            if (cudaEventCreate(&e) != cudaSuccess)
                return g->fail(PETB200_ERR_CUDA, "profile event creation failed");
        g->prof_slots = nslots;
        g->prof_pairs = pairs;
        g->prof_recorded.assign((size_t)nslots, 0);
    }
    g->prof_recorded[(size_t)slot] = 1;
    return g->run_all(st, false, slot);
}

extern "C" int petb200_graph_profile_other_ms(petb200_graph *g, int nslots, float *other_ms) {
    if (!g || !other_ms || nslots != g->prof_slots)
        return PETB200_ERR_INVALID;
    double total = 0;
    for (int slot = 0; slot < nslots; ++slot) {
        if (!g->prof_recorded[(size_t)slot])
            continue;
        g->prof_recorded[(size_t)slot] = 0;
        for (int pair = 0; pair < g->prof_pairs; ++pair) {
            const size_t i = ((size_t)slot * g->prof_pairs + pair) * 2;
            float ms = 0.f;
            if (cudaEventSynchronize(g->prof_events[i + 1]) != cudaSuccess ||
                cudaEventElapsedTime(&ms, g->prof_events[i], g->prof_events[i + 1]) != cudaSuccess)
                return g->fail(PETB200_ERR_CUDA, "profile event read failed");
            total += ms;
        }
    }
    *other_ms = (float)total;
    return PETB200_OK;
}

extern "C" int petb200_graph_num_launches(const petb200_graph *g) {
    int n = 0;
    if (g)
        for (auto &s : g->steps)
            if (!s.weight_only)
                n += s.launches;
    return n;
}
extern "C" int petb200_graph_num_steps(const petb200_graph *g) { return g ? (int)g->steps.size() : 0; }
extern "C" const char *petb200_graph_step_name(const petb200_graph *g, int i) {
    return (g && i >= 0 && i < (int)g->steps.size()) ? g->steps[i].name.c_str() : "";
}
extern "C" const char *petb200_graph_step_kernel(const petb200_graph *g, int i) {
    return (g && i >= 0 && i < (int)g->steps.size()) ? g->steps[i].kernel : "";
}

extern "C" int petb200_graph_perf(petb200_graph *g, int rounds, int warmup, float *total_ms, float *per_step_ms) {
    if (!g || !total_ms || rounds <= 0)
        return PETB200_ERR_INVALID;
    if (!g->compiled)
        return g->fail(PETB200_ERR_INVALID, "perf before compile");
    float total = 0.f;
    for (size_t i = 0; i < g->steps.size(); ++i) {
        Step &s = g->steps[i];
        float ms = 0.f;
        if (s.weight_only) {
            ms = 0.f; // ref: TransposeOp::perf returns 0 for weight inputs (src/Graph/operator.cc:2384-2386)
        } else if (s.plan) {
            // memo key: step type + every shape/attribute that determines the plan
            std::vector<int> key = {(int)s.type, (int)s.ops.size()};
            for (int o : s.ops) {
                const Operator &op = g->ops[o];
                for (int t : op.inputs) {
                    key.insert(key.end(), g->tensors[t].dims.begin(), g->tensors[t].dims.end());
                    key.push_back(g->tensors[t].weight ? -1 : -2); // (a constant operand is packed once, outside the timed launch)
                }
                int attrs[] = {op.ph, op.pw, op.sh, op.sw, op.dh, op.dw, op.act, op.bias >= 0, op.transA, op.transB, op.dim, op.num,
                               op.tr.split, op.tr.factor, op.tr.ngroups, op.win[0], op.win[1], op.win[2], op.win[3], op.oph, op.opw, op.width, op.dilation, op.halo[0], op.halo[1], op.halo[2], op.halo[3]};
                key.insert(key.end(), attrs, attrs + sizeof attrs / sizeof attrs[0]);
                key.insert(key.end(), op.tr.flat, op.tr.flat + 8);
                key.insert(key.end(), op.tr.group_sizes, op.tr.group_sizes + 8);
                key.insert(key.end(), op.pad3, op.pad3 + 3);
                key.insert(key.end(), op.stride3, op.stride3 + 3);
                key.insert(key.end(), op.begin.begin(), op.begin.end());
                key.insert(key.end(), op.end.begin(), op.end.end());
                // what else decides the plan: 3-D dilation, strided (folded-transpose) operands, a merged wide result
                key.insert(key.end(), op.dil3, op.dil3 + 3);
                key.push_back((int)op.seam_axis);
                key.push_back(op.mm_strided ? 1 : 0);
                for (int j = 0; j < 6; ++j) {
                    key.push_back((int)(op.mm_strides[j] & 0x7fffffff));
                    key.push_back((int)(op.mm_strides[j] >> 31));
                }
                if (op.merged_out >= 0)
                    key.insert(key.end(), g->tensors[op.merged_out].dims.begin(), g->tensors[op.merged_out].dims.end());
                key.push_back(-7); // separator: variable-length fields above
            }
            key.push_back(s.residual >= 0 ? 1 : 0);
            if (g->perf.check(key)) {
                ms = g->perf.get(key);
            } else {
                int rc = petb200_plan_time(s.plan, rounds, warmup, &ms, nullptr);
                if (rc == PETB200_ERR_UNSUPPORTED)
                    ms = 1e30f; // ref: unsupported algorithms cost INFINITY (src/Graph/operator.cc:428-433)
                else if (rc)
                    return g->pass(rc);
                g->perf.save(key, ms);
            }
        } else if (s.launches > 0) {
            // plan-less steps (elementwise, pooling, softmax, norms, concat/split) are timed in place on the graph's tensors
            cudaEvent_t e0, e1;
            cudaEventCreate(&e0);
            cudaEventCreate(&e1);
            for (int r = 0; r < std::max(1, warmup); ++r)
                g->run_step(s, nullptr);
            cudaEventRecord(e0, nullptr);
            for (int r = 0; r < rounds; ++r) {
                int rc = g->run_step(s, nullptr);
                if (rc)
                    return rc;
            }
            cudaEventRecord(e1, nullptr);
            cudaEventSynchronize(e1);
            cudaEventElapsedTime(&ms, e0, e1);
            ms /= (float)rounds;
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
        }
        if (per_step_ms)
            per_step_ms[i] = ms;
        total += ms;
    }
    *total_ms = total;
    return PETB200_OK;
}

extern "C" int petb200_graph_time(petb200_graph *g, int rounds, int warmup, float *ms, petb200_stream stream) {
    if (!g || !ms || rounds <= 0 || warmup < 0)
        return PETB200_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)stream;
    for (int i = 0; i < warmup + 1; ++i) {
        int rc = petb200_graph_run(g, stream);
        if (rc)
            return rc;
    }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, st);
    for (int i = 0; i < rounds; ++i) {
        int rc = petb200_graph_run(g, stream);
        if (rc) {
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            return rc;
        }
    }
    cudaEventRecord(e1, st);
    cudaEventSynchronize(e1);
    float total = 0.f;
    cudaEventElapsedTime(&total, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms = total / (float)rounds;
    return petb200_check_device_status(g->ctx, stream);
}
