// Reference-side binding: PET's operator classes costed by the petb200 backend.
//
// This translation unit is compiled against the reference's own headers and linked with the reference's own objects
// (compiled where they lie; see the Makefile beside this file).  It gives strong definitions to
//     tpm::<Op>::perf(PerfEngine*, int rounds, int warmupRounds)          (ref: include/operator.h:176-177)
// for every operator class the search costs through a library call or an analytic formula, and to
//     tpm::PerfEngine::allocMem()                                          (ref: src/Graph/perf_engine.cc:31-56)
// The reference's definitions of the same symbols are weakened at link time (objcopy --weaken-symbol on a copy of its
// objects; nothing of the reference is edited), so SearchEngine::getPerf / getMaxPerf / getTransPerf
// (ref: src/Graph/search_engine.cc:467-521) reach these bodies through the unchanged virtual call.  Contract kept:
// milliseconds per call; INFINITY for an operator the backend cannot run; results memoised through the unchanged
// PerfEngine::checkOpPerf / getOpPerf / saveOpPerf tables (ref: include/perf_engine.h:81-159).
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>
#include <cuda_runtime.h>

// The operator classes keep some of the parameters a backend needs (TransposeOp::split/factor, ConvTransOp::oph/opw, ...)
// private without getters; the binding reads them in place.
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
#include "graph.h"
#include "operator.h"
#include "perf_engine.h"
#include "tensor.h"
#undef private
#undef protected

#include "petb200.h"
#include "petb200_shim.h"

namespace {

std::atomic<long> g_perf_calls{0};
petb200_ctx *g_ctx = nullptr;
bool g_ctx_tried = false;

struct Scratch { // grow-only device buffers for the operators that are timed through run functions rather than plans
    float *p[3] = {nullptr, nullptr, nullptr};
    size_t n[3] = {0, 0, 0};
    float *get(int i, size_t floats) {
        if (floats > n[i]) {
            if (p[i])
                cudaFree(p[i]);
            p[i] = nullptr;
            n[i] = 0;
            if (cudaMalloc(&p[i], floats * sizeof(float)) != cudaSuccess)
                return nullptr;
            cudaMemset(p[i], 0, floats * sizeof(float));
            n[i] = floats;
        }
        return p[i];
    }
} g_scratch;

// Times `launch` (returns a petb200 status) with CUDA events on the default stream: the loop of the reference's perf
// bodies (ref: src/Graph/operator.cc:416-467) with device time instead of wall clock.
template <class F> double time_launches(F launch, int rounds, int warmup) {
    for (int i = 0; i < warmup; ++i)
        if (launch() != PETB200_OK)
            return INFINITY;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, nullptr);
    for (int i = 0; i < rounds; ++i)
        launch();
    cudaEventRecord(e1, nullptr);
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return petb200_check_device_status(g_ctx, nullptr) == PETB200_OK ? ms / rounds : INFINITY;
}

double time_plan(petb200_plan *plan, int rounds, int warmup) {
    float ms = 0.f;
    const int rc = petb200_plan_time(plan, rounds, warmup, &ms, nullptr);
    petb200_plan_destroy(plan);
    return rc == PETB200_OK ? (double)ms : INFINITY;
}

size_t numel(const tpm::Dim &d) {
    size_t n = 1;
    for (int v : d)
        n *= (size_t)v;
    return n;
}

int act_of(tpm::Operator::ActType a) { // the two enums list None/Relu/Sigmoid/Tanh in the same order
    return (int)a;
}

} // namespace

extern "C" petb200_ctx *petb200_shim_ctx(void) {
    if (!g_ctx_tried) {
        g_ctx_tried = true;
        int dev = 0;
        if (const char *e = getenv("PETB200_DEVICE"))
            dev = atoi(e);
        if (petb200_ctx_create(dev, &g_ctx) != PETB200_OK) {
            fprintf(stderr, "[petb200 shim] no backend context: %s\n", petb200_last_error(nullptr));
            g_ctx = nullptr;
        }
    }
    return g_ctx;
}
extern "C" long petb200_shim_perf_calls(void) { return g_perf_calls.load(); }

namespace tpm {

// The reference's generated banded-attention launchers (ref: src/custom_ops.cu:6-14) are referenced only by the timing
// bodies this file replaces; empty definitions keep the link closed without compiling its 5.8k lines of generated kernels.
void _sg2bmm(float *, float *, float *, int, int, int, int, int) {}
void _sgbmml(float *, float *, float *, int, int, int, int, int) {}

// PerfEngine's constructor takes 4 x 1 GiB + 7 GiB of device memory and fills 3 GiB with random numbers for the library
// calls to run on; the backend's plans own their operands, so nothing is taken here.  The destructor's cudaFree(nullptr)
// calls are no-ops.
void PerfEngine::allocMem() {
    inputPtr = weightPtr = outputPtr = biasPtr = workspace = nullptr;
    matA = matB = matC = nullptr;
}

double ConvOp::perf(PerfEngine *pe, int rounds, int warmupRounds) {
    ++g_perf_calls;
    const ConvArgs args = getArgs(pe ? pe->withPenalty() : 0);
    if (pe && pe->checkOpPerf(Conv, args))
        return pe->getOpPerf(Conv, args);
    const int a[16] = {std::get<0>(args), std::get<1>(args), std::get<2>(args), std::get<3>(args), std::get<4>(args), std::get<5>(args),
                       std::get<6>(args), std::get<7>(args), std::get<8>(args), std::get<9>(args), std::get<10>(args), std::get<11>(args),
                       std::get<12>(args), std::get<13>(args), std::get<14>(args), act_of((ActType)std::get<15>(args))};
    double t = INFINITY;
    petb200_plan *plan = nullptr;
    if (petb200_shim_ctx() && petb200_conv2d_plan(g_ctx, a, PETB200_ALGO_AUTO, &plan) == PETB200_OK)
        t = time_plan(plan, rounds, warmupRounds);
    if (pe) // algo and workspace mean nothing to this backend; the activation is always fused into the epilogue
        pe->saveOpPerf(Conv, args, ConvResult{t, CUDNN_CONVOLUTION_FWD_ALGO_IMPLICIT_GEMM, 0, true});
    return t;
}

double MatmulOp::perf(PerfEngine *pe, int rounds, int warmupRounds) {
    ++g_perf_calls;
    const MatmulArgs args = getArgs();
    if (pe && pe->checkOpPerf(Matmul, args))
        return pe->getOpPerf(Matmul, args);
    double t = INFINITY;
    petb200_plan *plan = nullptr;
    if (petb200_shim_ctx() &&
        petb200_matmul_plan(g_ctx, std::get<0>(args), std::get<1>(args), std::get<2>(args), std::get<3>(args), std::get<4>(args),
                            std::get<5>(args), bias != nullptr, act_of(act), PETB200_ALGO_AUTO, &plan) == PETB200_OK)
        t = time_plan(plan, rounds, warmupRounds);
    if (pe)
        pe->saveOpPerf(Matmul, args, MatmulResult{t, true, CUBLAS_GEMM_DEFAULT});
    return t;
}

double ConvTransOp::perf(PerfEngine *pe, int rounds, int warmupRounds) {
    ++g_perf_calls;
    const ConvArgs args = getArgs(pe ? pe->withPenalty() : 0);
    if (pe && pe->checkOpPerf(ConvTrans, args))
        return pe->getOpPerf(ConvTrans, args);
    const int a[18] = {std::get<0>(args), std::get<1>(args), std::get<2>(args), std::get<3>(args), std::get<4>(args), std::get<5>(args),
                       std::get<6>(args), std::get<7>(args), std::get<8>(args), std::get<9>(args), std::get<10>(args), std::get<11>(args),
                       std::get<12>(args), std::get<13>(args), std::get<14>(args), act_of((ActType)std::get<15>(args)), oph, opw};
    double t = INFINITY;
    petb200_plan *plan = nullptr;
    if (petb200_shim_ctx() && petb200_convtrans_plan(g_ctx, a, PETB200_ALGO_AUTO, &plan) == PETB200_OK)
        t = time_plan(plan, rounds, warmupRounds);
    if (pe)
        pe->saveOpPerf(ConvTrans, args, ConvTransResult{t, CUDNN_CONVOLUTION_BWD_DATA_ALGO_0, 0});
    return t;
}

double G2BMMOp::perf(PerfEngine *pe, int rounds, int warmupRounds) {
    ++g_perf_calls;
    const G2BMMGBMMLArgs args = getArgs();
    if (pe && pe->checkOpPerf(G2BMM, args))
        return pe->getOpPerf(G2BMM, args);
    float ms = INFINITY;
    const Dim &d = inputs[0]->getDims(); // [b, n, m]
    if (!petb200_shim_ctx() || petb200_banded_time(g_ctx, 0, d[0], d[1], d[2], width, dilation, rounds, warmupRounds, &ms, nullptr) != PETB200_OK)
        ms = INFINITY;
    if (pe)
        pe->saveOpPerf(G2BMM, args, ms);
    return ms;
}

double GBMMLOp::perf(PerfEngine *pe, int rounds, int warmupRounds) {
    ++g_perf_calls;
    const G2BMMGBMMLArgs args = getArgs();
    if (pe && pe->checkOpPerf(GBMML, args))
        return pe->getOpPerf(GBMML, args);
    float ms = INFINITY;
    const Dim &p = inputs[0]->getDims(), &v = inputs[1]->getDims(); // [b, n, 2w+1], [b, n, m]
    if (!petb200_shim_ctx() ||
        petb200_banded_time(g_ctx, 1, p[0], p[1], v[2], (p[2] - 1) / 2, dilation, rounds, warmupRounds, &ms, nullptr) != PETB200_OK)
        ms = INFINITY;
    if (pe)
        pe->saveOpPerf(GBMML, args, ms);
    return ms;
}

// The reference charges a transpose 2 * bytes / (200 MiB/ms), a constant tuned on another GPU, and nothing when it
// reads a weight or follows another transpose (those are hoisted / fused by its code generator; ref:
// src/Graph/operator.cc:2383-2400).  The two free cases are kept; the third is the measured time of the layout kernel.
double TransposeOp::perf(PerfEngine *pe, int rounds, int warmupRounds) {
    ++g_perf_calls;
    if (inputs[0]->getType() == Tensor::Weight)
        return 0;
    if (inputs[0]->getOutputOf() != nullptr && inputs[0]->getOutputOf()->getType() == Transpose)
        return 0;
    petb200_transpose_desc desc;
    if (!petb200_shim_fill_transpose_desc(this, &desc) || !petb200_shim_ctx())
        return INFINITY;
    const Dim &d = inputs[0]->getDims();
    petb200_plan *plan = nullptr;
    if (petb200_transpose_plan(g_ctx, (int)d.size(), d.data(), 1, &desc, &plan) != PETB200_OK)
        return INFINITY;
    return time_plan(plan, rounds, warmupRounds);
}

double PadOp::perf(PerfEngine *, int rounds, int warmupRounds) {
    ++g_perf_calls;
    const Dim &d = inputs[0]->getDims();
    petb200_plan *plan = nullptr;
    if (!petb200_shim_ctx() || petb200_pad_plan(g_ctx, (int)d.size(), d.data(), begin.data(), end.data(), &plan) != PETB200_OK)
        return INFINITY;
    return time_plan(plan, rounds, warmupRounds);
}

double SliceOp::perf(PerfEngine *, int rounds, int warmupRounds) {
    ++g_perf_calls;
    const Dim &d = inputs[0]->getDims();
    petb200_plan *plan = nullptr;
    if (!petb200_shim_ctx() || petb200_slice_plan(g_ctx, (int)d.size(), d.data(), begin.data(), end.data(), &plan) != PETB200_OK)
        return INFINITY;
    return time_plan(plan, rounds, warmupRounds);
}

static double pool_perf(Operator *op, PerfEngine *pe, int kind, int kh, int kw, int ph, int pw, int sh, int sw, int rounds, int warmup) {
    const Dim &d = op->getInputs()[0]->getDims(), &o = op->getOutputs()[0]->getDims();
    if (!petb200_shim_ctx() || d.size() != 4)
        return INFINITY;
    float *x = g_scratch.get(0, numel(d)), *y = g_scratch.get(1, numel(o));
    if (!x || !y)
        return INFINITY;
    return time_launches([&] { return petb200_pool2d_run(g_ctx, kind, x, y, d[0], d[1], d[2], d[3], kh, kw, ph, pw, sh, sw, nullptr); }, rounds,
                         warmup);
}

double MaxPoolOp::perf(PerfEngine *pe, int rounds, int warmupRounds) {
    ++g_perf_calls;
    const double t = pool_perf(this, pe, 0, kh, kw, ph, pw, sh, sw, rounds, warmupRounds);
    if (pe)
        pe->saveOpPerf(MaxPool, PoolArgs{kh, kw, ph, pw, sh, sw, dh, dw}, (float)t);
    return t;
}

double AvgPoolOp::perf(PerfEngine *pe, int rounds, int warmupRounds) {
    ++g_perf_calls;
    const double t = pool_perf(this, pe, 1, kh, kw, ph, pw, sh, sw, rounds, warmupRounds);
    if (pe)
        pe->saveOpPerf(AvgPool, PoolArgs{kh, kw, ph, pw, sh, sw, 1, 1}, (float)t);
    return t;
}

} // namespace tpm

// Element-wise operators and softmax: the reference's headers define these perf bodies inline (Add/Sub/Mul return 0,
// softmax charges dims[0] * 0.02 ms; ref: include/operator.h:1486-1577,1916-1918), i.e. as weak symbols in every object
// that uses them, so a strong symbol of the same name wins at link time.  A class member cannot be defined twice in one
// translation unit, hence plain functions carrying the members' mangled names (Itanium ABI: `this` is the first argument).
static double eltwise_perf(tpm::Operator *op, int kind, int rounds, int warmup) {
    ++g_perf_calls;
    if (!petb200_shim_ctx())
        return INFINITY;
    const size_t n_out = numel(op->getOutputs()[0]->getDims());
    const int n_in = (int)op->getInputs().size();
    if (n_in < 1 || n_in > 3)
        return INFINITY;
    const float *ins[3];
    size_t sizes[3];
    for (int i = 0; i < n_in; ++i) {
        sizes[i] = numel(op->getInputs()[i]->getDims());
        ins[i] = g_scratch.get(i == 0 ? 0 : 2, std::max(sizes[i], (size_t)1));
        if (!ins[i])
            return INFINITY;
    }
    float *out = g_scratch.get(1, n_out);
    if (!out)
        return INFINITY;
    return time_launches([&] { return petb200_eltwise_run(g_ctx, kind, n_in, ins, sizes, out, n_out, PETB200_ACT_NONE, nullptr); }, rounds, warmup);
}
extern "C" {
double petb200_shim_add_perf(tpm::AddOp *self, tpm::PerfEngine *, int rounds, int warmup) asm("_ZN3tpm5AddOp4perfEPNS_10PerfEngineEii");
double petb200_shim_sub_perf(tpm::SubOp *self, tpm::PerfEngine *, int rounds, int warmup) asm("_ZN3tpm5SubOp4perfEPNS_10PerfEngineEii");
double petb200_shim_mul_perf(tpm::MulOp *self, tpm::PerfEngine *, int rounds, int warmup) asm("_ZN3tpm5MulOp4perfEPNS_10PerfEngineEii");
double petb200_shim_softmax_perf(tpm::SoftmaxOp *self, tpm::PerfEngine *, int rounds, int warmup) asm("_ZN3tpm9SoftmaxOp4perfEPNS_10PerfEngineEii");
double petb200_shim_add_perf(tpm::AddOp *self, tpm::PerfEngine *, int rounds, int warmup) { return eltwise_perf(self, 0, rounds, warmup); }
double petb200_shim_sub_perf(tpm::SubOp *self, tpm::PerfEngine *, int rounds, int warmup) { return eltwise_perf(self, 1, rounds, warmup); }
double petb200_shim_mul_perf(tpm::MulOp *self, tpm::PerfEngine *, int rounds, int warmup) { return eltwise_perf(self, 2, rounds, warmup); }
double petb200_shim_softmax_perf(tpm::SoftmaxOp *self, tpm::PerfEngine *, int rounds, int warmup) {
    ++g_perf_calls;
    const tpm::Dim &d = self->getInputs()[0]->getDims();
    const int axis = self->getAxis();
    if (!petb200_shim_ctx() || d.empty() || (axis != (int)d.size() - 1 && axis != -1))
        return d.empty() ? 0.0 : d[0] * 0.02; // the reference's own charge where this backend has no kernel to time
    const size_t n = numel(d);
    float *x = g_scratch.get(0, n), *y = g_scratch.get(1, n);
    if (!x || !y)
        return INFINITY;
    return time_launches([&] { return petb200_softmax_run(g_ctx, x, y, n / (size_t)d.back(), d.back(), nullptr); }, rounds, warmup);
}
}

namespace tpm {
} // namespace tpm

// TransposeOp -> petb200_transpose_desc.  The constructor rewrote `after` into flat (post-split) indices: values above
// the split dim were shifted by one and -1 became split + 1 (ref: include/operator.h:1124-1144); the descriptor wants the
// constructor's own convention back.
extern "C" int petb200_shim_fill_transpose_desc(const void *transpose_op, petb200_transpose_desc *out) {
    const tpm::TransposeOp *op = static_cast<const tpm::TransposeOp *>(transpose_op);
    memset(out, 0, sizeof *out);
    out->split = op->split;
    out->factor = op->factor;
    const std::vector<tpm::PermItem> &groups = const_cast<tpm::TransposeOp *>(op)->after.getPerm();
    if (groups.size() > 8)
        return 0;
    out->ngroups = (int)groups.size();
    int k = 0;
    for (size_t i = 0; i < groups.size(); ++i) {
        const std::vector<int> &items = groups[i].getVec();
        out->group_sizes[i] = (int)items.size();
        for (int v : items) {
            if (k >= 8)
                return 0;
            if (op->split >= 0)
                v = (v == op->split + 1) ? -1 : (v > op->split + 1 ? v - 1 : v);
            out->flat[k++] = v;
        }
    }
    return 1;
}
