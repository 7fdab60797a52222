/* petb200 graph layer — C ABI of the host side that sits above the operator kernels (petb200.h).
 *
 * It mirrors, for the execution/timing path only, the reference's graph API and the two engines that consume it:
 *   - builder calls = tpm::Graph::{tensor,conv,matmul,transpose,pad,slice,concat,split,extend,add,sub,mul,relu,sigmoid,
 *     tanh,maxpool,avgpool,softmax,batchnorm,reshape,flatten,identity}  (ref: include/graph.h:38-190; the same set the
 *     pybind11 module exposes, ref: src/ffi/ffi_pet.cc:32-175), plus conv3d / gelu / layernorm / correction, which the
 *     reference lacks;
 *   - petb200_graph_compile + petb200_graph_run replace CodeEngine::genCode + the emitted program
 *     (ref: src/Graph/code_engine.cc:91-256): operators are ordered topologically (Kahn, as SubGraph::compute does,
 *     ref: src/Graph/graph.cc:1355-1386), chains of transposes with single consumers are fused into one kernel
 *     (ref: code_engine.cc:1428-1459), an activation that is the only consumer of a conv/matmul/add is folded into
 *     its epilogue (ref: SearchEngine::fuse, src/Graph/search_engine.cc:837-892), reshape/identity/flatten alias their
 *     input (ref: code_engine.cc:1681-1690), weight-only work is hoisted out of the replayed sequence
 *     (ref: code_engine.cc:187-193), and the whole sequence is captured in a CUDA graph;
 *   - petb200_graph_perf replaces SearchEngine::getPerf over Operator::perf (ref: src/Graph/search_engine.cc:467-495):
 *     per-operator measured milliseconds, memoised by argument tuple like PerfEngine's tables
 *     (ref: include/perf_engine.h:15-21,81-159); petb200_graph_time is the reference program's own protocol: warm-up
 *     + timed replays of the whole graph between two CUDA events (ref: code_engine.cc:195-217).
 * Tensors and operators are named by small integer ids; every call returns a petb200_status.
 */
#ifndef PETB200_GRAPH_H
#define PETB200_GRAPH_H
#include "petb200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct petb200_graph petb200_graph;

int petb200_graph_create(petb200_ctx *ctx, petb200_graph **out);
void petb200_graph_destroy(petb200_graph *g);
const char *petb200_graph_last_error(const petb200_graph *g);

/* Graph::tensor (ref: include/graph.h:19-20).  is_weight marks Tensor::Weight (ref: include/tensor.h:16-21). */
int petb200_graph_tensor(petb200_graph *g, int nd, const int *dims, int is_weight, int *tensor);
int petb200_graph_tensor_dims(const petb200_graph *g, int tensor, int *dims); /* returns the rank, or -1 */

/* Each builder appends one operator and returns the id(s) of its freshly created output tensor(s).
 * `bias` is a tensor id or -1; `act` is a PETB200_ACT_* value applied after the bias. */
int petb200_graph_conv(petb200_graph *g, int x, int w, int bias, int ph, int pw, int sh, int sw, int dh, int dw, int act,
                       int *out);
int petb200_graph_conv3d(petb200_graph *g, int x, int w, int bias, const int pad[3], const int stride[3], const int dil[3],
                         int act, int *out);
int petb200_graph_matmul(petb200_graph *g, int a, int b, int bias, int transA, int transB, int act, int *out);
/* ref: Graph::convTrans (src/Graph/graph.cc:120-131): x {n,h,w,f}, w {r,s,f,c} -> {n,oh,ow,c}; dilation must be 1. */
int petb200_graph_convtrans(petb200_graph *g, int x, int w, int bias, int ph, int pw, int sh, int sw, int dh, int dw, int oph,
                            int opw, int act, int *out);
/* ref: Graph::g2bmm / Graph::gbmml (include/graph.h:80-90): banded Q.K^T -> [b,n,2*width+1]; banded P.V -> [b,n,m]. */
int petb200_graph_g2bmm(petb200_graph *g, int a, int b, int width, int dilation, int *out);
int petb200_graph_gbmml(petb200_graph *g, int a, int b, int dilation, int *out);
int petb200_graph_transpose(petb200_graph *g, int x, const petb200_transpose_desc *desc, int *out);
/* TransposeOp with padding / halo parameters (ref: TransposeOp::setPaddingSize, include/operator.h:1187-1190); at most one of
 * extr/copys and one of pad/dels non-zero, see petb200_transpose_halo_plan. */
int petb200_graph_transpose_halo(petb200_graph *g, int x, const petb200_transpose_desc *desc, int pad, int extr, int copys,
                                 int dels, int *out);
int petb200_graph_pad(petb200_graph *g, int x, const int *begin, const int *end, int *out);
int petb200_graph_slice(petb200_graph *g, int x, const int *begin, const int *end, int *out);
int petb200_graph_extend(petb200_graph *g, int x, int dim, int num, int *out);
int petb200_graph_concat(petb200_graph *g, int n, const int *xs, int dim, int *out);
int petb200_graph_split(petb200_graph *g, int x, int dim, int n, const int *ratio_sizes, int *outs);
int petb200_graph_eltwise(petb200_graph *g, int kind /*0 add,1 sub,2 mul*/, int n, const int *xs, int *out);
int petb200_graph_activation(petb200_graph *g, int x, int act, int *out);
int petb200_graph_pool(petb200_graph *g, int kind /*0 max,1 avg*/, int x, int kh, int kw, int ph, int pw, int sh, int sw,
                       int *out);
int petb200_graph_softmax(petb200_graph *g, int x, int axis, int *out);
/* ref: Graph::div / pow / reduceMean / gather (src/ffi/ffi_pet.cc:110-125).  `indices` of gather is a tensor whose 32-bit
 * words are int32 values. */
int petb200_graph_div(petb200_graph *g, int a, int b, int *out);
int petb200_graph_pow(petb200_graph *g, int x, int p, int *out);
int petb200_graph_reducemean(petb200_graph *g, int x, int axis, int *out);
int petb200_graph_gather(petb200_graph *g, int data, int indices, int axis, int *out);
int petb200_graph_layernorm(petb200_graph *g, int x, int gamma, int beta, float eps, int *out);
int petb200_graph_batchnorm(petb200_graph *g, int x, int scale, int bias, int mean, int var, float eps, int *out);
int petb200_graph_reshape(petb200_graph *g, int x, int nd, const int *dims, int *out); /* alias; -1 infers one dim */
/* Correction of a partially equivalent rewrite: recomputes window rows [oh0,oh0+ohn) x cols [ow0,ow0+own) of `y`
 * (the rewritten sub-graph's output in the ORIGINAL layout) from the original conv operands.  The output tensor
 * aliases `y`.  No counterpart in the reference (it only models the cost, ref: include/tensor.h:138-159). */
int petb200_graph_correction(petb200_graph *g, int x, int w, int bias, int y, int ph, int pw, int sh, int sw, int dh,
                             int dw, int act, int oh0, int ohn, int ow0, int own, int *out);

/* Graph::setOutputs (ref: include/graph.h:184). Tensors nobody consumes are outputs by default. */
int petb200_graph_set_outputs(petb200_graph *g, int n, const int *tensors);

/* Orders, fuses, plans, allocates device memory.  flags: bit 0 = do not fuse; bit 1 = do not capture a CUDA graph;
 * bit 2 = keep every step on the caller's stream (no side stream for shortcut branches); bit 3 = keep an attention head
 * (Matmul(transB) -> Softmax -> Matmul) as three steps instead of one petb200_attention_run launch. */
int petb200_graph_compile(petb200_graph *g, int flags);
/* Host <-> device transfer of one tensor (n floats). set_data on a weight re-runs the weight preprocessing. */
int petb200_graph_set_data(petb200_graph *g, int tensor, const float *host, size_t n, petb200_stream stream);
int petb200_graph_get_data(petb200_graph *g, int tensor, float *host, size_t n, petb200_stream stream);
void *petb200_graph_device_ptr(petb200_graph *g, int tensor);
/* One forward pass on `stream` (a CUDA-graph launch unless compiled with bit 1). */
int petb200_graph_run(petb200_graph *g, petb200_stream stream);
/* One forward pass issued step by step on `stream` (no CUDA graph), instrumented for the roofline accounting of a
 * benchmark: a CUDA event is recorded on the stream before and after every step that is NOT a tensor-core launch (pooling,
 * element-wise, softmax, LayerNorm, layout, small-m matmul ...), into slot `slot` of `nslots` event sets, so that `nslots`
 * consecutive passes can be issued back to back without reading anything in between.  Tensor-core steps run exactly as
 * in petb200_graph_run, chained by programmatic dependent launch.  petb200_graph_profile_other_ms then returns the summed
 * duration of those other steps over the slots run since its previous call (it waits for them): the time of a region made of such passes, minus this sum, is the time the
 * tensor-core kernel was running.  The counterpart in the reference is the per-operator timing inside Operator::perf
 * (ref: src/Graph/operator.cc:416-467); the reference times whole programs only with wall clock (ref: code_engine.cc:195-217). */
int petb200_graph_run_profiled(petb200_graph *g, petb200_stream stream, int slot, int nslots);
int petb200_graph_profile_other_ms(petb200_graph *g, int nslots, float *other_ms);
/* Kernel launches one pass issues; operators left after fusion. */
int petb200_graph_num_launches(const petb200_graph *g);
int petb200_graph_num_steps(const petb200_graph *g);
/* Name ("conv", "transpose_chain", ...) and kernel family of step i, for reports. */
const char *petb200_graph_step_name(const petb200_graph *g, int i);
const char *petb200_graph_step_kernel(const petb200_graph *g, int i);

/* Sum over operators of the measured per-operator time (ms), each timed alone for `rounds` launches after `warmup`
 * and memoised by argument tuple; per_step_ms (may be NULL) receives the individual times. */
int petb200_graph_perf(petb200_graph *g, int rounds, int warmup, float *total_ms, float *per_step_ms);
/* Whole-graph replay: `warmup` passes, then `rounds` passes between two CUDA events; ms per pass. */
int petb200_graph_time(petb200_graph *g, int rounds, int warmup, float *ms, petb200_stream stream);

#ifdef __cplusplus
}
#endif
#endif
