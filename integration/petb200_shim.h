/* Entry points of the reference-side binding (integration/): the C-callable surface of a library that contains the
 * reference's own host code (graph, mutators, SearchEngine, CodeEngine, compiled where it lies) with its operator costs and
 * its execution served by libpetb200.  Used by tests and by a maintainer as the pattern for wiring the backend in. */
#ifndef PETB200_SHIM_H
#define PETB200_SHIM_H
#include <stddef.h>
#include "petb200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The process-wide backend context the perf bodies use (created on first use on device $PETB200_DEVICE, default 0);
 * NULL when no GPU / no sm_100 device is available — perf then returns INFINITY, the reference's "unsupported". */
petb200_ctx *petb200_shim_ctx(void);
/* How many times one of the overriding tpm::<Op>::perf bodies has run (proof that the virtual call lands here). */
long petb200_shim_perf_calls(void);
/* tpm::TransposeOp* -> descriptor of petb200_transpose_plan; returns 0 if the operator has more than 8 flat dims. */
int petb200_shim_fill_transpose_desc(const void *transpose_op, petb200_transpose_desc *out);

/* Calls perf(NULL, 1, 0) on a freshly built tpm::ConvOp / MatmulOp / TransposeOp / MaxPoolOp through the Operator base
 * pointer and returns the number of calls that reached the overriding bodies (4 when the link is right).  Needs no GPU:
 * without one every call answers INFINITY. */
int petb200_pet_perf_probe(double out_ms[4]);

/* Builds the one-convolution graph of the reference's rule tests (ref: src/Test/single_op_test_5.cc,
 * src/Test/single_rule_test_1_n2h.cc) — conv = {n,c,h,w,f,r,s,ph,pw,dh,dw}, stride 1 — and runs the reference's unchanged
 * SearchEngine::run on it (Generator as the mutation engine), every Operator::perf answered by the backend.  The graph it
 * chooses is then executed on the GPU by walking it into petb200_graph in CodeEngine::genCode's operator order
 * (ref: src/Graph/code_engine.cc:151-167), on host inputs x [n,c,h,w] and w [f,c,r,s]; y [n,f,oh,ow] receives the result
 * and y_direct (may be NULL) the result of the original single operator.  report receives the chosen graph's operator
 * list, one per line; perf_ms = {SearchEngine::getPerf of the original graph, of the chosen graph}. */
int petb200_pet_search_conv(const int conv[11], const float *x, const float *w, float *y, float *y_direct, char *report,
                            size_t report_len, double perf_ms[2]);

/* Builds, with the reference's own Graph API, the mutant its generator derives for that convolution — TransposeOp H->N,
 * ConvOp on the two stacked halves, TransposeOp N->H (ref: src/Mutant/generator.cc:1027-1046) — and evaluates it twice on
 * the same integer-valued inputs: with the reference's own host operators (SubGraph::compute, uint32 arithmetic,
 * ref: src/Graph/graph.cc:1353-1386) into y_host, and on the GPU through the walker into y_gpu.  The two agree exactly
 * (modulo 2^32), seam rows included: both compute the partially equivalent graph as written. */
int petb200_pet_run_h2n_rewrite(const int conv[11], const float *x, const float *w, float *y_gpu, unsigned *y_host, char *report,
                                size_t report_len);

#ifdef __cplusplus
}
#endif
#endif
