/* petb200 — C ABI of the Blackwell (sm_100a) execution and timing backend for PET operator graphs.
 *
 * Everything PET's  Operator::perf()  bodies and the program text emitted by  CodeEngine  obtain from
 * cuDNN / cuBLAS / TVM-generated kernels is offered here as plain C functions over device pointers.
 * Conventions (same as the reference at this boundary, include/operator.h:359 and src/Graph/operator.cc):
 *   - tensors are fp32, contiguous, NCHW / row-major; filters are [F, C/g, R, S]; groups = C / filter.dims[1];
 *   - conv is cross-correlation with symmetric padding; output extent (h - (r - sh)*dh + 2*ph) / sh;
 *   - every pointer argument named x/w/y/a/b/c/in/out is a DEVICE pointer owned by the caller;
 *   - every function returns a petb200_status; nothing exits the process and nothing synchronises the device
 *     except the *_time functions and petb200_ctx_destroy;
 *   - a ctx belongs to one host thread and one GPU; launches go to the stream passed in (0 = default stream).
 * Citations "ref:" are paths inside the reference project (thu-pacman/PET).
 */
#ifndef PETB200_H
#define PETB200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct petb200_ctx petb200_ctx;
typedef struct petb200_plan petb200_plan;
typedef void *petb200_stream; /* cudaStream_t */

typedef enum {
    PETB200_OK = 0,
    PETB200_ERR_INVALID = 1,     /* bad argument / shape the reference would also reject */
    PETB200_ERR_UNSUPPORTED = 2, /* valid operator this build has no kernel for; perf() maps it to INFINITY */
    PETB200_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed; text in petb200_last_error */
    PETB200_ERR_NOMEM = 4,
    PETB200_ERR_DEVICE = 5       /* a kernel reported an internal error (bounded wait expired, bad tile) */
} petb200_status;

/* ref: include/operator.h:95-100 (ActType None/Relu/Sigmoid/Tanh); GELU is an addition. */
enum { PETB200_ACT_NONE = 0, PETB200_ACT_RELU = 1, PETB200_ACT_SIGMOID = 2, PETB200_ACT_TANH = 3, PETB200_ACT_GELU = 4 };

/* Kernel families, the counterpart of the cuDNN algo enum ConvOp::perf sweeps (ref: src/Graph/operator.cc:297-306). */
enum {
    PETB200_ALGO_AUTO = 0,
    PETB200_ALGO_TC_3XTF32 = 1, /* tcgen05 implicit GEMM, error-compensated TF32 (fp32-grade accuracy) */
    PETB200_ALGO_SIMT_FP32 = 2, /* CUDA-core FFMA, exact fp32 products */
    PETB200_ALGO_TC_1XTF32 = 3, /* tcgen05, single TF32 pass (what cuDNN's default math mode does) */
    PETB200_ALGO_TC_BF16X3 = 4  /* tcgen05, error-compensated bf16: x = hi + lo in bf16, hi*hi + hi*lo + lo*hi with fp32
                                   accumulation; per-product error ~2^-17, half the tensor-core instructions of 3xTF32 */
};

/* ---- context ------------------------------------------------------------------------------------------------
 * Replaces PerfEngine's constructor-time state (ref: include/perf_engine.h:12-56, src/Graph/perf_engine.cc:31-56):
 * no 11 GiB scratch is taken; plans own what they need. */
int petb200_ctx_create(int device, petb200_ctx **out);
int petb200_ctx_destroy(petb200_ctx *ctx);
/* Text of the last error on this ctx (or of the last failed create when ctx is NULL). Never NULL. */
const char *petb200_last_error(const petb200_ctx *ctx);
const char *petb200_status_string(int status);
/* Number of kernel launches issued through this ctx since creation (bench bookkeeping). */
uint64_t petb200_launch_count(const petb200_ctx *ctx);
/* Synchronises `stream`, then reports PETB200_ERR_DEVICE if any kernel launched through this ctx gave up on one of
 * its bounded waits since the last check (every spin in the tensor-core kernels has an iteration limit and records
 * its give-up here instead of hanging the GPU).  The reference has no counterpart: it exits on any CUDA error
 * (ref: include/common.h:30-126). */
int petb200_check_device_status(petb200_ctx *ctx, petb200_stream stream);
void petb200_plan_destroy(petb200_plan *plan);
/* Bytes of device memory the plan owns (packed weights, scratch). */
size_t petb200_plan_device_bytes(const petb200_plan *plan);
/* Name of the kernel family the plan resolved to ("tc_3xtf32", "simt_fp32", "rowcopy", "tile", "gather" ...). */
const char *petb200_plan_kernel(const petb200_plan *plan);

/* ---- convolution --------------------------------------------------------------------------------------------
 * Replaces cudnnConvolutionForward / cudnnConvolutionBiasActivationForward as issued by ConvOp::perf
 * (ref: src/Graph/operator.cc:296-515) and emitted by CodeEngine (ref: src/Graph/code_engine.cc:797-831,869-977).
 * args = {n,c,h,w,f,r,s,ph,pw,sh,sw,dh,dw,g,bias,act}, the order of ConvArgs (ref: include/perf.h:9-25).
 * Semantics: ConvOp::compute (ref: src/Graph/operator.cc:94-158), then + bias[f], then activation. */
int petb200_conv2d_plan(petb200_ctx *ctx, const int args[16], int algo, petb200_plan **out);
/* Weight-only preprocessing hoisted out of the timed loop, like the reference's "preprocess operators for
 * weights" (ref: src/Graph/code_engine.cc:187-193).  Must be called once per weight tensor before *_run. */
int petb200_conv2d_set_weights(petb200_plan *plan, const float *w, petb200_stream stream);
int petb200_conv2d_run(petb200_plan *plan, const float *x, const float *bias, float *y, petb200_stream stream);
/* Output extents the plan computed (ref: ConvOp::computeShape, src/Graph/operator.cc:208-237). */
int petb200_conv2d_out_dims(const petb200_plan *plan, int out_nchw[4]);

/* Correction for partially equivalent rewrites.  The reference only *costs* the correction (Tensor::dimPenalty,
 * ref: include/tensor.h:138-159; markTransType, ref: src/Mutant/generator.cc:1889-1958); this recomputes, from the
 * ORIGINAL input x, the output window rows [oh0,oh0+ohn) x cols [ow0,ow0+own) of every image and filter of the
 * ORIGINAL-layout output y (other elements of y are left untouched).  It runs the same kernel as
 * petb200_conv2d_run with the same reduction order, so the rewritten graph + correction is bit-identical to
 * petb200_conv2d_run on the unsplit operator. */
int petb200_conv2d_correct(petb200_plan *plan, const float *x, const float *bias, float *y, int oh0, int ohn,
                           int ow0, int own, petb200_stream stream);

/* 3-D convolution (the reference has none; ref: src/Graph/operator.cc:23,283-294 asserts 4-D).
 * args = {n,c,d,h,w, f,t,r,s, pd,ph,pw, sd,sh,sw, dd,dh,dw, g,bias,act}. */
int petb200_conv3d_plan(petb200_ctx *ctx, const int args[21], int algo, petb200_plan **out);
int petb200_conv3d_set_weights(petb200_plan *plan, const float *w, petb200_stream stream);
int petb200_conv3d_run(petb200_plan *plan, const float *x, const float *bias, float *y, petb200_stream stream);
/* y = act(conv(x) + bias + residual) for a 2-D or 3-D convolution plan; residual has the shape of y (NULL: none).  The
 * reference runs the residual Add of a ResNet block as its own operator (ref: src/Graph/operator.cc, AddOp); this entry
 * lets an executor fold that Add (and the activation after it) into the convolution's epilogue.  Same arithmetic, in
 * the same order, as petb200_conv2d_run followed by petb200_eltwise_run(add, act). */
int petb200_conv_run_residual(petb200_plan *plan, const float *x, const float *bias, const float *residual, float *y,
                              petb200_stream stream);

/* ---- matmul ---------------------------------------------------------------------------------------------------
 * Replaces cublasGemmStridedBatchedEx / cublasGemmEx as issued by MatmulOp::perf (ref: src/Graph/operator.cc:728-832)
 * and emitted by CodeEngine (ref: src/Graph/code_engine.cc:1103-1169).  (transA,transB,b,m,n,k) is MatmulArgs
 * (ref: include/perf.h:40-46).  C[b,m,n] = op(A)·op(B) row-major (ref: MatmulOp::compute, operator.cc:620-654),
 * then + bias[n], then activation (bias before activation, unlike the emitted program, which is a reference bug). */
int petb200_matmul_plan(petb200_ctx *ctx, int transA, int transB, int b, int m, int n, int k, int has_bias, int act,
                        int algo, petb200_plan **out);
/* The same with operands that are strided views: strides = {A batch, A row, B batch, B row, C batch, C row} in elements,
 * the innermost dimension of each matrix contiguous ("B row" is the row stride of B as stored, [k][n] or [n][k]).  This
 * is how an executor folds the head split/merge transposes around attention matmuls (a [seq, heads, d] tensor read as
 * [heads, seq, d] is A batch = d, A row = heads*d) instead of running TransposeOp (ref: include/operator.h:1100-1202) as a
 * copy.  Served by the tensor-core kernel only: PETB200_ERR_UNSUPPORTED for transposed A, k % 4 != 0 or A strides that
 * are not multiples of 4 (the caller then keeps the copy).  A residual passed to petb200_matmul_run_residual uses the
 * C strides. */
int petb200_matmul_plan_strided(petb200_ctx *ctx, int transA, int transB, int b, int m, int n, int k, int has_bias, int act,
                                int algo, const long long strides[6], petb200_plan **out);
/* Declares B a weight: it is preprocessed once here (hoisted like the reference's weight-only operators,
 * ref: src/Graph/code_engine.cc:187-193) and petb200_matmul_run may then be called with b = NULL. */
int petb200_matmul_set_weights(petb200_plan *plan, const float *b, petb200_stream stream);
int petb200_matmul_run(petb200_plan *plan, const float *a, const float *b, const float *bias, float *c,
                       petb200_stream stream);
/* c = act(op(A)·op(B) + bias + residual); residual has the shape of c (NULL: none).  See petb200_conv_run_residual. */
int petb200_matmul_run_residual(petb200_plan *plan, const float *a, const float *b, const float *bias,
                                const float *residual, float *c, petb200_stream stream);

/* ---- layout / index operators (bit-exact copies of 32-bit words) ------------------------------------------
 * One TransposeOp (ref: include/operator.h:1100-1202; host definition src/Graph/operator.cc:2172-2210): input dim
 * `split` (or -1) is viewed as two dims by `factor` (factor>0: (D/factor,factor); factor<0: (|factor|,D/|factor|)),
 * then permuted/merged as `after` says.  `after` is given flattened: group i holds group_sizes[i] entries of
 * `flat`; the value -1 names the second of the two split dims, values > split name later input dims. */
typedef struct {
    int split;
    int factor;
    int ngroups;
    int group_sizes[8];
    int flat[8];
} petb200_transpose_desc;
/* A chain of n_ops TransposeOps applied left to right, fused into one kernel the way CodeEngine fuses
 * consecutive transposes (ref: src/Graph/code_engine.cc:1428-1459).  n_ops = 1 is a single TransposeOp. */
int petb200_transpose_plan(petb200_ctx *ctx, int nd, const int *dims, int n_ops, const petb200_transpose_desc *ops,
                           petb200_plan **out);
/* One TransposeOp carrying the reference's padding / halo parameters: what TransposeOp::getTTParam hands to the split
 * and merge micro-operations once TransposeOp::setPaddingSize is used (ref: include/operator.h:1184-1190,
 * src/Graph/operator.cc:2403-2441; index expressions src/Transpose/transpose.cc:22-42,70-106).  With n the inner extent
 * of the split or merged pair, at most one of extr/copys and one of pad/dels non-zero:
 *   extr  (split)  out[a][b] = in[a*(n+extr) + b]        skips the gaps a padded merge left       (Post of N2H/D2H/N2W/D2W)
 *   copys (split)  out[a][b] = in[a*n + b - a*copys]     dim == 2n, b < n+copys: halves overlapping by the halo (Pre of H2N/W2N)
 *   pad   (merge)  out[i] = i % (n+pad) < n ? in[i/(n+pad)][i%(n+pad)] : 0   extent A*(n+pad)-pad  (Pre of N2H/...)
 *   dels  (merge)  out[i] = in[i/(n-dels)][i%(n-dels) + (i/(n-dels))*dels]   A == 2               (Post of H2N/W2N)
 * pad/dels need the merged group to be a pair.  Run with petb200_layout_run; bit-exact. */
int petb200_transpose_halo_plan(petb200_ctx *ctx, int nd, const int *dims, const petb200_transpose_desc *op, int pad,
                                int extr, int copys, int dels, petb200_plan **out);
/* PadOp (ref: src/Graph/operator.cc:1640-1662), SliceOp (:1741-1773), ExtendOp (:2577-2597). */
int petb200_pad_plan(petb200_ctx *ctx, int nd, const int *dims, const int *begin, const int *end, petb200_plan **out);
int petb200_slice_plan(petb200_ctx *ctx, int nd, const int *dims, const int *begin, const int *end,
                       petb200_plan **out);
int petb200_extend_plan(petb200_ctx *ctx, int nd, const int *dims, int dim, int num, petb200_plan **out);
/* Output dims of a single-output layout plan; returns the rank. */
int petb200_layout_out_dims(const petb200_plan *plan, int *out_dims);
int petb200_layout_run(petb200_plan *plan, const void *in, void *out, petb200_stream stream);
/* ConcatOp (ref: src/Graph/operator.cc:1813-1850) / SplitOp with ratio sizes (ref: :1978-2020, shapes :2074-2101).
 * dims is the shape of the WHOLE tensor; extents[i] the extent of part i along `dim`. */
int petb200_concat_run(petb200_ctx *ctx, int nd, const int *dims, int dim, int n_parts, const int *extents,
                       const void *const *parts, void *whole, petb200_stream stream);
int petb200_split_run(petb200_ctx *ctx, int nd, const int *dims, int dim, int n_parts, const int *extents,
                      const void *whole, void *const *parts, petb200_stream stream);

/* ---- elementwise / activation / normalisation / pooling / softmax ------------------------------------------
 * AddOp/SubOp/MulOp with the reference's operand indexing in[j][i % size_j] (ref: src/Graph/operator.cc:2983-3002).
 * kind: 0 add, 1 sub, 2 mul.  Optional fused activation on the result. */
int petb200_eltwise_run(petb200_ctx *ctx, int kind, int n_in, const float *const *ins, const size_t *sizes, float *out,
                        size_t out_size, int act, petb200_stream stream);
/* ActivationOp (ref: include/operator.h:1940-2007; emitted as cudnnActivationForward, code_engine.cc:1248-1274). */
int petb200_activation_run(petb200_ctx *ctx, const float *x, float *y, size_t n, int act, petb200_stream stream);
/* BatchNormOp inference form (ref: src/Graph/operator.cc:2660-2681): x viewed as [outer, c, inner]. */
int petb200_batchnorm_run(petb200_ctx *ctx, const float *x, const float *scale, const float *bias, const float *mean,
                          const float *var, float *y, size_t outer, int c, size_t inner, float eps,
                          petb200_stream stream);
/* MaxPoolOp / AvgPoolOp with the cuDNN modes the reference selects (ref: src/Graph/code_engine.cc:1276-1329;
 * timing ref: src/Graph/operator.cc:2774-2967): max ignores padding, average excludes padding from the count.
 * kind 0 = max, 1 = average.  Output extent (h-(k-s)+2p)/s. */
int petb200_pool2d_run(petb200_ctx *ctx, int kind, const float *x, float *y, int n, int c, int h, int w, int kh, int kw,
                       int ph, int pw, int sh, int sw, petb200_stream stream);
/* Global average over all trailing dims: x [rows, cols] -> y [rows] (used for 3-D global pooling). */
int petb200_rowmean_run(petb200_ctx *ctx, const float *x, float *y, size_t rows, int cols, petb200_stream stream);
/* SoftmaxOp over the last axis (ref: online_softmax, src/Graph/code_engine.cc:424-486,1707-1731). */
int petb200_softmax_run(petb200_ctx *ctx, const float *x, float *y, size_t rows, int cols, petb200_stream stream);
/* The chain MatmulOp (transB) -> SoftmaxOp (last axis) -> MatmulOp of an attention head in one launch (ref: the three
 * operators' compute, src/Graph/operator.cc:632-651 and src/Graph/code_engine.cc:424-486): out[b] = softmax_rows(q[b] k[b]^T) v[b]
 * with q [bs, m, kd], k [bs, n, kd], v [bs, n, d], out [bs, m, d], in plain fp32 (no TF32), the softmax with the sums of
 * petb200_softmax_run.  strides = {q batch, q row, k batch, k row, v batch, v row, out batch, out row} in elements (rows
 * themselves contiguous), NULL for dense tensors.  Serves n, kd, d <= 128 (petb200_attention_supported returns 1);
 * anything else is PETB200_ERR_UNSUPPORTED and the caller runs the three operators. */
int petb200_attention_supported(int m, int n, int kd, int d);
int petb200_attention_run(petb200_ctx *ctx, const float *q, const float *k, const float *v, float *out, int bs, int m, int n,
                          int kd, int d, const long long *strides, petb200_stream stream);
/* SoftmaxOp over any axis (the operator carries one, ref: include/operator.h:1887-1938; the reference's emitted kernel
 * only serves the last): x viewed as [outer, len, inner], normalised over len.  inner == 1 is petb200_softmax_run. */
int petb200_softmax_axis_run(petb200_ctx *ctx, const float *x, float *y, size_t outer, int len, size_t inner,
                             petb200_stream stream);
/* LayerNorm over the last axis (no counterpart in the reference). gamma/beta may be NULL. */
int petb200_layernorm_run(petb200_ctx *ctx, const float *x, const float *gamma, const float *beta, float *y,
                          size_t rows, int cols, float eps, petb200_stream stream);

/* ---- the remaining small operators of the graph API ------------------------------------------------------------- */
/* DivOp (ref: include/operator.h:1580-1628): out[i] = a[i % size_a] / b[i % size_b].  The reference's host body subtracts
 * (ref: src/Graph/operator.cc:3258-3259) and its code generator has no case for the operator; this divides. */
int petb200_div_run(petb200_ctx *ctx, const float *a, size_t size_a, const float *b, size_t size_b, float *out,
                    size_t out_size, petb200_stream stream);
/* PowOp with its integer exponent (ref: include/operator.h:1630-1679; src/Graph/operator.cc:3330-3343). */
int petb200_pow_run(petb200_ctx *ctx, const float *x, float *y, size_t n, int p, petb200_stream stream);
/* ReduceMeanOp (ref: include/operator.h:1727-1782; shape src/Graph/operator.cc:3454-3458): x [outer, len, inner] -> y [outer, inner]. */
int petb200_reducemean_run(petb200_ctx *ctx, const float *x, float *y, size_t outer, int len, size_t inner,
                           petb200_stream stream);
/* GatherOp (ref: include/operator.h:1681-1725; shape src/Graph/operator.cc:3420-3428; index expression
 * src/Graph/code_engine.cc:1465-1487): data [outer, len, inner], n_idx int32 indices -> out [n_idx, outer, inner];
 * an index outside [0, len) yields 0.  Moves 32-bit words untouched. */
int petb200_gather_run(petb200_ctx *ctx, const void *data, const int *indices, void *out, size_t n_idx, size_t outer, int len,
                       size_t inner, petb200_stream stream);

/* ---- transposed convolution and banded attention products ------------------------------------------------------ */
/* ConvTransOp (ref: include/operator.h:466-614; host definition src/Graph/operator.cc:931-983; timing through
 * cudnnConvolutionBackwardData :1113-1287).  Channels-last tensors as the reference defines the operator:
 * x {n,h,w,f}, weight {r,s,f,c}, y {n,oh,ow,c}, oh = (h-1)*sh - 2*ph + (r-1) + oph + 1 (ref: operator.cc:1058-1059).
 * args = ConvTransOp::getArgs order (ref: include/operator.h:583-598) followed by the output padding, which the
 * reference leaves out of its tuple: {n,c,h,w,f,r,s,ph,pw,sh,sw,dh,dw,g,bias,act,oph,opw}.  Dilation other than 1 and
 * groups other than 1 return PETB200_ERR_UNSUPPORTED, as the reference refuses them (ref: operator.cc:1104,1134). */
int petb200_convtrans_plan(petb200_ctx *ctx, const int args[18], int algo, petb200_plan **out);
/* Weight-only work (filter flip, split for the tensor cores); once per weight tensor before *_run. */
int petb200_convtrans_set_weights(petb200_plan *plan, const float *w, petb200_stream stream);
int petb200_convtrans_run(petb200_plan *plan, const float *x, const float *bias, float *y, petb200_stream stream);
int petb200_convtrans_out_dims(const petb200_plan *plan, int out_nhwc[4]);

/* G2BMMOp / GBMMLOp (ref: include/operator.h:617-778), argument order of the reference's launchers
 * _sg2bmm / _sgbmml(a, b, y, bs, n, m, w, d) (ref: src/custom_ops.cu:6-14), any shape:
 *   g2bmm  y[b,i,j] = sum_k q[b,i,k] * k[b, i + d*(j-w), k]   q,k [bs,n,m] -> y [bs,n,2w+1]
 *   gbmml  y[b,i,k] = sum_j p[b,i,j] * v[b, i + d*(j-w), k]   p [bs,n,2w+1], v [bs,n,m] -> y [bs,n,m]
 * (ref: src/nnet/iterator_table.cc:597-633); rows outside [0,n) count as zero.
 * Dilation 1 with m a multiple of 4 and 16-byte aligned operands runs on the tensor cores (error-compensated TF32, the accuracy
 * of conv / matmul); the context then keeps one plan per shape, whose split copy of k / v is rewritten by every call: calls of
 * one shape on one context must not overlap (one stream, or one after the other).  Everything else runs the exact-fp32
 * CUDA-core kernels.  PETB200_BANDED_TC=0 in the environment keeps every call there. */
int petb200_g2bmm_run(petb200_ctx *ctx, const float *q, const float *k, float *y, int bs, int n, int m, int w, int d,
                      petb200_stream stream);
int petb200_gbmml_run(petb200_ctx *ctx, const float *p, const float *v, float *y, int bs, int n, int m, int w, int d,
                      petb200_stream stream);
/* Milliseconds per launch on library-owned operands, as G2BMMOp::perf / GBMMLOp::perf time the reference's kernels
 * (ref: src/Graph/operator.cc:1424-1465,1562-1598).  kind 0 = g2bmm, 1 = gbmml. */
int petb200_banded_time(petb200_ctx *ctx, int kind, int bs, int n, int m, int w, int d, int rounds, int warmup, float *ms,
                        petb200_stream stream);

/* ---- allocation-free entry point ------------------------------------------------------------------------------
 * Has no counterpart in the reference.  For callers that are not allowed to allocate device memory at the point where
 * they need a matmul — a thread that must not take the allocator's lock or its implicit device synchronisation, a
 * plug-in that was handed all of its buffers up front, code that runs after a memory pool has been sealed.  Such a
 * caller can create neither a context nor a plan (both own device memory), so this function takes neither: it gets
 * the operands and the result buffer, and the only other memory its two kernels touch is a fixed array of
 * PETB200_NOALLOC_SCRATCH_FLOATS floats that is part of the library image (every GPU that loads the library holds
 * those 8 MiB until the process exits).  It calls no cudaMalloc/cudaFree and no routine that allocates.
 *
 * C[b,m,n] = act(op(A)·op(B) + bias[n]), operands laid out as for petb200_matmul_run, computed by CUDA-core kernels in
 * two passes: partial sums of `ksplit` K slices go to the fixed array, a second kernel adds them in a fixed order.
 * Limit: ksplit * b * m * n <= PETB200_NOALLOC_SCRATCH_FLOATS, otherwise PETB200_ERR_UNSUPPORTED and a message saying so.
 * Sharing: all calls on a device use the same array and it keeps the last call's contents; nothing needs clearing,
 * because each call writes every word it later reads.  Calls that overlap on one GPU (two streams, two threads) race
 * on that array — issue them one after the other.
 * First call: the first call on each device looks up the array's device address and, since device code is loaded lazily,
 * makes the driver load the module that holds the array (the 8 MiB are reserved then, and the driver may synchronise).
 * Make one call on each device before entering the region where allocating or synchronising is not allowed, and before
 * starting a stream capture.  The address cache is safe against several host threads making that first call at once.
 * `err` (may be NULL) receives the reason when the status is not PETB200_OK. */
#define PETB200_NOALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)
int petb200_matmul_splitk_noalloc(int transA, int transB, int b, int m, int n, int k, int ksplit, const float *a_dev,
                                  const float *b_dev, const float *bias_dev, float *c_dev, int act, petb200_stream stream,
                                  char *err, size_t err_len);

/* ---- timing (the perf_engine side) --------------------------------------------------------------------------
 * Times `rounds` launches of a conv/matmul/layout plan after `warmup` launches on plan-owned scratch operands filled
 * with a fixed pattern, with CUDA events on the given stream; the counterpart of the loops in ConvOp::perf /
 * MatmulOp::perf (ref: src/Graph/operator.cc:416-467,770-812), which use wall clock around cudaDeviceSynchronize.
 * Returns milliseconds per launch through *ms. */
int petb200_plan_time(petb200_plan *plan, int rounds, int warmup, float *ms, petb200_stream stream);

#ifdef __cplusplus
}
#endif
#endif
