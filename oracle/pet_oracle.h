/* TEST INFRASTRUCTURE ONLY — CPU restatement of the reference's host operator semantics.
 * Nothing in the product links or imports this; tests/, the smoke check and bench.py's cpu_baseline leg do.
 * Citations are paths inside the reference project (thu-pacman/PET). */
#ifndef PET_ORACLE_H
#define PET_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORACLE_ACT_NONE = 0, ORACLE_ACT_RELU = 1, ORACLE_ACT_SIGMOID = 2, ORACLE_ACT_TANH = 3, ORACLE_ACT_GELU = 4 };

int oracle_num_threads(void);

/* ConvOp::compute, src/Graph/operator.cc:94-158 (loop order cc,rr,ss; out-of-image taps skipped);
 * output extent src/Graph/operator.cc:208-237.  x [n,c,h,w], wt [f,cpg,r,s], y [n,f,oh,ow]. */
void oracle_conv2d_u32(const uint32_t *x, const uint32_t *wt, uint32_t *y, int n, int c, int h, int w, int f,
                       int cpg, int r, int s, int ph, int pw, int sh, int sw, int dh, int dw);
/* Same loop nest in float; accumulate in float (wide=0) or double (wide=1); then +bias[f], then activation. */
void oracle_conv2d_f32(const float *x, const float *wt, const float *bias, float *y, int n, int c, int h, int w,
                       int f, int cpg, int r, int s, int ph, int pw, int sh, int sw, int dh, int dw, int act,
                       int wide);
/* Only output rows [row0,row1) of every image/channel are written (the seam rows a correction recomputes). */
void oracle_conv2d_rows_f32(const float *x, const float *wt, const float *bias, float *y, int n, int c, int h,
                            int w, int f, int cpg, int r, int s, int ph, int pw, int sh, int sw, int dh, int dw,
                            int act, int wide, int row0, int row1);
int oracle_conv_out(int in, int k, int pad, int stride, int dil);

/* 3-D extension of the same definition (the reference has no Conv3d): x [n,c,d,h,w], wt [f,cpg,t,r,s]. */
void oracle_conv3d_f32(const float *x, const float *wt, const float *bias, float *y, int n, int c, int d, int h,
                       int w, int f, int cpg, int t, int r, int s, int pd, int ph, int pw, int sd, int sh, int sw,
                       int dd, int dh, int dw, int act, int wide);

/* MatmulOp::compute, src/Graph/operator.cc:620-654.  A [b,m,k] (or [b,k,m] if transA), B [b,k,n] (or [b,n,k]). */
void oracle_matmul_u32(const uint32_t *a, const uint32_t *b, uint32_t *c, int bs, int m, int n, int k, int transA,
                       int transB);
void oracle_matmul_f32(const float *a, const float *b, const float *bias, float *c, int bs, int m, int n, int k,
                       int transA, int transB, int act, int wide);

/* TransposeOp::compute, src/Graph/operator.cc:2172-2210: split dim `split` by `factor` (sign picks which half is
 * the factor), scatter in[i] to the row-major position of the permuted coordinates.  `flat` lists the after-perm
 * with the constructor's numbering (-1 = second half of the split dim, indices > split shifted), grouped by
 * group_sizes.  Returns the number of output dims, or -1 if the split does not divide. */
int oracle_transpose_u32(const uint32_t *in, int nd, const int *dims, int split, int ngroups,
                         const int *group_sizes, const int *flat, int factor, uint32_t *out, int *out_dims);

/* PadOp operator.cc:1640-1662, SliceOp :1741-1773, ExtendOp :2577-2597. */
void oracle_pad_u32(const uint32_t *in, int nd, const int *dims, const int *begin, const int *end, uint32_t *out);
void oracle_slice_u32(const uint32_t *in, int nd, const int *dims, const int *begin, const int *end, uint32_t *out);
void oracle_extend_u32(const uint32_t *in, int nd, const int *dims, int dim, int num, uint32_t *out);
/* One part of ConcatOp (operator.cc:1813-1850) / SplitOp (operator.cc:1978-2020): copies a block whose extent along
 * `dim` is part_extent, placed at `offset` along `dim` of the whole tensor whose extent there is whole_extent.
 * to_whole=1 writes part->whole (concat), 0 reads whole->part (split).  outer = prod(dims[:dim]),
 * inner = prod(dims[dim+1:]). */
void oracle_axis_block_u32(const uint32_t *src, uint32_t *dst, size_t outer, size_t inner, int part_extent,
                           int whole_extent, int offset, int to_whole);

/* AddOp/SubOp/MulOp: operand j is read at i % size_j (operator.cc:2983-3002).  kind 0 add, 1 sub, 2 mul. */
void oracle_eltwise_u32(int kind, int n_in, const uint32_t *const *ins, const size_t *sizes, uint32_t *out,
                        size_t out_size);
void oracle_eltwise_f32(int kind, int n_in, const float *const *ins, const size_t *sizes, float *out,
                        size_t out_size);
/* BatchNormOp::compute operator.cc:2660-2681: (x-mean)*scale/sqrt(var+eps)+bias per channel (dim 1), the factor
 * formed in double as the reference does. */
void oracle_batchnorm_f32(const float *x, const float *scale, const float *bias, const float *mean,
                          const float *var, float *y, size_t outer, int c, size_t inner, float eps);
void oracle_activation_f32(const float *x, float *y, size_t n, int act);

/* Pooling as the reference's code generator configures cuDNN (src/Graph/code_engine.cc:1281-1311):
 * max ignores padding, average divides by the number of in-image taps.  Output extent (h-(k-s)+2p)/s. */
void oracle_maxpool_f32(const float *x, float *y, int n, int c, int h, int w, int kh, int kw, int ph, int pw, int sh,
                        int sw);
void oracle_avgpool_f32(const float *x, float *y, int n, int c, int h, int w, int kh, int kw, int ph, int pw, int sh,
                        int sw);
/* Softmax over the last axis as the reference's online_softmax kernel defines it (code_engine.cc:424-486). */
void oracle_softmax_f32(const float *x, float *y, size_t rows, int cols);
/* LayerNorm over the last axis (no counterpart in the reference; defined by the usual formula). */
void oracle_layernorm_f32(const float *x, const float *gamma, const float *beta, float *y, size_t rows, int cols,
                          float eps);

/* ConvTransOp, src/Graph/operator.cc:931-983 (whole tensor) and :1006-1040 (one position): x [n,h,w,f] (channels
 * last), wt [r,s,f,c], y [n,oh,ow,c] with oh = (h-1)*sh - 2*ph + dh*(r-1) + oph + 1 (:1058-1059).  Output (hh,ww)
 * gathers tap (rr,ss) from input row (hh + rr*dh - (r-ph-1)) / sh when that is a whole in-range number, times
 * wt[r-1-rr][s-1-ss]; taps with r - ((h+2ph-r) % sh) < rr (same for columns) are skipped, as the reference does.
 * The whole-tensor body of the reference reads its loop bounds from output dims 2 and 3 (ow and c); this
 * restatement uses oh and ow, which is what the one-position body computes. */
int oracle_convtrans_out(int in, int k, int pad, int stride, int dil, int out_pad);
void oracle_convtrans_u32(const uint32_t *x, const uint32_t *wt, uint32_t *y, int n, int h, int w, int f, int r, int s,
                          int c, int ph, int pw, int sh, int sw, int dh, int dw, int oph, int opw);
void oracle_convtrans_f32(const float *x, const float *wt, float *y, int n, int h, int w, int f, int r, int s, int c,
                          int ph, int pw, int sh, int sw, int dh, int dw, int oph, int opw, int wide);

/* Banded attention products.  The reference only has generated GPU kernels for one shape (include/custom_ops.cuh);
 * the definitions are the expressions its own rewriter uses for these operators (src/nnet/iterator_table.cc:597-633):
 *   G2BMM  y[b,i,j] = sum_k q[b,i,k] * kk[b, i + d*(j-w), k],  j in [0, 2w], rows outside [0,n) count as zero;
 *   GBMML  y[b,i,k] = sum_j p[b,i,j] * v[b, i + d*(j-w), k].
 * q, kk, v are [b,n,m]; the band tensors are [b,n,2w+1] (shapes: src/Graph/operator.cc:1415-1422). */
void oracle_g2bmm_f32(const float *q, const float *kk, float *y, int bs, int n, int m, int w, int d, int wide);
void oracle_gbmml_f32(const float *p, const float *v, float *y, int bs, int n, int m, int w, int d, int wide);

#ifdef __cplusplus
}
#endif
#endif
