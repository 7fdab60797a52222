/* TEST INFRASTRUCTURE ONLY — CPU restatement of the reference's host operator semantics (see pet_oracle.h).
 * Pinned against the reference's own host operators (oracle/_ref/libpetref.so) and against the fixtures under
 * tests/golden/ by tests/test_oracle.py.  Not linked, imported or executed by the product. */
#include "pet_oracle.h"
#include <math.h>
#include <omp.h>
#include <stdlib.h>
#include <string.h>

int oracle_num_threads(void) { return omp_get_max_threads(); }

int oracle_conv_out(int in, int k, int pad, int stride, int dil) {
    /* src/Graph/operator.cc:220-221: oh = (h - (r - sh) * dh + ph * 2) / sh */
    return (in - (k - stride) * dil + pad * 2) / stride;
}

static inline float act_f32(float v, int act) {
    switch (act) {
    case ORACLE_ACT_RELU:
        return v > 0.f ? v : 0.f;
    case ORACLE_ACT_SIGMOID:
        return 1.f / (1.f + expf(-v));
    case ORACLE_ACT_TANH:
        return tanhf(v);
    case ORACLE_ACT_GELU:
        return 0.5f * v * (1.f + erff(v * 0.70710678118654752440f));
    default:
        return v;
    }
}

void oracle_conv2d_u32(const uint32_t *x, const uint32_t *wt, uint32_t *y, int n, int c, int h, int w, int f,
                       int cpg, int r, int s, int ph, int pw, int sh, int sw, int dh, int dw) {
    int g = c / cpg;
    int oh = oracle_conv_out(h, r, ph, sh, dh), ow = oracle_conv_out(w, s, pw, sw, dw);
    for (int nn = 0; nn < n; nn++) {
#pragma omp parallel for
        for (int ff = 0; ff < f; ff++) {
            int gidx = ff / (f / g);
            for (int hh = 0; hh < oh; hh++)
                for (int ww = 0; ww < ow; ww++) {
                    uint32_t val = 0;
                    for (int cc = 0; cc < cpg; cc++)
                        for (int rr = 0; rr < r; rr++)
                            for (int ss = 0; ss < s; ss++) {
                                int posH = hh * sh + rr * dh - ph, posW = ww * sw + ss * dw - pw;
                                if (posH < 0 || posH >= h || posW < 0 || posW >= w)
                                    continue;
                                size_t io = posW + (size_t)w * (posH + (size_t)h * ((cc + gidx * cpg) + (size_t)c * nn));
                                size_t wo = ss + (size_t)s * (rr + (size_t)r * (cc + (size_t)cpg * ff));
                                val += wt[wo] * x[io];
                            }
                    y[ww + (size_t)ow * (hh + (size_t)oh * (ff + (size_t)f * nn))] = val;
                }
        }
    }
}

void oracle_conv2d_rows_f32(const float *x, const float *wt, const float *bias, float *y, int n, int c, int h,
                            int w, int f, int cpg, int r, int s, int ph, int pw, int sh, int sw, int dh, int dw,
                            int act, int wide, int row0, int row1) {
    int g = c / cpg;
    int oh = oracle_conv_out(h, r, ph, sh, dh), ow = oracle_conv_out(w, s, pw, sw, dw);
    if (row0 < 0)
        row0 = 0;
    if (row1 > oh)
        row1 = oh;
    for (int nn = 0; nn < n; nn++) {
#pragma omp parallel for
        for (int ff = 0; ff < f; ff++) {
            int gidx = ff / (f / g);
            for (int hh = row0; hh < row1; hh++)
                for (int ww = 0; ww < ow; ww++) {
                    float accf = 0.f;
                    double accd = 0.0;
                    for (int cc = 0; cc < cpg; cc++)
                        for (int rr = 0; rr < r; rr++)
                            for (int ss = 0; ss < s; ss++) {
                                int posH = hh * sh + rr * dh - ph, posW = ww * sw + ss * dw - pw;
                                if (posH < 0 || posH >= h || posW < 0 || posW >= w)
                                    continue;
                                size_t io = posW + (size_t)w * (posH + (size_t)h * ((cc + gidx * cpg) + (size_t)c * nn));
                                size_t wo = ss + (size_t)s * (rr + (size_t)r * (cc + (size_t)cpg * ff));
                                if (wide)
                                    accd += (double)wt[wo] * (double)x[io];
                                else
                                    accf += wt[wo] * x[io];
                            }
                    float v = wide ? (float)(accd + (bias ? (double)bias[ff] : 0.0)) : accf + (bias ? bias[ff] : 0.f);
                    y[ww + (size_t)ow * (hh + (size_t)oh * (ff + (size_t)f * nn))] = act_f32(v, act);
                }
        }
    }
}

void oracle_conv2d_f32(const float *x, const float *wt, const float *bias, float *y, int n, int c, int h, int w,
                       int f, int cpg, int r, int s, int ph, int pw, int sh, int sw, int dh, int dw, int act,
                       int wide) {
    oracle_conv2d_rows_f32(x, wt, bias, y, n, c, h, w, f, cpg, r, s, ph, pw, sh, sw, dh, dw, act, wide, 0,
                           oracle_conv_out(h, r, ph, sh, dh));
}

void oracle_conv3d_f32(const float *x, const float *wt, const float *bias, float *y, int n, int c, int d, int h,
                       int w, int f, int cpg, int t, int r, int s, int pd, int ph, int pw, int sd, int sh, int sw,
                       int dd, int dh, int dw, int act, int wide) {
    int g = c / cpg;
    int od = oracle_conv_out(d, t, pd, sd, dd), oh = oracle_conv_out(h, r, ph, sh, dh),
        ow = oracle_conv_out(w, s, pw, sw, dw);
    for (int nn = 0; nn < n; nn++) {
#pragma omp parallel for collapse(2)
        for (int ff = 0; ff < f; ff++)
            for (int zz = 0; zz < od; zz++) {
                int gidx = ff / (f / g);
                for (int hh = 0; hh < oh; hh++)
                    for (int ww = 0; ww < ow; ww++) {
                        float accf = 0.f;
                        double accd = 0.0;
                        for (int cc = 0; cc < cpg; cc++)
                            for (int tt = 0; tt < t; tt++)
                                for (int rr = 0; rr < r; rr++)
                                    for (int ss = 0; ss < s; ss++) {
                                        int posD = zz * sd + tt * dd - pd, posH = hh * sh + rr * dh - ph,
                                            posW = ww * sw + ss * dw - pw;
                                        if (posD < 0 || posD >= d || posH < 0 || posH >= h || posW < 0 || posW >= w)
                                            continue;
                                        size_t io = posW + (size_t)w * (posH + (size_t)h * (posD + (size_t)d * ((cc + gidx * cpg) + (size_t)c * nn)));
                                        size_t wo = ss + (size_t)s * (rr + (size_t)r * (tt + (size_t)t * (cc + (size_t)cpg * ff)));
                                        if (wide)
                                            accd += (double)wt[wo] * (double)x[io];
                                        else
                                            accf += wt[wo] * x[io];
                                    }
                        float v = wide ? (float)(accd + (bias ? (double)bias[ff] : 0.0)) : accf + (bias ? bias[ff] : 0.f);
                        y[ww + (size_t)ow * (hh + (size_t)oh * (zz + (size_t)od * (ff + (size_t)f * nn)))] = act_f32(v, act);
                    }
            }
    }
}

void oracle_matmul_u32(const uint32_t *a, const uint32_t *b, uint32_t *c, int bs, int m, int n, int k, int transA,
                       int transB) {
#pragma omp parallel for collapse(2)
    for (int bb = 0; bb < bs; ++bb)
        for (int mm = 0; mm < m; ++mm)
            for (int nn = 0; nn < n; ++nn) {
                uint32_t tmp = 0;
                for (int kk = 0; kk < k; ++kk) {
                    uint32_t lhs = transA ? a[mm + (size_t)m * (kk + (size_t)k * bb)] : a[kk + (size_t)k * (mm + (size_t)m * bb)];
                    uint32_t rhs = transB ? b[kk + (size_t)k * (nn + (size_t)n * bb)] : b[nn + (size_t)n * (kk + (size_t)k * bb)];
                    tmp += lhs * rhs;
                }
                c[nn + (size_t)n * (mm + (size_t)m * bb)] = tmp;
            }
}

void oracle_matmul_f32(const float *a, const float *b, const float *bias, float *c, int bs, int m, int n, int k,
                       int transA, int transB, int act, int wide) {
#pragma omp parallel for collapse(2)
    for (int bb = 0; bb < bs; ++bb)
        for (int mm = 0; mm < m; ++mm)
            for (int nn = 0; nn < n; ++nn) {
                float accf = 0.f;
                double accd = 0.0;
                for (int kk = 0; kk < k; ++kk) {
                    float lhs = transA ? a[mm + (size_t)m * (kk + (size_t)k * bb)] : a[kk + (size_t)k * (mm + (size_t)m * bb)];
                    float rhs = transB ? b[kk + (size_t)k * (nn + (size_t)n * bb)] : b[nn + (size_t)n * (kk + (size_t)k * bb)];
                    if (wide)
                        accd += (double)lhs * (double)rhs;
                    else
                        accf += lhs * rhs;
                }
                float v = wide ? (float)(accd + (bias ? (double)bias[nn] : 0.0)) : accf + (bias ? bias[nn] : 0.f);
                c[nn + (size_t)n * (mm + (size_t)m * bb)] = act_f32(v, act);
            }
}

int oracle_transpose_u32(const uint32_t *in, int nd, const int *dims, int split, int ngroups,
                         const int *group_sizes, const int *flat, int factor, uint32_t *out, int *out_dims) {
    int fd[16], nflat = 0;
    for (int i = 0; i < nd; ++i) {
        if (i != split) {
            fd[nflat++] = dims[i];
        } else if (factor > 0) { /* operator.cc:2182-2185 */
            if (dims[i] % factor != 0 || dims[i] < factor)
                return -1;
            fd[nflat++] = dims[i] / factor;
            fd[nflat++] = factor;
        } else { /* operator.cc:2187-2191 */
            int af = -factor;
            if (af == 0 || dims[i] % af != 0 || dims[i] < af)
                return -1;
            fd[nflat++] = af;
            fd[nflat++] = dims[i] / af;
        }
    }
    /* renumber `after` as TransposeOp::setParam does, include/operator.h:1133-1143 */
    int after[16], na = 0;
    for (int gi = 0, p = 0; gi < ngroups; ++gi) {
        int ext = 1;
        for (int j = 0; j < group_sizes[gi]; ++j, ++p) {
            int item = flat[p];
            if (split >= 0) {
                if (item > split)
                    item += 1;
                if (item == -1)
                    item = split + 1;
            }
            after[na++] = item;
            ext *= fd[item];
        }
        if (out_dims)
            out_dims[gi] = ext;
    }
    size_t total = 1;
    for (int i = 0; i < nflat; ++i)
        total *= (size_t)fd[i];
    if (out == NULL)
        return ngroups;
#pragma omp parallel for
    for (size_t i = 0; i < total; ++i) {
        int it[16];
        size_t rem = i;
        for (int d = nflat - 1; d >= 0; --d) {
            it[d] = (int)(rem % (size_t)fd[d]);
            rem /= (size_t)fd[d];
        }
        size_t o = 0;
        for (int j = 0; j < na; ++j)
            o = o * (size_t)fd[after[j]] + (size_t)it[after[j]];
        out[o] = in[i];
    }
    return ngroups;
}

void oracle_pad_u32(const uint32_t *in, int nd, const int *dims, const int *begin, const int *end, uint32_t *out) {
    int od[16];
    size_t total = 1;
    for (int i = 0; i < nd; ++i) {
        od[i] = dims[i] + begin[i] + end[i];
        total *= (size_t)od[i];
    }
#pragma omp parallel for
    for (size_t i = 0; i < total; ++i) {
        size_t rem = i, io = 0, mul = 1;
        int inside = 1;
        for (int d = nd - 1; d >= 0; --d) {
            int oi = (int)(rem % (size_t)od[d]);
            rem /= (size_t)od[d];
            int ii = oi - begin[d];
            if (ii < 0 || ii >= dims[d])
                inside = 0;
            io += (size_t)(ii < 0 ? 0 : ii) * mul;
            mul *= (size_t)dims[d];
        }
        out[i] = inside ? in[io] : 0u;
    }
}

void oracle_slice_u32(const uint32_t *in, int nd, const int *dims, const int *begin, const int *end, uint32_t *out) {
    int od[16];
    size_t total = 1;
    for (int i = 0; i < nd; ++i) {
        od[i] = dims[i] - begin[i] - end[i];
        total *= (size_t)od[i];
    }
#pragma omp parallel for
    for (size_t i = 0; i < total; ++i) {
        size_t rem = i, io = 0, mul = 1;
        for (int d = nd - 1; d >= 0; --d) {
            int oi = (int)(rem % (size_t)od[d]);
            rem /= (size_t)od[d];
            io += (size_t)(oi + begin[d]) * mul;
            mul *= (size_t)dims[d];
        }
        out[i] = in[io];
    }
}

void oracle_extend_u32(const uint32_t *in, int nd, const int *dims, int dim, int num, uint32_t *out) {
    size_t blk = 1, total = 1;
    for (int i = nd - 1; i >= dim; --i)
        blk *= (size_t)dims[i];
    for (int i = 0; i < nd; ++i)
        total *= (size_t)dims[i];
    size_t outer = (size_t)(num + 1) * blk;
    total *= (size_t)(num + 1);
#pragma omp parallel for
    for (size_t o = 0; o < total; ++o)
        out[o] = in[o % blk + o / outer * blk];
}

void oracle_axis_block_u32(const uint32_t *src, uint32_t *dst, size_t outer, size_t inner, int part_extent,
                           int whole_extent, int offset, int to_whole) {
    size_t local = (size_t)part_extent * inner;  /* localBlockOffset */
    size_t block = (size_t)whole_extent * inner; /* blockOffset */
    size_t shift = inner * (size_t)offset;       /* innerOffset */
    size_t total = outer * local;
#pragma omp parallel for
    for (size_t p = 0; p < total; ++p) {
        size_t wpos = p % local + shift + p / local * block;
        if (to_whole)
            dst[wpos] = src[p];
        else
            dst[p] = src[wpos];
    }
}

void oracle_eltwise_u32(int kind, int n_in, const uint32_t *const *ins, const size_t *sizes, uint32_t *out,
                        size_t out_size) {
#pragma omp parallel for
    for (size_t i = 0; i < out_size; ++i) {
        uint32_t v = (kind == 2) ? 1u : 0u;
        if (kind == 1)
            v = ins[0][i % sizes[0]] - ins[1][i % sizes[1]];
        else
            for (int j = 0; j < n_in; ++j) {
                uint32_t e = ins[j][i % sizes[j]];
                v = (kind == 2) ? v * e : v + e;
            }
        out[i] = v;
    }
}

void oracle_eltwise_f32(int kind, int n_in, const float *const *ins, const size_t *sizes, float *out,
                        size_t out_size) {
#pragma omp parallel for
    for (size_t i = 0; i < out_size; ++i) {
        float v;
        if (kind == 1) {
            v = ins[0][i % sizes[0]] - ins[1][i % sizes[1]];
        } else {
            v = ins[0][i % sizes[0]];
            for (int j = 1; j < n_in; ++j) {
                float e = ins[j][i % sizes[j]];
                v = (kind == 2) ? v * e : v + e;
            }
        }
        out[i] = v;
    }
}

void oracle_batchnorm_f32(const float *x, const float *scale, const float *bias, const float *mean,
                          const float *var, float *y, size_t outer, int c, size_t inner, float eps) {
#pragma omp parallel for collapse(2)
    for (size_t o = 0; o < outer; ++o)
        for (int cc = 0; cc < c; ++cc) {
            double k = (double)scale[cc] / sqrt((double)var[cc] + (double)eps);
            const float *xp = x + (o * (size_t)c + (size_t)cc) * inner;
            float *yp = y + (o * (size_t)c + (size_t)cc) * inner;
            for (size_t i = 0; i < inner; ++i)
                yp[i] = (float)(((double)xp[i] - (double)mean[cc]) * k + (double)bias[cc]);
        }
}

void oracle_activation_f32(const float *x, float *y, size_t n, int act) {
#pragma omp parallel for
    for (size_t i = 0; i < n; ++i)
        y[i] = act_f32(x[i], act);
}

static int pool_out(int in, int k, int p, int s) { return (in - (k - s) + 2 * p) / s; }

void oracle_maxpool_f32(const float *x, float *y, int n, int c, int h, int w, int kh, int kw, int ph, int pw, int sh,
                        int sw) {
    int oh = pool_out(h, kh, ph, sh), ow = pool_out(w, kw, pw, sw);
#pragma omp parallel for
    for (int nc = 0; nc < n * c; ++nc)
        for (int i = 0; i < oh; ++i)
            for (int j = 0; j < ow; ++j) {
                float best = -INFINITY;
                for (int a = 0; a < kh; ++a)
                    for (int b = 0; b < kw; ++b) {
                        int yy = i * sh + a - ph, xx = j * sw + b - pw;
                        if (yy < 0 || yy >= h || xx < 0 || xx >= w)
                            continue;
                        float v = x[((size_t)nc * h + yy) * w + xx];
                        if (v > best)
                            best = v;
                    }
                y[((size_t)nc * oh + i) * ow + j] = best;
            }
}

void oracle_avgpool_f32(const float *x, float *y, int n, int c, int h, int w, int kh, int kw, int ph, int pw, int sh,
                        int sw) {
    int oh = pool_out(h, kh, ph, sh), ow = pool_out(w, kw, pw, sw);
#pragma omp parallel for
    for (int nc = 0; nc < n * c; ++nc)
        for (int i = 0; i < oh; ++i)
            for (int j = 0; j < ow; ++j) {
                double acc = 0.0;
                int cnt = 0;
                for (int a = 0; a < kh; ++a)
                    for (int b = 0; b < kw; ++b) {
                        int yy = i * sh + a - ph, xx = j * sw + b - pw;
                        if (yy < 0 || yy >= h || xx < 0 || xx >= w)
                            continue;
                        acc += (double)x[((size_t)nc * h + yy) * w + xx];
                        cnt++;
                    }
                y[((size_t)nc * oh + i) * ow + j] = cnt ? (float)(acc / cnt) : 0.f;
            }
}

void oracle_softmax_f32(const float *x, float *y, size_t rows, int cols) {
#pragma omp parallel for
    for (size_t r = 0; r < rows; ++r) {
        const float *xp = x + r * (size_t)cols;
        float *yp = y + r * (size_t)cols;
        float mx = -INFINITY;
        for (int i = 0; i < cols; ++i)
            if (xp[i] > mx)
                mx = xp[i];
        double den = 0.0;
        for (int i = 0; i < cols; ++i)
            den += exp((double)xp[i] - (double)mx);
        for (int i = 0; i < cols; ++i)
            yp[i] = (float)(exp((double)xp[i] - (double)mx) / den);
    }
}

void oracle_layernorm_f32(const float *x, const float *gamma, const float *beta, float *y, size_t rows, int cols,
                          float eps) {
#pragma omp parallel for
    for (size_t r = 0; r < rows; ++r) {
        const float *xp = x + r * (size_t)cols;
        float *yp = y + r * (size_t)cols;
        double mean = 0.0, var = 0.0;
        for (int i = 0; i < cols; ++i)
            mean += xp[i];
        mean /= cols;
        for (int i = 0; i < cols; ++i)
            var += ((double)xp[i] - mean) * ((double)xp[i] - mean);
        var /= cols;
        double inv = 1.0 / sqrt(var + (double)eps);
        for (int i = 0; i < cols; ++i)
            yp[i] = (float)(((double)xp[i] - mean) * inv * (gamma ? (double)gamma[i] : 1.0) + (beta ? (double)beta[i] : 0.0));
    }
}

/* ---- ConvTransOp ------------------------------------------------------------------------------------------------ */
int oracle_convtrans_out(int in, int k, int pad, int stride, int dil, int out_pad) {
    /* src/Graph/operator.cc:1058-1059 */
    return (in - 1) * stride - 2 * pad + dil * (k - 1) + out_pad + 1;
}

#define CONVTRANS_BODY(TYPE, ACC)                                                                                    \
    int oh = oracle_convtrans_out(h, r, ph, sh, dh, oph), ow = oracle_convtrans_out(w, s, pw, sw, dw, opw);           \
    int ah = (h + 2 * ph - r) % sh, aw = (w + 2 * pw - s) % sw;                                                       \
    for (int nn = 0; nn < n; nn++) {                                                                                  \
        _Pragma("omp parallel for") for (int cc = 0; cc < c; cc++) {                                                  \
            for (int hh = 0; hh < oh; hh++)                                                                           \
                for (int ww = 0; ww < ow; ww++) {                                                                     \
                    ACC val = 0;                                                                                      \
                    for (int ff = 0; ff < f; ff++)                                                                    \
                        for (int rr = 0; rr < r; rr++)                                                                \
                            for (int ss = 0; ss < s; ss++) {                                                          \
                                if (r - ah < rr || s - aw < ss)                                                       \
                                    continue;                                                                         \
                                int posH = hh + rr * dh - (r - ph - 1), posW = ww + ss * dw - (s - pw - 1);           \
                                if (posH % sh != 0 || posW % sw != 0)                                                 \
                                    continue;                                                                         \
                                posH /= sh;                                                                           \
                                posW /= sw;                                                                           \
                                if (posH < 0 || posH >= h || posW < 0 || posW >= w)                                   \
                                    continue;                                                                         \
                                TYPE xv = x[ff + (size_t)f * (posW + (size_t)w * (posH + (size_t)h * nn))];           \
                                TYPE wv = wt[cc + (size_t)c * (ff + (size_t)f * ((s - 1 - ss) + (size_t)s * (r - 1 - rr)))]; \
                                val += (ACC)wv * (ACC)xv;                                                             \
                            }                                                                                         \
                    y[cc + (size_t)c * (ww + (size_t)ow * (hh + (size_t)oh * nn))] = (TYPE)val;                       \
                }                                                                                                     \
        }                                                                                                             \
    }

void oracle_convtrans_u32(const uint32_t *x, const uint32_t *wt, uint32_t *y, int n, int h, int w, int f, int r, int s,
                          int c, int ph, int pw, int sh, int sw, int dh, int dw, int oph, int opw) {
    CONVTRANS_BODY(uint32_t, uint32_t)
}

void oracle_convtrans_f32(const float *x, const float *wt, float *y, int n, int h, int w, int f, int r, int s, int c,
                          int ph, int pw, int sh, int sw, int dh, int dw, int oph, int opw, int wide) {
    if (wide) {
        CONVTRANS_BODY(float, double)
    } else {
        CONVTRANS_BODY(float, float)
    }
}

/* ---- banded attention products ---------------------------------------------------------------------------------- */
void oracle_g2bmm_f32(const float *q, const float *kk, float *y, int bs, int n, int m, int w, int d, int wide) {
    const int bw = 2 * w + 1;
#pragma omp parallel for collapse(2)
    for (int b = 0; b < bs; b++)
        for (int i = 0; i < n; i++)
            for (int j = 0; j < bw; j++) {
                long row = (long)i + (long)d * (j - w);
                double accd = 0;
                float accf = 0.f;
                if (row >= 0 && row < n)
                    for (int k = 0; k < m; k++) {
                        float a = q[((size_t)b * n + i) * m + k], c = kk[((size_t)b * n + row) * m + k];
                        if (wide)
                            accd += (double)a * (double)c;
                        else
                            accf += a * c;
                    }
                y[((size_t)b * n + i) * bw + j] = wide ? (float)accd : accf;
            }
}

void oracle_gbmml_f32(const float *p, const float *v, float *y, int bs, int n, int m, int w, int d, int wide) {
    const int bw = 2 * w + 1;
#pragma omp parallel for collapse(2)
    for (int b = 0; b < bs; b++)
        for (int i = 0; i < n; i++)
            for (int k = 0; k < m; k++) {
                double accd = 0;
                float accf = 0.f;
                for (int j = 0; j < bw; j++) {
                    long row = (long)i + (long)d * (j - w);
                    if (row < 0 || row >= n)
                        continue;
                    float a = p[((size_t)b * n + i) * bw + j], c = v[((size_t)b * n + row) * m + k];
                    if (wide)
                        accd += (double)a * (double)c;
                    else
                        accf += a * c;
                }
                y[((size_t)b * n + i) * m + k] = wide ? (float)accd : accf;
            }
}
