// Convolution and matmul plans: argument checking as the reference's operators do it, kernel-family selection
// (tcgen05 3xTF32 implicit GEMM, or the CUDA-core fp32 kernels below for shapes the tensor-core path does not
// take), weight preprocessing, correction windows, and the operands used by the timing entry point.
#include "common.h"
#include <algorithm>

namespace petb200 {

// implemented in igemm_tc.cu
int tc_conv_create(petb200_ctx *ctx, int nsp, const int *in_dims, int f, const int *k, const int *pad, const int *stride,
                   const int *dil, int groups, int has_bias, int act, int passes, void **out, size_t *dev_bytes, int channels_last_out);
void tc_conv_destroy(void *h);
int tc_conv_set_weights(void *h, const float *w, cudaStream_t s);
int tc_conv_run(void *h, const float *x, const float *bias, const float *res, float *y, const int *win, cudaStream_t s);
int tc_conv_row_pitch(void *h);
void tc_conv_set_prof(void *h, long long *p);
void tc_conv_set_starve(void *h, int on);
int tc_set_wait_limit_ns(unsigned long long ns);
void tc_matmul_set_prof(void *h, long long *p);
const char *tc_conv_variant(void *h);
int tc_matmul_create(petb200_ctx *ctx, int bs, int m, int n, int k, int transA, int transB, int has_bias, int act, int passes,
                     const long long *strides, void **out, size_t *dev_bytes);
int tc_matmul_native_a(void *h);
void tc_matmul_destroy(void *h);
int tc_matmul_pack_b(void *h, const float *b, cudaStream_t s);
int tc_matmul_run(void *h, const float *a_t, const float *bias, const float *res, float *cmat, cudaStream_t s);

// -------------------------------------------------------------------------------------------------------------
// CUDA-core kernels (exact fp32 products, sequential accumulation in the reference's loop order cc,tt,rr,ss)
// -------------------------------------------------------------------------------------------------------------
struct SimtConv {
    int N, C, D, H, W, F, T, R, S, pd, ph, pw, sd, sh, sw, dd, dh, dw, groups, OD, OH, OW;
    int oh0, ohn, ow0, own;
    int act, has_bias;
    int cl_out; // output [n,(od,)oh,ow,f] instead of [n,f,(od,)oh,ow]
};

__global__ void __launch_bounds__(256) k_conv_simt(const float *__restrict__ x, const float *__restrict__ w,
                                                   const float *__restrict__ bias, const float *__restrict__ res,
                                                   float *__restrict__ y, SimtConv c) {
    pdl_prologue();
    const int cpg = c.C / c.groups, fpg = c.F / c.groups;
    const long long total = (long long)c.N * c.F * c.OD * c.ohn * c.own;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        long long rem = i;
        const int ww = c.ow0 + (int)(rem % c.own);
        rem /= c.own;
        const int hh = c.oh0 + (int)(rem % c.ohn);
        rem /= c.ohn;
        const int zz = (int)(rem % c.OD);
        rem /= c.OD;
        const int ff = (int)(rem % c.F);
        const int nn = (int)(rem / c.F);
        const int gidx = ff / fpg;
        float acc = 0.f;
        for (int cc = 0; cc < cpg; ++cc)
            for (int tt = 0; tt < c.T; ++tt) {
                const int pz = zz * c.sd + tt * c.dd - c.pd;
                if (pz < 0 || pz >= c.D)
                    continue;
                for (int rr = 0; rr < c.R; ++rr) {
                    const int py = hh * c.sh + rr * c.dh - c.ph;
                    if (py < 0 || py >= c.H)
                        continue;
                    for (int ss = 0; ss < c.S; ++ss) {
                        const int px = ww * c.sw + ss * c.dw - c.pw;
                        if (px < 0 || px >= c.W)
                            continue;
                        const long long io = px + (long long)c.W * (py + (long long)c.H * (pz + (long long)c.D * ((cc + gidx * cpg) + (long long)c.C * nn)));
                        const long long wo = ss + (long long)c.S * (rr + (long long)c.R * (tt + (long long)c.T * (cc + (long long)cpg * ff)));
                        acc = fmaf(__ldg(w + wo), __ldg(x + io), acc);
                    }
                }
            }
        if (c.has_bias)
            acc += __ldg(bias + ff);
        const long long yo = c.cl_out ? ff + (long long)c.F * (ww + (long long)c.OW * (hh + (long long)c.OH * (zz + (long long)c.OD * nn)))
                                      : ww + (long long)c.OW * (hh + (long long)c.OH * (zz + (long long)c.OD * (ff + (long long)c.F * nn)));
        if (res)
            acc += __ldg(res + yo);
        y[yo] = apply_act(acc, c.act);
    }
}

__global__ void __launch_bounds__(256) k_matmul_simt(const float *__restrict__ a, const float *__restrict__ b,
                                                     const float *__restrict__ bias, const float *__restrict__ res,
                                                     float *__restrict__ c, int bs, int m, int n, int k, int transA, int transB,
                                                     int act) {
    pdl_prologue();
    const long long total = (long long)bs * m * n;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int nn = (int)(i % n);
        const int mm = (int)((i / n) % m);
        const int bb = (int)(i / ((long long)n * m));
        float acc = 0.f;
        for (int kk = 0; kk < k; ++kk) {
            const float lhs = transA ? __ldg(a + mm + (long long)m * (kk + (long long)k * bb)) : __ldg(a + kk + (long long)k * (mm + (long long)m * bb));
            const float rhs = transB ? __ldg(b + kk + (long long)k * (nn + (long long)n * bb)) : __ldg(b + nn + (long long)n * (kk + (long long)k * bb));
            acc = fmaf(lhs, rhs, acc);
        }
        if (bias)
            acc += __ldg(bias + nn);
        if (res)
            acc += __ldg(res + i);
        c[i] = apply_act(acc, act);
    }
}

// Matrix-vector shapes (m <= 8 rows of A, e.g. a classifier head at batch 1): the 128-row tensor-core tile would be
// almost empty, and the work is one pass over B.  A block owns 32 columns of C for all rows; exact fp32 FMA.
//   B as [k][n]: lanes = columns (coalesced rows of B), the 8 warps split K and are added up through shared memory.
//   B as [n][k]: a warp owns 4 columns, lanes split K (coalesced rows of B), lanes are added up by shuffles.
constexpr int kGemvRows = 8, kGemvWarps = 16, kGemvKTile = 768;
__global__ void __launch_bounds__(kGemvWarps * 32) k_gemv_small_m(const float *__restrict__ a, const float *__restrict__ b,
                                                                 const float *__restrict__ bias, const float *__restrict__ res,
                                                                 float *__restrict__ c, int m, int n, int k, int transA, int transB,
                                                                 int act) {
    pdl_prologue();
    __shared__ float sa[kGemvRows][kGemvKTile];        // a K tile of A, row r at sa[r]
    __shared__ float red[kGemvWarps][kGemvRows][33];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, bb = blockIdx.y;
    const float *ab = a + (long long)bb * m * k, *bm = b + (long long)bb * k * n;
    float acc[kGemvRows];
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r)
        acc[r] = 0.f;
    const int col0 = blockIdx.x * 32;
    for (int kt = 0; kt < k; kt += kGemvKTile) {
        const int kn = min(kGemvKTile, k - kt);
        __syncthreads(); // the previous tile has been consumed
        for (int i = threadIdx.x; i < m * kn; i += kGemvWarps * 32) {
            int r, kk;
            if (transA) // A is [k][m]: consecutive threads read consecutive addresses
                kk = i / m, r = i - kk * m;
            else
                r = i / kn, kk = i - r * kn;
            sa[r][kk] = __ldg(transA ? ab + (long long)(kt + kk) * m + r : ab + (long long)r * k + kt + kk);
        }
        __syncthreads();
        if (!transB) {
            // B as [k][n]: lanes = columns (coalesced rows of B), the warps split the tile's K range
            const int col = col0 + lane;
            const int kbeg = kn * warp / kGemvWarps, kend = kn * (warp + 1) / kGemvWarps;
            for (int k0 = kbeg; k0 < kend; k0 += 16) {
                float bv[16]; // sixteen rows of B in flight per lane
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    bv[u] = (k0 + u < kend && col < n) ? __ldg(bm + (long long)(kt + k0 + u) * n + col) : 0.f;
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const int kk = min(k0 + u, kend - 1); // rows past the end carry bv = 0
#pragma unroll
                    for (int r = 0; r < kGemvRows; ++r)
                        acc[r] = fmaf(sa[r][kk], bv[u], acc[r]);
                }
            }
        } else {
            // B as [n][k]: a warp owns columns warp and warp + 16 of the block, lanes split K (coalesced rows of B);
            // two accumulator sets would be needed to keep both: process the tile column by column instead
            for (int cc = 0; cc < 2; ++cc) {
                const int col = col0 + warp + cc * kGemvWarps;
                if (col >= n)
                    break;
                float part[kGemvRows];
#pragma unroll
                for (int r = 0; r < kGemvRows; ++r)
                    part[r] = 0.f;
                for (int k0 = lane; k0 < kn; k0 += 8 * 32) {
                    float bv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        bv[u] = k0 + 32 * u < kn ? __ldg(bm + (long long)col * k + kt + k0 + 32 * u) : 0.f;
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int kk = min(k0 + 32 * u, kn - 1);
#pragma unroll
                        for (int r = 0; r < kGemvRows; ++r)
                            part[r] = fmaf(sa[r][kk], bv[u], part[r]);
                    }
                }
                // per-column partial sums of this K tile go through shared memory, slot [cc*16 + warp... ] is this column
#pragma unroll
                for (int r = 0; r < kGemvRows; ++r) {
                    float v = part[r];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1)
                        v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (lane == 0)
                        red[cc][r][warp] = (kt == 0 ? 0.f : red[cc][r][warp]) + v;
                }
            }
        }
    }
    if (!transB) {
#pragma unroll
        for (int r = 0; r < kGemvRows; ++r)
            red[warp][r][lane] = acc[r];
    }
    __syncthreads();
    // thread (warp = row, lane = column) finishes one output
    if (warp < m) {
        const int r = warp;
        float v = 0.f;
        int col;
        if (!transB) {
            col = col0 + lane;
#pragma unroll
            for (int w = 0; w < kGemvWarps; ++w) // K slices in order
                v += red[w][r][lane];
        } else {
            col = col0 + (lane & 15) + (lane >> 4) * kGemvWarps;
            v = red[lane >> 4][r][lane & 15];
        }
        if (col < n) {
            if (bias)
                v += __ldg(bias + col);
            const long long co = ((long long)bb * m + r) * n + col;
            if (res)
                v += __ldg(res + co);
            c[co] = apply_act(v, act);
        }
    }
}

// Re-pitches [planes, H, W] rows to a pitch divisible by 4 (zero fill), so TMA's 16-byte stride rule holds.
__global__ void __launch_bounds__(256) k_repitch(const float *__restrict__ x, float *__restrict__ y, long long rows, int w, int wp) {
    pdl_prologue();
    const long long total = rows * wp;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int col = (int)(i % wp);
        const long long row = i / wp;
        y[i] = col < w ? __ldg(x + row * w + col) : 0.f;
    }
}

// [b][m][k] -> [b][k][mp]  (row pitch mp >= m, padding columns zero)
__global__ void __launch_bounds__(256) k_transpose_a(const float *__restrict__ a, float *__restrict__ at, int bs, int m, int k, int mp) {
    pdl_prologue();
    __shared__ float tile[32][33];
    const int tiles_k = (k + 31) / 32, tiles_m = (mp + 31) / 32;
    const long long ntiles = (long long)bs * tiles_k * tiles_m;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const int tk = (int)(t % tiles_k);
        const int tm = (int)((t / tiles_k) % tiles_m);
        const int bb = (int)(t / ((long long)tiles_k * tiles_m));
        for (int r = ty; r < 32; r += 8) {
            const int mm = tm * 32 + r, kk = tk * 32 + tx;
            tile[r][tx] = (mm < m && kk < k) ? __ldg(a + ((long long)bb * m + mm) * k + kk) : 0.f;
        }
        __syncthreads();
        for (int r = ty; r < 32; r += 8) {
            const int kk = tk * 32 + r, mm = tm * 32 + tx;
            if (kk < k && mm < mp)
                at[((long long)bb * k + kk) * mp + mm] = tile[tx][r];
        }
        __syncthreads();
    }
}

static int grid_for(petb200_ctx *ctx, long long work, int per_block) {
    long long blocks = (work + per_block - 1) / per_block;
    return (int)std::max<long long>(1, std::min<long long>(blocks, (long long)ctx->sm_count * 16));
}

// -------------------------------------------------------------------------------------------------------------
struct ConvPlan : petb200_plan {
    DevBuf xpad; // re-pitched input, for the shapes whose rows TMA cannot address (see tc_conv_row_pitch)
    int wp = 0;
    int nsp = 2;
    SimtConv sc{};
    int algo = 0; // resolved: PETB200_ALGO_TC_3XTF32 or PETB200_ALGO_SIMT_FP32
    void *tc = nullptr;
    const float *w_simt = nullptr; // SIMT path keeps the caller's weight pointer
    DevBuf bx, bw, bb, by; // timing operands
    ~ConvPlan() override {
        if (tc)
            tc_conv_destroy(tc);
    }
    int bench_launch(cudaStream_t s) override;
};

int make_conv_plan(petb200_ctx *ctx, int nsp, const int *in_dims, int f, const int *k, const int *pad, const int *stride,
                   const int *dil, int groups, int has_bias, int act, int algo, petb200_plan **out, int channels_last_out) {
    if (!ctx || !out)
        return PETB200_ERR_INVALID;
    const int nd = nsp + 2;
    for (int i = 0; i < nd; ++i)
        if (in_dims[i] <= 0)
            return fail(ctx, PETB200_ERR_INVALID, "conv plan: non-positive input dim");
    for (int i = 0; i < nsp; ++i)
        if (k[i] <= 0 || stride[i] <= 0 || dil[i] <= 0 || pad[i] < 0)
            return fail(ctx, PETB200_ERR_INVALID, "conv plan: bad kernel/stride/dilation/pad");
    const int C = in_dims[1];
    // ref: ConvOp::compute returns nullptr when f % g != 0 (src/Graph/operator.cc:108-110); groups = C / cpg
    if (f <= 0 || groups <= 0 || C % groups != 0 || f % groups != 0)
        return fail(ctx, PETB200_ERR_INVALID, "conv plan: channels %d / filters %d not divisible by groups %d", C, f, groups);
    if (act < 0 || act > PETB200_ACT_GELU)
        return fail(ctx, PETB200_ERR_INVALID, "conv plan: unknown activation %d", act);
    auto *pl = new ConvPlan();
    pl->ctx = ctx;
    pl->nsp = nsp;
    SimtConv &c = pl->sc;
    c.N = in_dims[0];
    c.C = C;
    c.F = f;
    c.groups = groups;
    c.act = act;
    c.has_bias = has_bias;
    c.cl_out = channels_last_out ? 1 : 0;
    if (nsp == 3) {
        c.D = in_dims[2], c.H = in_dims[3], c.W = in_dims[4];
        c.T = k[0], c.R = k[1], c.S = k[2];
        c.pd = pad[0], c.ph = pad[1], c.pw = pad[2];
        c.sd = stride[0], c.sh = stride[1], c.sw = stride[2];
        c.dd = dil[0], c.dh = dil[1], c.dw = dil[2];
    } else {
        c.D = 1, c.H = in_dims[2], c.W = in_dims[3];
        c.T = 1, c.R = k[0], c.S = k[1];
        c.pd = 0, c.ph = pad[0], c.pw = pad[1];
        c.sd = 1, c.sh = stride[0], c.sw = stride[1];
        c.dd = 1, c.dh = dil[0], c.dw = dil[1];
    }
    // ref: ConvOp::computeShape, src/Graph/operator.cc:220-221
    c.OD = (c.D - (c.T - c.sd) * c.dd + 2 * c.pd) / c.sd;
    c.OH = (c.H - (c.R - c.sh) * c.dh + 2 * c.ph) / c.sh;
    c.OW = (c.W - (c.S - c.sw) * c.dw + 2 * c.pw) / c.sw;
    if (c.OD <= 0 || c.OH <= 0 || c.OW <= 0) {
        delete pl;
        return fail(ctx, PETB200_ERR_INVALID, "conv plan: empty output");
    }
    c.oh0 = 0, c.ohn = c.OH, c.ow0 = 0, c.own = c.OW;
    int rc = PETB200_ERR_UNSUPPORTED;
    if (tc_is_tc_algo(algo)) {
        size_t bytes = 0;
        rc = tc_conv_create(ctx, nsp, in_dims, f, k, pad, stride, dil, groups, has_bias, act, tc_passes_for(algo),
                            &pl->tc, &bytes, c.cl_out);
        if (rc == PETB200_OK) {
            pl->algo = PETB200_ALGO_TC_3XTF32;
            pl->kernel = tc_conv_variant(pl->tc);
            pl->device_bytes = bytes;
            pl->wp = tc_conv_row_pitch(pl->tc);
            if (pl->wp != c.W) {
                size_t n = (size_t)c.N * c.C * c.D * c.H * pl->wp * 4;
                if (pl->xpad.alloc(n) != cudaSuccess) {
                    delete pl;
                    return fail(ctx, PETB200_ERR_NOMEM, "re-pitch scratch allocation failed");
                }
                pl->device_bytes += n;
            }
        } else if (algo != PETB200_ALGO_AUTO || rc != PETB200_ERR_UNSUPPORTED) {
            delete pl;
            return rc;
        }
    }
    if (rc != PETB200_OK) {
        pl->algo = PETB200_ALGO_SIMT_FP32;
        pl->kernel = "simt_fp32";
    }
    *out = pl;
    return PETB200_OK;
}

int conv_set_weights(petb200_plan *plan, const float *w, cudaStream_t s) {
    auto *pl = dynamic_cast<ConvPlan *>(plan);
    if (!pl || !w)
        return PETB200_ERR_INVALID;
    if (pl->algo == PETB200_ALGO_TC_3XTF32)
        return tc_conv_set_weights(pl->tc, w, s);
    pl->w_simt = w;
    return PETB200_OK;
}

int conv_run(petb200_plan *plan, const float *x, const float *bias, float *y, const int *win, cudaStream_t s, const float *res) {
    auto *pl = dynamic_cast<ConvPlan *>(plan);
    if (!pl)
        return PETB200_ERR_INVALID;
    petb200_ctx *ctx = pl->ctx;
    if (!x || !y)
        return fail(ctx, PETB200_ERR_INVALID, "conv run: null buffer");
    if (pl->sc.has_bias && !bias)
        return fail(ctx, PETB200_ERR_INVALID, "conv run: plan was made with a bias but none was passed");
    if (pl->algo == PETB200_ALGO_TC_3XTF32) {
        const float *xin = x;
        if (pl->xpad.p) {
            const SimtConv &c = pl->sc;
            long long rows = (long long)c.N * c.C * c.D * c.H;
            launch_pdl(k_repitch, grid_for(ctx, rows * pl->wp, 256), 256, 0, s, x, (float *)pl->xpad.p, rows, c.W, pl->wp);
            int rc = launched(ctx, "k_repitch");
            if (rc)
                return rc;
            xin = (const float *)pl->xpad.p;
        }
        return tc_conv_run(pl->tc, xin, bias, res, y, win, s);
    }
    if (!pl->w_simt)
        return fail(ctx, PETB200_ERR_INVALID, "conv run before set_weights");
    SimtConv c = pl->sc;
    if (win) {
        if (win[0] < 0 || win[1] <= 0 || win[0] + win[1] > c.OH || win[2] < 0 || win[3] <= 0 || win[2] + win[3] > c.OW)
            return fail(ctx, PETB200_ERR_INVALID, "correction window outside the output");
        c.oh0 = win[0], c.ohn = win[1], c.ow0 = win[2], c.own = win[3];
    }
    long long total = (long long)c.N * c.F * c.OD * c.ohn * c.own;
    launch_pdl(k_conv_simt, grid_for(ctx, total, 256), 256, 0, s, x, pl->w_simt, bias, res, y, c);
    return launched(ctx, "k_conv_simt");
}

int conv_out_dims(const petb200_plan *plan, int *d5) {
    auto *pl = dynamic_cast<const ConvPlan *>(plan);
    if (!pl)
        return PETB200_ERR_INVALID;
    d5[0] = pl->sc.N, d5[1] = pl->sc.F, d5[2] = pl->sc.OD, d5[3] = pl->sc.OH, d5[4] = pl->sc.OW;
    return PETB200_OK;
}

int ConvPlan::bench_launch(cudaStream_t s) {
    const SimtConv &c = sc;
    if (!bx.p) {
        size_t nx = (size_t)c.N * c.C * c.D * c.H * c.W, nw = (size_t)c.F * (c.C / c.groups) * c.T * c.R * c.S;
        size_t ny = (size_t)c.N * c.F * c.OD * c.OH * c.OW;
        if (bx.alloc(nx * 4) != cudaSuccess || bw.alloc(nw * 4) != cudaSuccess || by.alloc(ny * 4) != cudaSuccess ||
            bb.alloc((size_t)c.F * 4) != cudaSuccess)
            return fail(ctx, PETB200_ERR_NOMEM, "scratch allocation for timing failed");
        // 0x3c3c3c3c is 0.0115 as fp32: finite, non-trivial operands
        cudaMemsetAsync(bx.p, 0x3c, nx * 4, s);
        cudaMemsetAsync(bw.p, 0x3c, nw * 4, s);
        cudaMemsetAsync(bb.p, 0, (size_t)c.F * 4, s);
        int rc = conv_set_weights(this, (const float *)bw.p, s);
        if (rc)
            return rc;
    }
    return conv_run(this, (const float *)bx.p, c.has_bias ? (const float *)bb.p : nullptr, (float *)by.p, nullptr, s);
}

// -------------------------------------------------------------------------------------------------------------
struct MatmulPlan : petb200_plan {
    int transA, transB, bs, m, n, k, has_bias, act;
    int algo = 0;
    void *tc = nullptr;
    DevBuf at; // A re-laid as [b][k][m] when the caller's A is [b][m][k]
    const float *b_weight = nullptr; // set by matmul_set_weights
    bool native_a = false;           // the kernel reads row-major A directly
    bool gemv = false;               // m <= 8: matrix-vector kernel
    bool strided = false;            // operands/result addressed through st[] (tensor-core kernel only)
    long long st[6] = {0, 0, 0, 0, 0, 0};
    DevBuf ba, bbm, bbias, bc;
    ~MatmulPlan() override {
        if (tc)
            tc_matmul_destroy(tc);
    }
    int bench_launch(cudaStream_t s) override;
};

int make_matmul_plan(petb200_ctx *ctx, int transA, int transB, int b, int m, int n, int k, int has_bias, int act, int algo,
                     petb200_plan **out, const long long *strides) {
    if (!ctx || !out)
        return PETB200_ERR_INVALID;
    if (b <= 0 || m <= 0 || n <= 0 || k <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "matmul plan: non-positive extent");
    if (act < 0 || act > PETB200_ACT_GELU)
        return fail(ctx, PETB200_ERR_INVALID, "matmul plan: unknown activation %d", act);
    auto *pl = new MatmulPlan();
    pl->ctx = ctx;
    pl->transA = transA != 0, pl->transB = transB != 0, pl->bs = b, pl->m = m, pl->n = n, pl->k = k;
    pl->has_bias = has_bias, pl->act = act;
    int rc = PETB200_ERR_UNSUPPORTED;
    if (strides) {
        for (int i = 0; i < 6; ++i) {
            if (strides[i] <= 0) {
                delete pl;
                return fail(ctx, PETB200_ERR_INVALID, "matmul plan: strides must be positive");
            }
            pl->st[i] = strides[i];
        }
        pl->strided = true;
    }
    if (algo == PETB200_ALGO_AUTO && m <= kGemvRows && !strides) {
        pl->algo = PETB200_ALGO_SIMT_FP32;
        pl->gemv = true;
        pl->kernel = "gemv_fp32";
        *out = pl;
        return PETB200_OK;
    }
    if (tc_is_tc_algo(algo)) {
        size_t bytes = 0;
        rc = tc_matmul_create(ctx, b, m, n, k, pl->transA, pl->transB, has_bias, act, tc_passes_for(algo), strides,
                              &pl->tc, &bytes);
        if (rc == PETB200_OK) {
            pl->algo = PETB200_ALGO_TC_3XTF32;
            pl->kernel = tc_passes_for(algo) == 1 ? "tc_1xtf32_ts" : (tc_passes_for(algo) == 16 ? "tc_bf16x3_ts" : "tc_3xtf32_ts");
            pl->device_bytes = bytes;
            pl->native_a = tc_matmul_native_a(pl->tc) != 0;
            if (!pl->native_a && (!pl->transA || m % 4 != 0)) {
                if (pl->at.alloc((size_t)b * ((m + 3) / 4 * 4) * k * 4) != cudaSuccess) {
                    delete pl;
                    return fail(ctx, PETB200_ERR_NOMEM, "A re-layout scratch allocation failed");
                }
                pl->device_bytes += pl->at.bytes;
            }
        } else if (algo != PETB200_ALGO_AUTO || rc != PETB200_ERR_UNSUPPORTED) {
            delete pl;
            return rc;
        }
    } else if (algo != PETB200_ALGO_SIMT_FP32) {
        delete pl;
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "matmul plan: algo %d is not built", algo);
    }
    if (rc != PETB200_OK) {
        if (strides) {
            delete pl;
            return fail(ctx, PETB200_ERR_UNSUPPORTED, "strided matmul operands are served by the tensor-core kernel only");
        }
        pl->algo = PETB200_ALGO_SIMT_FP32;
        pl->kernel = "simt_fp32";
    }
    *out = pl;
    return PETB200_OK;
}

int matmul_run(petb200_plan *plan, const float *a, const float *b, const float *bias, float *c, cudaStream_t s, const float *res) {
    auto *pl = dynamic_cast<MatmulPlan *>(plan);
    if (!pl)
        return PETB200_ERR_INVALID;
    petb200_ctx *ctx = pl->ctx;
    if (!b)
        b = pl->b_weight;
    if (!a || !b || !c)
        return fail(ctx, PETB200_ERR_INVALID, "matmul run: null buffer");
    if (pl->has_bias && !bias)
        return fail(ctx, PETB200_ERR_INVALID, "matmul run: plan was made with a bias but none was passed");
    if (pl->algo == PETB200_ALGO_TC_3XTF32) {
        int rc = (b == pl->b_weight) ? PETB200_OK : tc_matmul_pack_b(pl->tc, b, s);
        if (rc)
            return rc;
        const float *at = a;
        const int mp = (pl->m + 3) / 4 * 4;
        if (pl->native_a) {
            // nothing to do: the kernel's K-major mode consumes A as it is
        } else if (!pl->transA) {
            long long tiles = (long long)pl->bs * ((pl->k + 31) / 32) * ((mp + 31) / 32);
            launch_pdl(k_transpose_a, (int)std::min<long long>(tiles, (long long)ctx->sm_count * 8), 256, 0, s, a, (float *)pl->at.p, pl->bs, pl->m, pl->k, mp);
            rc = launched(ctx, "k_transpose_a");
            if (rc)
                return rc;
            at = (const float *)pl->at.p;
        } else if (mp != pl->m) {
            long long rows = (long long)pl->bs * pl->k;
            launch_pdl(k_repitch, grid_for(ctx, rows * mp, 256), 256, 0, s, a, (float *)pl->at.p, rows, pl->m, mp);
            rc = launched(ctx, "k_repitch");
            if (rc)
                return rc;
            at = (const float *)pl->at.p;
        }
        return tc_matmul_run(pl->tc, at, pl->has_bias ? bias : nullptr, res, c, s);
    }
    if (pl->gemv) {
        launch_pdl(k_gemv_small_m, dim3((unsigned)((pl->n + 31) / 32), (unsigned)pl->bs), kGemvWarps * 32, 0, s, 
            a, b, pl->has_bias ? bias : nullptr, res, c, pl->m, pl->n, pl->k, pl->transA, pl->transB, pl->act);
        return launched(ctx, "k_gemv_small_m");
    }
    long long total = (long long)pl->bs * pl->m * pl->n;
    launch_pdl(k_matmul_simt, grid_for(ctx, total, 256), 256, 0, s, a, b, pl->has_bias ? bias : nullptr, res, c, pl->bs, pl->m, pl->n, pl->k,
                                                            pl->transA, pl->transB, pl->act);
    return launched(ctx, "k_matmul_simt");
}

int matmul_set_weights(petb200_plan *plan, const float *b, cudaStream_t s) {
    auto *pl = dynamic_cast<MatmulPlan *>(plan);
    if (!pl || !b)
        return PETB200_ERR_INVALID;
    pl->b_weight = b;
    if (pl->algo == PETB200_ALGO_TC_3XTF32)
        return tc_matmul_pack_b(pl->tc, b, s);
    return PETB200_OK;
}

int MatmulPlan::bench_launch(cudaStream_t s) {
    if (!ba.p) {
        size_t na = (size_t)bs * m * k, nb = (size_t)bs * k * n, nc = (size_t)bs * m * n;
        if (strided) { // extents that cover the last addressed element
            na = (size_t)((bs - 1) * st[0] + (m - 1) * st[1] + k);
            nb = (size_t)((bs - 1) * st[2] + ((transB ? n : k) - 1) * st[3] + (transB ? k : n));
            nc = (size_t)((bs - 1) * st[4] + (m - 1) * st[5] + n);
        }
        if (ba.alloc(na * 4) != cudaSuccess || bbm.alloc(nb * 4) != cudaSuccess || bc.alloc(nc * 4) != cudaSuccess ||
            bbias.alloc((size_t)n * 4) != cudaSuccess)
            return fail(ctx, PETB200_ERR_NOMEM, "scratch allocation for timing failed");
        cudaMemsetAsync(ba.p, 0x3c, na * 4, s);
        cudaMemsetAsync(bbm.p, 0x3c, nb * 4, s);
        cudaMemsetAsync(bbias.p, 0, (size_t)n * 4, s);
    }
    // a plan that was given its B operand as weights is timed the way it runs in a graph: on the operand packed once
    return matmul_run(this, (const float *)ba.p, b_weight ? nullptr : (const float *)bbm.p, has_bias ? (const float *)bbias.p : nullptr,
                      (float *)bc.p, s);
}

} // namespace petb200

// Tuning aid (not part of the public header): per-CTA cycle counters of the tensor-core conv kernel, 8 per CTA.
extern "C" int petb200_debug_conv_prof(petb200_plan *plan, long long *dev_counters) {
    if (auto *mp = dynamic_cast<petb200::MatmulPlan *>(plan)) {
        if (!mp->tc)
            return PETB200_ERR_INVALID;
        petb200::tc_matmul_set_prof(mp->tc, dev_counters);
        return PETB200_OK;
    }
    auto *pl = dynamic_cast<petb200::ConvPlan *>(plan);
    if (!pl || !pl->tc)
        return PETB200_ERR_INVALID;
    petb200::tc_conv_set_prof(pl->tc, dev_counters);
    return PETB200_OK;
}

// Test hooks for the give-up path of the tensor-core kernel's bounded waits (not part of the public header).
// set_wait_limit: how long a wait on an mbarrier may last on the current device (default 2 s).  conv_starve: while on,
// the plan's filter producer announces 64 bytes more per stage than it loads — a flag that nothing sets — so the MMA
// warp's wait runs out, every role leaves through its abort path, and petb200_check_device_status reports
// PETB200_ERR_DEVICE.  Nothing faults and nothing hangs: the kernel returns after the limit.
extern "C" int petb200_debug_set_wait_limit(unsigned long long ns) { return petb200::tc_set_wait_limit_ns(ns); }
extern "C" int petb200_debug_conv_starve(petb200_plan *plan, int on) {
    auto *pl = dynamic_cast<petb200::ConvPlan *>(plan);
    if (!pl || !pl->tc)
        return PETB200_ERR_INVALID;
    petb200::tc_conv_set_starve(pl->tc, on);
    return PETB200_OK;
}
