// Transposed convolution (the reference's ConvTransOp, include/operator.h:466-614) on the convolution kernels.
//
// The reference defines the operator on channels-last tensors: x {n,h,w,f}, weight {r,s,f,c}, y {n,oh,ow,c} with
// oh = (h-1)*sh - 2*ph + (r-1) + oph + 1 (src/Graph/operator.cc:1058-1059); output (hh,ww) gathers tap (rr,ss) from input
// row (hh + rr - (r-ph-1)) / sh when that is a whole in-range number, times weight[r-1-rr][s-1-ss]
// (src/Graph/operator.cc:931-983).  Dilation other than 1 is refused, as the reference does (operator.cc:1104).
//
// That is an ordinary stride-1 cross-correlation of the zero-inserted input with the flipped filter, so it runs as
//   1. k_convtrans_expand: x {n,h,w,f} -> xe [n,f,oh+r-1,ow+s-1], zero-inserted and shifted so that no padding is left
//      (one pass: a 32x32 transpose through shared memory, channel-contiguous reads, row-contiguous writes);
//   2. the implicit-GEMM convolution over xe with the flipped filter, its epilogue writing y channels-last directly.
// The filter flip (and the reference's skipped taps) is weight-only work done once in set_weights.
//
// For strides above 1 on problems large enough to pay for the extra launches the zeros are not multiplied at all: output
// rows hh = a (mod sh) only meet the filter taps rr = rr0(a) (mod sh), so each of the sh*sw phases (a,b) is a stride-1
// convolution of the ORIGINAL input (brought to NCHW once) with a sub-filter of ceil-ish(r/sh) x (s/sw) taps, writing every
// sh-th row and sw-th column of y (tc_conv_create_view: signed padding, explicit window, free output strides).
#include "common.h"
#include <algorithm>
#include <vector>

namespace petb200 {

int tc_conv_create_view(petb200_ctx *ctx, int n, int c, int h, int w, int f, int r, int s, int pad_h, int pad_w, int ohn, int own,
                        int ow_nominal, long long ys_n, long long ys_f, long long ys_p, int has_bias, int act, int passes, void **out,
                        size_t *dev_bytes);
void tc_conv_destroy(void *h);
int tc_conv_set_weights(void *h, const float *w, cudaStream_t s);
int tc_conv_run(void *h, const float *x, const float *bias, const float *res, float *y, const int *win, cudaStream_t s);
const char *tc_conv_variant(void *h);

namespace {

struct ExpandGeom {
    int n, h, w, f, Hb, Wb, lead_h, lead_w, sh, sw;
};

// grid (ceil(Wb/32), Hb, n * ceil(f/32)), block (32, 8)
__global__ void __launch_bounds__(256) k_convtrans_expand(const float *__restrict__ x, float *__restrict__ xe, ExpandGeom g) {
    pdl_prologue();
    __shared__ float tile[32][33]; // [position][channel]
    const int ftiles = (g.f + 31) / 32;
    const int nn = blockIdx.z / ftiles, f0 = (blockIdx.z % ftiles) * 32;
    const int y = blockIdx.y, bx0 = blockIdx.x * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int ry = y - g.lead_h;
    const bool row_live = ry >= 0 && ry % g.sh == 0 && ry / g.sh < g.h;
    if (row_live) {
        const int iy = ry / g.sh;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int pos = ty + 8 * i, rx = bx0 + pos - g.lead_w;
            float v = 0.f;
            if (bx0 + pos < g.Wb && rx >= 0 && rx % g.sw == 0 && rx / g.sw < g.w && f0 + tx < g.f)
                v = __ldg(x + ((size_t)(nn * g.h + iy) * g.w + rx / g.sw) * g.f + f0 + tx);
            tile[pos][tx] = v;
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int ch = ty + 8 * i;
        if (f0 + ch < g.f && bx0 + tx < g.Wb)
            xe[((size_t)(nn * g.f + f0 + ch) * g.Hb + y) * g.Wb + bx0 + tx] = row_live ? tile[tx][ch] : 0.f;
    }
}

// weight {r,s,f,c} -> [c][f][r][s], flipped in r and s; taps the reference skips (operator.cc:954-957) become zeros.
__global__ void __launch_bounds__(256) k_convtrans_flip_w(const float *__restrict__ w, float *__restrict__ wf, int r, int s, int f,
                                                          int c, int ah, int aw) {
    pdl_prologue();
    const long long total = (long long)c * f * r * s;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        long long rem = i;
        const int ss = (int)(rem % s);
        rem /= s;
        const int rr = (int)(rem % r);
        rem /= r;
        const int ff = (int)(rem % f);
        const int cc = (int)(rem / f);
        float v = 0.f;
        if (!(r - ah < rr || s - aw < ss))
            v = __ldg(w + cc + (size_t)c * (ff + (size_t)f * ((s - 1 - ss) + (size_t)s * (r - 1 - rr))));
        wf[i] = v;
    }
}

// Sub-filter of one phase: [c][f][Ta][Tb], tap (t,t') = flipped tap (rr0 + sh*t, ss0 + sw*t') of the full filter.
__global__ void __launch_bounds__(256) k_convtrans_phase_w(const float *__restrict__ w, float *__restrict__ wf, int r, int s, int f,
                                                           int c, int ah, int aw, int rr0, int sh, int Ta, int ss0, int sw, int Tb) {
    pdl_prologue();
    const long long total = (long long)c * f * Ta * Tb;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        long long rem = i;
        const int tb = (int)(rem % Tb);
        rem /= Tb;
        const int ta = (int)(rem % Ta);
        rem /= Ta;
        const int ff = (int)(rem % f);
        const int cc = (int)(rem / f);
        const int rr = rr0 + sh * ta, ss = ss0 + sw * tb;
        float v = 0.f;
        if (!(r - ah < rr || s - aw < ss))
            v = __ldg(w + cc + (size_t)c * (ff + (size_t)f * ((s - 1 - ss) + (size_t)s * (r - 1 - rr))));
        wf[i] = v;
    }
}

struct Phase {
    void *tc = nullptr;
    DevBuf wsub;
    int a = 0, b = 0, rr0 = 0, ss0 = 0, Ta = 0, Tb = 0;
    ~Phase() {
        if (tc)
            tc_conv_destroy(tc);
    }
};

struct ConvTransPlan : petb200_plan {
    std::vector<Phase *> phases; // non-empty: the phase decomposition is used instead of `conv`
    // The phases write disjoint pixels of y and each fills only part of the GPU, so they run side by side: phase i goes to
    // stream i % 4 (0 = the caller's), forked after the layout pass and joined before the call returns to the stream.
    static constexpr int kSide = 3;
    cudaStream_t side[kSide] = {nullptr, nullptr, nullptr};
    cudaEvent_t ev_fork = nullptr, ev_join[kSide] = {nullptr, nullptr, nullptr};
    DevBuf xn;                   // x as NCHW for the phase convolutions
    int sh = 1, sw = 1;
    ExpandGeom g{};
    int r = 0, s = 0, c = 0, oh = 0, ow = 0, ah = 0, aw = 0, has_bias = 0;
    petb200_plan *conv = nullptr;
    DevBuf xe, wflip;
    DevBuf bx, bw, bb, by; // timing operands
    bool weights_ready = false;
    ~ConvTransPlan() override {
        delete conv;
        for (Phase *p : phases)
            delete p;
        for (int i = 0; i < kSide; ++i) {
            if (side[i])
                cudaStreamDestroy(side[i]);
            if (ev_join[i])
                cudaEventDestroy(ev_join[i]);
        }
        if (ev_fork)
            cudaEventDestroy(ev_fork);
    }
    int bench_launch(cudaStream_t s) override;
};

} // namespace

int make_convtrans_plan(petb200_ctx *ctx, const int *a /*n,c,h,w,f,r,s,ph,pw,sh,sw,dh,dw,g,bias,act,oph,opw*/, int algo,
                        petb200_plan **out) {
    if (!ctx || !a || !out)
        return fail(ctx, PETB200_ERR_INVALID, "convtrans plan: null argument");
    const int n = a[0], c = a[1], h = a[2], w = a[3], f = a[4], r = a[5], s = a[6], ph = a[7], pw = a[8], sh = a[9], sw = a[10];
    const int dh = a[11], dw = a[12], groups = a[13], has_bias = a[14], act = a[15], oph = a[16], opw = a[17];
    if (n <= 0 || c <= 0 || h <= 0 || w <= 0 || f <= 0 || r <= 0 || s <= 0 || sh <= 0 || sw <= 0 || ph < 0 || pw < 0 || oph < 0 || opw < 0)
        return fail(ctx, PETB200_ERR_INVALID, "convtrans plan: bad extent");
    if (dh != 1 || dw != 1) // ref: ConvTransOp::checkValid, src/Graph/operator.cc:1103-1104
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "convtrans plan: dilation must be 1 (the reference refuses dilated transposed convolutions)");
    if (groups != 1) // ref: ConvTransOp::perf, src/Graph/operator.cc:1132-1134
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "convtrans plan: groups must be 1");
    const int oh = (h - 1) * sh - 2 * ph + (r - 1) + oph + 1, ow = (w - 1) * sw - 2 * pw + (s - 1) + opw + 1;
    if (oh <= 0 || ow <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "convtrans plan: empty output");
    auto *pl = new ConvTransPlan();
    pl->ctx = ctx;
    pl->g = ExpandGeom{n, h, w, f, oh + r - 1, ow + s - 1, r - ph - 1, s - pw - 1, sh, sw};
    pl->r = r, pl->s = s, pl->c = c, pl->oh = oh, pl->ow = ow, pl->has_bias = has_bias;
    pl->ah = (h + 2 * ph - r) % sh, pl->aw = (w + 2 * pw - s) % sw;
    const int in_dims[4] = {n, f, pl->g.Hb, pl->g.Wb}, k[2] = {r, s}, zero[2] = {0, 0}, one[2] = {1, 1};
    int rc = make_conv_plan(ctx, 2, in_dims, c, k, zero, one, one, 1, has_bias, act, algo, &pl->conv, 1);
    if (rc) {
        delete pl;
        return rc;
    }
    const size_t xe_bytes = (size_t)n * f * pl->g.Hb * pl->g.Wb * 4, w_bytes = (size_t)c * f * r * s * 4;
    if (pl->xe.alloc(xe_bytes) != cudaSuccess || pl->wflip.alloc(w_bytes) != cudaSuccess) {
        delete pl;
        return fail(ctx, PETB200_ERR_NOMEM, "convtrans plan: scratch allocation (%zu bytes) failed", xe_bytes + w_bytes);
    }
    pl->kernel = pl->conv->kernel;
    pl->device_bytes = pl->conv->device_bytes + xe_bytes + w_bytes;
    pl->sh = sh, pl->sw = sw;
    // Phase decomposition: worth its sh*sw + 1 launches once the zero-inserted product is large (rough model from
    // measurements on B200: the zero-inserted conv sustains ~100 TFLOP/s of issued work, a phase conv ~170 with a floor
    // of ~8 us per launch).  Needs taps in every phase and a row stride of y that is a whole number of phase pixels.
    const double issued = 2.0 * n * c * (double)oh * ow * f * r * s;
    const double us_inserted = issued / 100e6, us_phased = sh * sw * std::max(8.0, issued / (sh * sw) / 170e6);
    const bool tc_algo = tc_is_tc_algo(algo);
    const char *env = getenv("PETB200_CONVTRANS_PHASES");
    const int want = env ? atoi(env) : -1; // 0 never, 1 whenever possible, unset: by size
    if (tc_algo && sh * sw > 1 && r >= sh && s >= sw && ((long long)sh * ow) % sw == 0 && want != 0 && (want == 1 || us_phased < us_inserted) &&
        ctx->cc_major == 10) {
        const int lead_h = r - ph - 1, lead_w = s - pw - 1;
        auto mod = [](int v, int m) { return ((v % m) + m) % m; };
        bool ok = true;
        size_t extra = 0;
        for (int a = 0; a < sh && ok; ++a)
            for (int b = 0; b < sw && ok; ++b) {
                if (a >= oh || b >= ow)
                    continue; // no output row / column in this phase
                auto *ps = new Phase();
                pl->phases.push_back(ps);
                ps->a = a, ps->b = b;
                ps->rr0 = mod(lead_h - a, sh), ps->ss0 = mod(lead_w - b, sw);
                ps->Ta = (r - ps->rr0 + sh - 1) / sh, ps->Tb = (s - ps->ss0 + sw - 1) / sw;
                const int off_a = (a + ps->rr0 - lead_h) / sh, off_b = (b + ps->ss0 - lead_w) / sw; // exact divisions
                const int Ua = (oh - a + sh - 1) / sh, Vb = (ow - b + sw - 1) / sw;
                size_t bytes = 0;
                int prc = tc_conv_create_view(ctx, n, f, h, w, c, ps->Ta, ps->Tb, -off_a, -off_b, Ua, Vb, (int)(((long long)sh * ow) / sw),
                                              (long long)oh * ow * c, 1, (long long)sw * c, has_bias, act,
                                              tc_passes_for(algo), &ps->tc, &bytes);
                if (prc != PETB200_OK || ps->wsub.alloc((size_t)c * f * ps->Ta * ps->Tb * 4) != cudaSuccess)
                    ok = false;
                extra += bytes + ps->wsub.bytes;
            }
        if (ok && pl->xn.alloc((size_t)n * f * h * w * 4) != cudaSuccess)
            ok = false;
        if (!ok) { // keep the zero-insertion path
            for (Phase *p : pl->phases)
                delete p;
            pl->phases.clear();
            pl->xn.alloc(0);
        } else {
            pl->device_bytes += extra + pl->xn.bytes;
            pl->kernel = tc_conv_variant(pl->phases.front()->tc);
        }
    }
    *out = pl;
    return PETB200_OK;
}

int convtrans_set_weights(petb200_plan *plan, const float *w, cudaStream_t s) {
    auto *pl = dynamic_cast<ConvTransPlan *>(plan);
    if (!pl || !w)
        return PETB200_ERR_INVALID;
    petb200_ctx *ctx = pl->ctx;
    const long long total = (long long)pl->c * pl->g.f * pl->r * pl->s;
    const int blocks = (int)std::max<long long>(1, std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 16));
    launch_pdl(k_convtrans_flip_w, blocks, 256, 0, s, w, (float *)pl->wflip.p, pl->r, pl->s, pl->g.f, pl->c, pl->ah, pl->aw);
    int rc = launched(ctx, "k_convtrans_flip_w");
    if (rc)
        return rc;
    rc = conv_set_weights(pl->conv, (const float *)pl->wflip.p, s);
    for (Phase *ps : pl->phases) {
        if (rc)
            break;
        const long long tot = (long long)pl->c * pl->g.f * ps->Ta * ps->Tb;
        const int nb = (int)std::max<long long>(1, std::min<long long>((tot + 255) / 256, (long long)ctx->sm_count * 16));
        launch_pdl(k_convtrans_phase_w, nb, 256, 0, s, w, (float *)ps->wsub.p, pl->r, pl->s, pl->g.f, pl->c, pl->ah, pl->aw, ps->rr0, pl->sh,
                   ps->Ta, ps->ss0, pl->sw, ps->Tb);
        rc = launched(ctx, "k_convtrans_phase_w");
        if (rc == PETB200_OK)
            rc = tc_conv_set_weights(ps->tc, (const float *)ps->wsub.p, s);
    }
    pl->weights_ready = rc == PETB200_OK;
    return rc;
}

int convtrans_run(petb200_plan *plan, const float *x, const float *bias, float *y, cudaStream_t s) {
    auto *pl = dynamic_cast<ConvTransPlan *>(plan);
    if (!pl)
        return PETB200_ERR_INVALID;
    petb200_ctx *ctx = pl->ctx;
    if (!x || !y)
        return fail(ctx, PETB200_ERR_INVALID, "convtrans run: null buffer");
    if (!pl->weights_ready)
        return fail(ctx, PETB200_ERR_INVALID, "convtrans run before set_weights");
    if (!pl->phases.empty()) {
        if (pl->has_bias && !bias)
            return fail(ctx, PETB200_ERR_INVALID, "convtrans run: plan was made with a bias but none was passed");
        // x {n,h,w,f} -> NCHW once (the expansion kernel without insertion), then one convolution per phase
        const ExpandGeom t{pl->g.n, pl->g.h, pl->g.w, pl->g.f, pl->g.h, pl->g.w, 0, 0, 1, 1};
        const dim3 tg((unsigned)((t.Wb + 31) / 32), (unsigned)t.Hb, (unsigned)(t.n * ((t.f + 31) / 32)));
        if (tg.y > 65535u || tg.z > 65535u)
            return fail(ctx, PETB200_ERR_UNSUPPORTED, "convtrans run: image too tall or too many channel tiles for one launch");
        launch_pdl(k_convtrans_expand, tg, dim3(32, 8), 0, s, x, (float *)pl->xn.p, t);
        int rc = launched(ctx, "k_convtrans_expand");
        if (rc)
            return rc;
        const int nside = std::min<int>(ConvTransPlan::kSide, (int)pl->phases.size() - 1);
        if (nside > 0 && !pl->ev_fork) {
            PETB200_CUDA(ctx, cudaEventCreateWithFlags(&pl->ev_fork, cudaEventDisableTiming));
            for (int i = 0; i < nside; ++i) {
                PETB200_CUDA(ctx, cudaStreamCreateWithFlags(&pl->side[i], cudaStreamNonBlocking));
                PETB200_CUDA(ctx, cudaEventCreateWithFlags(&pl->ev_join[i], cudaEventDisableTiming));
            }
        }
        if (nside > 0) {
            PETB200_CUDA(ctx, cudaEventRecord(pl->ev_fork, s));
            for (int i = 0; i < nside; ++i)
                PETB200_CUDA(ctx, cudaStreamWaitEvent(pl->side[i], pl->ev_fork, 0));
        }
        for (size_t i = 0; i < pl->phases.size() && rc == PETB200_OK; ++i) {
            Phase *ps = pl->phases[i];
            const int lane = (int)(i % (size_t)(nside + 1));
            rc = tc_conv_run(ps->tc, (const float *)pl->xn.p, bias, nullptr, y + ((size_t)ps->a * pl->ow + ps->b) * pl->c, nullptr,
                             lane == 0 ? s : pl->side[lane - 1]);
        }
        for (int i = 0; i < nside; ++i) { // join even after a failed launch, so that a capture in progress stays well-formed
            cudaEventRecord(pl->ev_join[i], pl->side[i]);
            cudaStreamWaitEvent(s, pl->ev_join[i], 0);
        }
        return rc;
    }
    const ExpandGeom &g = pl->g;
    const dim3 grid((unsigned)((g.Wb + 31) / 32), (unsigned)g.Hb, (unsigned)(g.n * ((g.f + 31) / 32)));
    if (grid.y > 65535u || grid.z > 65535u)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "convtrans run: expanded image too tall or too many channel tiles for one launch");
    launch_pdl(k_convtrans_expand, grid, dim3(32, 8), 0, s, x, (float *)pl->xe.p, g);
    int rc = launched(ctx, "k_convtrans_expand");
    if (rc)
        return rc;
    return conv_run(pl->conv, (const float *)pl->xe.p, bias, y, nullptr, s);
}

int convtrans_out_dims(const petb200_plan *plan, int *nhwc) {
    auto *pl = dynamic_cast<const ConvTransPlan *>(plan);
    if (!pl || !nhwc)
        return PETB200_ERR_INVALID;
    nhwc[0] = pl->g.n, nhwc[1] = pl->oh, nhwc[2] = pl->ow, nhwc[3] = pl->c;
    return PETB200_OK;
}

int ConvTransPlan::bench_launch(cudaStream_t st) {
    if (!bx.p) {
        const size_t nx = (size_t)g.n * g.h * g.w * g.f, nw = (size_t)r * s * g.f * c, ny = (size_t)g.n * oh * ow * c;
        if (bx.alloc(nx * 4) != cudaSuccess || bw.alloc(nw * 4) != cudaSuccess || by.alloc(ny * 4) != cudaSuccess ||
            bb.alloc((size_t)c * 4) != cudaSuccess)
            return fail(ctx, PETB200_ERR_NOMEM, "scratch allocation for timing failed");
        cudaMemsetAsync(bx.p, 0x3c, nx * 4, st); // 0x3c3c3c3c is 0.0115 as fp32
        cudaMemsetAsync(bw.p, 0x3c, nw * 4, st);
        cudaMemsetAsync(bb.p, 0, (size_t)c * 4, st);
        int rc = convtrans_set_weights(this, (const float *)bw.p, st);
        if (rc)
            return rc;
    }
    return convtrans_run(this, (const float *)bx.p, has_bias ? (const float *)bb.p : nullptr, (float *)by.p, st);
}

} // namespace petb200

using namespace petb200;

extern "C" int petb200_convtrans_plan(petb200_ctx *ctx, const int args[18], int algo, petb200_plan **out) {
    return make_convtrans_plan(ctx, args, algo, out);
}
extern "C" int petb200_convtrans_set_weights(petb200_plan *plan, const float *w, petb200_stream s) {
    return convtrans_set_weights(plan, w, (cudaStream_t)s);
}
extern "C" int petb200_convtrans_run(petb200_plan *plan, const float *x, const float *bias, float *y, petb200_stream s) {
    return convtrans_run(plan, x, bias, y, (cudaStream_t)s);
}
extern "C" int petb200_convtrans_out_dims(const petb200_plan *plan, int out_nhwc[4]) { return convtrans_out_dims(plan, out_nhwc); }
