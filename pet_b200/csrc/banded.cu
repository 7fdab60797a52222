// Banded attention products (the reference's G2BMMOp / GBMMLOp, include/operator.h:617-778).
//
// The reference ships generated kernels for one shape only (include/custom_ops.cuh, n=10000 m=64 w=1000 d in {1,4});
// the definitions used here are the ones its rewriter states for the two operators (src/nnet/iterator_table.cc:597-633):
//   G2BMM  y[b,i,j] = sum_k q[b,i,k] * kk[b, i + d*(j-w), k]      y [b,n,2w+1], rows outside [0,n) count as zero
//   GBMML  y[b,i,k] = sum_j p[b,i,j] * v[b, i + d*(j-w), k]       p [b,n,2w+1], y [b,n,m]
// Both kernels work on one dilation residue class at a time: rows i = rho + d*R only meet keys rho + d*(R + j - w), so
// inside a class the problem has dilation 1 and a tile of TI rows x TJ band columns touches TI+TJ-1 consecutive keys.
// Exact fp32 on the CUDA cores (fmaf), any shape.  At the reference's shape the band tensor is 80 MB against 2.6 GFLOP:
// 32 flops per byte, which puts both kernels on the compute side of the CUDA cores' roofline (the FMA pipe, not HBM).
#include "common.h"
#include <algorithm>

namespace petb200 {
namespace {

constexpr int kTI = 32;   // rows of one class per block
constexpr int kKC = 32;   // reduction chunk held in shared memory (G2BMM)
constexpr int kTJ = 224;  // band columns per block (G2BMM)
constexpr int kKeys = 256; // keys per block (G2BMM): kTI + kTJ
constexpr int kGJ = 96;   // band columns per reduction chunk (GBMML)
constexpr int kGKR = 128; // key rows per chunk: kTI + kGJ - 1, rounded up
constexpr int kGM = 64;   // output columns per block (GBMML)

struct BandGeom {
    int n, m, w, d, tiles_per_class;
    int mtiles, chunks_per_split; // GBMML: column tiles of y; band-column chunks summed by one block
};

// grid (ceil((2w+1)/kTJ), d * tiles_per_class, b), 128 threads.  In (row, key) coordinates the band is an ordinary product
// P[R][key] = q[R] . kk[key]: a block forms the kTI x kKeys rectangle of it that holds band columns [J0, J0 + kTJ) of its
// rows (the parallelogram key - R in [0, kTJ)) with an 8 x 8 register tile per thread — rows 8ti..8ti+7, keys
// 4tj..4tj+3 and 128+4tj..128+4tj+3, so that a warp's 16-byte reads of the key tile are consecutive — and writes the
// parallelogram out through shared memory, a warp storing 32 consecutive band columns of one row.
__global__ void __launch_bounds__(128) k_g2bmm(const float *__restrict__ q, const float *__restrict__ kk, float *__restrict__ y, BandGeom g) {
    pdl_prologue();
    __shared__ __align__(16) float Qs[kKC][kTI];
    __shared__ __align__(16) float Ks[kKC][kKeys]; // reused as the [kTI][kKeys] output stage
    const int tid = threadIdx.x, ti = tid >> 5, tj = tid & 31;
    const int rho = blockIdx.y / g.tiles_per_class, R0 = (blockIdx.y % g.tiles_per_class) * kTI, J0 = blockIdx.x * kTJ;
    const int bw = 2 * g.w + 1;
    const size_t bb = (size_t)blockIdx.z * g.n;
    float acc[8][8];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int c = 0; c < 8; ++c)
            acc[a][c] = 0.f;
    const bool vec = (g.m & 3) == 0 && ((reinterpret_cast<size_t>(q) | reinterpret_cast<size_t>(kk)) & 15) == 0;
    const int cls_lim = (g.n - rho + g.d - 1) / g.d; // class indices 0 .. cls_lim-1 are rows of the sequence
    for (int k0 = 0; k0 < g.m; k0 += kKC) {
        // One 16-byte piece of a row per thread and step: eight lanes read the 128 contiguous bytes of a row, a warp four
        // consecutive rows.  The tiles are stored transposed ([k][row]) with the 4-row groups of a k row XOR-swizzled by
        // k / 4, which makes both these scattered stores and the 16-byte reads of the product loop conflict-free.  Loads
        // are issued in batches so that their latencies overlap.
        {
            const int kq = (tid & 7) * 4, r_lo = tid >> 3; // this thread's piece of a row, and its first row (then every 16th)
            const bool full = vec && k0 + kq + 3 < g.m;
            auto fetch = [&](const float *base, int cls) {
                float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                if (cls >= 0 && cls < cls_lim) {
                    const float *src = base + (bb + (size_t)rho + (size_t)g.d * cls) * g.m + k0 + kq;
                    if (full) {
                        t = __ldg(reinterpret_cast<const float4 *>(src));
                    } else {
                        if (k0 + kq < g.m) t.x = __ldg(src);
                        if (k0 + kq + 1 < g.m) t.y = __ldg(src + 1);
                        if (k0 + kq + 2 < g.m) t.z = __ldg(src + 2);
                        if (k0 + kq + 3 < g.m) t.w = __ldg(src + 3);
                    }
                }
                return t;
            };
            auto put = [&](float *tile, int pitch, int row, const float4 &t) {
                float *dstp = tile + kq * pitch + ((((row >> 2) ^ (kq >> 2)) << 2) | (row & 3)); // swizzled inside each aligned run of 8 groups
                dstp[0] = t.x, dstp[pitch] = t.y, dstp[2 * pitch] = t.z, dstp[3 * pitch] = t.w;
            };
            const float4 q0 = fetch(q, R0 + r_lo), q1 = fetch(q, R0 + r_lo + 16);
            put(&Qs[0][0], kTI, r_lo, q0);
            put(&Qs[0][0], kTI, r_lo + 16, q1);
            const int kcls0 = R0 + r_lo + J0 - g.w;
#pragma unroll 1
            for (int it0 = 0; it0 < kKeys / 16; it0 += 8) {
                float4 buf[8];
#pragma unroll
                for (int b = 0; b < 8; ++b)
                    buf[b] = fetch(kk, kcls0 + 16 * (it0 + b));
#pragma unroll
                for (int b = 0; b < 8; ++b)
                    put(&Ks[0][0], kKeys, r_lo + 16 * (it0 + b), buf[b]);
            }
        }
        __syncthreads();
#pragma unroll 4
        for (int k = 0; k < kKC; ++k) {
            const int h = k >> 2; // the swizzle of this k row
            const float4 qa = *reinterpret_cast<const float4 *>(&Qs[k][((2 * ti) ^ h) << 2]);
            const float4 qb = *reinterpret_cast<const float4 *>(&Qs[k][((2 * ti + 1) ^ h) << 2]);
            const float4 ka = *reinterpret_cast<const float4 *>(&Ks[k][(tj ^ h) << 2]);
            const float4 kb = *reinterpret_cast<const float4 *>(&Ks[k][kKeys / 2 + ((tj ^ h) << 2)]);
            const float qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
            const float kv[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
#pragma unroll
            for (int a = 0; a < 8; ++a)
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    acc[a][c] = fmaf(qv[a], kv[c], acc[a][c]);
        }
        __syncthreads();
    }
    float(*stage)[kKeys] = Ks;
#pragma unroll
    for (int a = 0; a < 8; ++a) {
        *reinterpret_cast<float4 *>(&stage[8 * ti + a][4 * tj]) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
        *reinterpret_cast<float4 *>(&stage[8 * ti + a][kKeys / 2 + 4 * tj]) = make_float4(acc[a][4], acc[a][5], acc[a][6], acc[a][7]);
    }
    __syncthreads();
    for (int r = ti; r < kTI; r += 4) {
        const long long i = (long long)rho + (long long)g.d * (R0 + r);
        if (i >= g.n)
            continue;
        float *dst = y + (bb + (size_t)i) * bw + J0;
#pragma unroll
        for (int c = 0; c < kTJ / 32; ++c) {
            const int j = tj + 32 * c;
            if (J0 + j < bw)
                dst[j] = stage[r][r + j]; // band column j of row r is key r + j of the tile
        }
    }
}
static_assert(kKeys == kTI + kTJ && kTJ % 32 == 0 && kKeys == 256 && kKC == kTI, "tile geometry of k_g2bmm");

// grid (ceil(m/kGM) * splits, d * tiles_per_class, b), 128 threads.  The band columns are split over `splits` blocks so that
// a long band still fills the GPU; split s writes its partial sums to y + s * (b*n*m) (the caller passes scratch there and
// k_band_reduce adds the parts in split order).  Thread (ti = tid/16, tk = tid%16) owns rows 4ti..4ti+3 and
// output columns 4tk..4tk+3.  A chunk of kGJ band columns is re-indexed by key: Ps[key][R] = p[R][key - R] (zero outside
// the chunk), which turns the chunk into a plain [kTI x kGKR] x [kGKR x kGM] product.
__global__ void __launch_bounds__(128) k_gbmml(const float *__restrict__ p, const float *__restrict__ v, float *__restrict__ y, BandGeom g) {
    pdl_prologue();
    extern __shared__ __align__(16) float band_smem[];
    float(*Ps)[kTI + 4] = reinterpret_cast<float(*)[kTI + 4]>(band_smem);                     // [kGKR][kTI + 4]
    float(*Vs)[kGM] = reinterpret_cast<float(*)[kGM]>(band_smem + kGKR * (kTI + 4));          // [kGKR][kGM]
    const int tid = threadIdx.x, ti = tid >> 4, tk = tid & 15;
    const int rho = blockIdx.y / g.tiles_per_class, R0 = (blockIdx.y % g.tiles_per_class) * kTI;
    const int M0 = ((int)blockIdx.x % g.mtiles) * kGM, split = (int)blockIdx.x / g.mtiles;
    const int bw = 2 * g.w + 1;
    const size_t bb = (size_t)blockIdx.z * g.n;
    y += (size_t)split * gridDim.z * g.n * g.m;
    const int J_begin = split * g.chunks_per_split * kGJ, J_end = min(bw, J_begin + g.chunks_per_split * kGJ);
    const bool vec = (g.m & 3) == 0 && ((reinterpret_cast<size_t>(v) | reinterpret_cast<size_t>(y)) & 15) == 0;
    const int cls_lim = (g.n - rho + g.d - 1) / g.d;    // class indices 0 .. cls_lim-1 are rows of the sequence
    const int rows_valid = min(kTI, cls_lim - R0);      // rows of this tile inside the sequence
    const size_t p_step = (size_t)g.d * bw - 1;         // next row of the class, one band column to the left
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c)
            acc[a][c] = 0.f;
    for (int J0 = J_begin; J0 < J_end; J0 += kGJ) {
        // Key row kr of the chunk is class index R0 + kr + J0 - w.  Thread `tid` fills key row tid of Ps: for row r that
        // is band column tid - r of the chunk — consecutive threads read consecutive band columns.  Loads are issued in
        // batches so that their latencies overlap.
        {
            const int kcls = R0 + tid + J0 - g.w;
            const bool key_ok = kcls >= 0 && kcls < cls_lim;
            const float *src = p + (bb + (size_t)rho + (size_t)g.d * R0) * bw + J0 + tid;
#pragma unroll 1
            for (int r0 = 0; r0 < kTI; r0 += 8) {
                float buf[8];
#pragma unroll
                for (int b = 0; b < 8; ++b) {
                    const int r = r0 + b, jj = tid - r;
                    buf[b] = (key_ok && r < rows_valid && jj >= 0 && jj < kGJ && J0 + jj < J_end) ? __ldg(src + r * p_step) : 0.f;
                }
#pragma unroll
                for (int b = 0; b < 8; ++b)
                    Ps[tid][r0 + b] = buf[b];
            }
        }
        {
            const int c4 = (tid & 15) * 4;
            const int kcls0 = R0 + (tid >> 4) + J0 - g.w; // this thread's key rows: kcls0 + 8 * it
            const bool full = vec && M0 + c4 + 3 < g.m;
#pragma unroll 1
            for (int it0 = 0; it0 < kGKR / 8; it0 += 4) {
                float4 buf[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const int kcls = kcls0 + 8 * (it0 + b);
                    float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (kcls >= 0 && kcls < cls_lim) {
                        const float *src = v + (bb + (size_t)rho + (size_t)g.d * kcls) * g.m + M0 + c4;
                        if (full) {
                            t = __ldg(reinterpret_cast<const float4 *>(src));
                        } else {
                            if (M0 + c4 < g.m) t.x = __ldg(src);
                            if (M0 + c4 + 1 < g.m) t.y = __ldg(src + 1);
                            if (M0 + c4 + 2 < g.m) t.z = __ldg(src + 2);
                            if (M0 + c4 + 3 < g.m) t.w = __ldg(src + 3);
                        }
                    }
                    buf[b] = t;
                }
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    *reinterpret_cast<float4 *>(&Vs[(tid >> 4) + 8 * (it0 + b)][c4]) = buf[b];
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int kr = 0; kr < kGKR; ++kr) {
            const float4 pa = *reinterpret_cast<const float4 *>(&Ps[kr][4 * ti]);
            const float4 va = *reinterpret_cast<const float4 *>(&Vs[kr][4 * tk]);
            const float pv[4] = {pa.x, pa.y, pa.z, pa.w};
            const float vv[4] = {va.x, va.y, va.z, va.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    acc[a][c] = fmaf(pv[a], vv[c], acc[a][c]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const long long i = (long long)rho + (long long)g.d * (R0 + 4 * ti + a);
        if (i >= g.n)
            continue;
        float *dst = y + (bb + (size_t)i) * g.m + M0 + 4 * tk;
        if (vec && M0 + 4 * tk + 3 < g.m) {
            *reinterpret_cast<float4 *>(dst) = make_float4(acc[a][0], acc[a][1], acc[a][2], acc[a][3]);
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (M0 + 4 * tk + c < g.m)
                    dst[c] = acc[a][c];
        }
    }
}
constexpr size_t kGbmmlSmem = sizeof(float) * kGKR * (kTI + 4 + kGM);
static_assert(kGKR >= kTI + kGJ - 1 && kGKR == 128 && kTI % 8 == 0, "key rows of a chunk: one per thread of k_gbmml");

// y[i] = parts[0][i] + parts[1][i] + ... in split order (the sum does not depend on timing).
__global__ void __launch_bounds__(256) k_band_reduce(const float *__restrict__ parts, float *__restrict__ y, size_t total, int splits) {
    pdl_prologue();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float acc = parts[i];
        for (int s = 1; s < splits; ++s)
            acc += parts[(size_t)s * total + i];
        y[i] = acc;
    }
}

int check_band(petb200_ctx *ctx, const void *a, const void *b, const void *y, int bs, int n, int m, int w, int d, BandGeom *g, int *ytiles) {
    if (!ctx)
        return PETB200_ERR_INVALID;
    if (!a || !b || !y)
        return fail(ctx, PETB200_ERR_INVALID, "banded product: null buffer");
    // ref: G2BMMOp::checkValid, src/Graph/operator.cc:1390-1412 (width may be 0; dilation is a positive step)
    if (bs <= 0 || n <= 0 || m <= 0 || w < 0 || d <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "banded product: bad extent (b=%d n=%d m=%d w=%d d=%d)", bs, n, m, w, d);
    const int per_class = (n + d - 1) / d;
    g->n = n, g->m = m, g->w = w, g->d = d, g->tiles_per_class = (per_class + kTI - 1) / kTI;
    const long long rows = (long long)std::min(d, n) * g->tiles_per_class;
    if (rows > 65535 || bs > 65535)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "banded product: too many row tiles (%lld) or batches (%d) for one launch", rows, bs);
    *ytiles = (int)rows;
    return PETB200_OK;
}

} // namespace
} // namespace petb200

// implemented in igemm_tc.cu
namespace petb200 {
int tc_g2bmm_create(petb200_ctx *ctx, int bs, int n, int m, int w, void **out);
int tc_gbmml_create(petb200_ctx *ctx, int bs, int n, int m, int w, void **out);
int tc_gbmml_run(void *h, const float *p, float *y, cudaStream_t s);
void tc_matmul_destroy(void *h);
int tc_matmul_pack_b(void *h, const float *b, cudaStream_t s);
int tc_matmul_run(void *h, const float *a_t, const float *bias, const float *res, float *cmat, cudaStream_t s);
} // namespace petb200

using namespace petb200;

// The tensor-core plan of a banded product of this shape, made on first use; null where that path does not apply (then the
// CUDA-core kernels below run): dilation 1, m a multiple of 4, 16-byte aligned operands, PETB200_BANDED_TC=0 not set.
static void *band_tc_plan(petb200_ctx *ctx, int kind, const void *a, const void *b, int bs, int n, int m, int w, int d) {
    static const bool enabled = !(getenv("PETB200_BANDED_TC") && atoi(getenv("PETB200_BANDED_TC")) == 0);
    if (!enabled || d != 1 || w < 1 || ctx->cc_major != 10 || (m & 3) || (((size_t)a | (size_t)b) & 15))
        return nullptr;
    for (auto &e : ctx->band_tc)
        if (e.key[0] == kind && e.key[1] == bs && e.key[2] == n && e.key[3] == m && e.key[4] == w)
            return e.plan;
    void *plan = nullptr;
    if ((kind == 0 ? tc_g2bmm_create(ctx, bs, n, m, w, &plan) : tc_gbmml_create(ctx, bs, n, m, w, &plan)) != PETB200_OK)
        plan = nullptr; // remembered as "not on this path"
    ctx->band_tc_destroy = tc_matmul_destroy;
    ctx->band_tc.push_back({{kind, bs, n, m, w}, plan});
    return plan;
}

// Tuning only: per-CTA counters of the tensor-core plans made so far (see IgemmParams::prof), null to stop.
namespace petb200 {
void tc_matmul_set_prof(void *h, long long *p);
}
extern "C" int petb200_debug_band_prof(petb200_ctx *ctx, long long *dev_counters) {
    for (auto &e : ctx->band_tc)
        if (e.plan)
            tc_matmul_set_prof(e.plan, dev_counters);
    return PETB200_OK;
}

// Argument order of the reference's launchers: _sg2bmm(q, k, y, bs, n, m, w, d), src/custom_ops.cu:6-9.
extern "C" int petb200_g2bmm_run(petb200_ctx *ctx, const float *q, const float *k, float *y, int bs, int n, int m, int w, int d,
                                 petb200_stream stream) {
    BandGeom g;
    int ytiles;
    int rc = check_band(ctx, q, k, y, bs, n, m, w, d, &g, &ytiles);
    if (rc)
        return rc;
    if (void *plan = band_tc_plan(ctx, 0, q, k, bs, n, m, w, d)) {
        // keys split into hi/lo once per call (they are an activation), then the tensor-core kernel with the banded epilogue
        rc = tc_matmul_pack_b(plan, k, (cudaStream_t)stream);
        return rc ? rc : tc_matmul_run(plan, q, nullptr, nullptr, y, (cudaStream_t)stream);
    }
    const dim3 grid((unsigned)((2 * w + 1 + kTJ - 1) / kTJ), (unsigned)ytiles, (unsigned)bs);
    launch_pdl(k_g2bmm, grid, dim3(128), 0, (cudaStream_t)stream, q, k, y, g);
    return launched(ctx, "k_g2bmm");
}

// _sgbmml(prob, v, y, bs, n, m, w, d), src/custom_ops.cu:11-14.
extern "C" int petb200_gbmml_run(petb200_ctx *ctx, const float *p, const float *v, float *y, int bs, int n, int m, int w, int d,
                                 petb200_stream stream) {
    BandGeom g;
    int ytiles;
    int rc = check_band(ctx, p, v, y, bs, n, m, w, d, &g, &ytiles);
    if (rc)
        return rc;
    if (void *plan = band_tc_plan(ctx, 1, p, v, bs, n, m, w, d)) {
        // value rows split into hi/lo once per call, then the tensor-core kernel gathering the band from global memory
        rc = tc_matmul_pack_b(plan, v, (cudaStream_t)stream);
        return rc ? rc : tc_gbmml_run(plan, p, y, (cudaStream_t)stream);
    }
    // Split the band columns over blocks so that the last wave of blocks is not nearly empty: cost of a choice = waves of
    // resident blocks (four per SM) x chunks per block, plus a little per split for the reduction pass.
    const int chunks = (2 * w + 1 + kGJ - 1) / kGJ;
    g.mtiles = (m + kGM - 1) / kGM;
    const long long base = (long long)g.mtiles * ytiles * bs, slots = 4LL * ctx->sm_count;
    int splits = 1;
    double best = 0;
    for (int sp = 1; sp <= std::min(chunks, 16); ++sp) {
        const int cps = (chunks + sp - 1) / sp, real = (chunks + cps - 1) / cps;
        const double cost = (double)((base * real + slots - 1) / slots) * cps + 0.3 * (real - 1);
        if (sp == 1 || cost < best * 0.98)
            best = cost, splits = real, g.chunks_per_split = cps;
    }
    const size_t total = (size_t)bs * n * m;
    float *dst = y;
    if (splits > 1) {
        if (ctx->band_scratch.bytes < total * splits * 4) {
            // the outgrown buffer is retired, not freed: an earlier captured graph may still hold its address
            if (ctx->band_scratch.p)
                ctx->band_retired.push_back(ctx->band_scratch.release());
            if (ctx->band_scratch.alloc(total * splits * 4) != cudaSuccess)
                return fail(ctx, PETB200_ERR_NOMEM, "gbmml: scratch for %d partial sums failed", splits);
        }
        dst = (float *)ctx->band_scratch.p;
    }
    const dim3 grid((unsigned)(g.mtiles * splits), (unsigned)ytiles, (unsigned)bs);
    if (!ctx->band_attr_set) {
        PETB200_CUDA(ctx, cudaFuncSetAttribute(k_gbmml, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGbmmlSmem));
        ctx->band_attr_set = true;
    }
    launch_pdl(k_gbmml, grid, dim3(128), kGbmmlSmem, (cudaStream_t)stream, p, v, dst, g);
    rc = launched(ctx, "k_gbmml");
    if (rc || splits == 1)
        return rc;
    const int blocks = (int)std::min<size_t>((total + 255) / 256, (size_t)ctx->sm_count * 8);
    launch_pdl(k_band_reduce, blocks, 256, 0, (cudaStream_t)stream, (const float *)dst, y, total, splits);
    return launched(ctx, "k_band_reduce");
}

// Milliseconds per launch on library-owned operands, the way G2BMMOp::perf / GBMMLOp::perf time the reference's kernels
// (src/Graph/operator.cc:1424-1465, :1562-1598).  kind 0 = G2BMM, 1 = GBMML.
extern "C" int petb200_banded_time(petb200_ctx *ctx, int kind, int bs, int n, int m, int w, int d, int rounds, int warmup, float *ms,
                                   petb200_stream stream) {
    if (!ctx || !ms || rounds <= 0 || warmup < 0 || (kind != 0 && kind != 1))
        return fail(ctx, PETB200_ERR_INVALID, "banded_time: bad argument");
    if (bs <= 0 || n <= 0 || m <= 0 || w < 0 || d <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "banded_time: bad extent");
    const size_t thin = (size_t)bs * n * m * 4, band = (size_t)bs * n * (2 * (size_t)w + 1) * 4;
    DevBuf a, b, y;
    if (a.alloc(kind == 0 ? thin : band) != cudaSuccess || b.alloc(thin) != cudaSuccess || y.alloc(kind == 0 ? band : thin) != cudaSuccess)
        return fail(ctx, PETB200_ERR_NOMEM, "banded_time: operand allocation failed");
    cudaStream_t s = (cudaStream_t)stream;
    cudaMemsetAsync(a.p, 0x3c, a.bytes, s); // 0x3c3c3c3c is 0.0115 as fp32
    cudaMemsetAsync(b.p, 0x3c, b.bytes, s);
    cudaEvent_t e0, e1;
    PETB200_CUDA(ctx, cudaEventCreate(&e0));
    PETB200_CUDA(ctx, cudaEventCreate(&e1));
    int rc = PETB200_OK;
    for (int i = 0; i < warmup + rounds && rc == PETB200_OK; ++i) {
        if (i == warmup)
            cudaEventRecord(e0, s);
        rc = kind == 0 ? petb200_g2bmm_run(ctx, (const float *)a.p, (const float *)b.p, (float *)y.p, bs, n, m, w, d, stream)
                       : petb200_gbmml_run(ctx, (const float *)a.p, (const float *)b.p, (float *)y.p, bs, n, m, w, d, stream);
    }
    cudaEventRecord(e1, s);
    cudaError_t e = cudaEventSynchronize(e1);
    float t = 0.f;
    if (e == cudaSuccess)
        cudaEventElapsedTime(&t, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc)
        return rc;
    if (e != cudaSuccess)
        return fail(ctx, PETB200_ERR_CUDA, "banded_time: %s", cudaGetErrorString(e));
    *ms = t / rounds;
    return PETB200_OK;
}
