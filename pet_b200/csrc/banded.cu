// Banded attention products (the reference's G2BMMOp / GBMMLOp, include/operator.h:617-778).
//
// The reference ships generated kernels for one shape only (include/custom_ops.cuh, n=10000 m=64 w=1000 d in {1,4});
// the definitions used here are the ones its rewriter states for the two operators (src/nnet/iterator_table.cc:597-633):
//   G2BMM  y[b,i,j] = sum_k q[b,i,k] * kk[b, i + d*(j-w), k]      y [b,n,2w+1], rows outside [0,n) count as zero
//   GBMML  y[b,i,k] = sum_j p[b,i,j] * v[b, i + d*(j-w), k]       p [b,n,2w+1], y [b,n,m]
// Both kernels work on one dilation residue class at a time: rows i = rho + d*R only meet keys rho + d*(R + j - w), so
// inside a class the problem has dilation 1 and a tile of TI rows x TJ band columns touches TI+TJ-1 consecutive keys.
// Exact fp32 on the CUDA cores (fmaf), any shape.  At the reference's shape G2BMM is bound by writing y and GBMML by
// reading p (both 80 MB against 2.6 GFLOP).
#include "common.h"
#include <algorithm>

namespace petb200 {
namespace {

constexpr int kTI = 32;   // rows of one class per block
constexpr int kKC = 32;   // reduction chunk held in shared memory (G2BMM)
constexpr int kTJ = 128;  // band columns per block (G2BMM)
constexpr int kGJ = 64;   // band columns per reduction chunk (GBMML)
constexpr int kGKR = 96;  // key rows per chunk: kTI + kGJ - 1, rounded up
constexpr int kGM = 64;   // output columns per block (GBMML)

struct BandGeom {
    int n, m, w, d, tiles_per_class;
};

// grid (ceil((2w+1)/kTJ), d * tiles_per_class, b), 256 threads.  Thread (ti = tid/32, tj = tid%32) owns rows 4ti..4ti+3 and
// band columns 4tj..4tj+3 of the tile: out(R, J) = sum_k Qs[k][R] * Ks[k][R + J], key rows 4(ti+tj) .. +6 per step.
__global__ void __launch_bounds__(256) k_g2bmm(const float *__restrict__ q, const float *__restrict__ kk, float *__restrict__ y, BandGeom g) {
    pdl_prologue();
    __shared__ __align__(16) float Qs[kKC][kTI];
    __shared__ __align__(16) float Ks[kKC][kTI + kTJ]; // reused as the [kTI][kTJ + 1] output stage
    const int tid = threadIdx.x, ti = tid >> 5, tj = tid & 31;
    const int rho = blockIdx.y / g.tiles_per_class, R0 = (blockIdx.y % g.tiles_per_class) * kTI, J0 = blockIdx.x * kTJ;
    const int bw = 2 * g.w + 1;
    const size_t bb = (size_t)blockIdx.z * g.n;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c)
            acc[a][c] = 0.f;
    const bool vec = (g.m & 3) == 0 && ((reinterpret_cast<size_t>(q) | reinterpret_cast<size_t>(kk)) & 15) == 0;
    for (int k0 = 0; k0 < g.m; k0 += kKC) {
        // rows of the class: one 16-byte piece of a row per thread and step; consecutive lanes take consecutive rows, so
        // the transposing stores into [k][row] are conflict-free
        for (int e = tid; e < (kTI + (kTI + kTJ)) * (kKC / 4); e += 256) {
            const bool is_q = e < kTI * (kKC / 4);
            const int e2 = is_q ? e : e - kTI * (kKC / 4);
            const int rows = is_q ? kTI : kTI + kTJ;
            const int row = e2 % rows, kq = (e2 / rows) * 4;
            const long long cls = is_q ? (long long)R0 + row : (long long)R0 + row + J0 - g.w; // index inside the class
            const long long i = (long long)rho + (long long)g.d * cls;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (cls >= 0 && i < g.n) {
                const float *src = (is_q ? q : kk) + (bb + (size_t)i) * g.m + k0 + kq;
                if (vec && k0 + kq + 3 < g.m) {
                    const float4 t = __ldg(reinterpret_cast<const float4 *>(src));
                    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
                } else {
#pragma unroll
                    for (int x = 0; x < 4; ++x)
                        if (k0 + kq + x < g.m)
                            v[x] = __ldg(src + x);
                }
            }
#pragma unroll
            for (int x = 0; x < 4; ++x) {
                if (is_q)
                    Qs[kq + x][row] = v[x];
                else
                    Ks[kq + x][row] = v[x];
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < kKC; ++k) {
            const float4 qa = *reinterpret_cast<const float4 *>(&Qs[k][4 * ti]);
            const float4 ka = *reinterpret_cast<const float4 *>(&Ks[k][4 * (ti + tj)]);
            const float4 kb = *reinterpret_cast<const float4 *>(&Ks[k][4 * (ti + tj) + 4]);
            const float qv[4] = {qa.x, qa.y, qa.z, qa.w};
            const float kv[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    acc[a][c] = fmaf(qv[a], kv[a + c], acc[a][c]);
        }
        __syncthreads();
    }
    // through shared memory so that a warp writes 32 consecutive band columns of one row
    float(*stage)[kTJ + 1] = reinterpret_cast<float(*)[kTJ + 1]>(&Ks[0][0]);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c)
            stage[4 * ti + a][4 * tj + c] = acc[a][c];
    __syncthreads();
    for (int r = ti; r < kTI; r += 8) {
        const long long i = (long long)rho + (long long)g.d * (R0 + r);
        if (i >= g.n)
            continue;
        float *dst = y + (bb + (size_t)i) * bw + J0;
#pragma unroll
        for (int c = 0; c < kTJ / 32; ++c) {
            const int j = tj + 32 * c;
            if (J0 + j < bw)
                dst[j] = stage[r][j];
        }
    }
}
static_assert(sizeof(float) * kKC * (kTI + kTJ) >= sizeof(float) * kTI * (kTJ + 1), "output stage must fit the key tile");

// grid (ceil(m/kGM), d * tiles_per_class, b), 128 threads.  Thread (ti = tid/16, tk = tid%16) owns rows 4ti..4ti+3 and
// output columns 4tk..4tk+3.  A chunk of kGJ band columns is re-indexed by key: Ps[key][R] = p[R][key - R] (zero outside
// the chunk), which turns the chunk into a plain [kTI x kGKR] x [kGKR x kGM] product.
__global__ void __launch_bounds__(128) k_gbmml(const float *__restrict__ p, const float *__restrict__ v, float *__restrict__ y, BandGeom g) {
    pdl_prologue();
    __shared__ __align__(16) float Ps[kGKR][kTI + 4];
    __shared__ __align__(16) float Vs[kGKR][kGM];
    const int tid = threadIdx.x, ti = tid >> 4, tk = tid & 15;
    const int rho = blockIdx.y / g.tiles_per_class, R0 = (blockIdx.y % g.tiles_per_class) * kTI, M0 = blockIdx.x * kGM;
    const int bw = 2 * g.w + 1;
    const size_t bb = (size_t)blockIdx.z * g.n;
    const bool vec = (g.m & 3) == 0 && ((reinterpret_cast<size_t>(v) | reinterpret_cast<size_t>(y)) & 15) == 0;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < 4; ++c)
            acc[a][c] = 0.f;
    for (int J0 = 0; J0 < bw; J0 += kGJ) {
        // key row `kr` of the chunk is class index R0 + kr + J0 - w
        for (int e = tid; e < kGKR * kTI; e += 128) {
            const int r = e / kGKR, kr = e % kGKR, jj = kr - r; // consecutive threads: consecutive band columns of one row
            const long long i = (long long)rho + (long long)g.d * (R0 + r);
            const long long kcls = (long long)R0 + kr + J0 - g.w, ki = (long long)rho + (long long)g.d * kcls;
            float val = 0.f;
            if (jj >= 0 && jj < kGJ && J0 + jj < bw && i < g.n && kcls >= 0 && ki < g.n)
                val = __ldg(p + (bb + (size_t)i) * bw + J0 + jj);
            Ps[kr][r] = val;
        }
        for (int e = tid; e < kGKR * (kGM / 4); e += 128) {
            const int kr = e / (kGM / 4), c4 = (e % (kGM / 4)) * 4;
            const long long kcls = (long long)R0 + kr + J0 - g.w, ki = (long long)rho + (long long)g.d * kcls;
            float t[4] = {0.f, 0.f, 0.f, 0.f};
            if (kcls >= 0 && ki < g.n) {
                const float *src = v + (bb + (size_t)ki) * g.m + M0 + c4;
                if (vec && M0 + c4 + 3 < g.m) {
                    const float4 t4 = __ldg(reinterpret_cast<const float4 *>(src));
                    t[0] = t4.x, t[1] = t4.y, t[2] = t4.z, t[3] = t4.w;
                } else {
#pragma unroll
                    for (int x = 0; x < 4; ++x)
                        if (M0 + c4 + x < g.m)
                            t[x] = __ldg(src + x);
                }
            }
            *reinterpret_cast<float4 *>(&Vs[kr][c4]) = make_float4(t[0], t[1], t[2], t[3]);
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
static_assert(kGKR >= kTI + kGJ - 1 && kGKR % 8 == 0, "key rows of a chunk");

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

using namespace petb200;

// Argument order of the reference's launchers: _sg2bmm(q, k, y, bs, n, m, w, d), src/custom_ops.cu:6-9.
extern "C" int petb200_g2bmm_run(petb200_ctx *ctx, const float *q, const float *k, float *y, int bs, int n, int m, int w, int d,
                                 petb200_stream stream) {
    BandGeom g;
    int ytiles;
    int rc = check_band(ctx, q, k, y, bs, n, m, w, d, &g, &ytiles);
    if (rc)
        return rc;
    const dim3 grid((unsigned)((2 * w + 1 + kTJ - 1) / kTJ), (unsigned)ytiles, (unsigned)bs);
    launch_pdl(k_g2bmm, grid, dim3(256), 0, (cudaStream_t)stream, q, k, y, g);
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
    const dim3 grid((unsigned)((m + kGM - 1) / kGM), (unsigned)ytiles, (unsigned)bs);
    launch_pdl(k_gbmml, grid, dim3(128), 0, (cudaStream_t)stream, p, v, y, g);
    return launched(ctx, "k_gbmml");
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
