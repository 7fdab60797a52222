// Elementwise, activation, batch-norm, pooling, softmax and LayerNorm kernels.  All are bandwidth-bound:
// 128-bit accesses where the shape allows, grids sized in multiples of the SM count, warp-shuffle reductions.
#include "common.h"
#include <algorithm>
#include <cfloat>

namespace petb200 {

constexpr int kMaxIn = 4;
struct EltArgs {
    const float *in[kMaxIn];
    unsigned long long size[kMaxIn];
    int n_in, kind, act;
};

__device__ __forceinline__ float combine(int kind, float a, float b) {
    return kind == 0 ? a + b : (kind == 1 ? a - b : a * b);
}

// Operand j is read at i % size_j (the reference's broadcast rule).  vec4 path: every operand either spans the whole
// output or has a size divisible by 4 that divides into aligned groups.
__global__ void __launch_bounds__(256) k_eltwise_v4(EltArgs a, float4 *__restrict__ out, size_t n4) {
    pdl_prologue();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        size_t e = i * 4;
        float4 v = __ldg(reinterpret_cast<const float4 *>(a.in[0] + e % a.size[0]));
#pragma unroll
        for (int j = 1; j < kMaxIn; ++j)
            if (j < a.n_in) {
                float4 w = __ldg(reinterpret_cast<const float4 *>(a.in[j] + e % a.size[j]));
                v.x = combine(a.kind, v.x, w.x);
                v.y = combine(a.kind, v.y, w.y);
                v.z = combine(a.kind, v.z, w.z);
                v.w = combine(a.kind, v.w, w.w);
            }
        v.x = apply_act(v.x, a.act);
        v.y = apply_act(v.y, a.act);
        v.z = apply_act(v.z, a.act);
        v.w = apply_act(v.w, a.act);
        out[i] = v;
    }
}

__global__ void __launch_bounds__(256) k_eltwise(EltArgs a, float *__restrict__ out, size_t n) {
    pdl_prologue();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = __ldg(a.in[0] + i % a.size[0]);
#pragma unroll
        for (int j = 1; j < kMaxIn; ++j)
            if (j < a.n_in)
                v = combine(a.kind, v, __ldg(a.in[j] + i % a.size[j]));
        out[i] = apply_act(v, a.act);
    }
}

__global__ void __launch_bounds__(256) k_batchnorm(const float *__restrict__ x, const float *__restrict__ scale,
                                                   const float *__restrict__ bias, const float *__restrict__ mean,
                                                   const float *__restrict__ var, float *__restrict__ y, size_t total,
                                                   int c, size_t inner, float eps) {
    pdl_prologue();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int cc = (int)((i / inner) % c);
        // the reference forms scale/sqrt(var+eps) in double (src/Graph/operator.cc:2669-2671)
        double k = (double)__ldg(scale + cc) / sqrt((double)__ldg(var + cc) + (double)eps);
        y[i] = (float)(((double)__ldg(x + i) - (double)__ldg(mean + cc)) * k + (double)__ldg(bias + cc));
    }
}

// One thread per output; blockIdx.z walks the (image, channel) planes and a 32x8 thread block covers a patch of one
// plane's outputs, so there is no division anywhere and neighbouring threads read neighbouring inputs.
__global__ void __launch_bounds__(256) k_pool2d(int kind, const float *__restrict__ x, float *__restrict__ y, int nc,
                                                int h, int w, int oh, int ow, int kh, int kw, int ph, int pw, int sh,
                                                int sw) {
    pdl_prologue();
    const int j = blockIdx.x * 32 + threadIdx.x, ii = blockIdx.y * 8 + threadIdx.y;
    if (j >= ow || ii >= oh)
        return;
    for (int plane = blockIdx.z; plane < nc; plane += gridDim.z) {
        const float *xp = x + (size_t)plane * h * w;
        float best = -INFINITY, acc = 0.f;
        int cnt = 0;
        for (int a = 0; a < kh; ++a) {
            const int yy = ii * sh + a - ph;
            if (yy < 0 || yy >= h)
                continue;
            const float *row = xp + (size_t)yy * w;
            for (int b = 0; b < kw; ++b) {
                const int xx = j * sw + b - pw;
                if (xx < 0 || xx >= w)
                    continue;
                const float v = __ldg(row + xx);
                best = fmaxf(best, v);
                acc += v;
                cnt++;
            }
        }
        y[((size_t)plane * oh + ii) * ow + j] = kind == 0 ? best : (cnt ? acc / (float)cnt : 0.f);
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Large windows (global pooling): one warp per output, the window spread over the lanes.  One thread per output would
// walk the window serially, one dependent L2 access after another.
__global__ void __launch_bounds__(256) k_pool2d_warp(int kind, const float *__restrict__ x, float *__restrict__ y, int nc,
                                                     int h, int w, int oh, int ow, int kh, int kw, int ph, int pw, int sh,
                                                     int sw) {
    pdl_prologue();
    const size_t total = (size_t)nc * oh * ow;
    const int lane = threadIdx.x & 31;
    for (size_t i = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5; i < total; i += ((size_t)gridDim.x * blockDim.x) >> 5) {
        const int j = (int)(i % ow);
        const size_t r = i / ow;
        const int ii = (int)(r % oh);
        const float *xp = x + (r / oh) * (size_t)h * w;
        float best = -INFINITY, acc = 0.f;
        int cnt = 0;
        for (int e = lane; e < kh * kw; e += 32) {
            const int a = e / kw, b = e - a * kw;
            const int yy = ii * sh + a - ph, xx = j * sw + b - pw;
            if (yy < 0 || yy >= h || xx < 0 || xx >= w)
                continue;
            const float v = __ldg(xp + (size_t)yy * w + xx);
            best = fmaxf(best, v);
            acc += v;
            cnt++;
        }
        best = warp_max(best);
        acc = warp_sum(acc);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
        if (lane == 0)
            y[i] = kind == 0 ? best : (cnt ? acc / (float)cnt : 0.f);
    }
}

// One warp per row; rows are short (<= a few thousand) in every PET workload, so the row stays in registers/L1.
__global__ void __launch_bounds__(256) k_rowmean(const float *__restrict__ x, float *__restrict__ y, size_t rows, int cols) {
    pdl_prologue();
    size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t r = warp; r < rows; r += nwarps) {
        const float *xp = x + r * (size_t)cols;
        float s = 0.f;
        for (int i = lane; i < cols; i += 32)
            s += __ldg(xp + i);
        s = warp_sum(s);
        if (lane == 0)
            y[r] = s / (float)cols;
    }
}

__global__ void __launch_bounds__(256) k_softmax(const float *__restrict__ x, float *__restrict__ y, size_t rows, int cols) {
    pdl_prologue();
    size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t r = warp; r < rows; r += nwarps) {
        const float *xp = x + r * (size_t)cols;
        float *yp = y + r * (size_t)cols;
        float mx = -INFINITY;
        for (int i = lane; i < cols; i += 32)
            mx = fmaxf(mx, __ldg(xp + i));
        mx = warp_max(mx);
        float den = 0.f;
        for (int i = lane; i < cols; i += 32)
            den += expf(__ldg(xp + i) - mx);
        den = warp_sum(den);
        float inv = 1.f / den;
        for (int i = lane; i < cols; i += 32)
            yp[i] = expf(__ldg(xp + i) - mx) * inv;
    }
}

// Softmax along an axis that is not the innermost one: x viewed as [outer, len, inner], normalised over `len`.  One
// thread per (outer, inner) column; neighbouring threads hold neighbouring `inner` positions, so every step of the walk
// along `len` is one coalesced row of the tensor.  Same arithmetic per column as k_softmax (max, sum of exp, scale).
__global__ void __launch_bounds__(256) k_softmax_strided(const float *__restrict__ x, float *__restrict__ y, size_t outer, int len,
                                                         size_t inner) {
    pdl_prologue();
    const size_t cols = outer * inner;
    for (size_t c = blockIdx.x * (size_t)blockDim.x + threadIdx.x; c < cols; c += (size_t)gridDim.x * blockDim.x) {
        const size_t o = c / inner, i = c - o * inner;
        const float *xp = x + o * (size_t)len * inner + i;
        float *yp = y + o * (size_t)len * inner + i;
        float mx = -INFINITY;
        for (int l = 0; l < len; ++l)
            mx = fmaxf(mx, __ldg(xp + (size_t)l * inner));
        float den = 0.f;
        for (int l = 0; l < len; ++l)
            den += expf(__ldg(xp + (size_t)l * inner) - mx);
        const float inv = 1.f / den;
        for (int l = 0; l < len; ++l)
            yp[(size_t)l * inner] = expf(__ldg(xp + (size_t)l * inner) - mx) * inv;
    }
}

__global__ void __launch_bounds__(256) k_layernorm(const float *__restrict__ x, const float *__restrict__ gamma,
                                                   const float *__restrict__ beta, float *__restrict__ y, size_t rows,
                                                   int cols, float eps) {
    pdl_prologue();
    size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t r = warp; r < rows; r += nwarps) {
        const float *xp = x + r * (size_t)cols;
        float *yp = y + r * (size_t)cols;
        float s = 0.f;
        for (int i = lane; i < cols; i += 32)
            s += __ldg(xp + i);
        float mean = warp_sum(s) / (float)cols;
        float v = 0.f;
        for (int i = lane; i < cols; i += 32) {
            float d = __ldg(xp + i) - mean;
            v += d * d;
        }
        float inv = rsqrtf(warp_sum(v) / (float)cols + eps);
        for (int i = lane; i < cols; i += 32) {
            float o = (__ldg(xp + i) - mean) * inv;
            if (gamma)
                o *= __ldg(gamma + i);
            if (beta)
                o += __ldg(beta + i);
            yp[i] = o;
        }
    }
}

// Block-wide sum / max of one value per thread (blockDim.x = 256), result broadcast to every thread.
__device__ __forceinline__ float block_sum(float v, float *red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        t += red[i];
    return t;
}
__device__ __forceinline__ float block_max(float v, float *red) {
    v = warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0)
        red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i)
        t = fmaxf(t, red[i]);
    return t;
}

// One 256-thread block per row: used when there are too few rows to fill the GPU with one warp per row.
__global__ void __launch_bounds__(256) k_softmax_block(const float *__restrict__ x, float *__restrict__ y, size_t rows, int cols) {
    pdl_prologue();
    __shared__ float red[8];
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float *xp = x + r * (size_t)cols;
        float *yp = y + r * (size_t)cols;
        float mx = -INFINITY;
        for (int i = threadIdx.x; i < cols; i += 256)
            mx = fmaxf(mx, __ldg(xp + i));
        mx = block_max(mx, red);
        float den = 0.f;
        for (int i = threadIdx.x; i < cols; i += 256)
            den += expf(__ldg(xp + i) - mx);
        const float inv = 1.f / block_sum(den, red);
        for (int i = threadIdx.x; i < cols; i += 256)
            yp[i] = expf(__ldg(xp + i) - mx) * inv;
    }
}

__global__ void __launch_bounds__(256) k_layernorm_block(const float *__restrict__ x, const float *__restrict__ gamma,
                                                         const float *__restrict__ beta, float *__restrict__ y, size_t rows,
                                                         int cols, float eps) {
    pdl_prologue();
    __shared__ float red[8];
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float *xp = x + r * (size_t)cols;
        float *yp = y + r * (size_t)cols;
        float s = 0.f;
        for (int i = threadIdx.x; i < cols; i += 256)
            s += __ldg(xp + i);
        const float mean = block_sum(s, red) / (float)cols;
        float v = 0.f;
        for (int i = threadIdx.x; i < cols; i += 256) {
            const float d = __ldg(xp + i) - mean;
            v += d * d;
        }
        const float inv = rsqrtf(block_sum(v, red) / (float)cols + eps);
        for (int i = threadIdx.x; i < cols; i += 256) {
            float o = (__ldg(xp + i) - mean) * inv;
            if (gamma)
                o *= __ldg(gamma + i);
            if (beta)
                o += __ldg(beta + i);
            yp[i] = o;
        }
    }
}

static int grid_for(petb200_ctx *ctx, size_t work_items, int per_block) {
    size_t blocks = (work_items + per_block - 1) / per_block;
    size_t cap = (size_t)ctx->sm_count * 16;
    return (int)std::max<size_t>(1, std::min(blocks, cap));
}

} // namespace petb200

using namespace petb200;

extern "C" int petb200_eltwise_run(petb200_ctx *ctx, int kind, int n_in, const float *const *ins, const size_t *sizes,
                                   float *out, size_t out_size, int act, petb200_stream stream) {
    if (!ctx || !ins || !sizes || !out || kind < 0 || kind > 2 || n_in < 1 || n_in > kMaxIn || (kind == 1 && n_in != 2))
        return fail(ctx, PETB200_ERR_INVALID, "eltwise_run: bad arguments");
    if (out_size == 0)
        return PETB200_OK;
    EltArgs a{};
    a.n_in = n_in;
    a.kind = kind;
    a.act = act;
    bool v4 = (out_size % 4 == 0) && (((uintptr_t)out & 15) == 0);
    for (int j = 0; j < n_in; ++j) {
        if (!ins[j] || sizes[j] == 0)
            return fail(ctx, PETB200_ERR_INVALID, "eltwise_run: operand %d empty", j);
        a.in[j] = ins[j];
        a.size[j] = sizes[j];
        v4 = v4 && (sizes[j] % 4 == 0) && (((uintptr_t)ins[j] & 15) == 0);
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (v4) {
        launch_pdl(k_eltwise_v4, grid_for(ctx, out_size / 4, 256), 256, 0, s, a, (float4 *)out, out_size / 4);
        return launched(ctx, "k_eltwise_v4");
    }
    launch_pdl(k_eltwise, grid_for(ctx, out_size, 256), 256, 0, s, a, out, out_size);
    return launched(ctx, "k_eltwise");
}

extern "C" int petb200_activation_run(petb200_ctx *ctx, const float *x, float *y, size_t n, int act,
                                      petb200_stream stream) {
    const float *ins[1] = {x};
    size_t sizes[1] = {n};
    if (!x || !y)
        return fail(ctx, PETB200_ERR_INVALID, "activation_run: null buffer");
    if (act < 0 || act > PETB200_ACT_GELU)
        return fail(ctx, PETB200_ERR_INVALID, "activation_run: unknown activation %d", act);
    return petb200_eltwise_run(ctx, 0, 1, ins, sizes, y, n, act, stream);
}

extern "C" int petb200_batchnorm_run(petb200_ctx *ctx, const float *x, const float *scale, const float *bias,
                                     const float *mean, const float *var, float *y, size_t outer, int c, size_t inner,
                                     float eps, petb200_stream stream) {
    if (!ctx || !x || !scale || !bias || !mean || !var || !y || c <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "batchnorm_run: bad arguments");
    size_t total = outer * (size_t)c * inner;
    if (!total)
        return PETB200_OK;
    launch_pdl(k_batchnorm, grid_for(ctx, total, 256), 256, 0, (cudaStream_t)stream, x, scale, bias, mean, var, y, total, c,
                                                                             inner, eps);
    return launched(ctx, "k_batchnorm");
}

extern "C" int petb200_pool2d_run(petb200_ctx *ctx, int kind, const float *x, float *y, int n, int c, int h, int w,
                                  int kh, int kw, int ph, int pw, int sh, int sw, petb200_stream stream) {
    if (!ctx || !x || !y || kind < 0 || kind > 1 || n <= 0 || c <= 0 || h <= 0 || w <= 0 || kh <= 0 || kw <= 0 ||
        sh <= 0 || sw <= 0 || ph < 0 || pw < 0)
        return fail(ctx, PETB200_ERR_INVALID, "pool2d_run: bad arguments");
    int oh = (h - (kh - sh) + 2 * ph) / sh, ow = (w - (kw - sw) + 2 * pw) / sw;
    if (oh <= 0 || ow <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "pool2d_run: empty output");
    size_t total = (size_t)n * c * oh * ow;
    if (kh * kw >= 32) {
        launch_pdl(k_pool2d_warp, grid_for(ctx, total, 8), 256, 0, (cudaStream_t)stream, kind, x, y, n * c, h, w, oh, ow, kh, kw, ph,
                                                                                  pw, sh, sw);
        return launched(ctx, "k_pool2d_warp");
    }
    launch_pdl(k_pool2d, dim3((unsigned)((ow + 31) / 32), (unsigned)((oh + 7) / 8), (unsigned)std::min(n * c, 65535)), dim3(32, 8), 0,
               (cudaStream_t)stream, kind, x, y, n * c, h, w, oh, ow, kh, kw, ph, pw, sh, sw);
    return launched(ctx, "k_pool2d");
}

extern "C" int petb200_rowmean_run(petb200_ctx *ctx, const float *x, float *y, size_t rows, int cols,
                                   petb200_stream stream) {
    if (!ctx || !x || !y || cols <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "rowmean_run: bad arguments");
    if (!rows)
        return PETB200_OK;
    launch_pdl(k_rowmean, grid_for(ctx, rows, 8), 256, 0, (cudaStream_t)stream, x, y, rows, cols);
    return launched(ctx, "k_rowmean");
}

extern "C" int petb200_softmax_run(petb200_ctx *ctx, const float *x, float *y, size_t rows, int cols,
                                   petb200_stream stream) {
    if (!ctx || !x || !y || cols <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "softmax_run: bad arguments");
    if (!rows)
        return PETB200_OK;
    if (cols >= 256 && rows <= (size_t)ctx->sm_count * 64) {
        launch_pdl(k_softmax_block, (int)std::min<size_t>(rows, (size_t)ctx->sm_count * 8), 256, 0, (cudaStream_t)stream, x, y, rows, cols);
        return launched(ctx, "k_softmax_block");
    }
    launch_pdl(k_softmax, grid_for(ctx, rows, 8), 256, 0, (cudaStream_t)stream, x, y, rows, cols);
    return launched(ctx, "k_softmax");
}

extern "C" int petb200_softmax_axis_run(petb200_ctx *ctx, const float *x, float *y, size_t outer, int len, size_t inner,
                                        petb200_stream stream) {
    if (!ctx || !x || !y || len <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "softmax_axis_run: bad arguments");
    if (!outer || !inner)
        return PETB200_OK;
    if (inner == 1)
        return petb200_softmax_run(ctx, x, y, outer, len, stream);
    launch_pdl(k_softmax_strided, grid_for(ctx, outer * inner, 256), 256, 0, (cudaStream_t)stream, x, y, outer, len, inner);
    return launched(ctx, "k_softmax_strided");
}

extern "C" int petb200_layernorm_run(petb200_ctx *ctx, const float *x, const float *gamma, const float *beta, float *y,
                                     size_t rows, int cols, float eps, petb200_stream stream) {
    if (!ctx || !x || !y || cols <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "layernorm_run: bad arguments");
    if (!rows)
        return PETB200_OK;
    if (cols >= 256 && rows <= (size_t)ctx->sm_count * 64) {
        launch_pdl(k_layernorm_block, (int)std::min<size_t>(rows, (size_t)ctx->sm_count * 8), 256, 0, (cudaStream_t)stream, x, gamma, beta, y, rows,
                                                                                                           cols, eps);
        return launched(ctx, "k_layernorm_block");
    }
    launch_pdl(k_layernorm, grid_for(ctx, rows, 8), 256, 0, (cudaStream_t)stream, x, gamma, beta, y, rows, cols, eps);
    return launched(ctx, "k_layernorm");
}
