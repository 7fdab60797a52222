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

// The same with one (outer, channel) plane per block iteration: scale / sqrt(var + eps) — a double-precision division and
// square root — is formed once per plane instead of once per element, and the plane is streamed with coalesced accesses.
__global__ void __launch_bounds__(256) k_batchnorm_plane(const float *__restrict__ x, const float *__restrict__ scale,
                                                         const float *__restrict__ bias, const float *__restrict__ mean,
                                                         const float *__restrict__ var, float *__restrict__ y, size_t planes, int c,
                                                         size_t inner, float eps) {
    pdl_prologue();
    for (size_t p = blockIdx.x; p < planes; p += gridDim.x) {
        const int cc = (int)(p % (size_t)c);
        const double k = (double)__ldg(scale + cc) / sqrt((double)__ldg(var + cc) + (double)eps);
        const double m = (double)__ldg(mean + cc), b = (double)__ldg(bias + cc);
        const float *xp = x + p * inner;
        float *yp = y + p * inner;
        for (size_t i = threadIdx.x; i < inner; i += 256)
            yp[i] = (float)(((double)__ldg(xp + i) - m) * k + b);
    }
}

// Pooling with small windows, the input rows of a band of output rows staged in shared memory: the band is one contiguous
// run of the plane, so it is fetched with fully coalesced loads once, and the window walks (strided, overlapping) hit
// shared memory instead of L1.  blockIdx.x = band of `ohb` output rows, blockIdx.y walks the planes.  MAX3S2: the window is
// 3x3, the stride 2 and the operator max (ResNet's stem pool), all at compile time: nine unrolled, predicated compares.
template <bool MAX3S2>
__global__ void __launch_bounds__(256) k_pool2d_tiled(int kind, const float *__restrict__ x, float *__restrict__ y, int nc, int h,
                                                      int w, int oh, int ow, int kh, int kw, int ph, int pw, int sh, int sw,
                                                      int ohb, int rows_in) {
    pdl_prologue();
    extern __shared__ __align__(16) float tile[];
    const int o0 = blockIdx.x * ohb, on = min(ohb, oh - o0);
    const int y0 = o0 * sh - ph;                        // first input row of the band (may be negative: padding)
    const int ylo = max(y0, 0), yhi = min(y0 + rows_in, h); // rows that exist
    const int count = max(yhi - ylo, 0) * w;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int plane = blockIdx.y; plane < nc; plane += gridDim.y) {
        const float *src = x + ((size_t)plane * h + ylo) * w;
        float *dst = tile + (ylo - y0) * w;
        // 16-byte copies need BOTH ends aligned: the global run and its place in the tile (rows skipped as padding shift it)
        if ((((uintptr_t)src) & 15) == 0 && (count & 3) == 0 && ((((ylo - y0) * w) & 3) == 0)) {
            for (int i = threadIdx.x; i < count / 4; i += 256)
                reinterpret_cast<float4 *>(dst)[i] = __ldg(reinterpret_cast<const float4 *>(src) + i);
        } else {
            for (int i = threadIdx.x; i < count; i += 256)
                dst[i] = __ldg(src + i);
        }
        __syncthreads();
        for (int ii = warp; ii < on; ii += 8) {
            for (int j = lane; j < ow; j += 32) {
                // the window clipped to the input once, then two plain loops
                const int ys = (o0 + ii) * sh - ph, xs = j * sw - pw;
                const int a0 = max(0, -ys), a1 = min(kh, h - ys), b0 = max(0, -xs), b1 = min(kw, w - xs);
                float best = -INFINITY, acc = 0.f;
                for (int a = a0; a < a1 && !MAX3S2; ++a) {
                    const float *row = tile + (ys + a - y0) * w + xs;
                    for (int b = b0; b < b1; ++b) {
                        const float v = row[b];
                        best = fmaxf(best, v);
                        acc += v;
                    }
                }
                const int cnt = max(a1 - a0, 0) * max(b1 - b0, 0);
                if (MAX3S2) {
                    best = -INFINITY;
                    const float *row = tile + (ys - y0) * w + xs;
#pragma unroll
                    for (int a = 0; a < 3; ++a)
#pragma unroll
                        for (int b = 0; b < 3; ++b)
                            if (a >= a0 && a < a1 && b >= b0 && b < b1)
                                best = fmaxf(best, row[a * w + b]);
                    y[((size_t)plane * oh + o0 + ii) * ow + j] = best;
                    continue;
                }
                y[((size_t)plane * oh + o0 + ii) * ow + j] = kind == 0 ? best : (cnt ? acc / (float)cnt : 0.f);
            }
        }
        __syncthreads();
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

// Short rows (global average pooling of 7x7 planes: 49 values): a block stages `rb` whole rows — one contiguous run of the
// tensor — in shared memory with coalesced loads, then every thread adds up one row.  Thread r starts at column r so that
// the threads of a warp hit different banks whatever the row length.
__global__ void __launch_bounds__(256) k_rowmean_staged(const float *__restrict__ x, float *__restrict__ y, size_t rows, int cols, int rb) {
    pdl_prologue();
    extern __shared__ __align__(16) float stage[];
    for (size_t r0 = (size_t)blockIdx.x * rb; r0 < rows; r0 += (size_t)gridDim.x * rb) {
        const int nr = (int)min((size_t)rb, rows - r0), count = nr * cols;
        const float *src = x + r0 * (size_t)cols;
        if ((((uintptr_t)src) & 15) == 0 && (count & 3) == 0) {
            for (int i = threadIdx.x; i < count / 4; i += 256)
                reinterpret_cast<float4 *>(stage)[i] = __ldg(reinterpret_cast<const float4 *>(src) + i);
        } else {
            for (int i = threadIdx.x; i < count; i += 256)
                stage[i] = __ldg(src + i);
        }
        __syncthreads();
        for (int r = threadIdx.x; r < nr; r += 256) {
            const float *row = stage + r * cols;
            float s = 0.f;
            int c = r % cols;
            for (int i = 0; i < cols; ++i) {
                s += row[c];
                c = c + 1 == cols ? 0 : c + 1;
            }
            y[r0 + r] = s / (float)cols;
        }
        __syncthreads();
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

// Rows of at most 32 * NPL values: one warp per row keeps the row in registers, so the tensor is read once and written
// once (8 bytes per element) and every exponential is evaluated once.  Same sums in the same order as k_softmax below.
template <int NPL>
__global__ void __launch_bounds__(256) k_softmax_reg(const float *__restrict__ x, float *__restrict__ y, size_t rows, int cols) {
    pdl_prologue();
    const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    for (size_t r = warp; r < rows; r += nwarps) {
        const float *xp = x + r * (size_t)cols;
        float *yp = y + r * (size_t)cols;
        float v[NPL];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int c = lane + 32 * i;
            v[i] = c < cols ? __ldg(xp + c) : -INFINITY;
            mx = fmaxf(mx, v[i]);
        }
        mx = warp_max(mx);
        float den = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int c = lane + 32 * i;
            v[i] = c < cols ? expf(v[i] - mx) : 0.f;
            den += v[i];
        }
        den = warp_sum(den);
        const float inv = 1.f / den;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int c = lane + 32 * i;
            if (c < cols)
                yp[c] = v[i] * inv;
        }
    }
}

template <int NPL>
__global__ void __launch_bounds__(256) k_layernorm_reg(const float *__restrict__ x, const float *__restrict__ gamma,
                                                       const float *__restrict__ beta, float *__restrict__ y, size_t rows, int cols,
                                                       float eps) {
    pdl_prologue();
    const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const int lane = threadIdx.x & 31;
    for (size_t r = warp; r < rows; r += nwarps) {
        const float *xp = x + r * (size_t)cols;
        float *yp = y + r * (size_t)cols;
        float v[NPL];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int c = lane + 32 * i;
            v[i] = c < cols ? __ldg(xp + c) : 0.f;
            s += v[i];
        }
        const float mean = warp_sum(s) / (float)cols;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int c = lane + 32 * i;
            const float d = c < cols ? v[i] - mean : 0.f;
            q += d * d;
        }
        const float inv = rsqrtf(warp_sum(q) / (float)cols + eps);
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int c = lane + 32 * i;
            if (c < cols) {
                float o = (v[i] - mean) * inv;
                if (gamma)
                    o *= __ldg(gamma + c);
                if (beta)
                    o += __ldg(beta + c);
                yp[c] = o;
            }
        }
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

// Softmax along an axis that is not the innermost one: x viewed as [outer, len, inner], normalised over `len`.  A 32 x 8
// block owns 32 neighbouring `inner` positions of one `outer` index: threadIdx.x walks `inner` (every access of a warp is
// one contiguous 128-byte piece of a row), the 8 values of threadIdx.y split `len`, and the maxima / sums of the 8 parts
// meet in shared memory.  Per column the same arithmetic as k_softmax: max, sum of exp(x - max), scale.
__global__ void __launch_bounds__(256) k_softmax_strided(const float *__restrict__ x, float *__restrict__ y, size_t outer, int len,
                                                         size_t inner) {
    pdl_prologue();
    __shared__ float red[8][33];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const size_t tiles_in = (inner + 31) / 32, tiles = outer * tiles_in;
    for (size_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const size_t o = t / tiles_in, i = (t - o * tiles_in) * 32 + tx;
        const bool live = i < inner;
        const float *xp = x + o * (size_t)len * inner + i;
        float *yp = y + o * (size_t)len * inner + i;
        float mx = -INFINITY;
        if (live)
            for (int l = ty; l < len; l += 8)
                mx = fmaxf(mx, __ldg(xp + (size_t)l * inner));
        red[ty][tx] = mx;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 8; ++k)
            mx = fmaxf(mx, red[k][tx]);
        __syncthreads();
        float den = 0.f;
        if (live)
            for (int l = ty; l < len; l += 8)
                den += expf(__ldg(xp + (size_t)l * inner) - mx);
        red[ty][tx] = den;
        __syncthreads();
        den = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            den += red[k][tx];
        __syncthreads();
        const float inv = 1.f / den;
        if (live)
            for (int l = ty; l < len; l += 8)
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

// Rows of 256..1024 values on 16-byte boundaries (a transformer's hidden width): one CTA per row, one quad per thread held
// in registers, so the row is read once and gamma / beta are in flight during the two reductions.
__global__ void __launch_bounds__(256) k_layernorm_row4(const float *__restrict__ x, const float *__restrict__ gamma,
                                                        const float *__restrict__ beta, float *__restrict__ y, size_t rows,
                                                        int cols, float eps) {
    pdl_prologue();
    __shared__ float red[8];
    const int t = (int)threadIdx.x;
    const bool on = t < (cols >> 2);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 g = (on && gamma) ? __ldg(reinterpret_cast<const float4 *>(gamma) + t) : make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 b = (on && beta) ? __ldg(reinterpret_cast<const float4 *>(beta) + t) : zero;
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float4 v = on ? __ldg(reinterpret_cast<const float4 *>(x + r * (size_t)cols) + t) : zero;
        const float mean = block_sum((v.x + v.y) + (v.z + v.w), red) / (float)cols;
        const float dx = on ? v.x - mean : 0.f, dy = on ? v.y - mean : 0.f, dz = on ? v.z - mean : 0.f, dw = on ? v.w - mean : 0.f;
        const float inv = rsqrtf(block_sum((dx * dx + dy * dy) + (dz * dz + dw * dw), red) / (float)cols + eps);
        if (on)
            reinterpret_cast<float4 *>(y + r * (size_t)cols)[t] =
                make_float4(dx * inv * g.x + b.x, dy * inv * g.y + b.y, dz * inv * g.z + b.z, dw * inv * g.w + b.w);
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
    if (inner >= 256) {
        const size_t planes = outer * (size_t)c;
        launch_pdl(k_batchnorm_plane, (int)std::min<size_t>(planes, (size_t)ctx->sm_count * 16), 256, 0, (cudaStream_t)stream, x, scale, bias, mean,
                   var, y, planes, c, inner, eps);
        return launched(ctx, "k_batchnorm_plane");
    }
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
    if (kind == 1 && kh == h && kw == w && ph == 0 && pw == 0) // global average: the mean of each contiguous plane
        return petb200_rowmean_run(ctx, x, y, (size_t)n * c, h * w, stream);
    if (kh * kw < 32) { // small windows: stage a band of input rows in shared memory when one fits in 24 KB
        const int ohb = std::min(16, (6144 / w - kh) / sh + 1);
        if (ohb >= 1) {
            const int rows_in = (ohb - 1) * sh + kh;
            if (kind == 0 && kh == 3 && kw == 3 && sh == 2 && sw == 2)
                launch_pdl(k_pool2d_tiled<true>, dim3((unsigned)((oh + ohb - 1) / ohb), (unsigned)std::min(n * c, 16384)), dim3(256),
                           (size_t)rows_in * w * sizeof(float), (cudaStream_t)stream, kind, x, y, n * c, h, w, oh, ow, kh, kw, ph, pw, sh, sw,
                           ohb, rows_in);
            else
                launch_pdl(k_pool2d_tiled<false>, dim3((unsigned)((oh + ohb - 1) / ohb), (unsigned)std::min(n * c, 16384)), dim3(256),
                           (size_t)rows_in * w * sizeof(float), (cudaStream_t)stream, kind, x, y, n * c, h, w, oh, ow, kh, kw, ph, pw, sh, sw,
                           ohb, rows_in);
            return launched(ctx, "k_pool2d_tiled");
        }
    }
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
    if (cols <= 96 && rows >= 1024) { // short rows, many of them
        const int rb = std::min(256, 8192 / cols);
        launch_pdl(k_rowmean_staged, (int)std::min<size_t>((rows + rb - 1) / rb, (size_t)ctx->sm_count * 8), 256, (size_t)rb * cols * sizeof(float),
                   (cudaStream_t)stream, x, y, rows, cols, rb);
        return launched(ctx, "k_rowmean_staged");
    }
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
    const int grid = grid_for(ctx, rows, 8);
    if (cols <= 128)
        launch_pdl(k_softmax_reg<4>, grid, 256, 0, (cudaStream_t)stream, x, y, rows, cols);
    else if (cols <= 256)
        launch_pdl(k_softmax_reg<8>, grid, 256, 0, (cudaStream_t)stream, x, y, rows, cols);
    else if (cols <= 512)
        launch_pdl(k_softmax_reg<16>, grid, 256, 0, (cudaStream_t)stream, x, y, rows, cols);
    else if (cols <= 768)
        launch_pdl(k_softmax_reg<24>, grid, 256, 0, (cudaStream_t)stream, x, y, rows, cols);
    else if (cols <= 1024)
        launch_pdl(k_softmax_reg<32>, grid, 256, 0, (cudaStream_t)stream, x, y, rows, cols);
    else
        launch_pdl(k_softmax, grid, 256, 0, (cudaStream_t)stream, x, y, rows, cols);
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
    const size_t tiles = outer * ((inner + 31) / 32);
    launch_pdl(k_softmax_strided, (int)std::min<size_t>(tiles, (size_t)ctx->sm_count * 16), dim3(32, 8), 0, (cudaStream_t)stream, x, y, outer, len,
               inner);
    return launched(ctx, "k_softmax_strided");
}

extern "C" int petb200_layernorm_run(petb200_ctx *ctx, const float *x, const float *gamma, const float *beta, float *y,
                                     size_t rows, int cols, float eps, petb200_stream stream) {
    if (!ctx || !x || !y || cols <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "layernorm_run: bad arguments");
    if (!rows)
        return PETB200_OK;
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (cols >= 256 && cols <= 1024 && cols % 4 == 0 && rows <= (size_t)ctx->sm_count * 64 && al16(x) && al16(y) && al16(gamma) && al16(beta)) {
        launch_pdl(k_layernorm_row4, (int)std::min<size_t>(rows, (size_t)ctx->sm_count * 8), 256, 0, (cudaStream_t)stream, x, gamma, beta, y, rows, cols,
                   eps);
        return launched(ctx, "k_layernorm_row4");
    }
    if (cols >= 256 && rows <= (size_t)ctx->sm_count * 64) {
        launch_pdl(k_layernorm_block, (int)std::min<size_t>(rows, (size_t)ctx->sm_count * 8), 256, 0, (cudaStream_t)stream, x, gamma, beta, y, rows,
                                                                                                           cols, eps);
        return launched(ctx, "k_layernorm_block");
    }
    const int grid = grid_for(ctx, rows, 8);
    if (cols <= 128)
        launch_pdl(k_layernorm_reg<4>, grid, 256, 0, (cudaStream_t)stream, x, gamma, beta, y, rows, cols, eps);
    else if (cols <= 256)
        launch_pdl(k_layernorm_reg<8>, grid, 256, 0, (cudaStream_t)stream, x, gamma, beta, y, rows, cols, eps);
    else if (cols <= 512)
        launch_pdl(k_layernorm_reg<16>, grid, 256, 0, (cudaStream_t)stream, x, gamma, beta, y, rows, cols, eps);
    else if (cols <= 768)
        launch_pdl(k_layernorm_reg<24>, grid, 256, 0, (cudaStream_t)stream, x, gamma, beta, y, rows, cols, eps);
    else if (cols <= 1024)
        launch_pdl(k_layernorm_reg<32>, grid, 256, 0, (cudaStream_t)stream, x, gamma, beta, y, rows, cols, eps);
    else
        launch_pdl(k_layernorm, grid, 256, 0, (cudaStream_t)stream, x, gamma, beta, y, rows, cols, eps);
    return launched(ctx, "k_layernorm");
}
