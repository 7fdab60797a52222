// The remaining small operators of the reference's graph API: Div, Pow, ReduceMean, Gather (ref: include/operator.h:1580-1780).
// The reference's code generator emits none of Div / Pow / ReduceMean (src/Graph/code_engine.cc:742-800 asserts on them) and
// lowers Gather through a TVM lambda (code_engine.cc:1465-1499); these kernels give the graph layer something to run
// for every operator its builder methods can create.  All are bound by HBM: 4*(inputs + output) bytes per launch.
#include "common.h"
#include <algorithm>

namespace petb200 {
namespace {

int blocks_for(petb200_ctx *ctx, size_t work, int per_block) {
    const size_t b = (work + per_block - 1) / per_block;
    return (int)std::max<size_t>(1, std::min<size_t>(b, (size_t)ctx->sm_count * 16));
}

// out[i] = a[i % sa] / b[i % sb]: the modulo broadcast of the reference's element-wise operators (operator.cc:2996-2998).
__global__ void __launch_bounds__(256) k_div(const float *__restrict__ a, size_t sa, const float *__restrict__ b, size_t sb,
                                             float *__restrict__ out, size_t n) {
    pdl_prologue();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __ldg(a + i % sa) / __ldg(b + i % sb);
}

// y = x^p by repeated multiplication, the order of powVType (ref: include/common.h:157-162); p < 0 gives 1 / x^|p|.
__global__ void __launch_bounds__(256) k_pow(const float *__restrict__ x, float *__restrict__ y, size_t n, int p) {
    pdl_prologue();
    const int q = p < 0 ? -p : p;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = __ldg(x + i);
        float r = 1.f;
        for (int k = 0; k < q; ++k)
            r *= v;
        y[i] = p < 0 ? 1.f / r : r;
    }
}

// y[o][i] = mean over a of x[o][a][i]; consecutive threads take consecutive i (coalesced for inner > 1).
__global__ void __launch_bounds__(256) k_reduce_mean(const float *__restrict__ x, float *__restrict__ y, size_t outer, int len,
                                                     size_t inner) {
    pdl_prologue();
    const size_t total = outer * inner;
    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        const size_t o = t / inner, i = t % inner;
        const float *src = x + o * (size_t)len * inner + i;
        float acc = 0.f;
        for (int a = 0; a < len; ++a)
            acc += __ldg(src + (size_t)a * inner);
        y[t] = acc / (float)len;
    }
}

// out[ib][o][i] = data[o][idx[ib]][i] (32-bit words moved untouched); an index outside [0, len) gives 0.
__global__ void __launch_bounds__(256) k_gather_axis(const uint32_t *__restrict__ data, const int *__restrict__ idx,
                                                     uint32_t *__restrict__ out, size_t n_idx, size_t outer, int len, size_t inner) {
    pdl_prologue();
    const size_t rest = outer * inner, total = n_idx * rest;
    for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
        const size_t ib = t / rest, r = t % rest, o = r / inner, i = r % inner;
        const int k = __ldg(idx + ib);
        out[t] = (k >= 0 && k < len) ? __ldg(data + (o * (size_t)len + (size_t)k) * inner + i) : 0u;
    }
}

} // namespace
} // namespace petb200

using namespace petb200;

/* DivOp (ref: include/operator.h:1580-1628).  The reference's host body subtracts instead of dividing
 * (src/Graph/operator.cc:3258-3259) and its code generator has no case for it; this is the division the operator names. */
extern "C" int petb200_div_run(petb200_ctx *ctx, const float *a, size_t size_a, const float *b, size_t size_b, float *out,
                               size_t out_size, petb200_stream stream) {
    if (!ctx || !a || !b || !out || !size_a || !size_b)
        return fail(ctx, PETB200_ERR_INVALID, "div_run: bad arguments");
    if (!out_size)
        return PETB200_OK;
    launch_pdl(k_div, blocks_for(ctx, out_size, 256), 256, 0, (cudaStream_t)stream, a, size_a, b, size_b, out, out_size);
    return launched(ctx, "k_div");
}

/* PowOp (ref: include/operator.h:1630-1679, host body src/Graph/operator.cc:3330-3343): integer exponent. */
extern "C" int petb200_pow_run(petb200_ctx *ctx, const float *x, float *y, size_t n, int p, petb200_stream stream) {
    if (!ctx || !x || !y)
        return fail(ctx, PETB200_ERR_INVALID, "pow_run: bad arguments");
    if (!n)
        return PETB200_OK;
    launch_pdl(k_pow, blocks_for(ctx, n, 256), 256, 0, (cudaStream_t)stream, x, y, n, p);
    return launched(ctx, "k_pow");
}

/* ReduceMeanOp (ref: include/operator.h:1727-1782; shape src/Graph/operator.cc:3454-3458: the reduced axis stays with
 * extent 1).  x is [outer, len, inner] around the axis. */
extern "C" int petb200_reducemean_run(petb200_ctx *ctx, const float *x, float *y, size_t outer, int len, size_t inner,
                                      petb200_stream stream) {
    if (!ctx || !x || !y || len <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "reducemean_run: bad arguments");
    if (!outer || !inner)
        return PETB200_OK;
    launch_pdl(k_reduce_mean, blocks_for(ctx, outer * inner, 256), 256, 0, (cudaStream_t)stream, x, y, outer, len, inner);
    return launched(ctx, "k_reduce_mean");
}

/* GatherOp (ref: include/operator.h:1681-1725; shape src/Graph/operator.cc:3420-3428: indices dims, then the data dims
 * without the axis; index expression src/Graph/code_engine.cc:1465-1487).  data is [outer, len, inner] around the axis,
 * indices are n_idx int32 values; out is [n_idx, outer, inner]. */
extern "C" int petb200_gather_run(petb200_ctx *ctx, const void *data, const int *indices, void *out, size_t n_idx, size_t outer,
                                  int len, size_t inner, petb200_stream stream) {
    if (!ctx || !data || !indices || !out || len <= 0)
        return fail(ctx, PETB200_ERR_INVALID, "gather_run: bad arguments");
    if (!n_idx || !outer || !inner)
        return PETB200_OK;
    launch_pdl(k_gather_axis, blocks_for(ctx, n_idx * outer * inner, 256), 256, 0, (cudaStream_t)stream, (const uint32_t *)data, indices,
               (uint32_t *)out, n_idx, outer, len, inner);
    return launched(ctx, "k_gather_axis");
}
