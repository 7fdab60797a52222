// Harness (not part of the product): the vendor-library calls PET's operators time themselves with, issued the way the
// reference issues them, so that their time and their output can stand beside this backend's on the same GPU.
//
//   refcalls_conv2d   ConvOp::perf (src/Graph/operator.cc:296-515): NCHW float descriptors, a convolution descriptor with
//                     CUDNN_CONVOLUTION mode (so the filter is applied flipped), float compute type and NO math type set
//                     (so the library's default math applies: TF32 tensor cores on this GPU), optional group count, then cudnnConvolutionForward for each of the eight forward
//                     algorithms the reference lists; the fastest one that runs wins.
//   refcalls_matmul   MatmulOp::perf (src/Graph/operator.cc:728-832): C^T = B^T A^T in column-major terms through
//                     cublasGemmStridedBatchedEx with fp32 data and fp32 compute (no TF32), the default algorithm and the
//                     legacy algorithm ids 0..23 (those the library no longer accepts are skipped, as the reference skips them).
//
// Differences from the reference, on purpose: times are CUDA events around the timed launches (the reference reads the host
// clock around them), the workspace is allocated here per call (the reference carves it from PerfEngine's one big buffer),
// and the result of the winning algorithm is left in the caller's output buffer so that it can be compared.
#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <cudnn.h>
#include <cmath>
#include <cstdio>

namespace {

cudnnHandle_t g_dnn = nullptr;
cublasHandle_t g_blas = nullptr;

float time_launches(int rounds, int warmup, bool (*launch)(void *), void *arg) {
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    bool ok = true;
    for (int i = 0; i < warmup && ok; ++i)
        ok = launch(arg);
    cudaEventRecord(e0);
    for (int i = 0; i < rounds && ok; ++i)
        ok = launch(arg);
    cudaEventRecord(e1);
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (!ok || cudaGetLastError() != cudaSuccess)
        return INFINITY;
    return ms / rounds;
}

struct ConvCall {
    cudnnTensorDescriptor_t in, out;
    cudnnFilterDescriptor_t kn;
    cudnnConvolutionDescriptor_t conv;
    cudnnConvolutionFwdAlgo_t algo;
    const float *x, *w;
    float *y;
    void *ws;
    size_t ws_size;
};
bool conv_launch(void *p) {
    auto *c = (ConvCall *)p;
    const float alpha = 1.f, beta = 0.f;
    return cudnnConvolutionForward(g_dnn, &alpha, c->in, c->x, c->kn, c->w, c->conv, c->algo, c->ws, c->ws_size, &beta, c->out, c->y) ==
           CUDNN_STATUS_SUCCESS;
}

struct GemmCall {
    cublasOperation_t opA, opB;
    int b, m, n, k, lda, ldb, ldc;
    const float *A, *B;
    float *C;
    cublasGemmAlgo_t algo;
    bool batched;
};
bool gemm_launch(void *p) {
    auto *g = (GemmCall *)p;
    const float alpha = 1.f, beta = 0.f;
    if (g->batched)
        return cublasGemmStridedBatchedEx(g_blas, g->opB, g->opA, g->n, g->m, g->k, &alpha, g->B, CUDA_R_32F, g->ldb, (long long)g->k * g->n,
                                          g->A, CUDA_R_32F, g->lda, (long long)g->m * g->k, &beta, g->C, CUDA_R_32F, g->ldc,
                                          (long long)g->m * g->n, g->b, CUBLAS_COMPUTE_32F, g->algo) == CUBLAS_STATUS_SUCCESS;
    return cublasGemmEx(g_blas, g->opB, g->opA, g->n, g->m, g->k, &alpha, g->B, CUDA_R_32F, g->ldb, g->A, CUDA_R_32F, g->lda, &beta, g->C,
                        CUDA_R_32F, g->ldc, CUBLAS_COMPUTE_32F, g->algo) == CUBLAS_STATUS_SUCCESS;
}

} // namespace

// x [n,c,h,w], w [f,c/g,r,s], y [n,f,oh,ow] device pointers.  Returns 0 and the best time / algorithm index (position in the
// reference's list), or -1 if no algorithm ran.
extern "C" int refcalls_conv2d(const float *x, const float *w, float *y, int n, int c, int h, int wd, int f, int cpg, int r, int s, int ph,
                               int pw, int sh, int sw, int dh, int dw, int rounds, int warmup, float *best_ms, int *best_algo) {
    static const cudnnConvolutionFwdAlgo_t kAlgos[8] = {
        CUDNN_CONVOLUTION_FWD_ALGO_IMPLICIT_GEMM, CUDNN_CONVOLUTION_FWD_ALGO_IMPLICIT_PRECOMP_GEMM,
        CUDNN_CONVOLUTION_FWD_ALGO_GEMM,          CUDNN_CONVOLUTION_FWD_ALGO_DIRECT,
        CUDNN_CONVOLUTION_FWD_ALGO_FFT,           CUDNN_CONVOLUTION_FWD_ALGO_FFT_TILING,
        CUDNN_CONVOLUTION_FWD_ALGO_WINOGRAD,      CUDNN_CONVOLUTION_FWD_ALGO_WINOGRAD_NONFUSED};
    if (!g_dnn && cudnnCreate(&g_dnn) != CUDNN_STATUS_SUCCESS)
        return -1;
    ConvCall call{};
    call.x = x, call.w = w, call.y = y;
    cudnnCreateTensorDescriptor(&call.in);
    cudnnCreateTensorDescriptor(&call.out);
    cudnnCreateFilterDescriptor(&call.kn);
    cudnnCreateConvolutionDescriptor(&call.conv);
    int rc = -1;
    int on, oc, oh, ow;
    if (cudnnSetTensor4dDescriptor(call.in, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, n, c, h, wd) == CUDNN_STATUS_SUCCESS &&
        cudnnSetFilter4dDescriptor(call.kn, CUDNN_DATA_FLOAT, CUDNN_TENSOR_NCHW, f, cpg, r, s) == CUDNN_STATUS_SUCCESS &&
        cudnnSetConvolution2dDescriptor(call.conv, ph, pw, sh, sw, dh, dw, CUDNN_CONVOLUTION, CUDNN_DATA_FLOAT) == CUDNN_STATUS_SUCCESS &&
        (c / cpg == 1 || cudnnSetConvolutionGroupCount(call.conv, c / cpg) == CUDNN_STATUS_SUCCESS) &&
        cudnnGetConvolution2dForwardOutputDim(call.conv, call.in, call.kn, &on, &oc, &oh, &ow) == CUDNN_STATUS_SUCCESS &&
        cudnnSetTensor4dDescriptor(call.out, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, on, oc, oh, ow) == CUDNN_STATUS_SUCCESS) {
        float best = INFINITY;
        int best_i = -1;
        for (int i = 0; i < 8; ++i) {
            size_t ws = 0;
            if (cudnnGetConvolutionForwardWorkspaceSize(g_dnn, call.in, call.kn, call.conv, call.out, kAlgos[i], &ws) != CUDNN_STATUS_SUCCESS)
                continue;
            if (ws >= ((size_t)4 << 30)) // (the reference's bound is 10 GiB of its own scratch)
                continue;
            void *buf = nullptr;
            if (ws && cudaMalloc(&buf, ws) != cudaSuccess) {
                (void)cudaGetLastError();
                continue;
            }
            call.algo = kAlgos[i], call.ws = buf, call.ws_size = ws;
            const float ms = time_launches(rounds, warmup, conv_launch, &call);
            if (ms < best)
                best = ms, best_i = i;
            cudaDeviceSynchronize();
            if (buf)
                cudaFree(buf);
        }
        if (best_i >= 0) { // leave the winner's result in y
            size_t ws = 0;
            cudnnGetConvolutionForwardWorkspaceSize(g_dnn, call.in, call.kn, call.conv, call.out, kAlgos[best_i], &ws);
            void *buf = nullptr;
            if (!ws || cudaMalloc(&buf, ws) == cudaSuccess) {
                call.algo = kAlgos[best_i], call.ws = buf, call.ws_size = ws;
                conv_launch(&call);
                cudaDeviceSynchronize();
                if (buf)
                    cudaFree(buf);
                *best_ms = best, *best_algo = best_i;
                rc = 0;
            }
        }
    }
    cudnnDestroyTensorDescriptor(call.in);
    cudnnDestroyTensorDescriptor(call.out);
    cudnnDestroyFilterDescriptor(call.kn);
    cudnnDestroyConvolutionDescriptor(call.conv);
    return rc;
}

// a [b,m,k] (or [b,k,m] with transA), bm [b,k,n] (or [b,n,k] with transB), cm [b,m,n], row-major device pointers.
// best_algo: -1 = CUBLAS_GEMM_DEFAULT, 0..23 the legacy ids; 100 + id when the unbatched call (b == 1) won.
extern "C" int refcalls_matmul(const float *a, const float *bm, float *cm, int b, int m, int n, int k, int transA, int transB, int rounds,
                               int warmup, float *best_ms, int *best_algo) {
    if (!g_blas && cublasCreate(&g_blas) != CUBLAS_STATUS_SUCCESS)
        return -1;
    GemmCall g{};
    g.opA = transA ? CUBLAS_OP_T : CUBLAS_OP_N, g.opB = transB ? CUBLAS_OP_T : CUBLAS_OP_N;
    g.b = b, g.m = m, g.n = n, g.k = k;
    g.lda = transA ? m : k, g.ldb = transB ? k : n, g.ldc = n;
    g.A = a, g.B = bm, g.C = cm;
    float best = INFINITY;
    int best_i = -2;
    for (int pass = 0; pass < (b == 1 ? 2 : 1); ++pass) {
        g.batched = pass == 0;
        for (int i = g.batched ? -1 : 0; i < 24; ++i) {
            g.algo = (cublasGemmAlgo_t)i; // CUBLAS_GEMM_DEFAULT = -1, CUBLAS_GEMM_ALGO0.. = 0..
            const float ms = time_launches(rounds, warmup, gemm_launch, &g);
            if (ms < best)
                best = ms, best_i = g.batched ? i : 100 + i;
        }
    }
    if (best_i == -2)
        return -1;
    g.batched = best_i < 100;
    g.algo = (cublasGemmAlgo_t)(best_i < 100 ? best_i : best_i - 100);
    gemm_launch(&g);
    cudaDeviceSynchronize();
    *best_ms = best, *best_algo = best_i;
    return 0;
}
