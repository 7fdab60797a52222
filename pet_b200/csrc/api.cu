// C-ABI glue: context, plan lifetime, argument decoding for conv/matmul, timing.
#include "common.h"

using namespace petb200;

static std::string g_create_error;

extern "C" int petb200_ctx_create(int device, petb200_ctx **out) {
    if (!out) {
        g_create_error = "ctx_create: out is NULL";
        return PETB200_ERR_INVALID;
    }
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        g_create_error = std::string("no CUDA device: ") + cudaGetErrorString(e);
        cudaGetLastError();
        return PETB200_ERR_CUDA;
    }
    if (device < 0 || device >= count) {
        g_create_error = "ctx_create: device index out of range";
        return PETB200_ERR_INVALID;
    }
    if ((e = cudaSetDevice(device)) != cudaSuccess) {
        g_create_error = std::string("cudaSetDevice failed: ") + cudaGetErrorString(e);
        return PETB200_ERR_CUDA;
    }
    auto *ctx = new petb200_ctx();
    ctx->device = device;
    cudaDeviceProp prop;
    cudaGetDeviceProperties(&prop, device);
    ctx->sm_count = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    if (cudaMalloc(&ctx->d_status, sizeof(int)) != cudaSuccess) {
        g_create_error = "ctx_create: status word allocation failed";
        delete ctx;
        return PETB200_ERR_NOMEM;
    }
    cudaMemset(ctx->d_status, 0, sizeof(int));
    *out = ctx;
    return PETB200_OK;
}

extern "C" int petb200_ctx_destroy(petb200_ctx *ctx) {
    if (!ctx)
        return PETB200_ERR_INVALID;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    if (ctx->d_status)
        cudaFree(ctx->d_status);
    delete ctx;
    return PETB200_OK;
}

extern "C" const char *petb200_last_error(const petb200_ctx *ctx) { return ctx ? ctx->err.c_str() : g_create_error.c_str(); }

extern "C" const char *petb200_status_string(int status) {
    switch (status) {
    case PETB200_OK:
        return "ok";
    case PETB200_ERR_INVALID:
        return "invalid argument";
    case PETB200_ERR_UNSUPPORTED:
        return "unsupported";
    case PETB200_ERR_CUDA:
        return "CUDA error";
    case PETB200_ERR_NOMEM:
        return "out of memory";
    case PETB200_ERR_DEVICE:
        return "device-side error";
    default:
        return "unknown status";
    }
}

extern "C" uint64_t petb200_launch_count(const petb200_ctx *ctx) { return ctx ? ctx->launches : 0; }

extern "C" void petb200_plan_destroy(petb200_plan *plan) { delete plan; }
extern "C" size_t petb200_plan_device_bytes(const petb200_plan *plan) { return plan ? plan->device_bytes : 0; }
extern "C" const char *petb200_plan_kernel(const petb200_plan *plan) { return plan ? plan->kernel : "none"; }

// Reads (and clears) the word device kernels set when a bounded wait expired.  Synchronises the stream.
extern "C" int petb200_check_device_status(petb200_ctx *ctx, petb200_stream stream) {
    if (!ctx)
        return PETB200_ERR_INVALID;
    int v = 0;
    PETB200_CUDA(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    PETB200_CUDA(ctx, cudaMemcpy(&v, ctx->d_status, sizeof v, cudaMemcpyDeviceToHost));
    if (v) {
        cudaMemset(ctx->d_status, 0, sizeof v);
        return fail(ctx, PETB200_ERR_DEVICE, "a kernel gave up on a bounded wait (status %d)", v);
    }
    return PETB200_OK;
}

extern "C" int petb200_conv2d_plan(petb200_ctx *ctx, const int a[16], int algo, petb200_plan **out) {
    if (!ctx || !a || !out)
        return fail(ctx, PETB200_ERR_INVALID, "conv2d_plan: null argument");
    // {n,c,h,w,f,r,s,ph,pw,sh,sw,dh,dw,g,bias,act}
    int in_dims[4] = {a[0], a[1], a[2], a[3]};
    int k[2] = {a[5], a[6]}, pad[2] = {a[7], a[8]}, stride[2] = {a[9], a[10]}, dil[2] = {a[11], a[12]};
    return make_conv_plan(ctx, 2, in_dims, a[4], k, pad, stride, dil, a[13], a[14], a[15], algo, out);
}
extern "C" int petb200_conv2d_set_weights(petb200_plan *plan, const float *w, petb200_stream s) {
    return conv_set_weights(plan, w, (cudaStream_t)s);
}
extern "C" int petb200_conv2d_run(petb200_plan *plan, const float *x, const float *bias, float *y, petb200_stream s) {
    return conv_run(plan, x, bias, y, nullptr, (cudaStream_t)s);
}
extern "C" int petb200_conv2d_out_dims(const petb200_plan *plan, int o[4]) {
    int d5[5];
    int rc = conv_out_dims(plan, d5);
    if (rc)
        return rc;
    o[0] = d5[0], o[1] = d5[1], o[2] = d5[3], o[3] = d5[4];
    return PETB200_OK;
}
extern "C" int petb200_conv2d_correct(petb200_plan *plan, const float *x, const float *bias, float *y, int oh0, int ohn,
                                      int ow0, int own, petb200_stream s) {
    int win[4] = {oh0, ohn, ow0, own};
    return conv_run(plan, x, bias, y, win, (cudaStream_t)s);
}

extern "C" int petb200_conv3d_plan(petb200_ctx *ctx, const int a[21], int algo, petb200_plan **out) {
    if (!ctx || !a || !out)
        return fail(ctx, PETB200_ERR_INVALID, "conv3d_plan: null argument");
    // {n,c,d,h,w, f,t,r,s, pd,ph,pw, sd,sh,sw, dd,dh,dw, g,bias,act}
    int in_dims[5] = {a[0], a[1], a[2], a[3], a[4]};
    int k[3] = {a[6], a[7], a[8]}, pad[3] = {a[9], a[10], a[11]}, stride[3] = {a[12], a[13], a[14]},
        dil[3] = {a[15], a[16], a[17]};
    return make_conv_plan(ctx, 3, in_dims, a[5], k, pad, stride, dil, a[18], a[19], a[20], algo, out);
}
extern "C" int petb200_conv3d_set_weights(petb200_plan *plan, const float *w, petb200_stream s) {
    return conv_set_weights(plan, w, (cudaStream_t)s);
}
extern "C" int petb200_conv3d_run(petb200_plan *plan, const float *x, const float *bias, float *y, petb200_stream s) {
    return conv_run(plan, x, bias, y, nullptr, (cudaStream_t)s);
}

extern "C" int petb200_conv_run_residual(petb200_plan *plan, const float *x, const float *bias, const float *residual, float *y,
                                         petb200_stream s) {
    return conv_run(plan, x, bias, y, nullptr, (cudaStream_t)s, residual);
}

extern "C" int petb200_matmul_plan(petb200_ctx *ctx, int transA, int transB, int b, int m, int n, int k, int has_bias,
                                   int act, int algo, petb200_plan **out) {
    return make_matmul_plan(ctx, transA, transB, b, m, n, k, has_bias, act, algo, out);
}
extern "C" int petb200_matmul_plan_strided(petb200_ctx *ctx, int transA, int transB, int b, int m, int n, int k, int has_bias,
                                           int act, int algo, const long long strides[6], petb200_plan **out) {
    if (!strides)
        return fail(ctx, PETB200_ERR_INVALID, "matmul_plan_strided: null strides");
    return make_matmul_plan(ctx, transA, transB, b, m, n, k, has_bias, act, algo, out, strides);
}
extern "C" int petb200_matmul_set_weights(petb200_plan *plan, const float *b, petb200_stream s) {
    return matmul_set_weights(plan, b, (cudaStream_t)s);
}
extern "C" int petb200_matmul_run(petb200_plan *plan, const float *a, const float *b, const float *bias, float *c,
                                  petb200_stream s) {
    return matmul_run(plan, a, b, bias, c, (cudaStream_t)s);
}

extern "C" int petb200_matmul_run_residual(petb200_plan *plan, const float *a, const float *b, const float *bias,
                                           const float *residual, float *c, petb200_stream s) {
    return matmul_run(plan, a, b, bias, c, (cudaStream_t)s, residual);
}

extern "C" int petb200_plan_time(petb200_plan *plan, int rounds, int warmup, float *ms, petb200_stream stream) {
    if (!plan || !ms || rounds <= 0 || warmup < 0)
        return PETB200_ERR_INVALID;
    petb200_ctx *ctx = plan->ctx;
    cudaStream_t s = (cudaStream_t)stream;
    for (int i = 0; i < warmup; ++i) {
        int rc = plan->bench_launch(s);
        if (rc)
            return rc;
    }
    if (warmup == 0) { // scratch operands are created by the first launch; keep that out of the timed region
        int rc = plan->bench_launch(s);
        if (rc)
            return rc;
    }
    cudaEvent_t e0, e1;
    PETB200_CUDA(ctx, cudaEventCreate(&e0));
    PETB200_CUDA(ctx, cudaEventCreate(&e1));
    PETB200_CUDA(ctx, cudaEventRecord(e0, s));
    for (int i = 0; i < rounds; ++i) {
        int rc = plan->bench_launch(s);
        if (rc) {
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            return rc;
        }
    }
    PETB200_CUDA(ctx, cudaEventRecord(e1, s));
    PETB200_CUDA(ctx, cudaEventSynchronize(e1));
    float total = 0.f;
    PETB200_CUDA(ctx, cudaEventElapsedTime(&total, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms = total / (float)rounds;
    return petb200_check_device_status(ctx, stream);
}
