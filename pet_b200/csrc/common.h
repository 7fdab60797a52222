// Internal definitions shared by the kernels and the C-ABI glue of libpetb200.
#pragma once
#include <cstdlib>
#include "../../include/petb200.h"
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace petb200 {
struct DevBuf {
    void *p = nullptr;
    size_t bytes = 0;
    ~DevBuf() {
        if (p)
            cudaFree(p);
    }
    void *release() { // hands the memory to the caller
        void *q = p;
        p = nullptr;
        bytes = 0;
        return q;
    }
    cudaError_t alloc(size_t n) {
        if (p) {
            cudaFree(p);
            p = nullptr;
        }
        const cudaError_t e = n ? cudaMalloc(&p, n) : cudaSuccess;
        if (e != cudaSuccess)
            p = nullptr;
        bytes = e == cudaSuccess ? n : 0; // a failed allocation leaves an empty buffer, not a size without memory
        return e;
    }
};
} // namespace petb200

struct petb200_ctx {
    int device = 0;
    int sm_count = 148;
    int cc_major = 0, cc_minor = 0;
    size_t smem_optin = 0;
    uint64_t launches = 0;
    std::string err;
    int *d_status = nullptr; // device word kernels write when a bounded wait expires
    bool band_attr_set = false;   // the banded-product kernel's shared-memory limit was raised on this device
    petb200::DevBuf band_scratch; // partial sums of a banded product split over its band columns (grown on demand)
    // Buffers band_scratch outgrew.  They stay allocated until the context goes: a CUDA graph captured while one of them
    // was current has its address baked into its kernel nodes and may still be replayed.
    std::vector<void *> band_retired;
    // Tensor-core plans of banded products, made on first use of a shape (kind, bs, n, m, w) and kept until the context goes.
    struct BandTcPlan {
        int key[5];
        void *plan;
    };
    std::vector<BandTcPlan> band_tc;
    void (*band_tc_destroy)(void *) = nullptr;
    ~petb200_ctx() {
        for (void *p : band_retired)
            cudaFree(p);
        for (auto &e : band_tc)
            if (band_tc_destroy && e.plan)
                band_tc_destroy(e.plan);
    }
};

struct petb200_plan {
    petb200_ctx *ctx = nullptr;
    const char *kernel = "none";
    size_t device_bytes = 0;
    virtual ~petb200_plan() {}
    // Launch once on plan-owned scratch operands (for petb200_plan_time).
    virtual int bench_launch(cudaStream_t) { return PETB200_ERR_UNSUPPORTED; }
};

namespace petb200 {

inline int fail(petb200_ctx *ctx, int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx)
        ctx->err = buf;
    return status;
}

#define PETB200_CUDA(ctx, call)                                                                              \
    do {                                                                                                     \
        cudaError_t e_ = (call);                                                                             \
        if (e_ != cudaSuccess)                                                                               \
            return petb200::fail((ctx), PETB200_ERR_CUDA, "%s failed: %s (%s:%d)", #call,                    \
                                 cudaGetErrorString(e_), __FILE__, __LINE__);                                \
    } while (0)

// Records a launch and converts a launch error into a status.
inline int launched(petb200_ctx *ctx, const char *what) {
    ctx->launches++;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(ctx, PETB200_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return PETB200_OK;
}

// ---- programmatic dependent launch ---------------------------------------------------------------------------------
// Kernel families that run on the tensor-core kernel, and the arithmetic ("passes") each one asks of it: 3 = error-compensated
// TF32, 1 = one TF32 product, 16 = error-compensated bf16.  PETB200_ALGO_AUTO takes PETB200_TC_MATH from the environment
// ("3xtf32", "bf16x3"), else the default below.
inline bool tc_is_tc_algo(int algo) {
    return algo == PETB200_ALGO_AUTO || algo == PETB200_ALGO_TC_3XTF32 || algo == PETB200_ALGO_TC_1XTF32 || algo == PETB200_ALGO_TC_BF16X3;
}
inline int tc_passes_for(int algo) {
    if (algo == PETB200_ALGO_TC_1XTF32)
        return 1;
    if (algo == PETB200_ALGO_TC_BF16X3)
        return 16;
    if (algo == PETB200_ALGO_TC_3XTF32)
        return 3;
    const char *v = getenv("PETB200_TC_MATH");
    if (v && !strcmp(v, "bf16x3"))
        return 16;
    return 3;
}

// Every kernel of the library starts with pdl_prologue() and is launched through launch_pdl(): a kernel's CTAs may then
// be placed on free SMs while the kernel before it in the stream is still finishing, and wait (griddepcontrol.wait)
// until that kernel has completed and its writes are visible before they touch global memory.  PETB200_PDL=0 in the
// environment launches without the attribute (both instructions are then no-ops).
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_prologue() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif
inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("PETB200_PDL");
        v = e ? atoi(e) : 1;
    }
    return v != 0;
}
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    if (pdl_enabled()) {
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
    }
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...); // errors surface through launched()
}

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- shared activation definition ----
__device__ __forceinline__ float apply_act(float v, int act) {
    switch (act) {
    case PETB200_ACT_RELU:
        return fmaxf(v, 0.f);
    case PETB200_ACT_SIGMOID:
        return 1.f / (1.f + expf(-v));
    case PETB200_ACT_TANH:
        return tanhf(v);
    case PETB200_ACT_GELU:
        return 0.5f * v * (1.f + erff(v * 0.70710678118654752440f));
    default:
        return v;
    }
}

// ---- plan factories implemented in the kernel files ----
int make_conv_plan(petb200_ctx *ctx, int nsp, const int *in_dims /*n,c,[d],h,w*/, int f, const int *k /*[t],r,s*/,
                   const int *pad, const int *stride, const int *dil, int groups, int has_bias, int act, int algo,
                   petb200_plan **out, int channels_last_out = 0 /*y as [n,(od,)oh,ow,f]*/);
int conv_set_weights(petb200_plan *plan, const float *w, cudaStream_t s);
int conv_run(petb200_plan *plan, const float *x, const float *bias, float *y, const int *win /*oh0,ohn,ow0,own or null*/,
             cudaStream_t s, const float *res = nullptr /*optional residual, shaped like y*/);
int conv_out_dims(const petb200_plan *plan, int *dims5);

int make_matmul_plan(petb200_ctx *ctx, int transA, int transB, int b, int m, int n, int k, int has_bias, int act,
                     int algo, petb200_plan **out,
                     const long long *strides = nullptr /*{A batch, A row, B batch, B row, C batch, C row} in elements*/);
int matmul_set_weights(petb200_plan *plan, const float *b, cudaStream_t s);
int matmul_run(petb200_plan *plan, const float *a, const float *b, const float *bias, float *c, cudaStream_t s,
               const float *res = nullptr /*optional residual, shaped like c*/);

} // namespace petb200
