// Split-K matmul that allocates nothing.
//
// Who this is for: code that runs where device allocation is off the table — a host thread that must not take the
// allocator's lock or trigger an implicit synchronisation (cudaMalloc/cudaFree synchronise the device), a plug-in
// that lives inside another process's memory budget and was handed its buffers up front, a late stage of start-up
// that runs after the memory pool has been sealed.  Such callers cannot create a context or a plan (both own device
// memory), so this entry point takes no context and no plan: the caller passes the operands and the result buffer,
// and the only extra memory the kernels touch is the fixed array below, which is part of the library image.
//
// The array is shared by every call made on a device and keeps whatever the previous call left in it.  Nothing has to
// be cleared between calls: the first kernel of a call writes every word that the second kernel of the same call
// reads (one partial sum per output element and K slice), so stale contents are never observed.  Two calls that
// overlap on the same GPU (different streams, or different host threads) would write the same words and race; run
// them one after the other.
//
// The first call on each device does the set-up: it looks up the array's device address, and — because CUDA loads a
// library's device code lazily — it is also the moment the driver loads the module that holds the array, i.e. reserves
// the array's 8 MiB on that GPU and possibly synchronises.  So make one call on every device you will use BEFORE entering
// the region where allocation or synchronisation is not allowed (and before starting any stream capture); every later
// call only launches two kernels.  The per-device address cache may be filled by several host threads at once.
#include "../../include/petb200.h"
#include <cuda_runtime.h>
#include <atomic>
#include <cstdio>

namespace {

// 2 Mi floats = 8 MiB, held by every GPU that loads the library until the process exits.
constexpr size_t kScratchFloats = PETB200_NOALLOC_SCRATCH_FLOATS;
static __device__ __align__(256) float g_splitk_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::atomic<float *> g_scratch_addr[kMaxDevices]; // device address of the array per device (zero-initialised: not looked up yet);
                                                   // threads that race on the first call all store the same value
// Writes the reason into the caller's buffer (if one was given) and passes the status through.
int fail(char *err, size_t err_len, int status, const char *fmt, const char *a = "", long long b = 0, long long c = 0) {
    if (err && err_len)
        snprintf(err, err_len, fmt, a, b, c);
    return status;
}

__device__ __forceinline__ float act_of(float v, int act) {
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

// pass 1: partial[s][i] = sum over the s-th K slice of op(A)[.,k] * op(B)[k,.]   (i = output element)
__global__ void __launch_bounds__(256) k_noalloc_partial(const float *__restrict__ a, const float *__restrict__ b,
                                                         float *__restrict__ partial, int bs, int m, int n, int k, int transA,
                                                         int transB, int ksplit) {
    const long long outs = (long long)bs * m * n, total = outs * ksplit;
    for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
        const int s = (int)(t / outs);
        const long long i = t - (long long)s * outs;
        const int nn = (int)(i % n), mm = (int)((i / n) % m), bb = (int)(i / ((long long)n * m));
        const int k0 = (int)((long long)s * k / ksplit), k1 = (int)((long long)(s + 1) * k / ksplit);
        float acc = 0.f;
        for (int kk = k0; kk < k1; ++kk) {
            const float lhs = transA ? __ldg(a + mm + (long long)m * (kk + (long long)k * bb)) : __ldg(a + kk + (long long)k * (mm + (long long)m * bb));
            const float rhs = transB ? __ldg(b + kk + (long long)k * (nn + (long long)n * bb)) : __ldg(b + nn + (long long)n * (kk + (long long)k * bb));
            acc = fmaf(lhs, rhs, acc);
        }
        partial[t] = acc;
    }
}

// pass 2: c[i] = act(sum_s partial[s][i] + bias[n]) in a fixed order
__global__ void __launch_bounds__(256) k_noalloc_reduce(const float *__restrict__ partial, const float *__restrict__ bias,
                                                        float *__restrict__ c, long long outs, int n, int ksplit, int act) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < outs; i += (long long)gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < ksplit; ++s)
            acc += partial[(long long)s * outs + i];
        if (bias)
            acc += __ldg(bias + i % n);
        c[i] = act_of(acc, act);
    }
}

} // namespace

extern "C" int petb200_matmul_splitk_noalloc(int transA, int transB, int bs, int m, int n, int k, int ksplit, const float *a,
                                             const float *b, const float *bias, float *c, int act, petb200_stream stream,
                                             char *err, size_t err_len) {
    if (err && err_len)
        err[0] = 0;
    if (!a || !b || !c)
        return fail(err, err_len, PETB200_ERR_INVALID, "matmul_splitk_noalloc: null operand%s");
    if (bs <= 0 || m <= 0 || n <= 0 || k <= 0 || ksplit <= 0 || ksplit > k)
        return fail(err, err_len, PETB200_ERR_INVALID, "matmul_splitk_noalloc: extents must be positive and 1 <= ksplit <= k%s");
    if (act < 0 || act > PETB200_ACT_GELU)
        return fail(err, err_len, PETB200_ERR_INVALID, "matmul_splitk_noalloc: unknown activation%s");
    // ksplit * bs * m * n against the array's size, by division: the product of four ints can overflow 64 bits' worth of
    // caller mistakes long before it means anything
    const long long cap = (long long)kScratchFloats;
    if (bs > cap || m > cap / bs || n > cap / ((long long)bs * m) || ksplit > cap / ((long long)bs * m * n))
        return fail(err, err_len, PETB200_ERR_UNSUPPORTED,
                    "matmul_splitk_noalloc:%s ksplit*b*m*n partial sums (b*m = %lld) exceed the fixed scratch of %lld floats; "
                    "use a smaller ksplit or the plan-based petb200_matmul_run",
                    "", (long long)bs * m, cap);
    const long long outs = (long long)bs * m * n;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return fail(err, err_len, PETB200_ERR_CUDA, "matmul_splitk_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
    float *scratch = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!scratch) { // first call on this device (with that device current): the host-side symbol is not a device address
        e = cudaGetSymbolAddress((void **)&scratch, g_splitk_scratch);
        if (e != cudaSuccess || !scratch)
            return fail(err, err_len, PETB200_ERR_CUDA, "matmul_splitk_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_scratch_addr[dev].store(scratch, std::memory_order_release);
    }
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = outs * ksplit;
    const int g1 = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    const int g2 = (int)((outs + 255) / 256 < 148 * 16 ? (outs + 255) / 256 : 148 * 16);
    k_noalloc_partial<<<g1, 256, 0, s>>>(a, b, scratch, bs, m, n, k, transA != 0, transB != 0, ksplit);
    k_noalloc_reduce<<<g2, 256, 0, s>>>(scratch, bias, c, outs, n, ksplit, act);
    e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(err, err_len, PETB200_ERR_CUDA, "matmul_splitk_noalloc: launch failed: %s", cudaGetErrorString(e));
    return PETB200_OK;
}
