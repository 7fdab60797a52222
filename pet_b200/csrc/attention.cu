// Attention rows in one launch: out[b] = softmax_rows(q[b] k[b]^T) v[b] for short sequences (n <= 128 keys, head widths
// <= 128).  In the reference's graph this is MatmulOp (transB) -> SoftmaxOp -> MatmulOp (ref: src/Graph/operator.cc:632-651
// for the products, src/Graph/code_engine.cc:424-486 for the softmax), three library calls plus whatever moves the
// operands; at BERT's shapes (12 heads of 128 x 64) each of those is a few microseconds of fixed cost around ~2 MFLOP, so
// the graph executor replaces the chain by this kernel when the two intermediate tensors have no other reader.
//
// Arithmetic: plain fp32 FMA chains (ascending k for the scores, ascending key index for the second product), and the
// softmax of k_softmax_reg sum for sum (lane-strided columns, xor butterflies, one reciprocal): no TF32 anywhere.
//
// Layout: a CTA takes 8 * TR query rows of one batch entry; K (rows an odd number of floats apart, so that 32 lanes
// reading 32 different keys at the same k hit 32 banks) and V sit in shared memory, read once per CTA from L2.  A warp owns TR
// rows: lane l holds the scores of columns l, l + 32, ... in registers, the normalised row goes through a private
// shared-memory strip to be broadcast during the second product.  Bound by shared-memory bandwidth
// (every warp walks all of K and all of V).
#include "common.h"
#include <algorithm>

namespace petb200 {
namespace {

struct AttnArgs {
    int m, n, kd, d;
    int vec; // every row of q, k, v starts on a 16-byte boundary and kd, d are multiples of 4
    long long qb, qr, kb, kr, vb, vr, ob, orow; // element strides of a batch entry and of a row, per operand
};

__device__ __forceinline__ float attn_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float attn_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

constexpr int kAttnWarps = 8;

// TR consecutive floats of shared memory as one access (the strips are laid out so that these are aligned)
template <int TR>
__device__ __forceinline__ void attn_ld(const float *p, float (&o)[TR]) {
    if (TR == 4) {
        const float4 t = *reinterpret_cast<const float4 *>(p);
        o[0] = t.x, o[1] = t.y, o[2 % TR] = t.z, o[3 % TR] = t.w;
    } else {
        const float2 t = *reinterpret_cast<const float2 *>(p);
        o[0] = t.x, o[1] = t.y;
    }
}
template <int TR>
__device__ __forceinline__ void attn_st(float *p, const float (&o)[TR]) {
    if (TR == 4)
        *reinterpret_cast<float4 *>(p) = make_float4(o[0], o[1], o[2 % TR], o[3 % TR]);
    else
        *reinterpret_cast<float2 *>(p) = make_float2(o[0], o[1]);
}

// floats of shared memory: K [32 NI][kd | 1], V [32 NI][32 ND], the warps' query strips [kd][TR] and probability strips [32 NI][TR]
inline size_t attn_smem_floats(int NI, int ND, int TR, int kd) {
    const size_t kt = ((size_t)(NI * 32) * (kd | 1) + 3) & ~(size_t)3;
    return kt + (size_t)NI * 32 * ND * 32 + (size_t)kAttnWarps * kd * TR + (size_t)kAttnWarps * NI * 32 * TR;
}

template <int NI, int ND, int TR>
__global__ void __launch_bounds__(256) k_attention(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                   float *__restrict__ o, AttnArgs a) {
    pdl_prologue();
    extern __shared__ __align__(16) float attn_sm[];
    constexpr int NC = NI * 32, DC = ND * 32;
    const int KP = a.kd | 1; // odd row pitch of K: lane l reads row l, and 32 rows an odd pitch apart fall into 32 banks
    float *Ks = attn_sm;
    float *Vs = Ks + (((size_t)NC * KP + 3) & ~(size_t)3);
    float *Qs = Vs + (size_t)NC * DC;
    float *Ps = Qs + (size_t)kAttnWarps * a.kd * TR;
    const int tid = (int)threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int z = (int)blockIdx.y, row0 = (int)blockIdx.x * kAttnWarps * TR;
    const float *kz = k + (long long)z * a.kb, *vz = v + (long long)z * a.vb, *qz = q + (long long)z * a.qb;

    if (a.vec) {
        // rows are multiples of four floats on 16-byte boundaries: eight 16-byte loads in flight per thread and operand
        const int kq = a.kd >> 2, dq = a.d >> 2;
        for (int base = tid; base < NC * kq; base += 256 * 8) {
            float4 t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * 256, c = i / kq, j = i - c * kq;
                t[u] = (i < NC * kq && c < a.n) ? __ldg(reinterpret_cast<const float4 *>(kz + (long long)c * a.kr) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * 256, c = i / kq, j = i - c * kq;
                if (i < NC * kq) {
                    float *dst = Ks + c * KP + 4 * j;
                    dst[0] = t[u].x, dst[1] = t[u].y, dst[2] = t[u].z, dst[3] = t[u].w;
                }
            }
        }
        for (int base = tid; base < NC * (DC / 4); base += 256 * 8) {
            float4 t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * 256, c = i / (DC / 4), j = i - c * (DC / 4);
                t[u] = (i < NC * (DC / 4) && c < a.n && j < dq) ? __ldg(reinterpret_cast<const float4 *>(vz + (long long)c * a.vr) + j)
                                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * 256;
                if (i < NC * (DC / 4))
                    reinterpret_cast<float4 *>(Vs)[i] = t[u];
            }
        }
        for (int i = tid; i < kAttnWarps * TR * kq; i += 256) {
            const int r = i / kq, j = i - r * kq, row = row0 + r;
            const float4 t = row < a.m ? __ldg(reinterpret_cast<const float4 *>(qz + (long long)row * a.qr) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            float *dst = Qs + ((r / TR) * a.kd + 4 * j) * TR + (r % TR);
            dst[0] = t.x, dst[TR] = t.y, dst[2 * TR] = t.z, dst[3 * TR] = t.w;
        }
    } else {
        for (int i = tid; i < NC * a.kd; i += 256) {
            const int c = i / a.kd, kk = i - c * a.kd;
            Ks[c * KP + kk] = c < a.n ? __ldg(kz + (long long)c * a.kr + kk) : 0.f;
        }
        for (int i = tid; i < NC * DC; i += 256) {
            const int c = i / DC, j = i - c * DC;
            Vs[i] = (c < a.n && j < a.d) ? __ldg(vz + (long long)c * a.vr + j) : 0.f;
        }
        for (int i = tid; i < kAttnWarps * TR * a.kd; i += 256) {
            const int r = i / a.kd, kk = i - r * a.kd, row = row0 + r;
            Qs[((r / TR) * a.kd + kk) * TR + (r % TR)] = row < a.m ? __ldg(qz + (long long)row * a.qr + kk) : 0.f;
        }
    }
    __syncthreads();

    // scores of this warp's TR rows: lane l holds columns l + 32 i
    float s[TR][NI];
#pragma unroll
    for (int r = 0; r < TR; ++r)
#pragma unroll
        for (int i = 0; i < NI; ++i)
            s[r][i] = 0.f;
    const float *qw = Qs + (size_t)warp * a.kd * TR;
#pragma unroll 4
    for (int kk = 0; kk < a.kd; ++kk) {
        float qv[TR], kv[NI];
        attn_ld<TR>(qw + kk * TR, qv);
#pragma unroll
        for (int i = 0; i < NI; ++i)
            kv[i] = Ks[(lane + 32 * i) * KP + kk];
#pragma unroll
        for (int r = 0; r < TR; ++r)
#pragma unroll
            for (int i = 0; i < NI; ++i)
                s[r][i] = fmaf(qv[r], kv[i], s[r][i]);
    }
    // softmax per row, then the normalised row into the warp's strip as [column][TR]
    float *pw = Ps + (size_t)warp * NC * TR;
    float inv[TR];
#pragma unroll
    for (int r = 0; r < TR; ++r) {
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            if (lane + 32 * i >= a.n)
                s[r][i] = -INFINITY;
            mx = fmaxf(mx, s[r][i]);
        }
        mx = attn_warp_max(mx);
        float den = 0.f;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            s[r][i] = lane + 32 * i < a.n ? expf(s[r][i] - mx) : 0.f;
            den += s[r][i];
        }
        den = attn_warp_sum(den);
        inv[r] = 1.f / den;
    }
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        float pr[TR];
#pragma unroll
        for (int r = 0; r < TR; ++r)
            pr[r] = s[r][i] * inv[r];
        attn_st<TR>(pw + (lane + 32 * i) * TR, pr);
    }
    __syncwarp();

    float acc[TR][ND];
#pragma unroll
    for (int r = 0; r < TR; ++r)
#pragma unroll
        for (int j = 0; j < ND; ++j)
            acc[r][j] = 0.f;
#pragma unroll 4
    for (int c = 0; c < a.n; ++c) {
        float pv[TR], vv[ND];
        attn_ld<TR>(pw + c * TR, pv);
#pragma unroll
        for (int j = 0; j < ND; ++j)
            vv[j] = Vs[c * DC + lane + 32 * j];
#pragma unroll
        for (int r = 0; r < TR; ++r)
#pragma unroll
            for (int j = 0; j < ND; ++j)
                acc[r][j] = fmaf(pv[r], vv[j], acc[r][j]);
    }
    float *oz = o + (long long)z * a.ob;
#pragma unroll
    for (int r = 0; r < TR; ++r) {
        const int row = row0 + warp * TR + r;
        if (row >= a.m)
            continue;
#pragma unroll
        for (int j = 0; j < ND; ++j)
            if (lane + 32 * j < a.d)
                oz[(long long)row * a.orow + lane + 32 * j] = acc[r][j];
    }
}

// ---- the 16-byte-aligned case (every BERT head): operands fetched with asynchronous 16-byte copies, register tiles -------
// A CTA takes 16 query rows.  Scores: warp w owns key columns [16 w, 16 w + 16), lane (lr, lc) = (lane / 4, lane % 4) the
// rows lr and lr + 8 and the columns 16 w + lc + 4 j, reading q and k four k at a time (rows 4 floats longer than kd, so
// that the 16-byte reads of eight different rows fall into different banks).  The 16 x n scores meet in shared memory,
// warp w normalises rows 2 w and 2 w + 1 exactly like k_softmax_reg, and the second product gives lane (lr, lc) of warp w the
// same two rows and CW adjacent output columns, walking the probabilities four keys at a time.  Same sums in the same order
// as the generic kernel below it in this file, with about a third of its shared-memory traffic.
constexpr int kAttnRows = 16, kAttnSP = 132; // rows per CTA; row pitch of the score strip (128 columns + 4)

inline size_t attn_tiled_smem_floats(int n, int kd, int d) {
    const int n16 = (n + 15) & ~15;
    return (size_t)(kAttnRows + n16) * (kd + 4) + (size_t)kAttnRows * kAttnSP + (size_t)n16 * d;
}

__device__ __forceinline__ void attn_cp16(float *dst, const float *src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(valid ? 16 : 0)
                 : "memory");
}

// KD, DD: the head widths when known at compile time (64, BERT-base and most encoders), else 0 and read from the arguments.
template <int CW, int KD, int DD>
__global__ void __launch_bounds__(256) k_attention_tiled(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                         float *__restrict__ o, AttnArgs a) {
    pdl_prologue();
    extern __shared__ __align__(16) float attn_sm[];
    const int kd = KD ? KD : a.kd, dd = DD ? DD : a.d;
    const int KP = kd + 4, n16 = (a.n + 15) & ~15, kq = kd >> 2, dq = dd >> 2;
    float *Qs = attn_sm;                       // [16][KP]
    float *Ks = Qs + kAttnRows * KP;           // [n16][KP], rows past n zero
    float *Ss = Ks + (size_t)n16 * KP;         // [16][kAttnSP]
    float *Vs = Ss + kAttnRows * kAttnSP;      // [n16][dd], rows past n zero
    const int tid = (int)threadIdx.x, warp = tid >> 5, lane = tid & 31, lr = lane >> 2, lc = lane & 3;
    const int z = (int)blockIdx.y, row0 = (int)blockIdx.x * kAttnRows;
    const float *kz = k + (long long)z * a.kb, *vz = v + (long long)z * a.vb, *qz = q + (long long)z * a.qb;
    // thread t copies 16-byte piece t, t + 256, ... of each operand; (row, piece within the row) advance without dividing
    {
        const int dr = 256 / kq, dj = 256 - dr * kq;
        int r = tid / kq, j = tid - r * kq;
        for (; r < kAttnRows; r += dr, j += dj) {
            if (j >= kq)
                j -= kq, ++r;
            if (r < kAttnRows) {
                const bool ok = row0 + r < a.m;
                attn_cp16(Qs + r * KP + 4 * j, ok ? qz + (long long)(row0 + r) * a.qr + 4 * j : qz, ok);
            }
        }
        int c = tid / kq;
        j = tid - c * kq;
        for (; c < n16; c += dr, j += dj) {
            if (j >= kq)
                j -= kq, ++c;
            if (c < n16)
                attn_cp16(Ks + c * KP + 4 * j, c < a.n ? kz + (long long)c * a.kr + 4 * j : kz, c < a.n);
        }
        asm volatile("cp.async.commit_group;" ::: "memory"); // q and k: all the scores need; v follows as a second group
        const int er = 256 / dq, ej = 256 - er * dq;
        c = tid / dq;
        j = tid - c * dq;
        for (; c < n16; c += er, j += ej) {
            if (j >= dq)
                j -= dq, ++c;
            if (c < n16)
                attn_cp16(Vs + c * dd + 4 * j, c < a.n ? vz + (long long)c * a.vr + 4 * j : vz, c < a.n);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory"); // q and k have landed; v keeps arriving behind the scores
    __syncthreads();

    if (warp * 16 < n16) { // scores of rows lr, lr + 8 at columns 16 warp + lc + 4 j
        float acc[2][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            acc[0][j] = acc[1][j] = 0.f;
        const float *q0 = Qs + lr * KP, *q1 = q0 + 8 * KP, *kb = Ks + (warp * 16 + lc) * KP;
#pragma unroll 4
        for (int kk = 0; kk < kd; kk += 4) {
            const float4 x0 = *reinterpret_cast<const float4 *>(q0 + kk), x1 = *reinterpret_cast<const float4 *>(q1 + kk);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 y = *reinterpret_cast<const float4 *>(kb + 4 * j * KP + kk);
                acc[0][j] = fmaf(x0.w, y.w, fmaf(x0.z, y.z, fmaf(x0.y, y.y, fmaf(x0.x, y.x, acc[0][j]))));
                acc[1][j] = fmaf(x1.w, y.w, fmaf(x1.z, y.z, fmaf(x1.y, y.y, fmaf(x1.x, y.x, acc[1][j]))));
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            Ss[lr * kAttnSP + warp * 16 + lc + 4 * j] = acc[0][j];
            Ss[(lr + 8) * kAttnSP + warp * 16 + lc + 4 * j] = acc[1][j];
        }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 2; ++r) { // rows 2 warp, 2 warp + 1: lane l holds columns l + 32 i; columns past n become 0
        float *row = Ss + (2 * warp + r) * kAttnSP;
        float e[4], mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            e[i] = lane + 32 * i < a.n ? row[lane + 32 * i] : -INFINITY;
            mx = fmaxf(mx, e[i]);
        }
        mx = attn_warp_max(mx);
        float den = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            e[i] = lane + 32 * i < a.n ? expf(e[i] - mx) : 0.f;
            den += e[i];
        }
        den = attn_warp_sum(den);
        const float inv = 1.f / den;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            row[lane + 32 * i] = e[i] * inv;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory"); // this thread's pieces of v; the barrier makes everyone's visible
    __syncthreads();

    const int col = CW * (warp * 4 + lc);
    if (col < dd) {
        float acc[2][CW];
#pragma unroll
        for (int j = 0; j < CW; ++j)
            acc[0][j] = acc[1][j] = 0.f;
        const float *p0 = Ss + lr * kAttnSP, *p1 = p0 + 8 * kAttnSP, *vb = Vs + col;
#pragma unroll 4
        for (int c = 0; c < a.n; c += 4) { // (keys n .. n16 - 1 carry probability 0 and zero rows of v)
            const float4 x0 = *reinterpret_cast<const float4 *>(p0 + c), x1 = *reinterpret_cast<const float4 *>(p1 + c);
            const float w0[4] = {x0.x, x0.y, x0.z, x0.w}, w1[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float y[CW];
                attn_ld<CW>(vb + (c + u) * dd, y);
#pragma unroll
                for (int j = 0; j < CW; ++j) {
                    acc[0][j] = fmaf(w0[u], y[j], acc[0][j]);
                    acc[1][j] = fmaf(w1[u], y[j], acc[1][j]);
                }
            }
        }
        float *oz = o + (long long)z * a.ob;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int row = row0 + lr + 8 * r;
            if (row < a.m)
#pragma unroll
                for (int j = 0; j < CW; ++j)
                    oz[(long long)row * a.orow + col + j] = acc[r][j];
        }
    }
}

template <int NI, int ND, int TR>
int attn_launch(petb200_ctx *ctx, const float *q, const float *k, const float *v, float *o, int bs, const AttnArgs &a, cudaStream_t s) {
    const size_t smem = attn_smem_floats(NI, ND, TR, a.kd) * sizeof(float);
    if (smem > 48 * 1024 && cudaFuncSetAttribute(k_attention<NI, ND, TR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "attention_run: %zu bytes of shared memory refused", smem);
    }
    const dim3 grid((unsigned)((a.m + kAttnWarps * TR - 1) / (kAttnWarps * TR)), (unsigned)bs);
    launch_pdl(k_attention<NI, ND, TR>, grid, 256, smem, s, q, k, v, o, a);
    return launched(ctx, "k_attention");
}

template <int NI, int TR>
int attn_pick_nd(petb200_ctx *ctx, const float *q, const float *k, const float *v, float *o, int bs, const AttnArgs &a, cudaStream_t s) {
    switch ((a.d + 31) / 32) {
    case 1: return attn_launch<NI, 1, TR>(ctx, q, k, v, o, bs, a, s);
    case 2: return attn_launch<NI, 2, TR>(ctx, q, k, v, o, bs, a, s);
    case 3: return attn_launch<NI, 3, TR>(ctx, q, k, v, o, bs, a, s);
    default: return attn_launch<NI, 4, TR>(ctx, q, k, v, o, bs, a, s);
    }
}
template <int TR>
int attn_pick_ni(petb200_ctx *ctx, const float *q, const float *k, const float *v, float *o, int bs, const AttnArgs &a, cudaStream_t s) {
    switch ((a.n + 31) / 32) {
    case 1: return attn_pick_nd<1, TR>(ctx, q, k, v, o, bs, a, s);
    case 2: return attn_pick_nd<2, TR>(ctx, q, k, v, o, bs, a, s);
    case 3: return attn_pick_nd<3, TR>(ctx, q, k, v, o, bs, a, s);
    default: return attn_pick_nd<4, TR>(ctx, q, k, v, o, bs, a, s);
    }
}

} // namespace
} // namespace petb200

using namespace petb200;

extern "C" int petb200_attention_supported(int m, int n, int kd, int d) {
    return m > 0 && n > 0 && n <= 128 && kd > 0 && kd <= 128 && d > 0 && d <= 128;
}

extern "C" int petb200_attention_run(petb200_ctx *ctx, const float *q, const float *k, const float *v, float *out, int bs, int m, int n,
                                     int kd, int d, const long long *strides, petb200_stream stream) {
    if (!ctx || !q || !k || !v || !out || bs < 0)
        return fail(ctx, PETB200_ERR_INVALID, "attention_run: bad arguments");
    if (!petb200_attention_supported(m, n, kd, d))
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "attention_run: serves 1..128 keys and head widths 1..128 (got n=%d kd=%d d=%d)", n, kd, d);
    if (bs == 0)
        return PETB200_OK;
    if (bs > 65535)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "attention_run: more than 65535 batch entries");
    AttnArgs a{m, n, kd, d, 0, (long long)m * kd, kd, (long long)n * kd, kd, (long long)n * d, d, (long long)m * d, d};
    if (strides) {
        a.qb = strides[0], a.qr = strides[1], a.kb = strides[2], a.kr = strides[3];
        a.vb = strides[4], a.vr = strides[5], a.ob = strides[6], a.orow = strides[7];
        if (a.qr < kd || a.kr < kd || a.vr < d || a.orow < d || a.qb < 0 || a.kb < 0 || a.vb < 0 || a.ob < 0)
            return fail(ctx, PETB200_ERR_INVALID, "attention_run: a row stride shorter than its row, or a negative batch stride");
    }
    auto al = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    a.vec = (kd % 4 == 0 && d % 4 == 0 && al(q) && al(k) && al(v) && ((a.qb | a.qr | a.kb | a.kr | a.vb | a.vr) & 3) == 0) ? 1 : 0;
    static const int tiled = [] { const char *e = getenv("PETB200_ATTN_TILED"); return e ? atoi(e) : 1; }();
    if (a.vec && tiled) {
        const size_t smem = attn_tiled_smem_floats(n, kd, d) * sizeof(float);
        auto kern = (kd == 64 && d == 64) ? k_attention_tiled<2, 64, 64> : (d <= 64 ? k_attention_tiled<2, 0, 0> : k_attention_tiled<4, 0, 0>);
        if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(ctx, PETB200_ERR_UNSUPPORTED, "attention_run: %zu bytes of shared memory refused", smem);
        }
        launch_pdl(kern, dim3((unsigned)((m + kAttnRows - 1) / kAttnRows), (unsigned)bs), 256, smem, (cudaStream_t)stream, q, k, v, out, a);
        return launched(ctx, "k_attention_tiled");
    }
    // 4 rows per warp halve the shared-memory traffic per row; 2 rows per warp double the CTAs when 4 would leave most SMs idle
    const long long ctas4 = (long long)bs * ((m + 31) / 32);
    static const int forced = [] { const char *e = getenv("PETB200_ATTN_ROWS"); return e ? atoi(e) : 0; }();
    const bool two = forced ? forced == 2 : ctas4 * 2 <= ctx->sm_count;
    return two ? attn_pick_ni<2>(ctx, q, k, v, out, bs, a, (cudaStream_t)stream) : attn_pick_ni<4>(ctx, q, k, v, out, bs, a, (cudaStream_t)stream);
}
