// Layout / index operators: every copy-type PET operator (Transpose chains, Pad, Slice, Extend, Concat, Split)
// is lowered on the host to ONE "digit map": an iteration space of up to 8 mixed-radix digits, each with an
// input stride and an output stride (in 32-bit words), an optional per-digit guard (zero outside, for Pad), and
// base offsets.  Three kernels execute a digit map:
//   rowcopy  — innermost digit contiguous on both sides: 128-bit loads and stores, one uint4 per thread step;
//   tile     — the input-contiguous digit differs from the output-contiguous one: a shared-memory tile is read
//              along the input-contiguous digit and written along the output-contiguous digit, so both sides
//              are coalesced (the counterpart of the reference's kernel_transpose_3d, without its %32 restriction);
//   gather   — anything else (guards, odd strides): coalesced stores, scalar gathers.
// All three move raw 32-bit words, so results are bit-exact by construction.
#include "common.h"
#include <algorithm>

namespace petb200 {

constexpr int kMaxDigits = 8;

struct MapParams {
    int nd;
    long long total; // iteration-space size
    long long ibase, obase;
    int ext[kMaxDigits];
    long long istr[kMaxDigits];
    long long ostr[kMaxDigits];
    int glo[kMaxDigits], ghi[kMaxDigits]; // element is zero unless glo <= idx < ghi (only when guarded)
    int guarded;
};

// ---------------------------------------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------------------------------------
// Decomposes a linear index over the digits [0, nd) of `p` (last digit fastest) into input/output word offsets.
// I is the index type: 32-bit when the iteration space allows it (64-bit division is an order of magnitude slower).
template <typename I, int FIRST_SKIP>
__device__ __forceinline__ void decode(const MapParams &p, I rem, long long &io, long long &oo, bool &inside) {
#pragma unroll
    for (int d = kMaxDigits - 1 - FIRST_SKIP; d >= 0; --d) {
        if (d < p.nd - FIRST_SKIP) {
            const I q = rem / (I)p.ext[d];
            const int idx = (int)(rem - q * (I)p.ext[d]);
            rem = q;
            io += idx * p.istr[d];
            oo += idx * p.ostr[d];
            if (p.guarded && (idx < p.glo[d] || idx >= p.ghi[d]))
                inside = false;
        }
    }
}

constexpr int kRowU = 4;
template <typename I>
__global__ void __launch_bounds__(256) k_rowcopy_v4(const uint4 *__restrict__ in, uint4 *__restrict__ out, MapParams p) {
    pdl_prologue();
    // iteration space counted in uint4 units along the innermost digit; strides of outer digits are word strides
    // divisible by 4 (checked on the host).  kRowU independent 128-bit loads are in flight per thread.
    const I total4 = (I)(p.total >> 2);
    const I inner4 = (I)(p.ext[p.nd - 1] >> 2);
    const I step = (I)gridDim.x * blockDim.x;
    for (I i0 = (I)blockIdx.x * blockDim.x + threadIdx.x; i0 < total4; i0 += kRowU * step) {
        uint4 v[kRowU];
        long long oo[kRowU];
#pragma unroll
        for (int u = 0; u < kRowU; ++u) {
            const I i = i0 + (I)u * step;
            if (i < total4) {
                const I row = i / inner4;
                long long io = p.ibase + (long long)(i - row * inner4) * 4;
                oo[u] = p.obase + (long long)(i - row * inner4) * 4;
                bool inside = true;
                decode<I, 1>(p, row, io, oo[u], inside);
                v[u] = __ldg(in + (io >> 2));
            }
        }
#pragma unroll
        for (int u = 0; u < kRowU; ++u)
            if (i0 + (I)u * step < total4)
                out[oo[u] >> 2] = v[u];
    }
}

template <typename I>
__global__ void __launch_bounds__(256) k_gather(const uint32_t *__restrict__ in, uint32_t *__restrict__ out, MapParams p) {
    pdl_prologue();
    const I total = (I)p.total;
    for (I i = (I)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (I)gridDim.x * blockDim.x) {
        long long io = p.ibase, oo = p.obase;
        bool inside = true;
        decode<I, 0>(p, i, io, oo, inside);
        out[oo] = inside ? __ldg(in + io) : 0u;
    }
}

// Long rows (innermost digit contiguous on both sides): a warp takes a piece of ONE row, decodes the outer digits once for
// it, and then only adds lane offsets — no division per 16-byte element.  kPiece4 uint4 (2 KB) per warp step, four loads
// in flight per lane.
constexpr int kPiece4 = 128;
template <typename I>
__global__ void __launch_bounds__(256) k_rowcopy_rows_v4(const uint4 *__restrict__ in, uint4 *__restrict__ out, MapParams p) {
    pdl_prologue();
    const I inner4 = (I)(p.ext[p.nd - 1] >> 2);
    const I pieces = (inner4 + kPiece4 - 1) / kPiece4;
    const I rows = (I)(p.total / p.ext[p.nd - 1]);
    const I units = rows * pieces;
    const int lane = threadIdx.x & 31;
    const I nwarps = ((I)gridDim.x * blockDim.x) >> 5;
    for (I u = ((I)blockIdx.x * blockDim.x + threadIdx.x) >> 5; u < units; u += nwarps) {
        const I row = u / pieces;
        const I c0 = (u - row * pieces) * kPiece4;
        long long io = p.ibase, oo = p.obase;
        bool inside = true;
        decode<I, 1>(p, row, io, oo, inside);
        const uint4 *src = in + (io >> 2) + c0;
        uint4 *dst = out + (oo >> 2) + c0;
        const int n = (int)min((I)kPiece4, inner4 - c0);
        uint4 v[kPiece4 / 32];
#pragma unroll
        for (int j = 0; j < kPiece4 / 32; ++j)
            if (lane + 32 * j < n)
                v[j] = __ldg(src + lane + 32 * j);
#pragma unroll
        for (int j = 0; j < kPiece4 / 32; ++j)
            if (lane + 32 * j < n)
                dst[lane + 32 * j] = v[j];
    }
}

// Rows whose innermost digit is contiguous on both sides but not 16-byte friendly (odd extents or offsets: Pad and Slice
// of the innermost dimension) or carries a guard: the same warp-per-row-piece scheme with 32-bit accesses; the guard of
// the innermost digit is a comparison, those of the outer digits are decided once per row.
constexpr int kPieceW = 256;
template <typename I>
__global__ void __launch_bounds__(256) k_rowgather(const uint32_t *__restrict__ in, uint32_t *__restrict__ out, MapParams p) {
    pdl_prologue();
    const int last = p.nd - 1;
    const I inner = (I)p.ext[last];
    const I pieces = (inner + kPieceW - 1) / kPieceW;
    const I rows = (I)(p.total / p.ext[last]);
    const I units = rows * pieces;
    const int lane = threadIdx.x & 31;
    const I nwarps = ((I)gridDim.x * blockDim.x) >> 5;
    const int glo = p.guarded ? p.glo[last] : 0, ghi = p.guarded ? p.ghi[last] : p.ext[last];
    for (I u = ((I)blockIdx.x * blockDim.x + threadIdx.x) >> 5; u < units; u += nwarps) {
        const I row = u / pieces;
        const int c0 = (int)((u - row * pieces) * kPieceW);
        long long io = p.ibase, oo = p.obase;
        bool inside = true;
        decode<I, 1>(p, row, io, oo, inside);
        const uint32_t *src = in + io;
        uint32_t *dst = out + oo;
        const int n = (int)min((I)kPieceW, inner - c0);
        uint32_t v[kPieceW / 32];
#pragma unroll
        for (int j = 0; j < kPieceW / 32; ++j) {
            const int c = c0 + lane + 32 * j;
            v[j] = (lane + 32 * j < n && inside && c >= glo && c < ghi) ? __ldg(src + c) : 0u;
        }
#pragma unroll
        for (int j = 0; j < kPieceW / 32; ++j)
            if (lane + 32 * j < n)
                dst[c0 + lane + 32 * j] = v[j];
    }
}

// Resident tile blocks per SM (PETB200_TILE_BLOCKS for tuning): each block has one 8 KB tile in flight.
// Measured on B200 at >= 384 MiB: maps whose tiles take 16-byte accesses on both sides (plain permutations such as
// NCHW -> NHWC) run best with 6 resident blocks, one-sided ones (space-to-batch and its inverse) with 8.
static int env_tile_blocks(bool both_sides_v4) {
    const char *e = getenv("PETB200_TILE_BLOCKS");
    const int v = e ? atoi(e) : (both_sides_v4 ? 6 : 8);
    return v >= 1 && v <= 8 ? v : 8;
}

constexpr int kMaxTileDigits = 4;
constexpr int kTileElems = 2048;
constexpr int kTileEPT = kTileElems / 256; // elements per thread

// A tile is the cross product of up to four digits (one of them possibly cut into chunks).  The digits are chosen
// on the host so that the tile contains both a long run that is contiguous in the INPUT and a long run that is
// contiguous in the OUTPUT.  Each thread keeps, in registers, the input offset / staging slot of the elements it
// reads (enumerated in input-stride order) and the output offset of the elements it writes (output order); tiles
// are then streamed: coalesced reads -> shared memory -> coalesced writes.
struct TileParams {
    MapParams m;             // batch digits (everything outside the tile, plus the chunk counter)
    int nt;                  // tile digits, in output order (0 = outermost)
    int text[kMaxTileDigits];
    int tistr[kMaxTileDigits], tostr[kMaxTileDigits];
    int read_order[kMaxTileDigits]; // tile digit indices, fastest (smallest input stride) first
    unsigned tmagic[kMaxTileDigits]; // ceil(2^22 / text[k]): e / text[k] == (e * magic) >> 22 for e, text[k] <= 2048
    int tile_elems;          // prod(text)
    int ck;                  // tile digit that is chunked (-1: none)
    int chunk_ext;           // full extent of that digit (text[ck] is the chunk)
    int chunk_digit;         // index inside m of the batch digit that counts chunks (-1: single chunk)
    int inner_ck;            // prod(text[ck+1:]) — only used when ck == 0 (ragged last chunk allowed)
};

__device__ __forceinline__ int fast_div(int e, unsigned magic) { return (int)(((unsigned long long)e * magic) >> 22); }

__global__ void __launch_bounds__(256) k_tile(const uint32_t *__restrict__ in, uint32_t *__restrict__ out, TileParams t) {
    pdl_prologue();
    __shared__ uint32_t tile[kTileElems + kTileElems / 32]; // one pad word per 32: transposing scatters stay conflict-free
    int li[kTileEPT], lo[kTileEPT];
    uint32_t ls[kTileEPT];
    {
        int sstride[kMaxTileDigits];
        int acc = 1;
#pragma unroll
        for (int k = kMaxTileDigits - 1; k >= 0; --k)
            if (k < t.nt) {
                sstride[k] = acc;
                acc *= t.text[k];
            }
#pragma unroll
        for (int u = 0; u < kTileEPT; ++u) {
            const int e = threadIdx.x + u * 256;
            int rem = e, off_o = 0;
#pragma unroll
            for (int k = kMaxTileDigits - 1; k >= 0; --k)
                if (k < t.nt) {
                    const int q = fast_div(rem, t.tmagic[k]);
                    off_o += (rem - q * t.text[k]) * t.tostr[k];
                    rem = q;
                }
            lo[u] = off_o;
            rem = e;
            int off_i = 0, sidx = 0, cck = 0;
#pragma unroll
            for (int q = 0; q < kMaxTileDigits; ++q)
                if (q < t.nt) {
                    const int k = t.read_order[q];
                    const int d = fast_div(rem, t.tmagic[k]);
                    const int c = rem - d * t.text[k];
                    rem = d;
                    off_i += c * t.tistr[k];
                    sidx += c * sstride[k];
                    if (k == t.ck)
                        cck = c;
                }
            li[u] = off_i;
            ls[u] = (uint32_t)(sidx + (sidx >> 5)) | ((uint32_t)cck << 16);
        }
    }
    // contiguous range of tiles per CTA: one full decode, then an odometer
    const unsigned ntiles = (unsigned)t.m.total;
    const unsigned per = (ntiles + gridDim.x - 1) / gridDim.x;
    const unsigned first = blockIdx.x * per;
    const unsigned last = min(first + per, ntiles);
    if (first >= last)
        return;
    int idx[kMaxDigits];
    long long io = t.m.ibase, oo = t.m.obase;
    {
        unsigned rem = first;
#pragma unroll
        for (int d = kMaxDigits - 1; d >= 0; --d) {
            idx[d] = 0;
            if (d < t.m.nd) {
                const unsigned q = rem / (unsigned)t.m.ext[d];
                idx[d] = (int)(rem - q * (unsigned)t.m.ext[d]);
                rem = q;
                io += idx[d] * t.m.istr[d];
                oo += idx[d] * t.m.ostr[d];
            }
        }
    }
    // Software pipeline: the loads of tile t+1 are issued before tile t is written out, so that reads stay in flight
    // during the store phase.
    auto valid_of = [&]() {
        int chunk_idx = 0;
#pragma unroll
        for (int d = 0; d < kMaxDigits; ++d)
            if (d == t.chunk_digit)
                chunk_idx = idx[d];
        return t.ck >= 0 ? min(t.text[t.ck], t.chunk_ext - chunk_idx * t.text[t.ck]) : 0x7fffffff;
    };
    uint32_t v[kTileEPT];
    int valid = valid_of();
    {
        const uint32_t *ip = in + io;
#pragma unroll
        for (int u = 0; u < kTileEPT; ++u)
            if (threadIdx.x + u * 256 < t.tile_elems && (int)(ls[u] >> 16) < valid)
                v[u] = __ldg(ip + li[u]);
    }
    for (unsigned blk = first; blk < last; ++blk) {
#pragma unroll
        for (int u = 0; u < kTileEPT; ++u)
            if (threadIdx.x + u * 256 < t.tile_elems && (int)(ls[u] >> 16) < valid)
                tile[ls[u] & 0xffffu] = v[u];
        __syncthreads();
        const int lim = (t.ck == 0) ? valid * t.inner_ck : t.tile_elems;
        uint32_t *op = out + oo;
        // odometer: next tile
        bool carry = true;
#pragma unroll
        for (int d = kMaxDigits - 1; d >= 0; --d)
            if (d < t.m.nd && carry) {
                if (++idx[d] < t.m.ext[d]) {
                    io += t.m.istr[d];
                    oo += t.m.ostr[d];
                    carry = false;
                } else {
                    io -= (long long)(t.m.ext[d] - 1) * t.m.istr[d];
                    oo -= (long long)(t.m.ext[d] - 1) * t.m.ostr[d];
                    idx[d] = 0;
                }
            }
        if (blk + 1 < last) { // prefetch the next tile into registers
            valid = valid_of();
            const uint32_t *ip = in + io;
#pragma unroll
            for (int u = 0; u < kTileEPT; ++u)
                if (threadIdx.x + u * 256 < t.tile_elems && (int)(ls[u] >> 16) < valid)
                    v[u] = __ldg(ip + li[u]);
        }
#pragma unroll
        for (int u = 0; u < kTileEPT; ++u) {
            const int e = threadIdx.x + u * 256;
            if (e < lim)
                op[lo[u]] = tile[e + (e >> 5)];
        }
        __syncthreads();
    }
}

// The same tile kernel with 16-byte global accesses on the side(s) whose contiguous run allows it (VI: four consecutive
// input words per load, VO: four consecutive output words per store; host-checked: run lengths and every other stride
// multiples of 4, no ragged chunk).  Shared memory stays word-addressed (one pad word per 32), so the in-tile permutation
// is unchanged; a quarter of the global-memory instructions remain.
template <bool VI, bool VO>
__global__ void __launch_bounds__(256) k_tile_v4(const uint32_t *__restrict__ in, uint32_t *__restrict__ out, TileParams t) {
    pdl_prologue();
    __shared__ uint32_t tile[kTileElems + kTileElems / 32];
    constexpr int NI = VI ? kTileEPT / 4 : kTileEPT, NO = VO ? kTileEPT / 4 : kTileEPT;
    constexpr int WI = VI ? 4 : 1, WO = VO ? 4 : 1;
    int li[NI], lo[NO], ls[NI];
    int svin = 0; // shared-memory stride of the input-contiguous digit
    {
        int sstride[kMaxTileDigits];
        int acc = 1;
#pragma unroll
        for (int k = kMaxTileDigits - 1; k >= 0; --k)
            if (k < t.nt) {
                sstride[k] = acc;
                acc *= t.text[k];
            }
#pragma unroll
        for (int k = 0; k < kMaxTileDigits; ++k)
            if (k == t.read_order[0])
                svin = sstride[k];
#pragma unroll
        for (int u = 0; u < NO; ++u) {
            int rem = (threadIdx.x + u * 256) * WO, off_o = 0;
#pragma unroll
            for (int k = kMaxTileDigits - 1; k >= 0; --k)
                if (k < t.nt) {
                    const int q = fast_div(rem, t.tmagic[k]);
                    off_o += (rem - q * t.text[k]) * t.tostr[k];
                    rem = q;
                }
            lo[u] = off_o;
        }
#pragma unroll
        for (int u = 0; u < NI; ++u) {
            int rem = (threadIdx.x + u * 256) * WI, off_i = 0, sidx = 0;
#pragma unroll
            for (int q = 0; q < kMaxTileDigits; ++q)
                if (q < t.nt) {
                    const int k = t.read_order[q];
                    const int d = fast_div(rem, t.tmagic[k]);
                    const int c = rem - d * t.text[k];
                    rem = d;
                    off_i += c * t.tistr[k];
                    sidx += c * sstride[k];
                }
            li[u] = off_i;
            ls[u] = sidx;
        }
    }
    const unsigned ntiles = (unsigned)t.m.total;
    const unsigned per = (ntiles + gridDim.x - 1) / gridDim.x;
    const unsigned first = blockIdx.x * per;
    const unsigned last = min(first + per, ntiles);
    if (first >= last)
        return;
    int idx[kMaxDigits];
    long long io = t.m.ibase, oo = t.m.obase;
    {
        unsigned rem = first;
#pragma unroll
        for (int d = kMaxDigits - 1; d >= 0; --d) {
            idx[d] = 0;
            if (d < t.m.nd) {
                const unsigned q = rem / (unsigned)t.m.ext[d];
                idx[d] = (int)(rem - q * (unsigned)t.m.ext[d]);
                rem = q;
                io += idx[d] * t.m.istr[d];
                oo += idx[d] * t.m.ostr[d];
            }
        }
    }
    uint32_t v[kTileEPT];
    auto load_tile = [&](const uint32_t *ip) {
#pragma unroll
        for (int u = 0; u < NI; ++u)
            if ((threadIdx.x + u * 256) * WI < t.tile_elems) {
                if (VI) {
                    const uint4 q = __ldg(reinterpret_cast<const uint4 *>(ip + li[u]));
                    v[4 * u] = q.x, v[4 * u + 1] = q.y, v[4 * u + 2] = q.z, v[4 * u + 3] = q.w;
                } else {
                    v[u] = __ldg(ip + li[u]);
                }
            }
    };
    load_tile(in + io);
    for (unsigned blk = first; blk < last; ++blk) {
#pragma unroll
        for (int u = 0; u < NI; ++u)
            if ((threadIdx.x + u * 256) * WI < t.tile_elems) {
#pragma unroll
                for (int j = 0; j < WI; ++j) {
                    const int sdx = ls[u] + j * svin;
                    tile[sdx + (sdx >> 5)] = v[WI * u + j];
                }
            }
        __syncthreads();
        uint32_t *op = out + oo;
        bool carry = true; // odometer: next tile
#pragma unroll
        for (int d = kMaxDigits - 1; d >= 0; --d)
            if (d < t.m.nd && carry) {
                if (++idx[d] < t.m.ext[d]) {
                    io += t.m.istr[d];
                    oo += t.m.ostr[d];
                    carry = false;
                } else {
                    io -= (long long)(t.m.ext[d] - 1) * t.m.istr[d];
                    oo -= (long long)(t.m.ext[d] - 1) * t.m.ostr[d];
                    idx[d] = 0;
                }
            }
        if (blk + 1 < last) // the next tile's loads stay in flight during the store phase
            load_tile(in + io);
#pragma unroll
        for (int u = 0; u < NO; ++u) {
            const int e = (threadIdx.x + u * 256) * WO;
            if (e < t.tile_elems) {
                if (VO) {
                    uint4 q;
                    q.x = tile[e + (e >> 5)], q.y = tile[e + 1 + ((e + 1) >> 5)];
                    q.z = tile[e + 2 + ((e + 2) >> 5)], q.w = tile[e + 3 + ((e + 3) >> 5)];
                    *reinterpret_cast<uint4 *>(op + lo[u]) = q;
                } else {
                    op[lo[u]] = tile[e + (e >> 5)];
                }
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------------------
// host-side lowering
// ---------------------------------------------------------------------------------------------------------
struct Digit {
    long long ext, istr;
    int glo = 0, ghi = 0;
    bool guard = false;
};
using DigitList = std::vector<Digit>;

struct LayoutPlan : petb200_plan {
    int mode = 0; // 0 rowcopy, 1 tile, 2 gather
    bool long_rows = false;  // rowcopy: rows of at least 64 uint4, one decode per row piece (k_rowcopy_rows_v4)
    bool row_gather = false; // gather whose innermost digit is contiguous on both sides (k_rowgather)
    bool tile_vi = false, tile_vo = false; // tile mode: 16-byte global loads / stores are possible
    MapParams mp{};
    TileParams tp{};
    int out_nd = 0;
    int out_dims[kMaxDigits * 2]{};
    long long in_words = 0, out_words = 0;
    int grid = 1, grid_gather = 1;
    size_t smem = 0;
    DevBuf bin, bout; // scratch for timing only
    LayoutPlan *zero_fill = nullptr; // second map of the same output that writes zeros where the first writes nothing
    ~LayoutPlan() override { delete zero_fill; }
    int bench_launch(cudaStream_t s) override;
};

static long long prod(const std::vector<long long> &v) {
    long long p = 1;
    for (auto x : v)
        p *= x;
    return p;
}

// Turns an ordered digit list (iteration order, with explicit out strides) into kernel parameters and picks a kernel.
static int finalize_plan(petb200_ctx *ctx, LayoutPlan *pl, std::vector<Digit> digits, std::vector<long long> ostr,
                         long long ibase, long long obase) {
    // drop unit digits
    {
        std::vector<Digit> d2;
        std::vector<long long> o2;
        for (size_t i = 0; i < digits.size(); ++i)
            if (digits[i].ext != 1 || digits[i].guard) {
                d2.push_back(digits[i]);
                o2.push_back(ostr[i]);
            }
        digits.swap(d2);
        ostr.swap(o2);
    }
    // merge neighbours that are contiguous on both sides
    for (size_t i = 0; i + 1 < digits.size();) {
        Digit &a = digits[i], &b = digits[i + 1];
        if (!a.guard && !b.guard && a.istr == b.istr * b.ext && ostr[i] == ostr[i + 1] * b.ext) {
            a.ext *= b.ext;
            a.istr = b.istr;
            ostr[i] = ostr[i + 1];
            digits.erase(digits.begin() + i + 1);
            ostr.erase(ostr.begin() + i + 1);
        } else {
            ++i;
        }
    }
    if (digits.empty()) {
        digits.push_back(Digit{1, 1});
        ostr.push_back(1);
    }
    if ((int)digits.size() > kMaxDigits)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "layout map needs %d digits (max %d)", (int)digits.size(), kMaxDigits);
    MapParams &m = pl->mp;
    m.nd = (int)digits.size();
    m.total = 1;
    m.ibase = ibase;
    m.obase = obase;
    m.guarded = 0;
    for (int i = 0; i < m.nd; ++i) {
        if (digits[i].ext > 0x7fffffffLL)
            return fail(ctx, PETB200_ERR_UNSUPPORTED, "digit extent too large");
        m.ext[i] = (int)digits[i].ext;
        m.istr[i] = digits[i].istr;
        m.ostr[i] = ostr[i];
        m.glo[i] = digits[i].guard ? digits[i].glo : 0;
        m.ghi[i] = digits[i].guard ? digits[i].ghi : (int)digits[i].ext;
        if (digits[i].guard)
            m.guarded = 1;
        m.total *= digits[i].ext;
    }
    const int last = m.nd - 1;
    const int sms = ctx->sm_count;
    // rowcopy: innermost digit contiguous both sides and everything 16-byte aligned
    bool v4 = !m.guarded && m.istr[last] == 1 && m.ostr[last] == 1 && m.ext[last] % 4 == 0 && ibase % 4 == 0 &&
              obase % 4 == 0;
    for (int i = 0; i < last && v4; ++i)
        v4 = (m.istr[i] % 4 == 0) && (m.ostr[i] % 4 == 0);
    if (v4) {
        pl->mode = 0;
        pl->kernel = "rowcopy";
        pl->long_rows = m.ext[last] / 4 >= 64; // decode once per 2 KB row piece instead of once per 16 bytes
        pl->row_gather = m.ext[last] >= 32;    // (fallback for caller buffers that are not 16-byte aligned)
        long long blocks = (m.total / 16 + 255) / 256;
        pl->grid = (int)std::max<long long>(1, std::min<long long>(blocks, (long long)sms * 8));
        pl->grid_gather = (int)std::max<long long>(1, std::min<long long>((m.total + 255) / 256, (long long)sms * 16));
        return PETB200_OK;
    }
    // tile: the innermost output digit is not contiguous in the input
    if (!m.guarded && m.ostr[last] == 1 && m.istr[last] != 1 && m.total < (1ll << 31)) {
        // Long contiguous digits are first split (exactly, by a divisor) into an outer and a 32..64-wide inner digit, so
        // that a tile can take a moderate run on BOTH sides instead of one very long run on one side only.
        auto split_digit = [&](int i) {
            if (m.nd >= kMaxDigits || m.ext[i] <= 128)
                return false;
            int c = 0;
            for (int cand = 64; cand >= 32; --cand)
                if (m.ext[i] % cand == 0) {
                    c = cand;
                    break;
                }
            if (!c)
                return false;
            for (int j = m.nd; j > i + 1; --j) {
                m.ext[j] = m.ext[j - 1];
                m.istr[j] = m.istr[j - 1];
                m.ostr[j] = m.ostr[j - 1];
                m.glo[j] = m.glo[j - 1];
                m.ghi[j] = m.ghi[j - 1];
            }
            m.ext[i + 1] = c;
            m.istr[i + 1] = m.istr[i];
            m.ostr[i + 1] = m.ostr[i];
            m.glo[i + 1] = 0;
            m.ghi[i + 1] = c;
            m.ext[i] /= c;
            m.istr[i] *= c;
            m.ostr[i] *= c;
            m.ghi[i] = m.ext[i];
            m.nd++;
            return true;
        };
        int a_in = -1;
        for (int i = 0; i < m.nd - 1; ++i)
            if (m.istr[i] == 1)
                a_in = i;
        if (a_in >= 0 && m.ext[a_in] > 128 && m.ext[m.nd - 1] > 128) {
            split_digit(m.nd - 1);
            split_digit(a_in);
        }
        const int last = m.nd - 1; // shadows the outer `last`: the digit count may have grown
        std::vector<int> chosen; // indices into m, kept sorted at the end
        auto has = [&](int i) { return std::find(chosen.begin(), chosen.end(), i) != chosen.end(); };
        auto tile_size = [&]() {
            long long p = 1;
            for (int i : chosen)
                p *= m.ext[i];
            return p;
        };
        // (a) output run: innermost digits while they stay contiguous in the output, until >= 64 words
        long long run = 1;
        for (int i = last; i >= 0 && run < 64 && (int)chosen.size() < kMaxTileDigits - 1; --i) {
            if (m.ostr[i] != run)
                break;
            chosen.push_back(i);
            run *= m.ext[i];
        }
        // (b) input run: digits by ascending input stride while they chain contiguously, until >= 64 words
        std::vector<int> by_istr(m.nd);
        for (int i = 0; i < m.nd; ++i)
            by_istr[i] = i;
        std::sort(by_istr.begin(), by_istr.end(), [&](int x, int y) { return m.istr[x] < m.istr[y]; });
        run = 1;
        for (int q = 0; q < m.nd && run < 64; ++q) {
            int i = by_istr[q];
            if (m.istr[i] != run)
                break;
            if (!has(i)) {
                if ((int)chosen.size() >= kMaxTileDigits)
                    break;
                chosen.push_back(i);
            }
            run *= m.ext[i];
        }
        // (c) grow small tiles with further outer digits
        for (int i = last; i >= 0 && tile_size() < kTileElems / 2 && (int)chosen.size() < kMaxTileDigits; --i)
            if (!has(i))
                chosen.push_back(i);
        std::sort(chosen.begin(), chosen.end());
        // If the tile is too large, ONE digit is cut into chunks: the outermost chosen digit when cutting it is enough
        // (its last chunk may be ragged), otherwise the largest digit, which then needs a chunk that divides it.
        int ckq = -1, chunk = 0;
        bool ok = !chosen.empty() && m.total / std::max<long long>(1, tile_size()) < (1ll << 31);
        for (int i : chosen)
            ok = ok && (long long)m.ext[i] * std::max(m.istr[i], m.ostr[i]) < (1ll << 31);
        if (ok && tile_size() > kTileElems) {
            auto others_of = [&](size_t q) {
                long long o = 1;
                for (size_t r = 0; r < chosen.size(); ++r)
                    if (r != q)
                        o *= m.ext[chosen[r]];
                return o;
            };
            if (others_of(0) <= kTileElems / 2) {
                ckq = 0;
                chunk = (int)std::min<long long>(m.ext[chosen[0]], kTileElems / others_of(0));
                for (int c = chunk; c >= std::max(1, chunk / 2); --c)
                    if (m.ext[chosen[0]] % c == 0) {
                        chunk = c;
                        break;
                    }
            } else {
                size_t big = 0;
                for (size_t q = 1; q < chosen.size(); ++q)
                    if (m.ext[chosen[q]] > m.ext[chosen[big]])
                        big = q;
                const long long lim = kTileElems / std::max<long long>(1, others_of(big));
                for (long long c = std::min<long long>(lim, m.ext[chosen[big]]); c >= 1; --c)
                    if (m.ext[chosen[big]] % c == 0) {
                        chunk = (int)c;
                        break;
                    }
                ckq = (int)big;
                ok = lim >= 1 && chunk >= 1 && (chunk * others_of(big) >= kTileElems / 8 || big == 0);
            }
        }
        if (ok) {
            TileParams &t = pl->tp;
            t.nt = (int)chosen.size();
            t.tile_elems = 1;
            for (int q = 0; q < t.nt; ++q) {
                const int i = chosen[q];
                t.text[q] = q == ckq ? chunk : m.ext[i];
                t.tistr[q] = (int)m.istr[i];
                t.tostr[q] = (int)m.ostr[i];
                t.tile_elems *= t.text[q];
                t.tmagic[q] = (unsigned)(((1u << 22) + t.text[q] - 1) / t.text[q]);
            }
            t.ck = ckq;
            t.chunk_ext = ckq >= 0 ? m.ext[chosen[ckq]] : 0;
            t.inner_ck = ckq == 0 ? t.tile_elems / t.text[0] : 1;
            std::vector<int> ro(t.nt);
            for (int q = 0; q < t.nt; ++q)
                ro[q] = q;
            std::sort(ro.begin(), ro.end(), [&](int x, int y) { return t.tistr[x] < t.tistr[y]; });
            for (int q = 0; q < t.nt; ++q)
                t.read_order[q] = ro[q];
            // batch digits: everything not chosen, plus the chunk counter in place of the chunked digit
            t.m = m;
            int k = 0;
            t.m.total = 1;
            t.chunk_digit = -1;
            for (int i = 0; i < m.nd; ++i) {
                if (ckq >= 0 && i == chosen[ckq]) {
                    const int nchunks = ceil_div(m.ext[i], chunk);
                    if (nchunks == 1)
                        continue;
                    t.m.ext[k] = nchunks;
                    t.m.istr[k] = m.istr[i] * chunk;
                    t.m.ostr[k] = m.ostr[i] * chunk;
                    t.chunk_digit = k;
                } else if (has(i)) {
                    continue;
                } else {
                    t.m.ext[k] = m.ext[i];
                    t.m.istr[k] = m.istr[i];
                    t.m.ostr[k] = m.ostr[i];
                }
                t.m.total *= t.m.ext[k];
                ++k;
            }
            t.m.nd = k;
            // 16-byte global accesses where the contiguous run and every other stride allow them
            {
                const bool whole_chunks = t.ck < 0 || t.chunk_ext % t.text[t.ck] == 0;
                const int kin = t.read_order[0], kout = t.nt - 1;
                bool vi = whole_chunks && t.tile_elems % 4 == 0 && t.tistr[kin] == 1 && t.text[kin] % 4 == 0 && t.m.ibase % 4 == 0;
                bool vo = whole_chunks && t.tile_elems % 4 == 0 && t.tostr[kout] == 1 && t.text[kout] % 4 == 0 && t.m.obase % 4 == 0;
                for (int q = 0; q < t.nt; ++q) {
                    vi = vi && (q == kin || t.tistr[q] % 4 == 0);
                    vo = vo && (q == kout || t.tostr[q] % 4 == 0);
                }
                for (int d = 0; d < t.m.nd; ++d) {
                    vi = vi && t.m.istr[d] % 4 == 0;
                    vo = vo && t.m.ostr[d] % 4 == 0;
                }
                pl->tile_vi = vi;
                pl->tile_vo = vo;
            }
            pl->mode = 1;
            pl->kernel = "tile";
            pl->smem = 0;
            pl->grid = (int)std::min<long long>(t.m.total, (long long)sms * env_tile_blocks(pl->tile_vi && pl->tile_vo));
            return PETB200_OK;
        }
    }
    pl->mode = 2;
    pl->kernel = "gather";
    pl->row_gather = m.istr[last] == 1 && m.ostr[last] == 1 && m.ext[last] >= 32;
    long long blocks = (m.total + 255) / 256;
    pl->grid = pl->grid_gather = (int)std::max<long long>(1, std::min<long long>(blocks, (long long)sms * 16));
    return PETB200_OK;
}

static void launch_gather(LayoutPlan *pl, const void *in, void *out, cudaStream_t s) {
    if (pl->row_gather) {
        if (pl->mp.total < (1ll << 31))
            launch_pdl(k_rowgather<unsigned>, pl->grid_gather, 256, 0, s, (const uint32_t *)in, (uint32_t *)out, pl->mp);
        else
            launch_pdl(k_rowgather<unsigned long long>, pl->grid_gather, 256, 0, s, (const uint32_t *)in, (uint32_t *)out, pl->mp);
        return;
    }
    if (pl->mp.total < (1ll << 31))
        launch_pdl(k_gather<unsigned>, pl->grid_gather, 256, 0, s, (const uint32_t *)in, (uint32_t *)out, pl->mp);
    else
        launch_pdl(k_gather<unsigned long long>, pl->grid_gather, 256, 0, s, (const uint32_t *)in, (uint32_t *)out, pl->mp);
}

static int layout_launch(LayoutPlan *pl, const void *in, void *out, cudaStream_t s) {
    if (pl->zero_fill) {
        int rc = layout_launch(pl->zero_fill, in, out, s);
        if (rc)
            return rc;
    }
    if (pl->mp.total == 0)
        return PETB200_OK;
    if (pl->mode == 0) {
        if ((((uintptr_t)in) | ((uintptr_t)out)) & 15) { // unaligned caller buffers: fall back to the word kernel
            launch_gather(pl, in, out, s);
            return launched(pl->ctx, "k_gather");
        }
        if (pl->long_rows) {
            if (pl->mp.total < (1ll << 31))
                launch_pdl(k_rowcopy_rows_v4<unsigned>, pl->grid, 256, 0, s, (const uint4 *)in, (uint4 *)out, pl->mp);
            else
                launch_pdl(k_rowcopy_rows_v4<unsigned long long>, pl->grid, 256, 0, s, (const uint4 *)in, (uint4 *)out, pl->mp);
            return launched(pl->ctx, "k_rowcopy_rows_v4");
        }
        if (pl->mp.total < (1ll << 31))
            launch_pdl(k_rowcopy_v4<unsigned>, pl->grid, 256, 0, s, (const uint4 *)in, (uint4 *)out, pl->mp);
        else
            launch_pdl(k_rowcopy_v4<unsigned long long>, pl->grid, 256, 0, s, (const uint4 *)in, (uint4 *)out, pl->mp);
        return launched(pl->ctx, "k_rowcopy_v4");
    }
    if (pl->mode == 1) {
        const bool vi = pl->tile_vi && (((uintptr_t)in) & 15) == 0, vo = pl->tile_vo && (((uintptr_t)out) & 15) == 0;
        const uint32_t *ip = (const uint32_t *)in;
        uint32_t *op = (uint32_t *)out;
        if (vi && vo)
            launch_pdl(k_tile_v4<true, true>, pl->grid, 256, pl->smem, s, ip, op, pl->tp);
        else if (vi)
            launch_pdl(k_tile_v4<true, false>, pl->grid, 256, pl->smem, s, ip, op, pl->tp);
        else if (vo)
            launch_pdl(k_tile_v4<false, true>, pl->grid, 256, pl->smem, s, ip, op, pl->tp);
        else
            launch_pdl(k_tile, pl->grid, 256, pl->smem, s, ip, op, pl->tp);
        return launched(pl->ctx, "k_tile");
    }
    launch_gather(pl, in, out, s);
    return launched(pl->ctx, "k_gather");
}

int LayoutPlan::bench_launch(cudaStream_t s) {
    if (!bin.p) {
        if (bin.alloc((size_t)in_words * 4) != cudaSuccess || bout.alloc((size_t)out_words * 4) != cudaSuccess)
            return fail(ctx, PETB200_ERR_NOMEM, "scratch allocation for timing failed");
        cudaMemsetAsync(bin.p, 0x3c, bin.bytes, s);
        device_bytes = bin.bytes + bout.bytes;
    }
    return layout_launch(this, bin.p, bout.p, s);
}

static std::vector<long long> row_major_strides(const std::vector<long long> &dims) {
    std::vector<long long> s(dims.size(), 1);
    for (int i = (int)dims.size() - 2; i >= 0; --i)
        s[i] = s[i + 1] * dims[i + 1];
    return s;
}

// Contiguous output over `digits` in order: out stride of digit i = product of later extents.
static std::vector<long long> contiguous_ostr(const std::vector<Digit> &digits) {
    std::vector<long long> o(digits.size(), 1);
    for (int i = (int)digits.size() - 2; i >= 0; --i)
        o[i] = o[i + 1] * digits[i + 1].ext;
    return o;
}

} // namespace petb200

using namespace petb200;

// Splits `src` (outer->inner digit list of one logical dim) into (outer part, inner part of extent `inner`).
static bool split_dim(const DigitList &src, long long inner, DigitList &hi, DigitList &lo) {
    hi.clear();
    lo.clear();
    long long acc = 1;
    int i = (int)src.size() - 1;
    while (i >= 0 && acc < inner) {
        Digit d = src[i];
        if (d.guard)
            return false;
        if (inner % acc != 0)
            return false;
        long long need = inner / acc;
        if (d.ext <= need) {
            if (need % d.ext != 0)
                return false;
            lo.insert(lo.begin(), d);
            acc *= d.ext;
            --i;
        } else {
            if (d.ext % need != 0)
                return false;
            Digit dl = d, dh = d;
            dl.ext = need;
            dh.ext = d.ext / need;
            dh.istr = d.istr * need;
            lo.insert(lo.begin(), dl);
            acc *= need;
            --i;
            for (int j = 0; j <= i; ++j)
                hi.push_back(src[j]);
            hi.push_back(dh);
            return acc == inner;
        }
    }
    if (acc != inner)
        return false;
    for (int j = 0; j <= i; ++j)
        hi.push_back(src[j]);
    return true;
}

extern "C" int petb200_transpose_plan(petb200_ctx *ctx, int nd, const int *dims, int n_ops,
                                      const petb200_transpose_desc *ops, petb200_plan **out) {
    if (!ctx || !dims || !ops || !out || nd < 1 || nd > 8 || n_ops < 1)
        return fail(ctx, PETB200_ERR_INVALID, "transpose_plan: bad arguments");
    std::vector<long long> d0(dims, dims + nd);
    for (auto v : d0)
        if (v <= 0)
            return fail(ctx, PETB200_ERR_INVALID, "transpose_plan: non-positive dim");
    auto str = row_major_strides(d0);
    std::vector<DigitList> cur(nd);
    for (int i = 0; i < nd; ++i)
        cur[i] = {Digit{d0[i], str[i]}};
    auto extent = [](const DigitList &l) {
        long long e = 1;
        for (auto &d : l)
            e *= d.ext;
        return e;
    };
    for (int oi = 0; oi < n_ops; ++oi) {
        const petb200_transpose_desc &op = ops[oi];
        int cnd = (int)cur.size();
        if (op.split >= cnd || op.ngroups < 1 || op.ngroups > 8)
            return fail(ctx, PETB200_ERR_INVALID, "transpose op %d: bad split/groups", oi);
        std::vector<DigitList> flat;
        for (int i = 0; i < cnd; ++i) {
            if (i != op.split) {
                flat.push_back(cur[i]);
                continue;
            }
            long long D = extent(cur[i]);
            long long af = op.factor > 0 ? op.factor : -(long long)op.factor;
            // ref: TransposeOp::computeShape, src/Graph/operator.cc:2346-2364 — non-divisible split is invalid
            if (af == 0 || D % af != 0 || D < af)
                return fail(ctx, PETB200_ERR_INVALID, "transpose op %d: factor %d does not divide dim %lld", oi,
                            op.factor, D);
            long long inner = op.factor > 0 ? af : D / af;
            DigitList hi, lo;
            if (!split_dim(cur[i], inner, hi, lo))
                return fail(ctx, PETB200_ERR_UNSUPPORTED, "transpose op %d: split is not expressible after fusion", oi);
            flat.push_back(hi);
            flat.push_back(lo);
        }
        int nflat = (int)flat.size();
        std::vector<DigitList> next;
        std::vector<int> used(nflat, 0);
        int p = 0, merged_groups = 0;
        for (int g = 0; g < op.ngroups; ++g) {
            DigitList l;
            if (op.group_sizes[g] < 1 || p + op.group_sizes[g] > 8)
                return fail(ctx, PETB200_ERR_INVALID, "transpose op %d: bad group size", oi);
            if (op.group_sizes[g] > 1)
                merged_groups++;
            for (int j = 0; j < op.group_sizes[g]; ++j, ++p) {
                int item = op.flat[p];
                if (op.split >= 0) { // ref: TransposeOp::setParam, include/operator.h:1133-1143
                    if (item > op.split)
                        item += 1;
                    if (item == -1)
                        item = op.split + 1;
                }
                if (item < 0 || item >= nflat || used[item])
                    return fail(ctx, PETB200_ERR_INVALID, "transpose op %d: permutation entry %d invalid", oi, op.flat[p]);
                used[item] = 1;
                l.insert(l.end(), flat[item].begin(), flat[item].end());
            }
            next.push_back(l);
        }
        for (int i = 0; i < nflat; ++i)
            if (!used[i])
                return fail(ctx, PETB200_ERR_INVALID, "transpose op %d: permutation does not cover dim %d", oi, i);
        // ref: TransposeOp::checkValid, src/Graph/operator.cc:2324-2336 — at most one merged group
        if (merged_groups > 1)
            return fail(ctx, PETB200_ERR_INVALID, "transpose op %d: more than one merged group", oi);
        cur.swap(next);
    }
    auto *pl = new LayoutPlan();
    pl->ctx = ctx;
    pl->out_nd = (int)cur.size();
    std::vector<Digit> digits;
    for (size_t i = 0; i < cur.size(); ++i) {
        pl->out_dims[i] = (int)extent(cur[i]);
        digits.insert(digits.end(), cur[i].begin(), cur[i].end());
    }
    pl->in_words = pl->out_words = prod(d0);
    int rc = finalize_plan(ctx, pl, digits, contiguous_ostr(digits), 0, 0);
    if (rc) {
        delete pl;
        return rc;
    }
    *out = pl;
    return PETB200_OK;
}

// One TransposeOp whose split or merge carries the reference's padding / halo parameters (ref: TransposeOp::getTTParam,
// src/Graph/operator.cc:2403-2441; index expressions TransSplit::putTranspose / TransFuse::putTranspose,
// src/Transpose/transpose.cc:22-42,70-106).  With in = extent of the inner part of the split or merged pair:
//   extr  (split)  out[a][b] = in[a*(in+extr) + b]         a < (D-1)/(in+extr)+1: skips the gaps a padded merge left
//   copys (split)  out[a][b] = in[a*in + b - a*copys]      D == 2*in, b < in+copys: two halves that overlap by the halo
//   pad   (merge)  out[x] = x % (in+pad) < in ? in[x/(in+pad)][x%(in+pad)] : 0     extent A*(in+pad) - pad: zero gaps
//   dels  (merge)  out[x] = in[x/(in-dels)][x%(in-dels) + (x/(in-dels))*dels]      A == 2: drops the overlap again
extern "C" int petb200_transpose_halo_plan(petb200_ctx *ctx, int nd, const int *dims, const petb200_transpose_desc *op, int pad,
                                           int extr, int copys, int dels, petb200_plan **out) {
    if (!ctx || !dims || !op || !out || nd < 1 || nd > 7)
        return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: bad arguments");
    if (pad < 0 || extr < 0 || copys < 0 || dels < 0 || (extr && copys) || (pad && dels)) // ref: transpose.cc:25,74-76
        return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: extr/copys and pad/dels exclude each other");
    std::vector<long long> d0(dims, dims + nd);
    for (auto v : d0)
        if (v <= 0)
            return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: non-positive dim");
    auto str = row_major_strides(d0);
    if (op->split >= nd || op->ngroups < 1 || op->ngroups > 8)
        return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: bad split/groups");
    if ((extr || copys) && op->split < 0)
        return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: extr/copys need a split");
    std::vector<Digit> flat; // one digit per dim after the split
    for (int i = 0; i < nd; ++i) {
        if (i != op->split) {
            flat.push_back(Digit{d0[i], str[i]});
            continue;
        }
        const long long D = d0[i], af = op->factor > 0 ? op->factor : -(long long)op->factor;
        if (af == 0 || D < af || (!extr && D % af != 0))
            return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: factor %d does not divide dim %lld", op->factor, D);
        const long long in = op->factor > 0 ? af : D / af; // ref: splitFactor, operator.cc:2425
        if (copys) {
            if (D != 2 * in || copys > in) // ref: transpose.cc:34
                return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: a halo split needs a dim of exactly 2 x %lld", in);
            flat.push_back(Digit{2, (in - copys) * str[i]});
            flat.push_back(Digit{in + copys, str[i]});
        } else {
            if (in + extr > D && extr)
                return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: gap larger than the dim");
            const long long parts = extr ? (D - 1) / (in + extr) + 1 : D / in;
            if (extr && (parts - 1) * (in + extr) + in > D)
                return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: dim %lld is not parts*(%lld+%d)-%d", D, in, extr, extr);
            flat.push_back(Digit{parts, (in + extr) * str[i]});
            flat.push_back(Digit{in, str[i]});
        }
    }
    const int nflat = (int)flat.size();
    std::vector<std::vector<int>> groups;
    std::vector<int> used(nflat, 0);
    int p = 0, merged = -1;
    for (int g = 0; g < op->ngroups; ++g) {
        if (op->group_sizes[g] < 1 || p + op->group_sizes[g] > 8)
            return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: bad group size");
        std::vector<int> items;
        for (int j = 0; j < op->group_sizes[g]; ++j, ++p) {
            int item = op->flat[p];
            if (op->split >= 0) { // ref: TransposeOp::setParam, include/operator.h:1133-1143
                if (item > op->split)
                    item += 1;
                if (item == -1)
                    item = op->split + 1;
            }
            if (item < 0 || item >= nflat || used[item])
                return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: permutation entry %d invalid", op->flat[p]);
            used[item] = 1;
            items.push_back(item);
        }
        if (items.size() > 1) {
            if (merged >= 0) // ref: TransposeOp::checkValid, src/Graph/operator.cc:2324-2336
                return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: more than one merged group");
            merged = g;
        }
        groups.push_back(items);
    }
    for (int i = 0; i < nflat; ++i)
        if (!used[i])
            return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: permutation does not cover dim %d", i);
    if ((pad || dels) && (merged < 0 || groups[merged].size() != 2))
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "transpose_halo_plan: pad/dels need one merged pair of dims");
    // output dims, digits in output order, and the zero gaps of a padded merge
    auto *pl = new LayoutPlan();
    pl->ctx = ctx;
    pl->out_nd = op->ngroups;
    std::vector<Digit> digits, zdigits;
    std::vector<long long> oext; // extent of every output dim
    for (int g = 0; g < op->ngroups; ++g) {
        if (g != merged || !(pad || dels)) {
            long long e = 1;
            for (int it : groups[g])
                e *= flat[it].ext;
            oext.push_back(e);
            continue;
        }
        const Digit &a = flat[groups[g][0]], &b = flat[groups[g][1]];
        if (dels && (a.ext != 2 || dels >= b.ext)) { // ref: transpose.cc:76
            delete pl;
            return fail(ctx, PETB200_ERR_INVALID, "transpose_halo_plan: dels needs a merged pair [2][in] with in > dels");
        }
        oext.push_back(pad ? a.ext * (b.ext + pad) - pad : a.ext * (b.ext - dels));
    }
    std::vector<long long> ostride(op->ngroups, 1);
    for (int g = op->ngroups - 2; g >= 0; --g)
        ostride[g] = ostride[g + 1] * oext[g + 1];
    std::vector<long long> ostr, zostr;
    for (int g = 0; g < op->ngroups; ++g) {
        pl->out_dims[g] = (int)oext[g];
        if (g == merged && (pad || dels)) {
            Digit a = flat[groups[g][0]], b = flat[groups[g][1]];
            if (dels) {
                a.istr += dels * b.istr;
                b.ext -= dels;
            }
            digits.push_back(a);
            ostr.push_back((b.ext + pad) * ostride[g]);
            digits.push_back(b);
            ostr.push_back(ostride[g]);
            if (pad && a.ext > 1) { // the gaps: (a.ext - 1) runs of `pad` zeros, read through an always-closed guard
                Digit za{a.ext - 1, 0}, zb{pad, 0};
                zb.guard = true, zb.glo = 0, zb.ghi = 0;
                zdigits.push_back(za);
                zostr.push_back((b.ext + pad) * ostride[g]);
                zdigits.push_back(zb);
                zostr.push_back(ostride[g]);
            }
            continue;
        }
        long long inner = 1; // out stride inside the group: later members are inner
        std::vector<long long> os(groups[g].size());
        for (int j = (int)groups[g].size() - 1; j >= 0; --j) {
            os[j] = inner * ostride[g];
            inner *= flat[groups[g][j]].ext;
        }
        for (size_t j = 0; j < groups[g].size(); ++j) {
            digits.push_back(flat[groups[g][j]]);
            ostr.push_back(os[j]);
            Digit z = flat[groups[g][j]];
            z.istr = 0;
            zdigits.push_back(z);
            zostr.push_back(os[j]);
        }
    }
    pl->in_words = prod(d0);
    pl->out_words = prod(oext);
    int rc = finalize_plan(ctx, pl, digits, ostr, 0, 0);
    if (rc == PETB200_OK && pad && merged >= 0 && flat[groups[merged][0]].ext > 1) {
        const long long gap0 = flat[groups[merged][1]].ext * ostride[merged]; // first gap starts after the first block
        pl->zero_fill = new LayoutPlan();
        pl->zero_fill->ctx = ctx;
        pl->zero_fill->in_words = pl->in_words;
        pl->zero_fill->out_words = pl->out_words;
        rc = finalize_plan(ctx, pl->zero_fill, zdigits, zostr, 0, gap0);
    }
    if (rc) {
        delete pl;
        return rc;
    }
    *out = pl;
    return PETB200_OK;
}

extern "C" int petb200_pad_plan(petb200_ctx *ctx, int nd, const int *dims, const int *begin, const int *end,
                                petb200_plan **out) {
    if (!ctx || !dims || !begin || !end || !out || nd < 1 || nd > 8)
        return fail(ctx, PETB200_ERR_INVALID, "pad_plan: bad arguments");
    std::vector<long long> d0(dims, dims + nd);
    auto str = row_major_strides(d0);
    auto *pl = new LayoutPlan();
    pl->ctx = ctx;
    pl->out_nd = nd;
    std::vector<Digit> digits;
    long long ibase = 0;
    for (int i = 0; i < nd; ++i) {
        if (begin[i] < 0 || end[i] < 0 || dims[i] <= 0) {
            delete pl;
            return fail(ctx, PETB200_ERR_INVALID, "pad_plan: negative pad or empty dim");
        }
        Digit d{(long long)dims[i] + begin[i] + end[i], str[i]};
        d.guard = (begin[i] || end[i]);
        d.glo = begin[i];
        d.ghi = begin[i] + dims[i];
        ibase -= (long long)begin[i] * str[i];
        digits.push_back(d);
        pl->out_dims[i] = (int)d.ext;
    }
    pl->in_words = prod(d0);
    pl->out_words = 1;
    for (auto &d : digits)
        pl->out_words *= d.ext;
    int rc = finalize_plan(ctx, pl, digits, contiguous_ostr(digits), ibase, 0);
    if (rc) {
        delete pl;
        return rc;
    }
    *out = pl;
    return PETB200_OK;
}

extern "C" int petb200_slice_plan(petb200_ctx *ctx, int nd, const int *dims, const int *begin, const int *end,
                                  petb200_plan **out) {
    if (!ctx || !dims || !begin || !end || !out || nd < 1 || nd > 8)
        return fail(ctx, PETB200_ERR_INVALID, "slice_plan: bad arguments");
    std::vector<long long> d0(dims, dims + nd);
    auto str = row_major_strides(d0);
    auto *pl = new LayoutPlan();
    pl->ctx = ctx;
    pl->out_nd = nd;
    std::vector<Digit> digits;
    long long ibase = 0;
    for (int i = 0; i < nd; ++i) {
        long long e = (long long)dims[i] - begin[i] - end[i];
        if (begin[i] < 0 || end[i] < 0 || e <= 0) {
            delete pl;
            return fail(ctx, PETB200_ERR_INVALID, "slice_plan: window outside the tensor");
        }
        digits.push_back(Digit{e, str[i]});
        ibase += (long long)begin[i] * str[i];
        pl->out_dims[i] = (int)e;
    }
    pl->in_words = prod(d0);
    pl->out_words = 1;
    for (auto &d : digits)
        pl->out_words *= d.ext;
    int rc = finalize_plan(ctx, pl, digits, contiguous_ostr(digits), ibase, 0);
    if (rc) {
        delete pl;
        return rc;
    }
    *out = pl;
    return PETB200_OK;
}

extern "C" int petb200_extend_plan(petb200_ctx *ctx, int nd, const int *dims, int dim, int num, petb200_plan **out) {
    if (!ctx || !dims || !out || nd < 1 || nd > 8 || dim < 0 || dim >= nd || num < 0)
        return fail(ctx, PETB200_ERR_INVALID, "extend_plan: bad arguments");
    long long outer = 1, blk = 1;
    for (int i = 0; i < nd; ++i) {
        if (dims[i] <= 0)
            return fail(ctx, PETB200_ERR_INVALID, "extend_plan: empty dim");
        (i < dim ? outer : blk) *= dims[i];
    }
    auto *pl = new LayoutPlan();
    pl->ctx = ctx;
    pl->out_nd = nd;
    for (int i = 0; i < nd; ++i)
        pl->out_dims[i] = dims[i] * (i == dim ? num + 1 : 1);
    // out[o] = in[o % blk + o / ((num+1) blk) * blk]   (ref: ExtendOp::compute, src/Graph/operator.cc:2585-2594)
    std::vector<Digit> digits = {Digit{outer, blk}, Digit{(long long)num + 1, 0}, Digit{blk, 1}};
    pl->in_words = outer * blk;
    pl->out_words = outer * blk * (num + 1);
    int rc = finalize_plan(ctx, pl, digits, contiguous_ostr(digits), 0, 0);
    if (rc) {
        delete pl;
        return rc;
    }
    *out = pl;
    return PETB200_OK;
}

extern "C" int petb200_layout_out_dims(const petb200_plan *plan, int *out_dims) {
    auto *pl = dynamic_cast<const LayoutPlan *>(plan);
    if (!pl)
        return -1;
    if (out_dims)
        for (int i = 0; i < pl->out_nd; ++i)
            out_dims[i] = pl->out_dims[i];
    return pl->out_nd;
}

extern "C" int petb200_layout_run(petb200_plan *plan, const void *in, void *out, petb200_stream stream) {
    auto *pl = dynamic_cast<LayoutPlan *>(plan);
    if (!pl)
        return PETB200_ERR_INVALID;
    if (!in || !out)
        return fail(pl->ctx, PETB200_ERR_INVALID, "layout_run: null buffer");
    return layout_launch(pl, in, out, (cudaStream_t)stream);
}

// Concat / Split share one lowering: part i is a block [outer, extents[i], inner] living at offset off_i along
// `dim` of the whole tensor (ref: ConcatOp::compute src/Graph/operator.cc:1823-1846, SplitOp::computeV :1994-2014).
static int axis_blocks(petb200_ctx *ctx, int nd, const int *dims, int dim, int n_parts, const int *extents,
                       const void *const *parts_in, void *const *parts_out, const void *whole_in, void *whole_out,
                       cudaStream_t s) {
    if (!ctx || !dims || !extents || nd < 1 || nd > 8 || dim < 0 || dim >= nd || n_parts < 1)
        return fail(ctx, PETB200_ERR_INVALID, "concat/split: bad arguments");
    long long outer = 1, inner = 1, sum = 0;
    for (int i = 0; i < nd; ++i) {
        if (dims[i] <= 0)
            return fail(ctx, PETB200_ERR_INVALID, "concat/split: empty dim");
        if (i < dim)
            outer *= dims[i];
        if (i > dim)
            inner *= dims[i];
    }
    for (int i = 0; i < n_parts; ++i) {
        if (extents[i] <= 0)
            return fail(ctx, PETB200_ERR_INVALID, "concat/split: empty part");
        sum += extents[i];
    }
    if (sum != dims[dim])
        return fail(ctx, PETB200_ERR_INVALID, "concat/split: part extents sum to %lld, dim is %d", sum, dims[dim]);
    long long whole_stride = (long long)dims[dim] * inner, off = 0;
    for (int i = 0; i < n_parts; ++i) {
        LayoutPlan pl;
        pl.ctx = ctx;
        long long run = (long long)extents[i] * inner;
        std::vector<Digit> digits;
        std::vector<long long> ostr;
        int rc;
        if (whole_out) { // concat: part (contiguous) -> whole (strided)
            digits = {Digit{outer, run}, Digit{run, 1}};
            ostr = {whole_stride, 1};
            rc = finalize_plan(ctx, &pl, digits, ostr, 0, off * inner);
            if (!rc)
                rc = layout_launch(&pl, parts_in[i], whole_out, s);
        } else { // split: whole (strided) -> part (contiguous)
            digits = {Digit{outer, whole_stride}, Digit{run, 1}};
            ostr = {run, 1};
            rc = finalize_plan(ctx, &pl, digits, ostr, off * inner, 0);
            if (!rc)
                rc = layout_launch(&pl, whole_in, parts_out[i], s);
        }
        if (rc)
            return rc;
        off += extents[i];
    }
    return PETB200_OK;
}

extern "C" int petb200_concat_run(petb200_ctx *ctx, int nd, const int *dims, int dim, int n_parts, const int *extents,
                                  const void *const *parts, void *whole, petb200_stream stream) {
    if (!parts || !whole)
        return fail(ctx, PETB200_ERR_INVALID, "concat_run: null buffer");
    return axis_blocks(ctx, nd, dims, dim, n_parts, extents, parts, nullptr, nullptr, whole, (cudaStream_t)stream);
}

extern "C" int petb200_split_run(petb200_ctx *ctx, int nd, const int *dims, int dim, int n_parts, const int *extents,
                                 const void *whole, void *const *parts, petb200_stream stream) {
    if (!parts || !whole)
        return fail(ctx, PETB200_ERR_INVALID, "split_run: null buffer");
    return axis_blocks(ctx, nd, dims, dim, n_parts, extents, nullptr, parts, whole, nullptr, (cudaStream_t)stream);
}
