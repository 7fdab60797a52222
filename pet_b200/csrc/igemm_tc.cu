// Implicit-GEMM convolution / matmul on the 5th-generation tensor cores (tcgen05) with error-compensated TF32.
//
//   D[pixel, filter] = sum_k A[pixel, k] * B[filter, k]            k = (channel chunk, tap, channel in chunk)
//
// One CTA computes a 128-pixel x BN-filter tile; the fp32 accumulator lives in tensor memory (TMEM).
//   warp 0   : TMA producer for the packed weights: per 32-wide K stage one 2-D tile of B_hi and one of B_lo,
//              straight into 128-byte-swizzled K-major shared memory.
//   warp 2   : TMA producer for the RAW activation tile of one channel chunk (all taps share it): a 5-D box
//              [images, channels, depth, rows, cols] of the NC(D)HW input, zero-filled outside the tensor, which
//              is exactly the convolution's zero padding.  Box start along W is rounded down to 16 bytes.
//   warps 3-6, 7-10: two transform sets taking alternate K stages.  Thread p owns pixel p of the tile: for every K stage it
//              gathers its 32 values from the raw tile (fixed strides where the channel chunk allows, else through a
//              precomputed offset table: tap shift, dilation, channel plane), splits each fp32
//              into hi (top 19 bits) and lo = x - hi, and writes the two K-major operand tiles — into swizzled
//              shared memory (SS variant) or directly into TMEM with tcgen05.st (TS variant, which leaves the
//              shared-memory read port to B alone).  The same warps run the epilogue.
//   warp 1   : issues, per K=8 step, the three products of 3xTF32 as two MMAs — A_hi x [B_hi;B_lo] (one MMA of width
//              2*BN: the hi*hi sum and the hi*lo sum in adjacent accumulators) and A_lo x B_hi — and commits the stage
//              release barriers.
// Epilogue: tcgen05.ld -> +bias -> activation -> global stores, coalesced across the 32 pixels of a warp (conv)
// or 128-bit per thread (row-major matmul output).
//
// Variants (template parameters): 3xTF32 (default), one TF32 pass, error-compensated bf16 (64 K elements per stage, K = 16 per
// MMA); persistent "ping-pong" tiles for narrow filter tiles (a CTA walks several pixel tiles, the transform sets take
// alternate tiles, accumulators alternate between two TMEM regions).  Long K ranges drain the main accumulator into a
// running total every few stages (the tensor core truncates its fp32 accumulator after every MMA).
// Split-K: the ksplit CTAs of one output tile form a thread-block cluster and exchange their partial sums through
// distributed shared memory (pushes into the owner's landing area, one cluster barrier, reduction in rank order).
// Every wait on an mbarrier is bounded (~2 s) and reports through a status word instead of hanging the GPU.
// TMA loads are per CTA (no cluster-wide loads of any kind).
#include "common.h"
#include "tc_ptx.cuh"
#include <algorithm>
#include <array>
#include <cstdlib>
#include <map>

namespace petb200 {

constexpr int kTileM = 128;
constexpr int kStageK = 32;               // 32-bit words per K stage = one 128-byte swizzle row (32 TF32 values or 64 bf16)
// values of the kernel's PASSES parameter: error-compensated TF32 (three products per multiply), one TF32 product, and
// error-compensated bf16 (hi/lo bf16 halves, three products, K = 16 per instruction: half the MMAs of 3xTF32 per K)
constexpr int kMathTf32x3 = 3, kMathTf32x1 = 1, kMathBf16x3 = 16;
constexpr int kAHalfBytes = kTileM * 128; // one 128 x 32 operand tile
constexpr int kThreads = 352;   // warps: 0 B producer, 1 MMA, 2 raw producer, 3-6 and 7-10 two transform/epilogue sets
constexpr int kProfSlots = 24; // tuning counters per CTA (see IgemmParams::prof)
constexpr int kMaxNB = 6;
constexpr int kMaxNR = 6;

struct IgemmParams {
    int Pw, units;          // pixels of one output plane (one image, one depth slice); number of such planes
    int OD, OH, OW;         // full output extents (for addressing y)
    int ohn, own, oh0, ow0; // output window actually computed (ohn*own = Pw)
    int sd, sh, sw, pd, ph, pw;
    int x0;                 // box origin along W (multiple of 4, may be negative)
    int RN, RD, RH, RW, BC; // raw box extents
    int nchunks, spc;       // channel chunks; K stages per chunk
    int ke;                 // K elements per stage: 32 (TF32) or 64 (bf16, two per 32-bit word)
    int cpg, Fg, BN;        // channels per group, filters per group, tile N
    int z_is_batch;         // blockIdx.z: 0 = conv group, 1 = matmul batch
    int wide, row_tiles;    // wide mode: a tile is 128 consecutive pixels of ONE output row (rows wider than a tile)
    int tpi, ipt;           // otherwise: tiles per plane (plane larger than a tile) or whole planes per tile
    int ksplit;             // K is split over this many CTAs, launched as one thread-block cluster (2, 4, 8 or 16); partial
                            // tiles are added up through distributed shared memory
    int NA, NB, NR;         // ring depths: A stages, B stages, raw activation buffers
    int fl;                 // 3xTF32 only: every `fl` K stages the main accumulator is drained into a running total that
                            // is summed with round-to-nearest adds (0: never).  The tensor core truncates its accumulator
                            // after every MMA; restarting it keeps the truncated partial sums short and small
    int a_col;              // first TMEM column of the A-operand ring (TS variants)
    int fl_regs;            // 128-wide tiles: the running total lives in the registers of the second transform set, whose
                            // warps then do nothing but drain (the first set produces every A stage); narrower tiles
                            // keep the total in TMEM columns [2*BN,3*BN) and both sets drain between their stages
    int a_kmajor;           // matmul with row-major A: the raw tile is [128 rows][32 k], 128B-swizzled, one per K stage
    int m_rows;             // a_kmajor: rows of A per batch entry
    int raw_bytes;          // bytes of one raw buffer (128-aligned)
    int flat;               // rows of the input are not 16-byte multiples: the raw tile is BC whole channels of RN images,
                            // dense and unpadded, fetched as a 2-D box [flat_rows][flat_w] of the contiguous run; padding
                            // becomes a per-pixel mask over the filter taps (<= 32 taps)
    int flat_w, flat_rows;
    int cstride;            // BC % 32 == 0, or BC 16 / 8: floats between consecutive channels of the raw tile (else 0: table)
    int gruns;              // runs (filter taps) per 32-wide K stage in that mode: 1, 2 (BC 16) or 4 (BC 8)
    int T3[3], dil[3];      // filter extents and dilations (flat only: for the tap mask)
    int xD, xH, xW;         // input extents (flat only)
    long long ys_n, ys_f, ys_p;
    int act, has_bias;
    const int *koff;
    const float *bias;
    const float *res; // optional residual, laid out like y: y = act(sum + bias + res)
    float *y;
    int *status;
    long long *prof; // optional per-CTA counters (kProfSlots per CTA), for tuning only
    int pp;          // persistent "ping-pong" mode: the grid's x extent is smaller than the number of pixel tiles (mtiles); a CTA
                     // walks tiles blockIdx.x, + gridDim.x, ...; the two transform sets take alternate TILES (each set produces
                     // every A stage of its tile and then stores it) and the accumulators alternate between two TMEM
                     // regions, so one tile's epilogue and the next tile's start-up hide behind the MMAs of the other
    int mtiles;      // pixel tiles along x
    int band_w;      // > 0: banded product y[b,i,j] = q[b,i,:] . k[b,i+j-w,:] (row-major A = q, "filters" = the keys of the window
                     // [128*tile - w, 128*tile + 127 + w] of the tile's rows, blockIdx.y = 64-key piece of that window); the
                     // epilogue stores the band entries of each row at their skewed positions, zero where the key is outside [0,n)
    const float *band_p; // non-null: GBMML y[b,i,c] = sum_j p[b,i,j] * v[b,i+j-w,c]: the A operand is the band p [bs][n][2w+1] read
                     // straight from global memory by the transform threads (row i of the tile meets key k through p[i][k-i+w]),
                     // the "filters" are v's columns with the keys as K (window of the tile's rows, start rounded down to 4)
    int band_nt;     // banded product: 64-key pieces per row tile; the x tile index runs over (row tile, piece) pairs, piece fastest,
                     // so that the cheap pieces at the band's edges are spread over all CTAs
    int epi_direct;  // tuning: store the epilogue straight from registers (no transposition through shared memory)
    int starve;      // test hook: the filter producer announces more bytes than it loads, so the stage never completes
};

struct SmemLayout {
    uint32_t a_off, b_off, raw_off, koff_off, split_off, stage_off, bar_off, total;
};
__host__ __device__ inline SmemLayout smem_layout(const IgemmParams &P, bool a_tmem) {
    SmemLayout L;
    uint32_t o = 0;
    L.a_off = o;
    o += a_tmem ? 0 : (uint32_t)P.NA * 2 * kAHalfBytes;
    L.b_off = o;
    o += (uint32_t)P.NB * 2 * (uint32_t)P.BN * 128;
    L.raw_off = o;
    o += (uint32_t)P.NR * (uint32_t)P.raw_bytes;
    L.koff_off = o;
    o += (uint32_t)P.spc * (uint32_t)P.ke * 4;
    // split-K: landing area for the cluster's partial sums of this CTA's columns, [rank][BN/ksplit][128] floats.  Its
    // own region: peers push into it while this CTA may still be in its main loop.
    L.split_off = (o + 127) & ~127u;
    o = L.split_off + (P.ksplit > 1 ? 512u * (uint32_t)P.BN + 1024u : 0u); // + each tile row's offset in y (-1: none)
    // ping-pong mode: the epilogue's 32x32 transposition blocks need their own room (the B ring is never idle), one per warp
    L.stage_off = (o + 127) & ~127u;
    // (GBMML's operand fetch, which is not in ping-pong mode, keeps two blocks per warp: one stage in flight)
    o = L.stage_off + (P.pp ? 8u * 4096u : ((P.a_kmajor && P.band_w > 0) ? 16u * 4096u : 0u));
    L.bar_off = (o + 15) & ~15u;
    L.total = L.bar_off + 384;
    return L;
}

// Which rows of an output plane the pixels [q_lo, q_hi] of that plane touch (all of them when a tile holds several
// whole planes); shared by the raw producer, the transform threads and the host-side box sizing.
__host__ __device__ inline void tile_rows(const IgemmParams &P, int q_lo, int q_hi, bool whole, int &yl_lo, int &yl_hi) {
    yl_lo = 0;
    yl_hi = P.ohn - 1;
    if (whole)
        return;
    yl_lo = q_lo / P.own;
    yl_hi = q_hi / P.own;
}

template <int ACT> __device__ __forceinline__ float act_fn(float v) {
    if (ACT == PETB200_ACT_RELU)
        return fmaxf(v, 0.f);
    if (ACT == PETB200_ACT_SIGMOID)
        return 1.f / (1.f + expf(-v));
    if (ACT == PETB200_ACT_TANH)
        return tanhf(v);
    if (ACT == PETB200_ACT_GELU)
        return 0.5f * v * (1.f + erff(v * 0.70710678118654752440f));
    return v;
}

// Split-K, COLS (< 32) columns per CTA: the 32 columns in r[] belong to 32 / COLS consecutive CTAs of the cluster, starting
// with `owner0`; each group goes to its owner's landing area [this rank][column][pixel] (this CTA's own group by a plain
// shared-memory store).
template <int COLS>
__device__ __forceinline__ void push_groups(const uint32_t (&r)[32], uint32_t split_addr, int owner0, int me) {
#pragma unroll
    for (int g = 0; g < 32 / COLS; ++g) {
        const int owner = owner0 + g;
        if (owner == me) {
#pragma unroll
            for (int j = 0; j < COLS; ++j)
                ptx::st_shared_f32(split_addr + (uint32_t)(j * kTileM) * 4u, __uint_as_float(r[g * COLS + j]));
        } else {
            const uint32_t remote = ptx::map_to_cta(split_addr, (uint32_t)owner);
#pragma unroll
            for (int j = 0; j < COLS; ++j)
                ptx::st_dsmem_f32(remote + (uint32_t)(j * kTileM) * 4u, __uint_as_float(r[g * COLS + j]));
        }
    }
}

// TMEM accumulator rows -> (+bias, activation) -> global.  `yp` already points at this thread's pixel and the first
// filter of the group; column j of the tile is filter f_tile0 + j.  The activation is a template parameter so that
// the common no-activation case carries none of the transcendental code.
template <int ACT, int PASSES>
__device__ __forceinline__ void epilogue_store(uint32_t tacc, uint32_t tcross, int BN, int f_tile0, int Fg, bool valid, const float *bias,
                                               const float *rp /*residual at this pixel, or null*/, float *yp, long long ys_f, bool vec_ok, float *stage, int nvalid_warp, float *ybase_warp,
                                               const float *rbase_warp /*residual at the warp's first pixel, or null*/, int col0, int col1, uint32_t split_addr /*split-K: shared address of [this rank][0][this pixel]*/,
                                               int split_shift /*log2(columns per CTA)*/) {
    uint32_t r[32], nx[32], sm[32];
    if (col0 >= col1)
        return;
    ptx::tmem_ld_32x32(tacc + (uint32_t)col0, nx);
    if (PASSES != kMathTf32x1)
        ptx::tmem_ld_32x32(tcross + (uint32_t)col0, sm);
    for (int cc = col0; cc < col1; cc += 32) {
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) // hi*hi sum + (lo*hi + hi*lo) sum, one rounded fp32 add
            r[j] = PASSES != kMathTf32x1 ? __float_as_uint(__uint_as_float(nx[j]) + __uint_as_float(sm[j])) : nx[j];
        if (cc + 32 < col1) { // in flight while this chunk is stored
            ptx::tmem_ld_32x32(tacc + (uint32_t)(cc + 32), nx);
            if (PASSES != kMathTf32x1)
                ptx::tmem_ld_32x32(tcross + (uint32_t)(cc + 32), sm);
        }
        if (split_addr != 0u) {
            // Split-K: column c of the tile is summed by CTA c / cols of the cluster.  Push this CTA's partial sum into
            // that CTA's shared memory, slot [this rank][c % cols][pixel] (consecutive lanes = consecutive words).
            if (split_shift >= 5) {
                // at least 32 columns per CTA: the whole block has one owner — one address translation, and the block this
                // CTA owns itself stays out of the cluster network
                const int owner = cc >> split_shift, lc0 = cc & ((1 << split_shift) - 1);
                const uint32_t local = split_addr + (uint32_t)(lc0 * kTileM) * 4u;
                if (owner == (int)ptx::cluster_ctarank()) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        ptx::st_shared_f32(local + (uint32_t)(j * kTileM) * 4u, __uint_as_float(r[j]));
                } else {
                    const uint32_t remote = ptx::map_to_cta(local, (uint32_t)owner);
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        ptx::st_dsmem_f32(remote + (uint32_t)(j * kTileM) * 4u, __uint_as_float(r[j]));
                }
                continue;
            }
            if (split_shift == 4 || split_shift == 3) { // 16 or 8 columns per CTA: one translation per owner, not per column
                const int me = (int)ptx::cluster_ctarank(), owner0 = cc >> split_shift;
                if (split_shift == 4)
                    push_groups<16>(r, split_addr, owner0, me);
                else
                    push_groups<8>(r, split_addr, owner0, me);
                continue;
            }
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const int col = cc + j, owner = col >> split_shift, lc = col & ((1 << split_shift) - 1);
                ptx::st_dsmem_f32(ptx::map_to_cta(split_addr + (uint32_t)(lc * kTileM) * 4u, (uint32_t)owner), __uint_as_float(r[j]));
            }
            continue;
        }
        if (stage == nullptr && !valid)
            continue;
        const int f0 = f_tile0 + cc;
        // bias / residual / activation: each behind ONE test per block (a test per column costs more than the sums)
        if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (f0 + j < Fg)
                    r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldg(bias + f0 + j));
        }
        if (rp != nullptr && stage == nullptr) { // (only valid rows get here; the staged path adds the residual 16 bytes at a time)
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (f0 + j < Fg)
                    r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldg(rp + (long long)(f0 + j) * ys_f));
        }
        if (ACT != PETB200_ACT_NONE && (stage == nullptr || rbase_warp == nullptr)) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                r[j] = __float_as_uint(act_fn<ACT>(__uint_as_float(r[j])));
        }
        if (stage != nullptr) {
            // NCHW output, the warp's 32 pixels contiguous in memory: transpose the 32x32 block through shared memory so
            // that every lane stores 16 bytes (4 pixels of one filter) instead of 4 — a quarter of the store instructions.
            const int lane = threadIdx.x & 31;
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 32; ++j)
                stage[j * 32 + lane] = __uint_as_float(r[j]);
            __syncwarp();
            const int px = (lane & 7) * 4, cq = lane >> 3;
            const long long off = (long long)(f0 + cq) * ys_f + px; // from the warp's first pixel: filter f0 + cq, 4 filters apart per step
            float *dst = ybase_warp + off;
            const float *rsd = rbase_warp != nullptr ? rbase_warp + off : nullptr;
            const float *src = stage + cq * 32 + px;
            const int fmax = Fg - f0 - cq; // filters left from this lane's first one
#pragma unroll
            for (int i = 0; i < 8; ++i, dst += 4 * ys_f, src += 128) {
                if (4 * i < fmax) {
                    float4 v = *reinterpret_cast<const float4 *>(src);
                    if (rsd != nullptr) { // y = act(sum + bias + residual): the residual's four pixels sit where y's will
                        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
                        const float *rs = rsd + (long long)(4 * i) * ys_f;
                        if (px + 3 < nvalid_warp) {
                            q = __ldg(reinterpret_cast<const float4 *>(rs));
                        } else {
                            if (px < nvalid_warp) q.x = __ldg(rs);
                            if (px + 1 < nvalid_warp) q.y = __ldg(rs + 1);
                            if (px + 2 < nvalid_warp) q.z = __ldg(rs + 2);
                        }
                        v.x = act_fn<ACT>(v.x + q.x), v.y = act_fn<ACT>(v.y + q.y), v.z = act_fn<ACT>(v.z + q.z), v.w = act_fn<ACT>(v.w + q.w);
                    }
                    if (px + 3 < nvalid_warp) {
                        *reinterpret_cast<float4 *>(dst) = v;
                    } else {
                        if (px < nvalid_warp) dst[0] = v.x;
                        if (px + 1 < nvalid_warp) dst[1] = v.y;
                        if (px + 2 < nvalid_warp) dst[2] = v.z;
                    }
                }
            }
        } else if (vec_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                if (f0 + j < Fg)
                    *reinterpret_cast<uint4 *>(yp + f0 + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (f0 + j < Fg)
                    yp[(long long)(f0 + j) * ys_f] = __uint_as_float(r[j]);
        }
    }
}

// Banded product: the tile holds rows [128*bx, +128) x keys [128*bx - w + col_base, + BN) of q . k^T.  Entry (row pr, column c)
// is band column jb = col_base + c - pr of row i = 128*bx + pr (key i + jb - w); entries with jb outside [0, 2w] are not part
// of the band, entries whose key is outside [0, n) are stored as zero.  A warp passes 32 rows x 32 columns through shared
// memory (XOR-swizzled, conflict-free both ways) so that each store instruction writes 32 consecutive band columns of one row.
template <int PASSES>
__device__ __forceinline__ void epilogue_banded(uint32_t tacc, uint32_t tcross, int c_lo, int c_hi /*columns of the tile to store*/, int col_base,
                                                int p0, int bx, int zb, int n, int w, float *y, float *stage, int lane) {
    uint32_t nx[32], sm[32];
    const int bw = 2 * w + 1;
    const int i0 = bx * kTileM + p0;    // first row of this warp
    const int rows = min(32, n - i0);   // rows of it inside the tensor
    for (int cc = c_lo; cc < c_hi; cc += 32) {
        const int lo = col_base + cc - p0; // jb of (row 0, lane 0); the block spans jb in [lo - 31, lo + 31]
        if (rows <= 0 || lo + 31 < 0 || lo - 31 >= bw)
            continue; // nothing of this block lies in the band
        ptx::tmem_ld_32x32(tacc + (uint32_t)cc, nx);
        if (PASSES != kMathTf32x1)
            ptx::tmem_ld_32x32(tcross + (uint32_t)cc, sm);
        // this lane's column: band column of warp row r is jb0 - r, the key is the same for every row
        const int jb0 = col_base + cc + lane - p0, key = i0 + jb0 - w;
        const bool key_ok = key >= 0 && key < n;
        float *dst = y + ((long long)zb * n + i0) * bw + jb0; // row r: dst + r * (bw - 1)
        ptx::tmem_ld_wait();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float v = PASSES != kMathTf32x1 ? __uint_as_float(nx[j]) + __uint_as_float(sm[j]) : __uint_as_float(nx[j]);
            stage[lane * 32 + (j ^ lane)] = v;
        }
        __syncwarp();
        // every entry of the block inside the band and the tensor (the common case): no tests per store
        if (rows == 32 && lo - 31 >= 0 && lo + 31 < bw && __all_sync(0xffffffffu, key_ok)) {
#pragma unroll
            for (int r = 0; r < 32; ++r, dst += bw - 1)
                *dst = stage[r * 32 + (lane ^ r)];
        } else {
#pragma unroll 4
            for (int r = 0; r < 32; ++r, dst += bw - 1)
                if (r < rows && (unsigned)(jb0 - r) < (unsigned)bw)
                    *dst = key_ok ? stage[r * 32 + (lane ^ r)] : 0.f;
        }
    }
}

// One K stage of one tile row: fetch the stage's operands (32, or 64 for bf16) and split them into hi/lo parts — TF32:
// hi = top 19 bits, lo = x - hi, one value per word; bf16: hi = bf16(x), lo = bf16(x - hi), two values per word, the
// lower K index in the low half; a single pass rounds instead.  Where the operands come from:
//   kGatherTable   im2col through the offset table of the stage (entry < 0: no such element);
//   kGatherFlat    the same for unpadded whole-plane raw tiles: entries carry the filter tap in bits 24..30 and `tmask`
//                  tells which taps fall inside the input for this pixel;
//   kGatherStride  the stage is RUNS runs of consecutive channels, each of ONE tap, so the operands of a run sit
//                  `cstride` floats apart from the run's first table entry - no table reads, no per-element tests;
//   kGatherKMajor  matmul with row-major A: row p of the 128B-swizzled [128][32] tile (two tiles for a 64-wide stage).
enum { kGatherTable = 0, kGatherFlat = 1, kGatherStride = 2, kGatherKMajor = 3 };
template <int MODE, int PASSES, int RUNS = 1>
__device__ __forceinline__ void gather_split(const int4 *ko, const float *raw, const uint8_t *krow, int p, uint32_t tmask,
                                             int cstride, bool flat, const float *zero_word, uint32_t (&hi)[32],
                                             uint32_t (&lo)[32]) {
    constexpr bool BF = PASSES == kMathBf16x3;
    constexpr int KE = BF ? 64 : 32;  // operands per stage
    constexpr int kRun = KE / RUNS;   // channels per run
    const float *q[RUNS];
    int cs[RUNS];
#pragma unroll
    for (int r = 0; r < RUNS; ++r) {
        q[r] = raw;
        cs[r] = cstride;
        if (MODE == kGatherStride) {
            const int o0 = ko[r * (kRun / 4)].x; // first table entry of the run
            // past the end of the chunk's K range, or a tap outside the input for this pixel: read zeros
            const bool off = o0 < 0 || (flat && !((tmask >> (o0 >> 24)) & 1u));
            q[r] = off ? zero_word : raw + (flat ? (o0 & 0xffffff) : o0);
            cs[r] = off ? 0 : cstride;
        }
    }
#pragma unroll
    for (int c4 = 0; c4 < KE / 4; ++c4) {
        float v[4];
        if (MODE == kGatherKMajor) { // 16-byte chunk c of row p sits at c ^ (p & 7); the second tile follows the first
            const float4 t4 = *reinterpret_cast<const float4 *>(krow + (c4 >> 3) * kAHalfBytes + (((c4 & 7) ^ (p & 7)) << 4));
            v[0] = t4.x, v[1] = t4.y, v[2] = t4.z, v[3] = t4.w;
        } else if (MODE == kGatherStride) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                v[i] = q[(4 * c4 + i) / kRun][((4 * c4 + i) % kRun) * cs[(4 * c4 + i) / kRun]];
        } else {
            const int4 o4 = ko[c4];
            const int o[4] = {o4.x, o4.y, o4.z, o4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (MODE == kGatherFlat)
                    v[i] = (o[i] >= 0 && ((tmask >> (o[i] >> 24)) & 1u)) ? raw[o[i] & 0xffffff] : 0.f;
                else
                    v[i] = raw[o[i]]; // plain table mode has no negative entries
            }
        }
        if (BF) {
#pragma unroll
            for (int i = 0; i < 4; i += 2) {
                const uint32_t h = ptx::pack_bf16x2(v[i], v[i + 1]);
                hi[2 * c4 + i / 2] = h;
                lo[2 * c4 + i / 2] = ptx::pack_bf16x2(v[i] - __uint_as_float(h << 16), v[i + 1] - __uint_as_float(h & 0xffff0000u));
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (PASSES == kMathTf32x3) {
                    hi[4 * c4 + i] = __float_as_uint(v[i]) & 0xffffe000u;
                    lo[4 * c4 + i] = __float_as_uint(v[i] - __uint_as_float(hi[4 * c4 + i]));
                } else { // single pass: round to nearest TF32 instead of letting the tensor core truncate
                    hi[4 * c4 + i] = ptx::cvt_rna_tf32(v[i]);
                }
            }
        }
    }
}

// GBMML's operand fetch: one K stage = keys k0 .. k0 + 31; row i of the tile meets key k through the band entry p[i][k - i + w].
// The 32 entries of a row are contiguous in global memory but every row starts elsewhere, so the warp fetches them row by
// row (lane = key: one coalesced 128-byte read per row; entries outside the band, the row range or the sequence count as
// zero) into an XOR-swizzled 32 x 32 block of shared memory, from which each thread then takes its own row.  The fetch is
// asynchronous (cp.async, zero-filling what does not exist): band_issue starts the copies of a stage and closes a group,
// band_take waits for the group and splits; the caller keeps one stage in flight while it works on the one before.
__device__ __forceinline__ void band_issue(const float *pb /*band of this batch entry*/, int n, int w, int i0 /*first row of the warp*/, int k0,
                                           float *stage, int lane) {
    const int bw = 2 * w + 1, key = k0 + lane;
    const bool key_ok = key >= 0 && key < n;
    const float *src = pb + (long long)i0 * bw + (key - i0 + w); // row r: src + r * (bw - 1)
    const uint32_t dst = ptx::smem_u32(stage);
#pragma unroll
    for (int r = 0; r < 32; ++r, src += bw - 1) {
        const int j = key - (i0 + r) + w;
        const bool ok = key_ok && i0 + r < n && j >= 0 && j < bw;
        // 4 bytes per lane; a source size of 0 writes zeros and reads nothing (the address is then a harmless valid one)
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst + (uint32_t)(r * 32 + (lane ^ r)) * 4u), "l"(ok ? src : pb),
                     "r"(ok ? 4 : 0)
                     : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int PASSES>
__device__ __forceinline__ void band_take(const float *stage, bool newer_in_flight, int lane, uint32_t (&hi)[32], uint32_t (&lo)[32]) {
    if (newer_in_flight)
        asm volatile("cp.async.wait_group 1;" ::: "memory"); // all but the newest group: this stage has landed
    else
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp(); // every lane's copies
#pragma unroll
    for (int e = 0; e < 32; ++e) {
        const float x = stage[lane * 32 + (e ^ lane)];
        if (PASSES == kMathTf32x3) {
            hi[e] = __float_as_uint(x) & 0xffffe000u;
            lo[e] = __float_as_uint(x - __uint_as_float(hi[e]));
        } else {
            hi[e] = ptx::cvt_rna_tf32(x);
        }
    }
    __syncwarp(); // the block may be overwritten by a later stage's copies
}

// Split-K reduction inside a thread-block cluster.  The ksplit CTAs of one output tile form a cluster; CTA `rank` owns
// BN/ksplit columns of the tile, and every CTA has pushed its partial sums of those columns into this CTA's shared memory
// as [source rank][column][pixel].  A thread adds the ksplit copies of an element in rank order (the sum does not depend
// on timing) and stores act(sum + bias).
template <int ACT>
__device__ __forceinline__ void cluster_reduce_store(const float *stage, int ksplit, int rank, int BN, int et /*0..255*/,
                                                     int f_tile0, int Fg, const float *bias, const float *rp, float *yp /*this pixel, filter 0*/,
                                                     long long ys_f, bool vec_ok) {
    const int cols = BN / ksplit, px = et & (kTileM - 1), half = et >> 7;
    if (vec_ok) {
        // Filters are contiguous in y (row-major matmul output): a thread owns a run of cols/2 consecutive columns of its
        // pixel and stores them 16 bytes at a time; with the interleaved assignment below every 4-byte store would
        // touch its own 32-byte sector.
        const int run = cols >> 1; // 2, 4, 8, ... 32
        for (int c0 = half * run; c0 < (half + 1) * run; c0 += 4) {
            const int f = f_tile0 + rank * cols + c0, nv = min(4, run);
            if (f >= Fg)
                break;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            // (kept as a loop: this code runs once per CTA, straight out of a cold instruction cache, so its length is its cost)
            const float *sp = stage + c0 * kTileM + px;
#pragma unroll 1
            for (int r = 0; r < ksplit; ++r, sp += cols * kTileM)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (j < nv)
                        acc[j] += sp[j * kTileM]; // rank order for every element
            if (nv == 4) { // Fg % 4 == 0 and f % 4 == 0 here: the whole quad is inside the row, and 16-byte aligned in y / residual
                if (bias != nullptr) {
                    float4 b;
                    if ((reinterpret_cast<uintptr_t>(bias) & 15) == 0)
                        b = __ldg(reinterpret_cast<const float4 *>(bias + f));
                    else
                        b = make_float4(__ldg(bias + f), __ldg(bias + f + 1), __ldg(bias + f + 2), __ldg(bias + f + 3));
                    acc[0] += b.x, acc[1] += b.y, acc[2] += b.z, acc[3] += b.w;
                }
                if (rp != nullptr) {
                    const float4 r4 = __ldg(reinterpret_cast<const float4 *>(rp + f));
                    acc[0] += r4.x, acc[1] += r4.y, acc[2] += r4.z, acc[3] += r4.w;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    acc[j] = act_fn<ACT>(acc[j]);
                *reinterpret_cast<float4 *>(yp + f) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    if (bias != nullptr)
                        acc[j] += __ldg(bias + f + j);
                    if (rp != nullptr)
                        acc[j] += __ldg(rp + f + j);
                    acc[j] = act_fn<ACT>(acc[j]);
                }
                *reinterpret_cast<float2 *>(yp + f) = make_float2(acc[0], acc[1]);
            }
        }
        return;
    }
#pragma unroll 2
    for (int cl = half; cl < cols; cl += 2) {
        const int f = f_tile0 + rank * cols + cl;
        if (f >= Fg)
            break;
        const float *sp = stage + cl * kTileM + px;
        float acc = sp[0]; // rank order, as in the 16-byte path
#pragma unroll 1
        for (int r = 1; r < ksplit; ++r)
            acc += sp[r * cols * kTileM];
        if (bias != nullptr)
            acc += __ldg(bias + f);
        if (rp != nullptr)
            acc += __ldg(rp + (long long)f * ys_f);
        yp[(long long)f * ys_f] = act_fn<ACT>(acc);
    }
}

// Register-total flush mode, transform set 1: its threads keep the 128 columns of their tile row in registers, add the main
// accumulator of every completed group of K stages to them (round-to-nearest adds, in group order), and at the end write
// total + last group back over the main accumulator, which the epilogue of both sets then reads as if nothing had happened.
// Returns false if a wait gave up.
__device__ __noinline__ bool drain_only_set(uint32_t tq /*TMEM address of this warp's lane quarter, column 0*/, int groups,
                                            uint64_t *acc_ready, uint64_t *acc_full, uint64_t *flushed, volatile int *abort_flag,
                                            int lane, long long *t_wait, long long *t_work) {
    float racc[128];
#pragma unroll
    for (int j = 0; j < 128; ++j)
        racc[j] = 0.f;
    for (int g = 0; g < groups; ++g) {
        const bool last = g == groups - 1;
        const long long cd0 = t_wait ? clock64() : 0;
        if (!(last ? ptx::mbar_wait(acc_full, 0u, abort_flag) : ptx::mbar_wait(acc_ready, (uint32_t)(g & 1), abort_flag)))
            return false;
        const long long cd1 = t_wait ? clock64() : 0;
        ptx::tc_fence_after();
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            uint32_t v0[16], v1[16];
            ptx::tmem_ld_32x16(tq + (uint32_t)(b * 32), v0);
            ptx::tmem_ld_32x16(tq + (uint32_t)(b * 32 + 16), v1);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                racc[b * 32 + j] += __uint_as_float(v0[j]);
                racc[b * 32 + 16 + j] += __uint_as_float(v1[j]);
            }
            if (last) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    v0[j] = __float_as_uint(racc[b * 32 + j]);
                    v1[j] = __float_as_uint(racc[b * 32 + 16 + j]);
                }
                ptx::tmem_st_32x16(tq + (uint32_t)(b * 32), v0);
                ptx::tmem_st_32x16(tq + (uint32_t)(b * 32 + 16), v1);
            }
        }
        if (last)
            ptx::tmem_st_wait();
        ptx::tc_fence_before();
        __syncwarp();
        if (!last && lane == 0)
            ptx::mbar_arrive(flushed);
        if (t_wait) {
            *t_wait += cd1 - cd0;
            *t_work += clock64() - cd1;
        }
    }
    return true;
}

// BAND: 0 ordinary operands; 1 G2BMM (banded epilogue, key windows per tile; persistent row-major mode only); 2 GBMML (A operand
// gathered from the band in global memory; row-major mode only).  Kernels of their own, so that the others carry none of it.
template <bool A_TMEM, bool A_KMAJOR, int PASSES, bool PP = false, int BAND = 0>
__global__ void __launch_bounds__(kThreads, 1)
k_igemm(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_bhi,
        const __grid_constant__ CUtensorMap tmap_blo, const IgemmParams P) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled operand tiles
    uint8_t *smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const SmemLayout L = smem_layout(P, A_TMEM);
    uint8_t *sA = smem + L.a_off;
    uint8_t *sB = smem + L.b_off;
    uint8_t *sRaw = smem + L.raw_off;
    int *sKoff = reinterpret_cast<int *>(smem + L.koff_off);
    float *sSplit = reinterpret_cast<float *>(smem + L.split_off);
    long long *sYoff = reinterpret_cast<long long *>(smem + L.split_off + 512u * (uint32_t)P.BN); // split-K only
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L.bar_off);
    // barrier slots
    uint64_t *raw_full = bars, *raw_empty = bars + kMaxNR;
    uint64_t *b_full = bars + 2 * kMaxNR, *b_empty = b_full + kMaxNB; // up to kMaxNB stages
    uint64_t *a_full = b_empty + kMaxNB, *a_empty = a_full + 4;       // up to 4 stages
    uint64_t *acc_full = a_empty + 4;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(acc_full + 2);
    float *zero_word = reinterpret_cast<float *>(acc_full + 3); // holds 0.0f: what a masked-off filter tap reads
    uint64_t *acc_ready = acc_full + 4; // a group of `fl` K stages has been accumulated: the main accumulator may be drained
    uint64_t *flushed = acc_full + 5;   // all eight transform warps have drained it: the MMA warp may restart it
    uint64_t *acc_full1 = acc_full + 6; // ping-pong mode: the second accumulator region is complete
    uint64_t *acc_empty = acc_full + 7; // [2]: the owning transform set has read accumulator region 0 / 1 out

    constexpr bool SPLIT = PASSES != kMathTf32x1; // hi/lo operands, two accumulators
    constexpr bool BF = PASSES == kMathBf16x3;
    constexpr int KE = BF ? 64 : 32;              // K elements per stage
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long *prof_cta = nullptr; // wall-clock marks of this CTA (entry, prologue done, epilogue done, exit), tuning only
    if (P.prof && threadIdx.x == 96) {
        prof_cta = P.prof + ((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * kProfSlots;
        prof_cta[8] = (long long)ptx::globaltimer_ns();
    }
    const int ntile = blockIdx.y / P.ksplit;
    const int ksp = blockIdx.y - ntile * P.ksplit;
    const int zb = blockIdx.z;
    const uint32_t b_half = (uint32_t)P.BN * 128u;
    // TMEM columns: [0,BN) accumulator of the hi*hi products, [BN,2*BN) accumulator of the two small cross terms,
    // [2*BN,3*BN) the running total of drained main accumulators (P.fl > 0), [P.a_col,512) the A stages of the TS variant
    const uint32_t tmem_cols = A_TMEM ? 512u : 256u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kMaxNR; ++i) {
            ptx::mbar_init(raw_full + i, 1);
            ptx::mbar_init(raw_empty + i, P.fl_regs ? 4 : 8);
        }
        for (int i = 0; i < kMaxNB; ++i) {
            ptx::mbar_init(b_full + i, 1);
            ptx::mbar_init(b_empty + i, 1);
        }
        for (int i = 0; i < 4; ++i) {
            ptx::mbar_init(a_full + i, 4);
            ptx::mbar_init(a_empty + i, 1);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_ready, 1);
        ptx::mbar_init(flushed, P.fl_regs ? 4 : 8);
        ptx::mbar_init(acc_full1, 1);
        ptx::mbar_init(acc_empty, BAND == 1 ? 8 : 4); // (G2BMM: both sets read every tile out)
        ptx::mbar_init(acc_empty + 1, BAND == 1 ? 8 : 4);
        *abort_flag = 0;
        *zero_word = 0.f;
        ptx::fence_mbar_init();
        ptx::prefetch_tmap(&tmap_x);
        ptx::prefetch_tmap(&tmap_bhi);
        ptx::prefetch_tmap(&tmap_blo);
    }
    for (int i = threadIdx.x; i < P.spc * KE; i += kThreads)
        sKoff[i] = P.koff[i];
    if (warp == 2) {
        ptx::tmem_alloc(tmem_slot, tmem_cols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched only this CTA's own state and the plan's constant table, so under programmatic dependent
    // launch it overlaps the tail of the preceding kernel; from here on the kernel reads what that kernel wrote.
    ptx::grid_dep_launch_dependents();
    ptx::grid_dep_wait();
    if (prof_cta)
        prof_cta[9] = (long long)ptx::globaltimer_ns();

    // Tile origin in the input: first image, depth slice, row and (16-byte aligned) column of the raw box.  `bx` is the
    // pixel-tile index: blockIdx.x, or in ping-pong mode every gridDim.x-th tile from there.
    int bx = (int)blockIdx.x;
    const int ntl = PP ? (P.mtiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 1; // tiles of this CTA
    int n_lo = 0, q0 = 0, unit0 = 0, z_start = 0, y_start = 0, x_start = 0, w_zl = 0, w_yl = 0, w_tx = 0;
    int nt_cur = ntile; // filter tile of the current pixel tile (differs per tile only for banded products)
    auto set_tile = [&](int tile) {
        bx = tile;
        if (BAND == 1) {
            bx = tile / P.band_nt;
            nt_cur = tile - bx * P.band_nt;
        }
        n_lo = 0, q0 = 0, unit0 = 0, w_zl = 0, w_yl = 0, w_tx = 0;
        if (A_KMAJOR) {
            z_start = y_start = x_start = 0; // the tile is rows [bx*128, +128) of A[zb]
        } else if (P.wide) {
            const int row = bx / P.row_tiles;
            w_tx = bx - row * P.row_tiles;
            n_lo = row / (P.OD * P.ohn);
            w_zl = (row / P.ohn) % P.OD;
            w_yl = row % P.ohn;
            z_start = w_zl * P.sd - P.pd;
            y_start = (P.oh0 + w_yl) * P.sh - P.ph;
            const int xs = (P.ow0 + w_tx * kTileM) * P.sw - P.pw;
            x_start = (xs >= 0) ? (xs & ~3) : -(((-xs) + 3) & ~3);
        } else {
            const int tu = bx / P.tpi;
            q0 = (bx - tu * P.tpi) * kTileM;
            unit0 = tu * P.ipt;
            n_lo = unit0 / P.OD;
            int yl_lo, yl_hi;
            tile_rows(P, q0, min(q0 + kTileM, P.Pw) - 1, P.ipt > 1, yl_lo, yl_hi);
            z_start = (unit0 - n_lo * P.OD) * P.sd - P.pd;
            y_start = (P.oh0 + yl_lo) * P.sh - P.ph;
            x_start = P.x0;
        }
        if (!A_KMAJOR && P.flat)
            z_start = y_start = x_start = 0; // the raw tile holds whole planes
    };
    set_tile((int)blockIdx.x);
    // Row p of this CTA's tile: is it an output pixel, where does its receptive field start in the raw tile, where does
    // it go in y.
    auto pixel_geom = [&](int p, bool &valid, int &base_p, long long &y_off) {
        base_p = 0;
        y_off = 0;
        if (A_KMAJOR) {
            const int row = bx * kTileM + p;
            valid = row < P.m_rows;
            y_off = (long long)zb * P.ys_n + (long long)row * P.ys_p;
        } else if (P.wide) {
            const int xl = w_tx * kTileM + p;
            valid = xl < P.own;
            if (valid) {
                const int oh = P.oh0 + w_yl, ow = P.ow0 + xl;
                base_p = ow * P.sw - P.pw - x_start;
                const long long img = P.z_is_batch ? (long long)zb : (long long)n_lo;
                y_off = img * P.ys_n + ((long long)(w_zl * P.OH + oh) * P.OW + ow) * P.ys_p;
            }
        } else {
            int ul = 0, q = q0 + p;
            if (P.ipt > 1) {
                ul = p / P.Pw;
                q = p - ul * P.Pw;
            }
            const int unit = unit0 + ul;
            valid = (ul < P.ipt) && (unit < P.units) && (q < P.Pw);
            if (valid) {
                const int n = unit / P.OD;
                const int zl = unit - n * P.OD;
                const int yl = q / P.own;
                const int xl = q - yl * P.own;
                const int oh = P.oh0 + yl, ow = P.ow0 + xl;
                base_p = (((n - n_lo) * P.BC * P.RD + (zl * P.sd - P.pd - z_start)) * P.RH + (oh * P.sh - P.ph - y_start)) * P.RW +
                         (ow * P.sw - P.pw - x_start);
                const long long img = P.z_is_batch ? (long long)zb : (long long)n;
                y_off = img * P.ys_n + ((long long)(zl * P.OH + oh) * P.OW + ow) * P.ys_p;
            }
        }
    };
    // split-K: this CTA reduces the channel chunks [c0, c1)
    const int c0 = (int)((long long)ksp * P.nchunks / P.ksplit), c1 = (int)((long long)(ksp + 1) * P.nchunks / P.ksplit);
    const int KS = (c1 - c0) * P.spc;

    if (warp == 0) {
        // ---------------- packed-weight producer (one thread) ----------------
        if (lane == 0) {
            int row0 = zb * P.Fg + ntile * P.BN;
            int sb = 0;
            uint32_t pb = 1; // first pass over the ring: every slot is free
            for (int ks = 0; ks < KS * ntl; ++ks) { // the same KS filter tiles for every pixel tile of this CTA
                if (!ptx::mbar_wait(b_empty + sb, pb, abort_flag))
                    break;
                uint8_t *dst = sB + (size_t)sb * 2 * b_half;
                ptx::mbar_expect_tx(b_full + sb, (SPLIT ? 2u : 1u) * b_half + (P.starve ? 64u : 0u));
                const int kst = ntl > 1 ? ks % KS : ks;
                int kx = (c0 * P.spc + kst) * KE; // first K element of the stage
                if (BAND == 2) // the key window of the row tile, start rounded down to a multiple of 4
                    kx += (((int)blockIdx.x * kTileM - P.band_w) & ~3);
                if (BAND == 1) { // the key window moves with the row tile (rows before the tensor or past it read as zero / are masked)
                    const int tile = (int)blockIdx.x + (ks / KS) * (int)gridDim.x, rt = tile / P.band_nt;
                    row0 = zb * P.m_rows + rt * kTileM - P.band_w + (tile - rt * P.band_nt) * P.BN;
                }
                ptx::tma_load_2d(dst, &tmap_bhi, b_full + sb, kx, row0);
                if (SPLIT)
                    ptx::tma_load_2d(dst + b_half, &tmap_blo, b_full + sb, kx, row0);
                if (++sb == P.NB) {
                    sb = 0;
                    pb ^= 1u;
                }
            }
        }
    } else if (warp == 2) {
        // ---------------- raw activation producer ----------------
        const int c_base = P.z_is_batch ? 0 : zb * P.cpg;
        if (lane == 0) {
            const uint32_t bytes = (uint32_t)P.RN * P.BC * P.RD * P.RH * P.RW * 4u;
            int rb = 0;
            uint32_t pr = 1; // first pass over the ring: every buffer is free
            bool go = true;
            for (int tl = 0; tl < ntl && go && !(BAND == 2); ++tl) { // (GBMML reads its A operand from global memory)
            if (tl > 0)
                set_tile((int)blockIdx.x + tl * (int)gridDim.x);
            const int n_start = P.z_is_batch ? zb : n_lo;
            for (int ch = 0; ch < c1 - c0; ++ch) {
                if (!ptx::mbar_wait(raw_empty + rb, pr, abort_flag)) {
                    go = false;
                    break;
                }
                if (A_KMAJOR) { // one [128 rows][32 k] tile per 32 K elements of the stage (columns past K read as zero)
                    ptx::mbar_expect_tx(raw_full + rb, (uint32_t)kAHalfBytes * (KE / 32));
                    for (int h = 0; h < KE / 32; ++h)
                        ptx::tma_load_3d(sRaw + (size_t)rb * P.raw_bytes + (size_t)h * kAHalfBytes, &tmap_x, raw_full + rb,
                                         (c0 + ch) * KE + h * 32, bx * kTileM, zb);
                } else if (P.flat) {
                    ptx::mbar_expect_tx(raw_full + rb, bytes);
                    ptx::tma_load_3d(sRaw + (size_t)rb * P.raw_bytes, &tmap_x, raw_full + rb, 0,
                                     ((c_base + (c0 + ch) * P.BC) / P.BC) * P.flat_rows, n_start);
                } else {
                    ptx::mbar_expect_tx(raw_full + rb, bytes);
                    ptx::tma_load_5d(sRaw + (size_t)rb * P.raw_bytes, &tmap_x, raw_full + rb, x_start, y_start, z_start,
                                     c_base + (c0 + ch) * P.BC, n_start);
                }
                if (++rb == P.NR) {
                    rb = 0;
                    pr ^= 1u;
                }
            }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The whole warp runs this loop with uniform control flow and only the tcgen05 instructions sit under
        // elect_one: descriptors and TMEM addresses then live in uniform registers.  (With the loop confined to one
        // lane the same instruction stream was issue-bound: 94 instead of 64 cycles per 128x128x8 MMA.)
        // 3xTF32 with two MMAs per K=8 step instead of three: the hi and lo filter tiles of a stage are adjacent in shared
        // memory, i.e. one K-major tile of 2*BN rows, so  A_hi x [B_hi ; B_lo]  is ONE MMA of width 2*BN whose result columns
        // [0,BN) are the main accumulator and [BN,2BN) the accumulator of the cross terms; A_lo x B_hi then adds to the
        // latter.  Same tensor-pipe work, a third fewer instructions from the warp that every stage waits for.
        const uint32_t idesc = BF ? ptx::idesc_bf16(kTileM, P.BN) : ptx::idesc_tf32(kTileM, P.BN);
        const uint32_t idesc_wide = BF ? ptx::idesc_bf16(kTileM, 2 * P.BN) : ptx::idesc_tf32(kTileM, 2 * P.BN);
        // A from TMEM; per instruction K = 8 TF32 values or 16 bf16 values, either way 8 columns of A and 32 bytes of a B row
        auto mma_ts = [](uint32_t d, uint32_t a, uint64_t b, uint32_t id, uint32_t acc) {
            if (BF)
                ptx::mma_bf16_ts(d, a, b, id, acc);
            else
                ptx::mma_tf32_ts(d, a, b, id, acc);
        };
        const uint64_t bdesc0 = ptx::smem_desc_k128(ptx::smem_u32(sB));
        const uint64_t adesc0 = A_TMEM ? 0ull : ptx::smem_desc_k128(ptx::smem_u32(sA));
        const uint32_t b_half16 = b_half >> 4;
        uint32_t tmem_acc = tmem_base, tmem_small = tmem_base + (uint32_t)P.BN; // main and cross-term accumulators of the tile
        uint32_t accumulate = 0;
        int sa = 0, sb = 0, prev_sa = -1, prev_sb = -1;
        uint32_t pa = 0, pb = 0;
        long long t_wa = 0, t_wb = 0, t_wf = 0;
        const long long t_begin = P.prof ? clock64() : 0;
        bool ok = true, ready_next = false;
        const int FLm = PP ? 0 : P.fl;
        int gpos = 0, gidx = 0; // position of the stage inside its flush group, index of the group
        bool cross_prepaid = false; // the current stage's cross-term MMAs were issued ahead, during the previous stage
        // Ping-pong mode: each transform set fills its own half of the A ring (slots 2*set, 2*set + 1, alternately), so every
        // slot's barriers see one producer in order; bit i of `apar` is the parity of slot i's next completed fill.
        uint32_t apar = 0;
        for (int tl = 0; tl < ntl && ok; ++tl) {
        if (PP) {
            // accumulators alternate between two TMEM regions; before reusing one, its previous tile must have been read out
            tmem_acc = tmem_base + (uint32_t)((tl & 1) * 2 * P.BN);
            tmem_small = tmem_acc + (uint32_t)P.BN;
            if (tl >= 2) {
                ok = ptx::mbar_wait(acc_empty + (tl & 1), (uint32_t)(((tl >> 1) - 1) & 1), abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                ptx::tc_fence_after();
            }
            accumulate = 0;
            ready_next = false;
            prev_sa = -1;
        }
        for (int ks = 0; ks < KS; ++ks) {
            if (PP) {
                sa = (tl & 1) * 2 + (ks & 1);
                pa = (apar >> sa) & 1u;
            }
            if (!ready_next) { // not already seen complete by the poll issued in the shadow of the previous stage's MMAs
                if (P.prof) {
                    const long long q0c = clock64();
                    ok = ptx::mbar_wait(a_full + sa, pa, abort_flag);
                    const long long q1c = clock64();
                    ok = ok && ptx::mbar_wait(b_full + sb, pb, abort_flag);
                    t_wa += q1c - q0c;
                    t_wb += clock64() - q1c;
                } else {
                    ok = ptx::mbar_wait(a_full + sa, pa, abort_flag) && ptx::mbar_wait(b_full + sb, pb, abort_flag);
                }
                ok = __all_sync(0xffffffffu, ok);
            }
            if (!ok)
                break;
            ptx::tc_fence_after();
            const uint64_t bhi = bdesc0 + (uint64_t)((uint32_t)sb * 2u * b_half16);
            const uint32_t ahi_t = tmem_base + (uint32_t)P.a_col + (uint32_t)sa * 64u, alo_t = ahi_t + 32u;
            const uint64_t ahi_s = adesc0 + (uint64_t)((uint32_t)sa * 2u * (kAHalfBytes >> 4));
            const uint64_t alo_s = ahi_s + (kAHalfBytes >> 4);
            // next stage's ring positions, polled (non-blocking) while this stage's last MMAs are still queued
            int nsa = sa + 1, nsb = sb + 1;
            uint32_t npa = pa, npb = pb;
            if (nsa == P.NA) {
                nsa = 0;
                npa ^= 1u;
            }
            if (PP) { // the next stage of this tile sits in the set's other slot
                nsa = (tl & 1) * 2 + ((ks + 1) & 1);
                npa = (apar >> nsa) & 1u;
                apar ^= 1u << sa;
            }
            if (nsb == P.NB) {
                nsb = 0;
                npb ^= 1u;
            }
            // one K=8 step.  The cross terms have their own accumulator: the tensor core truncates (rounds toward zero) its
            // accumulator after every MMA, a bias proportional to the accumulator's magnitude; keeping the small terms
            // away from the big sum removes most of those truncations from it.
            auto issue_step = [&](int kk) {
                const uint32_t acc_kk = kk == 0 ? accumulate : 1u;
                if (SPLIT) {
                    if (A_TMEM)
                        mma_ts(tmem_acc, ahi_t + kk * 8, bhi + 2 * kk, idesc_wide, acc_kk);
                    else
                        ptx::mma_tf32_ss(tmem_acc, ahi_s + 2 * kk, bhi + 2 * kk, idesc_wide, acc_kk);
                } else {
                    mma_ts(tmem_acc, ahi_t + kk * 8, bhi + 2 * kk, idesc, acc_kk); // single TF32 pass
                }
                if (kk == 0 && prev_sa >= 0) { // release the previous stage once this stage's first MMA is queued
                    ptx::mma_commit(a_empty + prev_sa);
                    ptx::mma_commit(b_empty + prev_sb);
                }
                if (SPLIT) {
                    if (A_TMEM)
                        mma_ts(tmem_small, alo_t + kk * 8, bhi + 2 * kk, idesc, 1u);
                    else
                        ptx::mma_tf32_ss(tmem_small, alo_s + 2 * kk, bhi + 2 * kk, idesc, 1u);
                }
            };
            // First stage of a new flush group: the main accumulator restarts from zero, but only after the transform warps
            // have drained the previous group's sum.  The stage's eight cross-term MMAs do not touch the main accumulator
            // and are issued first, so the tensor pipe has work while the drain is in flight.
            auto issue_main_only = [&](int kk) {
                mma_ts(tmem_acc, ahi_t + kk * 8, bhi + 2 * kk, idesc, 1u);
                if (kk == 0 && prev_sa >= 0) {
                    ptx::mma_commit(a_empty + prev_sa);
                    ptx::mma_commit(b_empty + prev_sb);
                }
            };
            const bool group_start = SPLIT && FLm > 0 && ks > 0 && gpos == 0; // (no division: this warp's loop is latency bound)
            const bool prepaid_now = cross_prepaid;
            cross_prepaid = false;
            if (group_start) {
                const uint64_t blo = bhi + b_half16;
                if (ptx::elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        mma_ts(tmem_small, ahi_t + kk * 8, blo + 2 * kk, idesc, 1u);
                        if (kk == 0 && prev_sa >= 0) {
                            ptx::mma_commit(a_empty + prev_sa);
                            ptx::mma_commit(b_empty + prev_sb);
                        }
                        mma_ts(tmem_small, alo_t + kk * 8, bhi + 2 * kk, idesc, 1u);
                    }
                }
                __syncwarp();
                // ... and, if the stage after this one is already there, its eight cross-term MMAs as well: 2 x 8 MMAs of
                // cover for the drain (that stage then only issues its four main MMAs)
                bool pre = (ks + 1 < KS) && FLm >= 2 && ptx::mbar_test_wait(a_full + nsa, npa) && ptx::mbar_test_wait(b_full + nsb, npb);
                pre = __all_sync(0xffffffffu, pre);
                if (pre) {
                    ptx::tc_fence_after();
                    const uint64_t nbhi = bdesc0 + (uint64_t)((uint32_t)nsb * 2u * b_half16), nblo = nbhi + b_half16;
                    const uint32_t nahi = tmem_base + (uint32_t)P.a_col + (uint32_t)nsa * 64u, nalo = nahi + 32u;
                    if (ptx::elect_one()) {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            mma_ts(tmem_small, nahi + kk * 8, nblo + 2 * kk, idesc, 1u);
                            mma_ts(tmem_small, nalo + kk * 8, nbhi + 2 * kk, idesc, 1u);
                        }
                    }
                    __syncwarp();
                    cross_prepaid = true;
                }
                const long long qf0 = P.prof ? clock64() : 0;
                ok = ptx::mbar_wait(flushed, (uint32_t)((gidx - 1) & 1), abort_flag);
                if (P.prof)
                    t_wf += clock64() - qf0;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                ptx::tc_fence_after();
                if (ptx::elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < 3; ++kk)
                        mma_ts(tmem_acc, ahi_t + kk * 8, bhi + 2 * kk, idesc, kk == 0 ? 0u : 1u);
                }
                __syncwarp();
            } else if (prepaid_now) { // the cross terms of this stage were issued with the previous stage's
                if (ptx::elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < 3; ++kk)
                        issue_main_only(kk);
                }
                __syncwarp();
            } else {
                if (ptx::elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < 3; ++kk)
                        issue_step(kk);
                }
                __syncwarp();
            }
            ready_next = (ks + 1 < KS) && ptx::mbar_test_wait(a_full + nsa, npa) && ptx::mbar_test_wait(b_full + nsb, npb);
            ready_next = __all_sync(0xffffffffu, ready_next);
            const bool group_end = SPLIT && FLm > 0 && gpos == FLm - 1 && ks + 1 < KS;
            if (++gpos == FLm)
                gpos = 0, ++gidx;
            if (ptx::elect_one()) {
                if (group_start)
                    mma_ts(tmem_acc, ahi_t + 24, bhi + 6, idesc, 1u);
                else if (prepaid_now)
                    issue_main_only(3);
                else
                    issue_step(3);
                if (group_end) // fires once every MMA of the group has completed
                    ptx::mma_commit(acc_ready);
            }
            __syncwarp();
            accumulate = 1u;
            if (ready_next) {
                // MMA-bound: the release of this stage rides behind the next stage's first MMA (nothing to wait for)
                prev_sa = sa;
                prev_sb = sb;
            } else {
                // transform-bound: the next stage is not there yet, and its producers may be waiting for this slot
                if (ptx::elect_one()) {
                    ptx::mma_commit(a_empty + sa);
                    ptx::mma_commit(b_empty + sb);
                }
                __syncwarp();
                prev_sa = -1;
            }
            sa = nsa;
            sb = nsb;
            pa = npa;
            pb = npb;
        }
        if (ptx::elect_one()) {
            if (ok && prev_sa >= 0) {
                ptx::mma_commit(a_empty + prev_sa);
                ptx::mma_commit(b_empty + prev_sb);
            }
            if (ok)
                ptx::mma_commit((PP && (tl & 1)) ? acc_full1 : acc_full);
        }
        __syncwarp();
        }
        if (lane == 0 && P.prof) {
            long long *pr = P.prof + ((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * kProfSlots;
            pr[0] = t_wa;
            pr[1] = t_wb;
            pr[2] = clock64() - t_begin;
            pr[16] = t_wf;
        }
    } else {
        // ---------------- transform + epilogue: two sets of four warps (3..6 and 7..10) ----------------
        // The per-stage chain  wait -> gather -> tcgen05.st -> wait::st -> arrive  is latency bound (~600 cycles);
        // two sets taking alternate K stages double the rate at which A stages are produced.
        const int tset = (warp - 3) >> 2;     // 0 or 1
        const int quarter = warp & 3;         // TMEM lane quarter this warp may access
        const int p = quarter * 32 + lane;    // pixel row inside the tile
        bool alive = true;
        long long t_we = 0, t_wr = 0, t_g = 0, t_st = 0, t_dw = 0, t_dd = 0, t_loop = 0, t_epi0 = 0;
        const long long t_begin = P.prof ? clock64() : 0;
        const bool reg_total = !PP && SPLIT && A_TMEM && P.fl > 0 && P.fl_regs != 0; // (ping-pong plans never flush)
        const int FL = (!PP && SPLIT && A_TMEM && !reg_total) ? P.fl : 0;
        // Register-total mode: set 1 only drains (a function of its own: its 128 totals per thread want the whole register file)
        if (reg_total && tset == 1)
            alive = drain_only_set(tmem_base + ((uint32_t)(quarter * 32) << 16), (KS + P.fl - 1) / P.fl, acc_ready, acc_full, flushed,
                                   abort_flag, lane, P.prof ? &t_dw : nullptr, P.prof ? &t_dd : nullptr);
        // Ping-pong mode: this set takes every second TILE of the CTA (set 0 the even ones) and produces all of its stages;
        // otherwise there is one tile and the sets take alternate stages of it.
        // Ping-pong mode: parities of this set's two A slots (free at first), and how many raw chunks of the CTA (all tiles,
        // in load order) this set has seen complete.  The raw ring is shared by both sets and a parity wait cannot tell a fill
        // from the one two fills earlier, so BOTH sets wait for every fill in order and release it: a set does that for the
        // other set's tiles (which it does not read) in the pauses of its own work.
        uint32_t own_apar = 3u;
        int rseen = 0;
        auto observe_until = [&](int limit) {
            for (; rseen < limit && alive; ++rseen) {
                alive = ptx::mbar_wait(raw_full + rseen % P.NR, (uint32_t)((rseen / P.NR) & 1), abort_flag);
                __syncwarp();
                if (lane == 0 && alive)
                    ptx::mbar_arrive(raw_empty + rseen % P.NR);
            }
        };
        if (BAND == 1) {
            // G2BMM: a tile is two K stages and 32 KB of skewed stores, so the epilogue is the long part: both sets store half
            // of EVERY tile (32 of its 64 key columns each), and the set that owns tile t + 2's operands produces them right
            // after its half of tile t, i.e. while the MMA warp is on tile t + 1.
            const int nch = c1 - c0;
            auto produce = [&](int tl) {
                observe_until(tl * nch); // fills of the other set's tiles
                if (!alive)
                    return;
                rseen += nch;
                const int chunk0 = tl * nch;
                int rb = chunk0 % P.NR, sa = 2 * tset;
                uint32_t prw = (uint32_t)((chunk0 / P.NR) & 1);
                for (int ch = 0; ch < nch && alive; ++ch) {
                    alive = ptx::mbar_wait(raw_full + rb, prw, abort_flag);
                    if (!alive)
                        break;
                    uint32_t hi[32], lo[32];
                    gather_split<kGatherKMajor, PASSES>(nullptr, nullptr, sRaw + (size_t)rb * P.raw_bytes + (size_t)p * 128, p, 0u, 0, false,
                                                        zero_word, hi, lo);
                    alive = ptx::mbar_wait(a_empty + sa, (own_apar >> (sa & 1)) & 1u, abort_flag);
                    if (!alive)
                        break;
                    ptx::tc_fence_after();
                    const uint32_t t = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)P.a_col + (uint32_t)sa * 64u;
                    ptx::tmem_st_32x32(t, hi);
                    ptx::tmem_st_32x32(t + 32u, lo);
                    ptx::tmem_st_wait();
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::mbar_arrive(a_full + sa);
                        ptx::mbar_arrive(raw_empty + rb);
                    }
                    own_apar ^= 1u << (sa & 1);
                    sa ^= 1;
                    if (++rb == P.NR) {
                        rb = 0;
                        prw ^= 1u;
                    }
                }
            };
            if (tset < ntl)
                produce(tset);
            for (int tl = 0; tl < ntl && alive; ++tl) {
                alive = ptx::mbar_wait((tl & 1) ? acc_full1 : acc_full, (uint32_t)((tl >> 1) & 1), abort_flag);
                if (!alive)
                    break;
                ptx::tc_fence_after();
                set_tile((int)blockIdx.x + tl * (int)gridDim.x);
                const uint32_t tacc = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((tl & 1) * 2 * P.BN);
                epilogue_banded<PASSES>(tacc, tacc + (uint32_t)P.BN, tset * 32, tset * 32 + 32, nt_cur * P.BN, (warp & 3) * 32, bx, zb, P.m_rows,
                                        P.band_w, P.y, reinterpret_cast<float *>(smem + L.stage_off) + (warp - 3) * 1024, lane);
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(acc_empty + (tl & 1));
                if ((tl & 1) == tset && tl + 2 < ntl)
                    produce(tl + 2);
            }
            observe_until(ntl * nch);
        }
        if (BAND != 1)
        for (int tl = PP ? tset : 0; tl < ntl && alive; tl += PP ? 2 : 1) {
        set_tile((int)blockIdx.x + tl * (int)gridDim.x); // (also for the only tile: nothing of it stays live across the code above)
        bool valid;
        int base_p;
        long long y_off;
        pixel_geom(p, valid, base_p, y_off);
        if (P.ksplit > 1 && tset == 0)
            sYoff[p] = valid ? y_off : -1; // read by the split-K reduction, after the cluster barrier
        uint32_t tmask = 0;
        if (!A_KMAJOR && P.flat && valid) { // which filter taps of this pixel lie inside the (unpadded) input
            int ul = 0, q = q0 + p;
            if (P.ipt > 1) {
                ul = p / P.Pw;
                q = p - ul * P.Pw;
            }
            const int zl = (unit0 + ul) % P.OD, yl = q / P.own, xl = q - yl * P.own;
            const int z0 = zl * P.sd - P.pd, y0 = (P.oh0 + yl) * P.sh - P.ph, x0 = (P.ow0 + xl) * P.sw - P.pw;
            int tap = 0;
            for (int t = 0; t < P.T3[0]; ++t)
                for (int r = 0; r < P.T3[1]; ++r)
                    for (int sx = 0; sx < P.T3[2]; ++sx, ++tap) {
                        const int z = z0 + t * P.dil[0], y = y0 + r * P.dil[1], x = x0 + sx * P.dil[2];
                        if (z >= 0 && z < P.xD && y >= 0 && y < P.xH && x >= 0 && x < P.xW)
                            tmask |= 1u << tap;
                    }
        }
        if (PP) {
            observe_until(tl * (c1 - c0)); // fills that belong to the other set's tiles
            if (!alive)
                break;
            rseen += c1 - c0; // this tile's own chunks, waited for and released below
        }
        // raw buffer of the tile's first chunk and the parity of its fill
        const int chunk0 = PP ? tl * (c1 - c0) : 0;
        int rb = chunk0 % P.NR;
        uint32_t prw = (uint32_t)((chunk0 / P.NR) & 1);
        // Accumulator flush (P.fl > 0): the K stages form groups of P.fl; when the MMAs of group g have completed, the
        // eight transform warps add the main accumulator to the running total in TMEM (round-to-nearest fp32 adds, in
        // group order) and the MMA warp restarts the main accumulator for group g + 1.  A warp drains the columns its set
        // stores in the epilogue, of its own lane quarter.
        const int n_groups = FL > 0 ? (KS + FL - 1) / FL : 1;
        const int fcol0 = tset == 0 ? 0 : ((P.BN / 32 + 1) / 2) * 32, fcol1 = tset == 0 ? ((P.BN / 32 + 1) / 2) * 32 : P.BN;
        int fg = 0; // next group this warp has to drain
        auto drain_group = [&](int g, bool wait_mma, bool signal) -> bool {
            const long long cd0 = P.prof ? clock64() : 0;
            if (wait_mma && !ptx::mbar_wait(acc_ready, (uint32_t)(g & 1), abort_flag))
                return false;
            const long long cd1 = P.prof ? clock64() : 0;
            ptx::tc_fence_after();
            const uint32_t tq = tmem_base + ((uint32_t)(quarter * 32) << 16);
            for (int cc = fcol0; cc < fcol1; cc += 32) {
                uint32_t mn[32], tt[32];
                ptx::tmem_ld_32x32(tq + (uint32_t)cc, mn);
                if (g > 0)
                    ptx::tmem_ld_32x32(tq + 2u * (uint32_t)P.BN + (uint32_t)cc, tt);
                ptx::tmem_ld_wait();
                if (g > 0) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        mn[j] = __float_as_uint(__uint_as_float(tt[j]) + __uint_as_float(mn[j]));
                }
                ptx::tmem_st_32x32(tq + 2u * (uint32_t)P.BN + (uint32_t)cc, mn);
            }
            ptx::tmem_st_wait();
            ptx::tc_fence_before();
            __syncwarp();
            if (signal && lane == 0)
                ptx::mbar_arrive(flushed);
            if (P.prof) {
                t_dw += cd1 - cd0;
                t_dd += clock64() - cd1;
            }
            return true;
        };
        const bool all_stages = reg_total || PP; // this set produces every stage of the tile
        const int sstep = all_stages ? 1 : 2;  // stages between two stages of one set
        int gs = all_stages ? 0 : tset; // index of this set's next K stage among the tile's KS stages
        // This set owns every second K stage (tset, tset + 2, ...) or all of them: `st` is the next one's index inside the
        // current chunk, `sa`/`pa` its slot of the A ring and the parity to wait for (first pass over the ring: every slot is
        // free; ping-pong: the tile's first stage follows the tl * KS stages of the earlier tiles).
        int st = all_stages ? 0 : tset;
        int sa = PP ? 2 * tset : st;
        uint32_t pa = PP ? (own_apar & 1u) : 1u;
        for (int ch = 0; ch < ((reg_total && tset == 1) ? 0 : c1 - c0) && alive; ++ch, st -= P.spc) {
            const long long cr0 = P.prof ? clock64() : 0;
            const bool band_gather = BAND == 2; // no raw tiles: the operands come from global memory
            if (!band_gather)
                alive = ptx::mbar_wait(raw_full + rb, prw, abort_flag); // also by a set without a stage in this chunk
            if (P.prof)
                t_wr += clock64() - cr0;
            const float *raw = reinterpret_cast<const float *>(sRaw + (size_t)rb * P.raw_bytes) + base_p;
            for (; st < P.spc && alive; st += sstep, gs += sstep) {
                // Groups that ended before this stage: drain at once if their MMAs are done; otherwise produce one more
                // stage first (the MMA warp can start on it) and then wait for them.
                while (fg < n_groups - 1 && gs >= (fg + 1) * FL && alive) {
                    const bool done = __shfl_sync(0xffffffffu, ptx::mbar_test_wait(acc_ready, (uint32_t)(fg & 1)) ? 1 : 0, 0) != 0;
                    if (!done && gs < (fg + 1) * FL + 2)
                        break;
                    alive = drain_group(fg, !done, true);
                    ++fg;
                }
                if (!alive)
                    break;
                const int4 *ko = reinterpret_cast<const int4 *>(sKoff + st * KE);
                if (!A_TMEM) {
                    const long long ce0 = P.prof ? clock64() : 0;
                    alive = ptx::mbar_wait(a_empty + sa, pa, abort_flag);
                    if (P.prof)
                        t_we += clock64() - ce0;
                    if (!alive)
                        break;
                }
                if (A_TMEM) {
                    // The operands are gathered and split into registers BEFORE the wait for the stage's slot in tensor
                    // memory: when the slot frees, only the two tcgen05.st remain, so a set is one stage ahead in registers
                    // on top of its slots in the ring.
                    uint32_t hi[32], lo[32];
                    const uint8_t *krow = sRaw + (size_t)rb * P.raw_bytes + (size_t)p * 128;
                    const long long cg0 = P.prof ? clock64() : 0;
                    if (BAND == 2) {
                        // stage (c0 + ch) of the tile covers keys k0 .. k0 + 31 of the row tile's window; this set's next stage
                        // (two on) is fetched while this one is split and written
                        if (PASSES != kMathBf16x3) {
                            const int k0 = ((bx * kTileM - P.band_w) & ~3) + (c0 + ch) * kStageK, i0w = bx * kTileM + (warp & 3) * 32;
                            const float *pb = P.band_p + (long long)zb * P.m_rows * (2 * P.band_w + 1);
                            float *blk = reinterpret_cast<float *>(smem + L.stage_off) + (warp - 3) * 2048; // two blocks per warp
                            const bool more = ch + sstep < c1 - c0;
                            if (ch < sstep) // the set's first stage of the tile
                                band_issue(pb, P.m_rows, P.band_w, i0w, k0, blk + ((ch / sstep) & 1) * 1024, lane);
                            if (more)
                                band_issue(pb, P.m_rows, P.band_w, i0w, k0 + sstep * kStageK, blk + ((ch / sstep + 1) & 1) * 1024, lane);
                            band_take<PASSES>(blk + ((ch / sstep) & 1) * 1024, more, lane, hi, lo);
                        }
                    } else if (A_KMAJOR)
                        gather_split<kGatherKMajor, PASSES>(ko, raw, krow, p, tmask, 0, false, zero_word, hi, lo);
                    else if (P.cstride) // runs per stage: 1, 2 or 4 of 32 TF32 values; 2, 4 or 8 of 64 bf16 values
                        if (!BF && P.gruns == 1)
                            gather_split<kGatherStride, PASSES, 1>(ko, raw, krow, p, tmask, P.cstride, P.flat != 0, zero_word, hi, lo);
                        else if (P.gruns == 2)
                            gather_split<kGatherStride, PASSES, 2>(ko, raw, krow, p, tmask, P.cstride, P.flat != 0, zero_word, hi, lo);
                        else if (!BF || P.gruns == 4)
                            gather_split<kGatherStride, PASSES, 4>(ko, raw, krow, p, tmask, P.cstride, P.flat != 0, zero_word, hi, lo);
                        else
                            gather_split<kGatherStride, PASSES, 8>(ko, raw, krow, p, tmask, P.cstride, P.flat != 0, zero_word, hi, lo);
                    else if (P.flat)
                        gather_split<kGatherFlat, PASSES>(ko, raw, krow, p, tmask, 0, true, zero_word, hi, lo);
                    else
                        gather_split<kGatherTable, PASSES>(ko, raw, krow, p, tmask, 0, false, zero_word, hi, lo);
                    const long long ce0 = P.prof ? clock64() : 0;
                    alive = ptx::mbar_wait(a_empty + sa, pa, abort_flag);
                    if (!alive)
                        break;
                    ptx::tc_fence_after();
                    const uint32_t t = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)P.a_col + (uint32_t)sa * 64u;
                    ptx::tmem_st_32x32(t, hi);
                    const long long cg1 = P.prof ? clock64() : 0;
                    if (P.prof) {
                        t_we += cg1 - ce0;
                        t_g -= cg1 - ce0; // the gather time below is measured up to cg1
                    }
                    if (SPLIT)
                        ptx::tmem_st_32x32(t + 32u, lo);
                    ptx::tmem_st_wait();
                    ptx::tc_fence_before();
                    if (P.prof) {
                        t_g += cg1 - cg0;
                        t_st += clock64() - cg1;
                    }
                } else {
                    uint8_t *rowh = sA + (size_t)sa * 2 * kAHalfBytes + (size_t)p * 128;
                    uint8_t *rowl = rowh + kAHalfBytes;
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const int4 o = ko[c4];
                        float v0 = o.x >= 0 ? raw[o.x] : 0.f, v1 = o.y >= 0 ? raw[o.y] : 0.f;
                        float v2 = o.z >= 0 ? raw[o.z] : 0.f, v3 = o.w >= 0 ? raw[o.w] : 0.f;
                        float4 h, l;
                        h.x = __uint_as_float(__float_as_uint(v0) & 0xffffe000u);
                        h.y = __uint_as_float(__float_as_uint(v1) & 0xffffe000u);
                        h.z = __uint_as_float(__float_as_uint(v2) & 0xffffe000u);
                        h.w = __uint_as_float(__float_as_uint(v3) & 0xffffe000u);
                        l.x = v0 - h.x;
                        l.y = v1 - h.y;
                        l.z = v2 - h.z;
                        l.w = v3 - h.w;
                        const int phys = (c4 ^ (p & 7)) << 4;
                        *reinterpret_cast<float4 *>(rowh + phys) = h;
                        *reinterpret_cast<float4 *>(rowl + phys) = l;
                    }
                    ptx::fence_proxy_async_smem();
                }
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(a_full + sa);
                if (PP) { // the set's other slot next; a slot's parity flips with every use
                    own_apar ^= 1u << (sa & 1);
                    sa ^= 1;
                    pa = (own_apar >> (sa & 1)) & 1u;
                } else {
                    sa += sstep;
                    if (sa >= P.NA) {
                        sa -= P.NA;
                        pa ^= 1u;
                    }
                }
            }
            __syncwarp();
            if (lane == 0 && alive && !band_gather)
                ptx::mbar_arrive(raw_empty + rb);
            if (++rb == P.NR) {
                rb = 0;
                prw ^= 1u;
            }
        }
        // ---------------- epilogue ----------------
        t_loop = P.prof ? clock64() - t_begin : 0;
        if (PP) // the next tile's fills (the other set's): their loads only wait for buffers this tile has already released
            observe_until(min((tl + 2) * (c1 - c0), ntl * (c1 - c0)));
        // Addresses and store mode first: the MMA warp is still working through the last stages, so this costs nothing.
        const bool vec_ok = (P.ys_f == 1) && ((P.ys_p & 3) == 0) && ((P.ys_n & 3) == 0) && ((P.Fg & 3) == 0) &&
                            ((reinterpret_cast<uintptr_t>(P.y) & 15) == 0);
        const int f_tile0 = ntile * P.BN;
        const long long f_glob0 = P.z_is_batch ? 0 : (long long)zb * P.Fg;
        float *yp = P.y + y_off + f_glob0 * P.ys_f;
        const float *bp = (P.has_bias && P.ksplit == 1) ? P.bias + f_glob0 : nullptr;
        const float *rp = (P.res != nullptr && P.ksplit == 1) ? P.res + y_off + f_glob0 * P.ys_f : nullptr;
        // split-K: partial sums go to the landing areas of the cluster's CTAs, summed after the role branches
        const int split_cols = P.BN / P.ksplit, split_shift = 31 - __clz(split_cols);
        const uint32_t split_addr =
            P.ksplit > 1 ? ptx::smem_u32(sSplit) + (uint32_t)(((int)ptx::cluster_ctarank() * split_cols) * kTileM + p) * 4u : 0u;
        const uint32_t tacc0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (PP ? (uint32_t)((tl & 1) * 2 * P.BN) : 0u);
        const uint32_t tacc = tacc0 + (FL > 0 ? 2u * (uint32_t)P.BN : 0u);
        const uint32_t tcross = tacc0 + (uint32_t)P.BN;
        // staged 16-byte stores need: pixel-contiguous NCHW output, full-width rows (no column window), one plane per
        // tile, 16-byte aligned runs (of y and of the residual, which is laid out like y)
        float *stage = nullptr;
        int nvalid_warp = 0;
        const long long plane_elems = (long long)P.OD * P.OH * P.OW;
        const long long y_off0 = __shfl_sync(0xffffffffu, y_off, 0);
        float *ybase_warp = yp - y_off + y_off0;
        const float *rbase_warp = rp != nullptr ? rp - y_off + y_off0 : nullptr;
        if (P.ys_p == 1 && P.ipt == 1 && P.own == P.OW && P.ow0 == 0 && (plane_elems & 3) == 0 && (P.ys_n & 3) == 0 &&
            ((P.OH * P.OW) & 3) == 0 && (!P.wide || (P.OW & 3) == 0) &&
            (P.ys_f & 3) == 0 && ((P.oh0 * P.OW) & 3) == 0 && P.ksplit == 1 &&
            (reinterpret_cast<uintptr_t>(P.y) & 15) == 0 && (reinterpret_cast<uintptr_t>(P.res) & 15) == 0 && !P.epi_direct) {
            nvalid_warp = __popc(__ballot_sync(0xffffffffu, valid));
            if (nvalid_warp > 0) // B stages are idle once the accumulator is complete; in ping-pong mode they never are
                stage = reinterpret_cast<float *>(PP ? smem + L.stage_off : sB) + (warp - 3) * 1024;
            if (!PP && (uint32_t)(warp - 3 + 1) * 4096u > (uint32_t)P.NB * (SPLIT ? 2u : 1u) * b_half)
                stage = nullptr; // not enough idle shared memory for this warp's block
        }
        // the two sets split the tile's columns (whole 32-column blocks)
        const int nblk = P.BN / 32, half_blk = (nblk + 1) / 2;
        const int col0 = (PP || tset == 0) ? 0 : half_blk * 32, col1 = (!PP && tset == 0) ? half_blk * 32 : P.BN;
        for (; fg < n_groups - 1 && alive; ++fg)
            alive = drain_group(fg, true, true);
        if (alive)
            alive = ptx::mbar_wait((PP && (tl & 1)) ? acc_full1 : acc_full, PP ? (uint32_t)((tl >> 1) & 1) : 0u, abort_flag);
        if (alive && FL > 0) // the last group joins the total; the epilogue then reads the total in place of the accumulator
            drain_group(n_groups - 1, false, false);
        if (reg_total) { // set 1 has written total + last group over the main accumulator: both sets meet before reading it
            ptx::named_bar_sync(1, 256);
            ptx::tc_fence_after();
        }
        t_epi0 = P.prof ? clock64() : 0;
        if (alive) {
            ptx::tc_fence_after();
#define PETB200_EPI(ACT_)                                                                                              \
    epilogue_store<ACT_, PASSES>(tacc, tcross, P.BN, f_tile0, P.Fg, valid, bp, rp, yp, P.ys_f, vec_ok, stage, nvalid_warp, \
                                 ybase_warp, rbase_warp, col0, col1, split_addr, split_shift)
            switch (P.ksplit > 1 ? PETB200_ACT_NONE : P.act) {
            case PETB200_ACT_RELU: PETB200_EPI(PETB200_ACT_RELU); break;
            case PETB200_ACT_SIGMOID: PETB200_EPI(PETB200_ACT_SIGMOID); break;
            case PETB200_ACT_TANH: PETB200_EPI(PETB200_ACT_TANH); break;
            case PETB200_ACT_GELU: PETB200_EPI(PETB200_ACT_GELU); break;
            default: PETB200_EPI(PETB200_ACT_NONE); break;
            }
#undef PETB200_EPI
            if (PP) { // this tile's accumulators are in registers or stored: the MMA warp may reuse the region
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(acc_empty + (tl & 1));
            }
        }
        } // tiles of this set
        if (PP)
            observe_until(ntl * (c1 - c0)); // fills of tiles after this set's last one
        if (P.prof && threadIdx.x == 96) { // lane 0 of warp 3 (transform set 0)
            long long *pr = P.prof + ((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * kProfSlots;
            pr[3] = t_we;
            pr[4] = t_wr;
            pr[5] = t_loop;
            pr[6] = clock64() - t_epi0;
            pr[7] = t_epi0 - t_begin;
            pr[10] = (long long)ptx::globaltimer_ns();
            pr[12] = t_g;
            pr[13] = t_st;
            pr[17] = t_dw;
            pr[18] = t_dd;
        }
    }

    // ---------------- split-K: reduction across the cluster ----------------
    // Every thread of every CTA of the cluster reaches the barrier (all waits above are bounded).
    if (P.ksplit > 1) {
        if (warp >= 3 && warp < 7) {
            // The bias / residual values the reduction below adds start their way to L1 while the cluster meets.  Set 0's
            // threads do it, for the row each of them wrote into sYoff itself (both halves of the CTA's column slice).
            const int et = threadIdx.x - 96, cols = P.BN / P.ksplit;
            const long long y_off = sYoff[et];
            const int f = ntile * P.BN + (int)ptx::cluster_ctarank() * cols;
            const long long f_glob0 = P.z_is_batch ? 0 : (long long)zb * P.Fg;
            if (y_off >= 0 && P.ys_f == 1) {
                if (P.res != nullptr)
                    for (int i = 0; i < cols && f + i < P.Fg; i += 8)
                        ptx::prefetch_l1(P.res + y_off + f_glob0 + f + i);
                if (P.has_bias && et == 0)
                    for (int i = 0; i < cols && f + i < P.Fg; i += 8)
                        ptx::prefetch_l1(P.bias + f_glob0 + f + i);
            }
        }
        ptx::cluster_sync_all(); // every CTA's pushes have landed; nothing touches a peer's memory after this
        if (prof_cta)
            prof_cta[14] = (long long)ptx::globaltimer_ns();
        if (warp >= 3) {
            const int et = threadIdx.x - 96;
            const long long y_off = sYoff[et & (kTileM - 1)];
            if (y_off >= 0 && *abort_flag == 0) {
                const long long f_glob0 = P.z_is_batch ? 0 : (long long)zb * P.Fg;
                float *yp = P.y + y_off + f_glob0 * P.ys_f;
                const float *bp = P.has_bias ? P.bias + f_glob0 : nullptr;
                const float *rp = P.res != nullptr ? P.res + y_off + f_glob0 * P.ys_f : nullptr;
                const int rank = (int)ptx::cluster_ctarank();
                // 16-byte stores need filters contiguous in y, 16-byte aligned rows, and column runs of at least 2
                const bool red_vec = (P.ys_f == 1) && ((P.ys_p & 3) == 0) && ((P.ys_n & 3) == 0) && ((P.Fg & 3) == 0) &&
                                     ((reinterpret_cast<uintptr_t>(P.y) & 15) == 0) && (P.BN / P.ksplit >= 4) &&
                                     (P.res == nullptr || (reinterpret_cast<uintptr_t>(P.res) & 15) == 0);
#define PETB200_RED(ACT_) \
    cluster_reduce_store<ACT_>(sSplit, P.ksplit, rank, P.BN, et, ntile * P.BN, P.Fg, bp, rp, yp, P.ys_f, red_vec)
                switch (P.act) {
                case PETB200_ACT_RELU: PETB200_RED(PETB200_ACT_RELU); break;
                case PETB200_ACT_SIGMOID: PETB200_RED(PETB200_ACT_SIGMOID); break;
                case PETB200_ACT_TANH: PETB200_RED(PETB200_ACT_TANH); break;
                case PETB200_ACT_GELU: PETB200_RED(PETB200_ACT_GELU); break;
                default: PETB200_RED(PETB200_ACT_NONE); break;
                }
#undef PETB200_RED
            }
        }
        if (prof_cta)
            prof_cta[15] = (long long)ptx::globaltimer_ns();
    }

    // ---------------- teardown ----------------
    if (*abort_flag) {
        // give copies that may still be in flight time to land before the CTA's shared memory is released
        uint64_t t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 200000ull)
            __nanosleep(1000);
        if (threadIdx.x == 0 && P.status)
            atomicExch(P.status, 1);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 2)
        ptx::tmem_dealloc(tmem_base, tmem_cols);
    if (prof_cta)
        prof_cta[11] = (long long)ptx::globaltimer_ns();
}

// -------------------------------------------------------------------------------------------------------------
// weight packing: W[F][cpg][T] (conv) or B[b][k][n] / B[b][n][k] (matmul) -> hi/lo [rows][Ktot], K ordered as the
// kernel consumes it: k = chunk*Kc_pad + tap*BC + ci, zero where there is no such element.
// -------------------------------------------------------------------------------------------------------------
// hi/lo parts of one packed value: TF32 (hi = top 19 bits, or rounded for a single pass) as fp32 words, or bf16 halves
template <bool BF> __device__ __forceinline__ void store_split(void *hi, void *lo, long long i, float v, int rna) {
    if (BF) {
        const uint32_t h = ptx::pack_bf16x2(v, 0.f) & 0xffffu;
        reinterpret_cast<uint16_t *>(hi)[i] = (uint16_t)h;
        reinterpret_cast<uint16_t *>(lo)[i] = (uint16_t)(ptx::pack_bf16x2(v - __uint_as_float(h << 16), 0.f) & 0xffffu);
    } else {
        const float h = rna ? __uint_as_float(ptx::cvt_rna_tf32(v)) : __uint_as_float(__float_as_uint(v) & 0xffffe000u);
        reinterpret_cast<float *>(hi)[i] = h;
        reinterpret_cast<float *>(lo)[i] = v - h;
    }
}

template <bool BF>
__global__ void __launch_bounds__(256) k_pack_conv_w(const float *__restrict__ w, void *__restrict__ hi,
                                                     void *__restrict__ lo, int F, int cpg, int T, int BC, int Kc_pad,
                                                     int nchunks, int rna) {
    const long long Ktot = (long long)Kc_pad * nchunks;
    const long long total = (long long)F * Ktot;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int f = (int)(i / Ktot);
        const int k = (int)(i - (long long)f * Ktot);
        const int ch = k / Kc_pad, kc = k - ch * Kc_pad;
        const int tap = kc / BC, ci = kc - tap * BC;
        const int c = ch * BC + ci;
        float v = 0.f;
        if (tap < T && c < cpg)
            v = __ldg(w + ((long long)f * cpg + c) * T + tap);
        store_split<BF>(hi, lo, i, v, rna);
    }
}

template <bool BF>
__global__ void __launch_bounds__(256) k_pack_mm_b(const float *__restrict__ b, void *__restrict__ hi,
                                                   void *__restrict__ lo, int bs, int n, int k, int Kpad, int transB, int rna,
                                                   long long sb_batch, long long sb_row, int BC, int Kc_pad) {
    pdl_prologue();
    const long long total = (long long)bs * n * Kpad;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int kp = (int)(i % Kpad); // packed position: chunk * Kc_pad + element of the chunk (BC of them, then padding)
        const int ch = kp / Kc_pad, kc = kp - ch * Kc_pad, kk = ch * BC + kc;
        const long long row = i / Kpad;
        const int nn = (int)(row % n);
        const int bb = (int)(row / n);
        float v = 0.f;
        if (kc < BC && kk < k)
            v = transB ? __ldg(b + bb * sb_batch + nn * sb_row + kk) : __ldg(b + bb * sb_batch + kk * sb_row + nn);
        store_split<BF>(hi, lo, i, v, rna);
    }
}

// -------------------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

static int env_int_early(const char *name, int dflt) {
    const char *v = getenv(name);
    return v ? atoi(v) : dflt;
}

struct TcCore {
    petb200_ctx *ctx = nullptr;
    IgemmParams P{};
    bool a_tmem = false;
    int single_pass = 0;
    int bf16 = 0; // error-compensated bf16 (64 K elements per stage) instead of TF32
    dim3 grid;
    size_t smem = 0;
    // geometry needed to (re)encode the activation map
    int xd[5]{}; // W,H,D,C,N of the activation tensor as the kernel sees it
    long long a_row = 0, a_batch = 0; // row-major matmul A: element strides of a row and of a batch entry
    long long Ktot = 0;
    int rows_b = 0;
    DevBuf whi, wlo, koff;
    long long y_elems = 0;
    CUtensorMap map_x{}, map_bhi{}, map_blo{};
    const void *map_x_ptr = nullptr;
    bool weights_ready = false;
    long long *prof = nullptr;
    int starve = 0;

    void (*kernel() const)(CUtensorMap, CUtensorMap, CUtensorMap, IgemmParams) {
        if (P.a_kmajor && P.band_w > 0) // banded products: G2BMM in persistent mode with its own epilogue, GBMML with its own operand fetch
            return P.pp ? k_igemm<true, true, kMathTf32x3, true, 1> : k_igemm<true, true, kMathTf32x3, false, 2>;
        if (P.pp) { // conv plans on the TS variant
            if (single_pass)
                return k_igemm<true, false, kMathTf32x1, true>;
            return bf16 ? k_igemm<true, false, kMathBf16x3, true> : k_igemm<true, false, kMathTf32x3, true>;
        }
        if (single_pass)
            return P.a_kmajor ? k_igemm<true, true, kMathTf32x1> : k_igemm<true, false, kMathTf32x1>;
        if (bf16)
            return P.a_kmajor ? k_igemm<true, true, kMathBf16x3> : k_igemm<true, false, kMathBf16x3>;
        if (P.a_kmajor)
            return k_igemm<true, true, kMathTf32x3>;
        return a_tmem ? k_igemm<true, false, kMathTf32x3> : k_igemm<false, false, kMathTf32x3>;
    }
    int encode_x(const float *x) {
        if (x == map_x_ptr)
            return PETB200_OK;
        EncodeTiledFn enc = encode_fn();
        if (!enc)
            return fail(ctx, PETB200_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
        if (P.a_kmajor) { // A[b][m][k] row-major: dims (k, m, b), one 128B-swizzled [128 rows][32 k] box per K stage
            cuuint64_t d3[3] = {(cuuint64_t)xd[0], (cuuint64_t)xd[1], (cuuint64_t)xd[2]};
            cuuint64_t s3[2] = {(cuuint64_t)a_row * 4, (cuuint64_t)a_batch * 4};
            cuuint32_t b3[3] = {(cuuint32_t)kStageK, (cuuint32_t)kTileM, 1};
            cuuint32_t e3[3] = {1, 1, 1};
            CUresult r3 = enc(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(x), d3, s3, b3, e3,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r3 != CUDA_SUCCESS)
                return fail(ctx, PETB200_ERR_CUDA, "cuTensorMapEncodeTiled(row-major A) failed with %d", (int)r3);
            map_x_ptr = x;
            return PETB200_OK;
        }
        if (P.flat) { // each image is one run of C*D*H*W floats, viewed as rows of flat_w
            const cuuint64_t run = (cuuint64_t)xd[0] * xd[1] * xd[2] * xd[3];
            cuuint64_t d3[3] = {(cuuint64_t)P.flat_w, run / P.flat_w, (cuuint64_t)xd[4]};
            cuuint64_t s3[2] = {(cuuint64_t)P.flat_w * 4, run * 4};
            cuuint32_t b3[3] = {(cuuint32_t)P.flat_w, (cuuint32_t)P.flat_rows, (cuuint32_t)P.RN};
            cuuint32_t e3[3] = {1, 1, 1};
            CUresult r3 = enc(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(x), d3, s3, b3, e3,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r3 != CUDA_SUCCESS)
                return fail(ctx, PETB200_ERR_CUDA, "cuTensorMapEncodeTiled(flat activations) failed with %d", (int)r3);
            map_x_ptr = x;
            return PETB200_OK;
        }
        cuuint64_t dims[5] = {(cuuint64_t)xd[0], (cuuint64_t)xd[1], (cuuint64_t)xd[2], (cuuint64_t)xd[3], (cuuint64_t)xd[4]};
        cuuint64_t str[4] = {(cuuint64_t)xd[0] * 4, (cuuint64_t)xd[0] * xd[1] * 4, (cuuint64_t)xd[0] * xd[1] * xd[2] * 4,
                             (cuuint64_t)xd[0] * xd[1] * xd[2] * xd[3] * 4};
        cuuint32_t box[5] = {(cuuint32_t)P.RW, (cuuint32_t)P.RH, (cuuint32_t)P.RD, (cuuint32_t)P.BC, (cuuint32_t)P.RN};
        cuuint32_t es[5] = {1, 1, 1, 1, 1};
        CUresult r = enc(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float *>(x), dims, str, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(ctx, PETB200_ERR_CUDA, "cuTensorMapEncodeTiled(activations) failed with %d", (int)r);
        map_x_ptr = x;
        return PETB200_OK;
    }
    int encode_b() {
        EncodeTiledFn enc = encode_fn();
        if (!enc)
            return fail(ctx, PETB200_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
        cuuint64_t dims[2] = {(cuuint64_t)Ktot, (cuuint64_t)rows_b};
        cuuint64_t str[1] = {(cuuint64_t)Ktot * (bf16 ? 2 : 4)};
        cuuint32_t box[2] = {(cuuint32_t)P.ke, (cuuint32_t)P.BN}; // one 128-byte row of K per filter
        cuuint32_t es[2] = {1, 1};
        for (int i = 0; i < 2; ++i) {
            CUresult r = enc(i ? &map_blo : &map_bhi, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                             i ? wlo.p : whi.p, dims, str, box,
                             es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS)
                return fail(ctx, PETB200_ERR_CUDA, "cuTensorMapEncodeTiled(weights) failed with %d", (int)r);
        }
        return PETB200_OK;
    }
    int launch(const float *x, const float *bias, const float *res, float *y, cudaStream_t s) {
        int rc = encode_x(x);
        if (rc)
            return rc;
        IgemmParams p = P;
        p.bias = bias;
        p.res = res;
        p.y = y;
        p.koff = (const int *)koff.p;
        p.status = ctx->d_status;
        p.prof = prof;
        p.starve = starve;
        p.epi_direct = env_int_early("PETB200_TC_EPI_DIRECT", 0);
        p.has_bias = (P.has_bias && bias) ? 1 : 0;
        void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, IgemmParams) = kernel();
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[2] = {};
        int nattr = 0;
        if (P.ksplit > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(ctx, PETB200_ERR_UNSUPPORTED, "clusters of %d CTAs are not allowed on this device", P.ksplit);
        }
        if (P.ksplit > 1) { // the splits of one output tile are consecutive in blockIdx.y: one cluster
            attr[nattr].id = cudaLaunchAttributeClusterDimension;
            attr[nattr].val.clusterDim.x = 1;
            attr[nattr].val.clusterDim.y = (unsigned)P.ksplit;
            attr[nattr].val.clusterDim.z = 1;
            ++nattr;
        }
        if (pdl_enabled()) { // this kernel's set-up may overlap the end of the kernel before it in the stream
            attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[nattr].val.programmaticStreamSerializationAllowed = 1;
            ++nattr;
        }
        cfg.attrs = nattr ? attr : nullptr;
        cfg.numAttrs = (unsigned)nattr;
        cudaError_t le = cudaLaunchKernelEx(&cfg, kern, map_x, map_bhi, map_blo, p);
        if (le != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(ctx, PETB200_ERR_CUDA, "launch of k_igemm failed: %s", cudaGetErrorString(le));
        }
        return launched(ctx, "k_igemm");
    }
};

// Geometry of the convolution as the tensor-core kernel sees it.
struct ConvGeom {
    int N, C, D, H, W, Wst /*row pitch of the stored tensor, >= W*/, F, T3[3] /*t,r,s*/, pad[3], stride[3], dil[3], groups;
    int OD, OH, OW;
};

static int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return v ? atoi(v) : dflt;
}

// Fills core.P (tiling, raw box, stage counts) for a window [oh0,ohn) x [ow0,own) of the output; returns
// PETB200_ERR_UNSUPPORTED when the shape does not fit this kernel's constraints.
// Rough cycle model of one launch, used to pick the tile width and the K split for problems that cannot fill the GPU
// with 128-wide tiles.  Constants are measured on B200: a K stage costs its MMAs (N/2 cycles each, 12 per stage for
// 3xTF32, 4 for one pass) or, if larger, the transform chain of the stage (~330 cycles with two warp sets); a CTA pays
// ~3000 cycles before its first MMA and 1700 + 44*BN cycles of epilogue (split-K: the exchange through the cluster instead).
// How many clusters of `ks` CTAs of this kernel (one CTA per SM) the device can hold at once: asked of the driver once
// per size (clusters stay inside a GPC, which leaves some SMs of every GPC without a cluster).
static int cluster_slots(int sm_count, int ks) {
    static int cached[17] = {0};
    if (ks <= 1)
        return sm_count;
    if (cached[ks] == 0) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(1, (unsigned)ks * 64, 1);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = 200 * 1024; // enough that two CTAs never share an SM, as in every real plan
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1, attr[0].val.clusterDim.y = (unsigned)ks, attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr, cfg.numAttrs = 1;
        int n = 0;
        (void)cudaFuncSetAttribute(k_igemm<true, false, kMathTf32x3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (ks > 8) // clusters of 16 are beyond the portable size: allowed per function
            (void)cudaFuncSetAttribute(k_igemm<true, false, kMathTf32x3, false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (cudaOccupancyMaxActiveClusters(&n, k_igemm<true, false, kMathTf32x3, false>, &cfg) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            // what B200 was measured to hold; a cluster of 16 is only used where the driver itself says it fits
            n = ks > 8 ? -1 : std::max(1, (sm_count * (ks <= 2 ? 96 : 86) / 100) / ks);
        }
        cached[ks] = n;
    }
    return cached[ks];
}

static double est_cycles(int sm_count, long long base_ctas, int nchunks, int spc, int BN, int passes, int ks) {
    const double stage = std::max<double>((passes == 3 ? 12.0 : 4.0) * (BN / 2), 520.0);
    const long long stages = (long long)((nchunks + ks - 1) / ks) * spc;
    // split-K: (ks-1)/ks of the 512*BN-byte tile crosses to other SMs at ~10 bytes per cycle, then barrier + local sums
    const double per_cta = 3000.0 + (double)stages * stage + 1700.0 + (ks > 1 ? 1500.0 + 50.0 * BN * (ks - 1) / ks : 44.0 * BN);
    const long long slots = cluster_slots(sm_count, ks);
    if (slots <= 0)
        return 1e30; // this cluster size cannot be launched here
    const long long waves = (base_ctas + slots - 1) / slots;
    return (double)waves * per_cta;
}
// Split K over 1, 2, 4, 8 or 16 CTAs (a cluster; 16 is beyond the portable cluster size and allowed per function): the
// split must divide the tile width and leave every CTA a chunk.
static int choose_ksplit(int sm_count, long long base_ctas, const IgemmParams &P, int passes, int want, double *cycles) {
    auto ok = [&](int ks) { return ks == 1 || (ks <= P.nchunks && P.BN % ks == 0); };
    int best = 1;
    double best_c = est_cycles(sm_count, base_ctas, P.nchunks, P.spc, P.BN, passes, 1);
    static const int ks_cap = std::min(16, std::max(1, env_int_early("PETB200_TC_KSPLIT_MAX", 16)));
    if (want > 0) {
        for (best = 16; best > 1 && !(best <= want && ok(best) && cluster_slots(sm_count, best) > 0); best /= 2) {
        }
        best_c = est_cycles(sm_count, base_ctas, P.nchunks, P.spc, P.BN, passes, best);
    } else {
        for (int ks = 2; ks <= ks_cap; ks *= 2) {
            if (!ok(ks))
                continue;
            const double c = est_cycles(sm_count, base_ctas, P.nchunks, P.spc, P.BN, passes, ks);
            if (c < best_c * 0.97) // a deeper split has to pay for itself
                best = ks, best_c = c;
        }
    }
    if (cycles)
        *cycles = best_c;
    return best;
}

// Accumulator flush period (see IgemmParams::fl) and the TMEM column map that goes with it.  The truncation bias of the
// tensor core's fp32 accumulator grows with the number of MMAs added into one running sum: K ranges of more than
// `3 * period` stages per CTA are drained every `period` stages (PETB200_TC_FLUSH in the environment, 0 = never; measured
// without a flush: 2.4e-4 of the contract's 1e-3 at 18 stages, 3e-4..4e-4 at 36, 2e-3 at 54).  The
// running total takes BN more TMEM columns; a 128-wide tile then has room for two A stages instead of four.
static void choose_flush(TcCore &core) {
    IgemmParams &P = core.P;
    // (bf16: twice the K per stage and an accuracy class that the split, not the truncation, dominates: half as often)
    const int period = env_int("PETB200_TC_FLUSH", core.bf16 ? 16 : 8);
    const int ks_max = ((P.nchunks + P.ksplit - 1) / P.ksplit) * P.spc;
    P.fl = (!core.single_pass && core.a_tmem && period > 0 && ks_max > 3 * period) ? period : 0;
    // register totals make one transform set do all the A stages: only where the gather is the cheap kind (whole 32-channel
    // stages of one tap, or row-major matmul tiles); slower gathers need both sets and keep the total in TMEM
    const bool fast_gather = P.a_kmajor || (P.cstride != 0 && P.gruns == (core.bf16 ? 2 : 1));
    const int regs_env = env_int("PETB200_TC_FLUSH_REGS", -1);
    P.fl_regs = (P.fl > 0 && P.BN == 128 && (regs_env < 0 ? fast_gather : regs_env != 0)) ? 1 : 0;
    P.a_col = (P.fl > 0 && P.BN == 128 && !P.fl_regs) ? 384 : 256;
    if (core.a_tmem)
        P.NA = (512 - P.a_col) / 64;
    if (env_int("PETB200_TC_VERBOSE", 0))
        fprintf(stderr, "[petb200] igemm plan: BN %d BC %d chunks %d stages/chunk %d ksplit %d flush %d (regs %d) NA %d NB %d NR %d kmajor %d flat %d math %s\n",
                P.BN, P.BC, P.nchunks, P.spc, P.ksplit, P.fl, P.fl_regs, P.NA, P.NB, P.NR, P.a_kmajor, P.flat,
                core.single_pass ? "1xtf32" : (core.bf16 ? "bf16x3" : "3xtf32"));
}

// The dynamic shared-memory attribute is per function, not per launch: raise it once to the device limit so that plans
// with different needs can coexist.
static int raise_smem_limit(petb200_ctx *ctx) {
    static bool attr_set = false;
    if (attr_set)
        return PETB200_OK;
    const int lim = (int)std::min<size_t>(ctx->smem_optin, 227 * 1024);
    cudaError_t e = cudaFuncSetAttribute(k_igemm<true, false, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<false, false, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<true, true, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<true, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<true, true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<true, false, kMathBf16x3>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<true, true, kMathBf16x3>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<true, false, kMathTf32x3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<true, false, kMathBf16x3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<true, false, kMathTf32x1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<true, true, kMathTf32x3, true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(k_igemm<true, true, kMathTf32x3, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e != cudaSuccess)
        return fail(ctx, PETB200_ERR_CUDA, "cudaFuncSetAttribute(%d bytes) failed: %s", lim, cudaGetErrorString(e));
    attr_set = true;
    return PETB200_OK;
}

static int tc_configure(petb200_ctx *ctx, TcCore &core, const ConvGeom &g, int oh0, int ohn, int ow0, int own,
                        int z_is_batch, int images, long long ys_n, long long ys_f, long long ys_p, int has_bias, int act,
                        int force_bc = 0, int force_ksplit = 0, int force_bn = 0, int flat = 0, int max_ipt = 0) {
    IgemmParams &P = core.P;
    const int cpg = g.C / g.groups, Fg = g.F / g.groups;
    if (!flat && g.Wst % 4 != 0)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "the TMA box needs a row pitch divisible by 4, got %d", g.Wst);
    P.flat = flat ? 1 : 0;
    P.ke = core.bf16 ? 64 : kStageK;
    P.xD = g.D, P.xH = g.H, P.xW = g.W;
    for (int i = 0; i < 3; ++i)
        P.T3[i] = g.T3[i], P.dil[i] = g.dil[i];
    P.OD = g.OD;
    P.OH = g.OH;
    P.OW = g.OW;
    P.oh0 = oh0;
    P.ohn = ohn;
    P.ow0 = ow0;
    P.own = own;
    P.Pw = ohn * own;
    P.units = (z_is_batch ? 1 : images) * g.OD;
    P.sd = g.stride[0];
    P.sh = g.stride[1];
    P.sw = g.stride[2];
    P.pd = g.pad[0];
    P.ph = g.pad[1];
    P.pw = g.pad[2];
    P.cpg = cpg;
    P.Fg = Fg;
    P.z_is_batch = z_is_batch;
    P.ys_n = ys_n;
    P.ys_f = ys_f;
    P.ys_p = ys_p;
    P.has_bias = has_bias;
    P.act = act;
    // Planes smaller than half a tile are packed several to a tile: whole images for 2-D problems, consecutive depth
    // slices of one image (a divisor of the depth, so that no tile straddles two images) for 3-D problems.
    P.ipt = 1;
    if (!z_is_batch && 2 * P.Pw <= kTileM) {
        const int cap = kTileM / P.Pw;
        if (g.OD == 1) {
            P.ipt = std::min(cap, P.units); // no more images per tile than there are
        } else {
            for (int d = std::min(cap, g.OD); d >= 1; --d)
                if (g.OD % d == 0) {
                    P.ipt = d;
                    break;
                }
        }
    }
    if (max_ipt > 0) // a caller that must keep another plan's chunk size may not afford several images per raw tile
        P.ipt = std::min(P.ipt, max_ipt);
    P.tpi = (P.Pw + kTileM - 1) / kTileM;
    P.wide = (own > kTileM) ? 1 : 0;
    P.row_tiles = (own + kTileM - 1) / kTileM;
    const int xs = ow0 * P.sw - P.pw;
    P.x0 = (xs >= 0) ? (xs / 4) * 4 : -(((-xs) + 3) / 4) * 4;
    if (P.wide) {
        // one output row per tile: the box covers 128 pixels of one row (one depth slice, one image)
        const int wneed = (kTileM - 1) * P.sw + (g.T3[2] - 1) * g.dil[2] + 1 + (xs - P.x0);
        P.RW = (wneed + 3) / 4 * 4;
        P.RN = 1;
        P.RD = (g.T3[0] - 1) * g.dil[0] + 1;
        P.RH = (g.T3[1] - 1) * g.dil[1] + 1;
    } else {
        const int wneed = (own - 1) * P.sw + (g.T3[2] - 1) * g.dil[2] + 1 + (xs - P.x0);
        P.RW = (wneed + 3) / 4 * 4;
        // rows a tile touches: maximum over the tiles of one plane (in OUTPUT rows first)
        int RHo = 1;
        for (int tq = 0; tq < P.tpi; ++tq) {
            int yl_lo, yl_hi;
            tile_rows(P, tq * kTileM, std::min((tq + 1) * kTileM, P.Pw) - 1, P.ipt > 1, yl_lo, yl_hi);
            RHo = std::max(RHo, yl_hi - yl_lo + 1);
        }
        P.RN = (g.OD == 1) ? P.ipt : 1;
        P.RD = ((g.OD == 1) ? 0 : (P.ipt - 1) * P.sd) + (g.T3[0] - 1) * g.dil[0] + 1;
        P.RH = (RHo - 1) * P.sh + (g.T3[1] - 1) * g.dil[1] + 1;
    }
    const int T = g.T3[0] * g.T3[1] * g.T3[2];
    if (flat) {
        // whole, unpadded planes: BC channels x all depth slices of RN images; padding is a mask over the taps
        if (P.wide || T > 32 || g.Wst != g.W)
            return fail(ctx, PETB200_ERR_UNSUPPORTED, "flat raw tiles need rows of at most 128 pixels and at most 32 taps");
        P.x0 = 0;
        P.RW = g.W, P.RH = g.H, P.RD = g.D;
        P.RN = (g.OD == 1) ? P.ipt : 1;
    } else if (P.RW > 256 || P.RH > 256 || P.RD > 256 || P.RN > 256) {
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "raw activation box %dx%dx%dx%d exceeds the TMA box limit", P.RN, P.RD, P.RH, P.RW);
    }
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 1024; // alignment slack
    core.a_tmem = core.single_pass || core.bf16 || env_int("PETB200_TC_A_TMEM", 1) != 0; // other variants exist for TS only
    const int forced_bc = force_bc > 0 ? force_bc : env_int("PETB200_TC_BC", 0);
    // Channels per chunk (32, or more for filters with few taps so that one raw tile still feeds several K stages) and
    // ring depths for a given tile width; false if not even one channel's raw tile fits.
    auto fit = [&](int BN) -> bool {
        P.BN = BN;
        int bc_cap = 32 * std::max(1, std::min(4, 4 / T));
        int BC = std::min(cpg, bc_cap);
        if (BC > 32)
            BC = BC / 32 * 32;
        if (forced_bc > 0)
            BC = std::min(forced_bc, cpg);
        for (;; BC = std::max(1, BC / 2)) {
            P.BC = BC;
            P.spc = (T * BC + P.ke - 1) / P.ke;
            P.nchunks = (cpg + BC - 1) / BC;
            size_t raw = (size_t)P.RN * BC * P.RD * P.RH * P.RW * 4;
            P.raw_bytes = (int)((raw + 127) / 128 * 128);
            P.NA = core.a_tmem ? 4 : 2;
            P.NB = 2;
            P.NR = 2;
            P.a_kmajor = 0;
            P.m_rows = 0;
            bool shape_ok = true;
            if (flat) {
                // The BC*D*H*W floats of a chunk are one contiguous run: fetch it as a 2-D box [rows][w] with w a multiple
                // of 4 (16-byte rule), both extents within the TMA box limit; chunks must start on a box boundary.
                const long long L = (long long)BC * g.D * g.H * g.W;
                P.flat_w = 0;
                for (int w = 256; w >= 4 && !P.flat_w; w -= 4)
                    if (L % w == 0 && L / w <= 256)
                        P.flat_w = w, P.flat_rows = (int)(L / w);
                shape_ok = P.flat_w != 0 && cpg % BC == 0 && P.RN <= 256;
            }
            if (shape_ok && smem_layout(P, core.a_tmem).total <= budget) {
                // deepen the rings while there is room: B first (it hides TMA latency), then A
                for (bool grew = true; grew;) {
                    grew = false;
                    if (P.NB < kMaxNB) {
                        P.NB++;
                        if (smem_layout(P, core.a_tmem).total <= budget)
                            grew = true;
                        else
                            P.NB--;
                    }
                    if (!core.a_tmem && P.NA < 3 && P.NB >= 3) {
                        P.NA++;
                        if (smem_layout(P, core.a_tmem).total <= budget)
                            grew = true;
                        else
                            P.NA--;
                    }
                }
                return true;
            }
            if (BC == 1 || forced_bc > 0)
                return false;
        }
    };
    const int n_img = z_is_batch ? 1 : images;
    const int mtiles = P.wide ? n_img * g.OD * ohn * P.row_tiles : ((P.units + P.ipt - 1) / P.ipt) * P.tpi;
    const int gz = z_is_batch ? images : g.groups;
    // Tile width and K split: 128-wide tiles unless the problem has too few of them for the GPU, in which case narrower
    // tiles and/or a split of K spread the same MMA work over more SMs (see est_cycles).
    const int bn_max = Fg <= 32 ? 32 : (Fg <= 64 ? 64 : 128);
    const int forced_bn = force_bn > 0 ? force_bn : env_int("PETB200_TC_BN", 0);
    if (forced_bn != 0 && forced_bn != 32 && forced_bn != 64 && forced_bn != 128)
        return fail(ctx, PETB200_ERR_INVALID, "PETB200_TC_BN must be 32, 64 or 128");
    const int want_ks = force_ksplit > 0 ? force_ksplit : env_int("PETB200_TC_KSPLIT", 0);
    double best_cycles = 0;
    IgemmParams bestP{};
    bool have = false;
    for (int bn = 128; bn >= 32; bn /= 2) {
        if (forced_bn ? bn != forced_bn : bn > bn_max)
            continue;
        P.ksplit = 1;
        if (!fit(bn))
            continue;
        const long long base_ctas = (long long)mtiles * ((Fg + bn - 1) / bn) * gz;
        const int passes = core.single_pass ? 1 : 3;
        double cyc;
        const int ks = choose_ksplit(ctx->sm_count, base_ctas, P, passes, want_ks, &cyc);
        if (ks > 1) { // the landing area takes shared memory from the rings (or even from the chunk size): fit again
            P.ksplit = ks;
            if (!fit(bn))
                continue;
            if (P.nchunks < ks) {
                P.ksplit = 1;
                if (!fit(bn))
                    continue;
                cyc = est_cycles(ctx->sm_count, base_ctas, P.nchunks, P.spc, bn, passes, 1);
            }
        }
        if (!have || cyc < best_cycles * 0.97) { // prefer the wider tile unless the narrower one clearly wins
            have = true;
            best_cycles = cyc;
            bestP = P;
        }
    }
    if (!have)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "raw activation tile does not fit shared memory");
    P = bestP;
    // runs of consecutive channels (of one filter tap) per K stage, when the chunk size allows that kind of gather
    P.gruns = P.BC % kStageK == 0 ? P.ke / kStageK : (P.BC == 16 ? P.ke / 16 : (P.BC == 8 ? P.ke / 8 : 0));
    P.cstride = (P.gruns && env_int("PETB200_TC_TABLE", 0) == 0) ? P.RD * P.RH * P.RW : 0;
    choose_flush(core);
    if (flat && (!core.a_tmem || (long long)P.RN * P.BC * P.RD * P.RH * P.RW >= (1 << 24)))
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "flat raw tiles need the TS kernel variant");
    const int BN = P.BN;
    if (core.a_tmem && BN > 256)
        return fail(ctx, PETB200_ERR_INVALID, "TS variant supports BN <= 256");
    const int ntiles = (Fg + BN - 1) / BN;
    // Persistent ping-pong mode (see IgemmParams::pp) where every SM would otherwise run several CTAs in sequence: narrow
    // tiles (two accumulator regions must fit beside the A ring), no K split, no accumulator flush.
    P.mtiles = mtiles;
    P.pp = 0;
    int grid_x = mtiles;
    {
        const int slots = std::max(1, ctx->sm_count / (ntiles * gz));
        const int tiles_per_cta = (mtiles + slots - 1) / slots;
        if (core.a_tmem && env_int("PETB200_TC_PINGPONG", 1) && P.ksplit == 1 && P.fl == 0 && BN <= 64 && tiles_per_cta >= 2) {
            const int nb_was = P.NB;
            P.pp = 1;
            // (NA is 4 without a flush: two A slots per transform set)
            while (smem_layout(P, true).total > budget && P.NB > 2)
                P.NB--;
            if (smem_layout(P, true).total > budget || P.NA != 4)
                P.pp = 0, P.NB = nb_was;
            else
                grid_x = (mtiles + tiles_per_cta - 1) / tiles_per_cta;
        }
    }
    core.smem = smem_layout(P, core.a_tmem).total + 1024;
    core.y_elems = (z_is_batch ? (long long)images : (long long)n_img) * g.F * g.OD * g.OH * g.OW;
    if (z_is_batch)
        core.y_elems = (long long)images * ys_n;
    core.grid = dim3((unsigned)grid_x, (unsigned)(ntiles * P.ksplit), (unsigned)gz);
    core.Ktot = (long long)P.nchunks * P.spc * P.ke;
    core.xd[0] = g.Wst;
    core.xd[1] = g.H;
    core.xd[2] = g.D;
    core.xd[3] = g.C;
    core.xd[4] = g.N;
    // offset table for one chunk
    // Entries past the end of the chunk's K range (their packed weights are zero): -1 where the gather tests for it; in
    // plain table mode the pixel's own first element instead, so that the gather needs no test per element (the value only
    // ever meets a zero weight, and a NaN there would poison this pixel's sum anyway).
    std::vector<int> koff((size_t)P.spc * P.ke, (!flat && P.cstride == 0) ? 0 : -1);
    const int plane_w = P.RW, plane_h = P.RH * P.RW, plane_d = P.RD * plane_h;
    for (int tap = 0; tap < T; ++tap) {
        int t = tap / (g.T3[1] * g.T3[2]), r = (tap / g.T3[2]) % g.T3[1], s = tap % g.T3[2];
        for (int ci = 0; ci < P.BC; ++ci)
            koff[(size_t)tap * P.BC + ci] =
                (ci * plane_d + t * g.dil[0] * plane_h + r * g.dil[1] * plane_w + s * g.dil[2]) | (flat ? tap << 24 : 0);
    }
    if (core.koff.alloc(koff.size() * 4) != cudaSuccess)
        return fail(ctx, PETB200_ERR_NOMEM, "koff allocation failed");
    PETB200_CUDA(ctx, cudaMemcpy(core.koff.p, koff.data(), koff.size() * 4, cudaMemcpyHostToDevice));
    return raise_smem_limit(ctx);
}

// ---- exported to conv.cu -------------------------------------------------------------------------------------
struct TcConv {
    TcCore full;                 // the whole output
    ConvGeom g{};
    int has_bias = 0, act = 0;
    long long ys[3] = {0, 0, 0}; // output strides {image, filter, pixel}: {F*plane, plane, 1} (NCHW) or {F*plane, 1, F} (channels last)
    std::map<std::array<int, 4>, TcCore *> windows; // correction windows, keyed by (oh0,ohn,ow0,own)
    ~TcConv() {
        for (auto &kv : windows)
            delete kv.second;
    }
};

int tc_conv_create(petb200_ctx *ctx, int nsp, const int *in_dims, int f, const int *k, const int *pad, const int *stride,
                   const int *dil, int groups, int has_bias, int act, int passes, void **out, size_t *dev_bytes, int channels_last_out) {
    if (ctx->cc_major != 10)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "tcgen05 kernels need compute capability 10.x, device has %d.%d", ctx->cc_major, ctx->cc_minor);
    auto *t = new TcConv();
    ConvGeom &g = t->g;
    g.N = in_dims[0];
    g.C = in_dims[1];
    if (nsp == 3) {
        g.D = in_dims[2];
        g.H = in_dims[3];
        g.W = in_dims[4];
        for (int i = 0; i < 3; ++i) {
            g.T3[i] = k[i];
            g.pad[i] = pad[i];
            g.stride[i] = stride[i];
            g.dil[i] = dil[i];
        }
    } else {
        g.D = 1;
        g.H = in_dims[2];
        g.W = in_dims[3];
        g.T3[0] = 1;
        g.pad[0] = 0;
        g.stride[0] = 1;
        g.dil[0] = 1;
        for (int i = 0; i < 2; ++i) {
            g.T3[i + 1] = k[i];
            g.pad[i + 1] = pad[i];
            g.stride[i + 1] = stride[i];
            g.dil[i + 1] = dil[i];
        }
    }
    g.F = f;
    g.groups = groups;
    auto oext = [](int in, int kk, int p, int s, int d) { return (in - (kk - s) * d + 2 * p) / s; };
    g.OD = nsp == 3 ? oext(g.D, g.T3[0], g.pad[0], g.stride[0], g.dil[0]) : 1;
    g.OH = oext(g.H, g.T3[1], g.pad[1], g.stride[1], g.dil[1]);
    g.OW = oext(g.W, g.T3[2], g.pad[2], g.stride[2], g.dil[2]);
    g.Wst = g.W;
    t->has_bias = has_bias;
    t->act = act;
    t->full.ctx = ctx;
    t->full.single_pass = passes == kMathTf32x1;
    t->full.bf16 = passes == kMathBf16x3;
    const long long plane = (long long)g.OD * g.OH * g.OW;
    t->ys[0] = (long long)g.F * plane;
    t->ys[1] = channels_last_out ? 1 : plane;
    t->ys[2] = channels_last_out ? g.F : 1;
    // Rows that are not multiples of 16 bytes cannot be a TMA stride: small planes are fetched whole ("flat"), anything
    // else is re-pitched by the caller first (tc_conv_row_pitch tells it to what).
    int rc = PETB200_ERR_UNSUPPORTED;
    if (g.W % 4 != 0) {
        rc = tc_configure(ctx, t->full, g, 0, g.OH, 0, g.OW, 0, g.N, t->ys[0], t->ys[1], t->ys[2], has_bias, act, 0, 0, 0, 1);
        if (rc == PETB200_ERR_UNSUPPORTED) {
            g.Wst = (g.W + 3) / 4 * 4;
            memset(&t->full.P, 0, sizeof t->full.P);
        }
    }
    if (rc == PETB200_ERR_UNSUPPORTED)
        rc = tc_configure(ctx, t->full, g, 0, g.OH, 0, g.OW, 0, g.N, t->ys[0], t->ys[1], t->ys[2], has_bias, act);
    if (rc) {
        delete t;
        return rc;
    }
    TcCore &c = t->full;
    c.rows_b = g.F;
    size_t wbytes = (size_t)g.F * c.Ktot * (c.bf16 ? 2 : 4);
    if (c.whi.alloc(wbytes) != cudaSuccess || c.wlo.alloc(wbytes) != cudaSuccess) {
        delete t;
        return fail(ctx, PETB200_ERR_NOMEM, "packed weight allocation (%zu bytes) failed", 2 * wbytes);
    }
    rc = c.encode_b();
    if (rc) {
        delete t;
        return rc;
    }
    *dev_bytes = 2 * wbytes + c.koff.bytes;
    *out = t;
    return PETB200_OK;
}

// A stride-1, dilation-1 2-D convolution whose geometry is given explicitly instead of derived: signed padding (a negative
// value crops; whatever falls outside the input reads as zero on every side, so bottom/right padding is whatever the
// output extent asks for), an output window of ohn x own pixels, and free output strides {image, filter, row, pixel}
// with row = ow_nominal * pixel.  Used by the transposed convolution, whose sh*sw phases are such convolutions writing
// every sh-th row and sw-th column of a channels-last tensor.
int tc_conv_create_view(petb200_ctx *ctx, int n, int c, int h, int w, int f, int r, int s, int pad_h, int pad_w, int ohn, int own,
                        int ow_nominal, long long ys_n, long long ys_f, long long ys_p, int has_bias, int act, int passes, void **out,
                        size_t *dev_bytes) {
    if (ctx->cc_major != 10)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "tcgen05 kernels need compute capability 10.x, device has %d.%d", ctx->cc_major, ctx->cc_minor);
    if (ohn <= 0 || own <= 0 || own > ow_nominal)
        return fail(ctx, PETB200_ERR_INVALID, "conv view: empty or oversized window");
    auto *t = new TcConv();
    ConvGeom &g = t->g;
    g.N = n, g.C = c, g.D = 1, g.H = h, g.W = w, g.Wst = w, g.F = f, g.groups = 1;
    g.T3[0] = 1, g.T3[1] = r, g.T3[2] = s;
    g.pad[0] = 0, g.pad[1] = pad_h, g.pad[2] = pad_w;
    for (int i = 0; i < 3; ++i)
        g.stride[i] = 1, g.dil[i] = 1;
    g.OD = 1, g.OH = ohn, g.OW = ow_nominal;
    t->has_bias = has_bias;
    t->act = act;
    t->full.ctx = ctx;
    t->full.single_pass = passes == kMathTf32x1;
    t->full.bf16 = passes == kMathBf16x3;
    t->ys[0] = ys_n, t->ys[1] = ys_f, t->ys[2] = ys_p;
    int rc = PETB200_ERR_UNSUPPORTED;
    if (w % 4 != 0)
        rc = tc_configure(ctx, t->full, g, 0, ohn, 0, own, 0, n, ys_n, ys_f, ys_p, has_bias, act, 0, 0, 0, 1);
    else
        rc = tc_configure(ctx, t->full, g, 0, ohn, 0, own, 0, n, ys_n, ys_f, ys_p, has_bias, act);
    if (rc) {
        delete t;
        return rc;
    }
    TcCore &core = t->full;
    core.rows_b = f;
    const size_t wbytes = (size_t)f * core.Ktot * (core.bf16 ? 2 : 4);
    if (core.whi.alloc(wbytes) != cudaSuccess || core.wlo.alloc(wbytes) != cudaSuccess) {
        delete t;
        return fail(ctx, PETB200_ERR_NOMEM, "packed weight allocation (%zu bytes) failed", 2 * wbytes);
    }
    rc = core.encode_b();
    if (rc) {
        delete t;
        return rc;
    }
    *dev_bytes = 2 * wbytes + core.koff.bytes;
    *out = t;
    return PETB200_OK;
}

void tc_conv_destroy(void *h) { delete (TcConv *)h; }

int tc_conv_set_weights(void *h, const float *w, cudaStream_t s) {
    auto *t = (TcConv *)h;
    TcCore &c = t->full;
    const int cpg = t->g.C / t->g.groups, T = t->g.T3[0] * t->g.T3[1] * t->g.T3[2];
    long long total = (long long)t->g.F * c.Ktot;
    int blocks = (int)std::min<long long>((total + 255) / 256, (long long)c.ctx->sm_count * 16);
    if (c.bf16)
        k_pack_conv_w<true><<<blocks, 256, 0, s>>>(w, c.whi.p, c.wlo.p, t->g.F, cpg, T, c.P.BC, c.P.spc * c.P.ke, c.P.nchunks, 0);
    else
        k_pack_conv_w<false><<<blocks, 256, 0, s>>>(w, c.whi.p, c.wlo.p, t->g.F, cpg, T, c.P.BC, c.P.spc * c.P.ke, c.P.nchunks,
                                                    c.single_pass);
    c.weights_ready = true;
    return launched(c.ctx, "k_pack_conv_w");
}

int tc_conv_run(void *h, const float *x, const float *bias, const float *res, float *y, const int *win, cudaStream_t s) {
    auto *t = (TcConv *)h;
    if (!t->full.weights_ready)
        return fail(t->full.ctx, PETB200_ERR_INVALID, "conv run before set_weights");
    if (!win)
        return t->full.launch(x, bias, res, y, s);
    const ConvGeom &g = t->g;
    if (win[0] < 0 || win[1] <= 0 || win[0] + win[1] > g.OH || win[2] < 0 || win[3] <= 0 || win[2] + win[3] > g.OW)
        return fail(t->full.ctx, PETB200_ERR_INVALID, "correction window outside the output");
    const std::array<int, 4> key = {win[0], win[1], win[2], win[3]};
    TcCore *&wc = t->windows[key];
    if (!wc) {
        wc = new TcCore();
        wc->ctx = t->full.ctx;
        wc->single_pass = t->full.single_pass;
        wc->bf16 = t->full.bf16;
        // A window must consume K in exactly the order of the full operator (same BC / chunking), otherwise the
        // two would round differently; the raw box only shrinks for a window, so the full plan's BC always fits.
        int rc = tc_configure(wc->ctx, *wc, g, win[0], win[1], win[2], win[3], 0, g.N, t->ys[0], t->ys[1], t->ys[2],
                              t->has_bias, t->act, t->full.P.BC, t->full.P.ksplit, t->full.P.BN, t->full.P.flat);
        if (rc == PETB200_ERR_UNSUPPORTED) {
            // A small window packs several images into one tile, and with the full plan's chunk size forced the raw tile
            // of that many images may not fit: one image per tile always does (it is the full plan's raw tile or less).
            memset(&wc->P, 0, sizeof wc->P);
            rc = tc_configure(wc->ctx, *wc, g, win[0], win[1], win[2], win[3], 0, g.N, t->ys[0], t->ys[1], t->ys[2], t->has_bias,
                              t->act, t->full.P.BC, t->full.P.ksplit, t->full.P.BN, t->full.P.flat, std::max(1, t->full.P.ipt));
        }
        if (rc == PETB200_OK && (wc->P.BN != t->full.P.BN || wc->P.BC != t->full.P.BC || wc->Ktot != t->full.Ktot || wc->P.ksplit != t->full.P.ksplit))
            rc = fail(wc->ctx, PETB200_ERR_UNSUPPORTED, "window plan diverged from the full plan");
        if (rc) {
            delete wc;
            t->windows.erase(key);
            return rc;
        }
        wc->map_bhi = t->full.map_bhi;
        wc->map_blo = t->full.map_blo;
        wc->weights_ready = true;
    }
    return wc->launch(x, bias, res, y, s);
}

void tc_conv_out_dims(void *h, int *d5) {
    auto *t = (TcConv *)h;
    d5[0] = t->g.N;
    d5[1] = t->g.F;
    d5[2] = t->g.OD;
    d5[3] = t->g.OH;
    d5[4] = t->g.OW;
}
void tc_conv_set_prof(void *h, long long *p) { ((TcConv *)h)->full.prof = p; }
void tc_conv_set_starve(void *h, int on) { ((TcConv *)h)->full.starve = on; }
int tc_set_wait_limit_ns(unsigned long long ns) {
    return cudaMemcpyToSymbol(ptx::g_mbar_wait_limit_ns, &ns, sizeof ns) == cudaSuccess ? PETB200_OK : PETB200_ERR_CUDA;
}
int tc_conv_row_pitch(void *h) { return ((TcConv *)h)->g.Wst; }
const char *tc_conv_variant(void *h) {
    const TcCore &c = ((TcConv *)h)->full;
    return c.single_pass ? "tc_1xtf32_ts" : (c.bf16 ? "tc_bf16x3_ts" : (c.a_tmem ? "tc_3xtf32_ts" : "tc_3xtf32_ss"));
}

// ---- matmul on the same kernel ------------------------------------------------------------------------------
// C[b,m,n] = A·B with A supplied as [b,k,m] (i.e. transA): a 1x1 "convolution" whose image is one batch entry,
// channels = k, width = m; B is packed per call (or once, for weights) into hi/lo [b*n][Kpad].
struct TcMatmul {
    // element strides {A batch, A row, B batch, B row (of the stored matrix), C batch, C row}; innermost dims contiguous
    long long st[6] = {0, 0, 0, 0, 0, 0};
    TcCore core;
    int bs, m, n, k, transB;
    bool native_a = false; // A is consumed row-major as passed (no re-layout)
};

// Row-major A ([b][m][k], k % 4 == 0): the kernel's K-major mode, no re-layout of A.
static int tc_configure_kmajor(petb200_ctx *ctx, TcCore &core, int bs, int m, int n, int k, int has_bias, int act,
                               const long long *st) {
    IgemmParams &P = core.P;
    memset(&P, 0, sizeof P);
    core.a_tmem = true;
    P.a_kmajor = 1;
    P.ke = core.bf16 ? 64 : kStageK;
    P.m_rows = m;
    P.z_is_batch = 1;
    P.OD = P.OH = 1, P.OW = m, P.ohn = 1, P.own = m, P.Pw = m, P.units = 1, P.ipt = 1, P.tpi = (m + kTileM - 1) / kTileM;
    P.sd = P.sh = P.sw = 1;
    P.cpg = k, P.Fg = n;
    P.BC = P.ke, P.spc = 1, P.nchunks = (k + P.ke - 1) / P.ke;
    P.RN = P.RD = 1, P.RH = kTileM, P.RW = kStageK;
    P.raw_bytes = kAHalfBytes * (P.ke / kStageK); // one [128][32] fp32 tile per 32 K elements of a stage
    P.ys_n = st[4], P.ys_f = 1, P.ys_p = st[5];
    core.a_batch = st[0], core.a_row = st[1];
    P.has_bias = has_bias, P.act = act;
    P.NA = 4;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 1024;
    P.NB = 2, P.NR = 2;
    // tile width and K split by the cycle model (before the rings are sized: a split takes shared memory)
    {
        const int bn_max = n <= 32 ? 32 : (n <= 64 ? 64 : 128), forced_bn = env_int("PETB200_TC_BN", 0);
        double best = 0;
        int best_bn = 0, best_ks = 1;
        for (int bn = 128; bn >= 32; bn /= 2) {
            if (forced_bn ? bn != forced_bn : bn > bn_max)
                continue;
            P.BN = bn;
            double cyc;
            const int ks = choose_ksplit(ctx->sm_count, (long long)P.tpi * ((n + bn - 1) / bn) * bs, P, core.single_pass ? 1 : 3,
                                         env_int("PETB200_TC_KSPLIT", 0), &cyc);
            if (!best_bn || cyc < best * 0.97)
                best = cyc, best_bn = bn, best_ks = ks;
        }
        if (!best_bn)
            return fail(ctx, PETB200_ERR_INVALID, "PETB200_TC_BN must be 32, 64 or 128");
        P.BN = best_bn;
        P.ksplit = best_ks;
    }
    if (smem_layout(P, true).total > budget)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "matmul tile does not fit shared memory");
    for (bool grew = true; grew;) { // deepen both rings alternately: every K stage needs one B tile and one raw tile
        grew = false;
        if (P.NB < kMaxNB) {
            P.NB++;
            if (smem_layout(P, true).total <= budget)
                grew = true;
            else
                P.NB--;
        }
        if (P.NR < kMaxNR) {
            P.NR++;
            if (smem_layout(P, true).total <= budget)
                grew = true;
            else
                P.NR--;
        }
    }
    choose_flush(core);
    core.smem = smem_layout(P, true).total + 1024;
    core.Ktot = (long long)P.nchunks * P.ke;
    core.xd[0] = k, core.xd[1] = m, core.xd[2] = bs;
    std::vector<int> koff(P.ke, -1); // unused in this mode; the kernel still copies one stage worth of table
    if (core.koff.alloc(koff.size() * 4) != cudaSuccess)
        return fail(ctx, PETB200_ERR_NOMEM, "koff allocation failed");
    PETB200_CUDA(ctx, cudaMemcpy(core.koff.p, koff.data(), koff.size() * 4, cudaMemcpyHostToDevice));
    core.y_elems = (long long)bs * m * n;
    core.grid = dim3((unsigned)P.tpi, (unsigned)(((n + P.BN - 1) / P.BN) * P.ksplit), (unsigned)bs);
    return raise_smem_limit(ctx);
}

int tc_matmul_create(petb200_ctx *ctx, int bs, int m, int n, int k, int transA, int transB, int has_bias, int act, int passes,
                     const long long *strides, void **out, size_t *dev_bytes) {
    const int mp = (m + 3) / 4 * 4; // row pitch of A as [b][k][mp]
    if (ctx->cc_major != 10)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "tcgen05 kernels need compute capability 10.x");
    auto *t = new TcMatmul();
    t->bs = bs;
    t->m = m;
    t->n = n;
    t->k = k;
    t->transB = transB;
    t->core.ctx = ctx;
    t->core.single_pass = passes == kMathTf32x1;
    t->core.bf16 = passes == kMathBf16x3;
    const long long dense[6] = {(long long)m * k, transA ? m : k, (long long)k * n, transB ? k : n, (long long)m * n, n};
    for (int i = 0; i < 6; ++i)
        t->st[i] = strides ? strides[i] : dense[i];
    int rc;
    if (!transA && k % 4 == 0 && t->st[0] % 4 == 0 && t->st[1] % 4 == 0 && env_int("PETB200_TC_KMAJOR", 1)) {
        rc = tc_configure_kmajor(ctx, t->core, bs, m, n, k, has_bias, act, t->st);
        t->native_a = true;
    } else if (strides) {
        delete t;
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "strided matmul operands need row-major A with k and the A strides multiples of 4");
    } else {
        ConvGeom g{};
        g.N = bs;
        g.C = k;
        g.D = 1;
        g.H = 1;
        g.W = m;
        g.Wst = mp;
        g.F = n;
        g.groups = 1;
        for (int i = 0; i < 3; ++i) {
            g.T3[i] = 1;
            g.pad[i] = 0;
            g.stride[i] = 1;
            g.dil[i] = 1;
        }
        g.OD = 1;
        g.OH = 1;
        g.OW = m;
        rc = tc_configure(ctx, t->core, g, 0, 1, 0, m, 1, bs, (long long)m * n, 1, n, has_bias, act);
    }
    if (rc) {
        delete t;
        return rc;
    }
    TcCore &c = t->core;
    c.rows_b = bs * n;
    // rows of different batch entries are adjacent: Fg = n rows per z
    size_t wbytes = (size_t)bs * n * c.Ktot * (c.bf16 ? 2 : 4);
    if (c.whi.alloc(wbytes) != cudaSuccess || c.wlo.alloc(wbytes) != cudaSuccess) {
        delete t;
        return fail(ctx, PETB200_ERR_NOMEM, "packed B allocation failed");
    }
    rc = c.encode_b();
    if (rc) {
        delete t;
        return rc;
    }
    *dev_bytes = 2 * wbytes + c.koff.bytes;
    *out = t;
    return PETB200_OK;
}
// G2BMM on the tensor-core kernel (dilation 1): q [bs][n][m] is the row-major A operand, the keys k [bs][n][m] are packed like
// a matmul's B operand ([bs*n rows][K]); a CTA column (blockIdx.y) is one 64-key piece of the 2w + 128 keys a row tile can
// meet, and CTAs walk the row tiles in ping-pong mode.  `y` [bs][n][2w+1] is written by the banded epilogue.
int tc_g2bmm_create(petb200_ctx *ctx, int bs, int n, int m, int w, void **out) {
    if (ctx->cc_major != 10)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "tcgen05 kernels need compute capability 10.x");
    if (m % 4 != 0 || w <= 0)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "tensor-core g2bmm needs m divisible by 4");
    auto *t = new TcMatmul();
    t->bs = bs, t->m = n, t->n = n, t->k = m, t->transB = 1;
    t->st[2] = (long long)n * m, t->st[3] = m; // keys: batch and row strides
    t->native_a = true;
    TcCore &core = t->core;
    core.ctx = ctx;
    IgemmParams &P = core.P;
    memset(&P, 0, sizeof P);
    core.a_tmem = true;
    P.a_kmajor = 1, P.ke = kStageK, P.m_rows = n, P.z_is_batch = 1, P.band_w = w;
    P.OD = P.OH = 1, P.OW = n, P.ohn = 1, P.own = n, P.Pw = n, P.units = 1, P.ipt = 1, P.tpi = (n + kTileM - 1) / kTileM;
    P.sd = P.sh = P.sw = 1;
    P.cpg = m, P.Fg = n, P.BN = 64, P.ksplit = 1;
    P.BC = P.ke, P.spc = 1, P.nchunks = (m + P.ke - 1) / P.ke;
    P.RN = P.RD = 1, P.RH = kTileM, P.RW = kStageK, P.raw_bytes = kAHalfBytes;
    P.ys_n = (long long)n * (2 * w + 1), P.ys_f = 1, P.ys_p = 2 * w + 1;
    core.a_batch = (long long)n * m, core.a_row = m;
    P.NA = 4, P.a_col = 256, P.fl = 0, P.fl_regs = 0;
    const int key_tiles = (2 * w + kTileM + P.BN - 1) / P.BN;
    P.pp = 1, P.band_nt = key_tiles, P.mtiles = P.tpi * key_tiles;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 1024;
    P.NB = 2, P.NR = 2;
    if (smem_layout(P, true).total > budget) {
        delete t;
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "g2bmm tile does not fit shared memory");
    }
    for (bool grew = true; grew;) {
        grew = false;
        if (P.NB < kMaxNB) {
            P.NB++;
            if (smem_layout(P, true).total <= budget)
                grew = true;
            else
                P.NB--;
        }
        if (P.NR < kMaxNR) {
            P.NR++;
            if (smem_layout(P, true).total <= budget)
                grew = true;
            else
                P.NR--;
        }
    }
    core.smem = smem_layout(P, true).total + 1024;
    core.Ktot = (long long)P.nchunks * P.ke;
    core.xd[0] = m, core.xd[1] = n, core.xd[2] = bs;
    std::vector<int> koff(P.ke, -1);
    if (core.koff.alloc(koff.size() * 4) != cudaSuccess) {
        delete t;
        return fail(ctx, PETB200_ERR_NOMEM, "koff allocation failed");
    }
    cudaMemcpy(core.koff.p, koff.data(), koff.size() * 4, cudaMemcpyHostToDevice);
    const int slots = std::max(1, ctx->sm_count / bs);
    const int tiles_per_cta = (P.mtiles + slots - 1) / slots;
    core.grid = dim3((unsigned)((P.mtiles + tiles_per_cta - 1) / tiles_per_cta), 1u, (unsigned)bs);
    core.y_elems = (long long)bs * n * (2 * w + 1);
    core.rows_b = bs * n;
    const size_t wbytes = (size_t)bs * n * core.Ktot * 4;
    int rc = raise_smem_limit(ctx);
    if (rc == PETB200_OK && (core.whi.alloc(wbytes) != cudaSuccess || core.wlo.alloc(wbytes) != cudaSuccess))
        rc = fail(ctx, PETB200_ERR_NOMEM, "packed key allocation failed");
    if (rc == PETB200_OK)
        rc = core.encode_b();
    if (rc) {
        delete t;
        return rc;
    }
    if (env_int("PETB200_TC_VERBOSE", 0))
        fprintf(stderr, "[petb200] g2bmm plan: grid %u x %u x %u, NB %d NR %d\n", core.grid.x, core.grid.y, core.grid.z, P.NB, P.NR);
    *out = t;
    return PETB200_OK;
}

// GBMML on the tensor-core kernel (dilation 1): y [bs][n][m] = band p [bs][n][2w+1] times the value rows v [bs][n][m] it points at.
// Rows are the M dimension, v's columns the filters (packed like a matmul's B operand with the keys as K), and the K range
// of a row tile is the key window [128*tile - w, 128*tile + 127 + w]; the transform threads read the band from global memory.
int tc_gbmml_create(petb200_ctx *ctx, int bs, int n, int m, int w, void **out) {
    if (ctx->cc_major != 10)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "tcgen05 kernels need compute capability 10.x");
    if (m % 4 != 0 || m > 128 || w <= 0)
        return fail(ctx, PETB200_ERR_UNSUPPORTED, "tensor-core gbmml needs m divisible by 4 and at most 128");
    auto *t = new TcMatmul();
    t->bs = bs, t->m = n, t->n = m, t->k = n, t->transB = 0;
    t->st[2] = (long long)n * m, t->st[3] = m; // v: batch stride, stride of a key row
    t->native_a = true;
    TcCore &core = t->core;
    core.ctx = ctx;
    IgemmParams &P = core.P;
    memset(&P, 0, sizeof P);
    core.a_tmem = true;
    P.a_kmajor = 1, P.ke = kStageK, P.m_rows = n, P.z_is_batch = 1, P.band_w = w;
    P.OD = P.OH = 1, P.OW = n, P.ohn = 1, P.own = n, P.Pw = n, P.units = 1, P.ipt = 1, P.tpi = (n + kTileM - 1) / kTileM;
    P.sd = P.sh = P.sw = 1;
    P.cpg = n, P.Fg = m, P.BN = m <= 32 ? 32 : (m <= 64 ? 64 : 128), P.ksplit = 1;
    P.BC = P.ke, P.spc = 1, P.nchunks = (2 * w + kTileM + 3 + P.ke - 1) / P.ke; // K stages of one row tile's key window
    P.RN = P.RD = 1, P.RH = kTileM, P.RW = kStageK, P.raw_bytes = 128; // no raw tiles
    P.ys_n = (long long)n * m, P.ys_f = 1, P.ys_p = m;
    P.NA = 4, P.NB = 2, P.NR = 2;
    P.mtiles = P.tpi;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 1024;
    for (bool grew = true; grew;) {
        grew = false;
        if (P.NB < kMaxNB) {
            P.NB++;
            if (smem_layout(P, true).total <= budget)
                grew = true;
            else
                P.NB--;
        }
    }
    choose_flush(core);
    core.smem = smem_layout(P, true).total + 1024;
    core.Ktot = ((long long)n + P.ke - 1) / P.ke * P.ke; // the packed operand covers all keys; a tile reads its window of them
    core.xd[0] = kStageK, core.xd[1] = kTileM, core.xd[2] = 1; // (the activation map is not used: any valid extents)
    core.a_batch = kStageK * kTileM, core.a_row = kStageK;
    std::vector<int> koff(P.ke, -1);
    if (core.koff.alloc(koff.size() * 4) != cudaSuccess) {
        delete t;
        return fail(ctx, PETB200_ERR_NOMEM, "koff allocation failed");
    }
    cudaMemcpy(core.koff.p, koff.data(), koff.size() * 4, cudaMemcpyHostToDevice);
    core.grid = dim3((unsigned)P.tpi, (unsigned)((m + P.BN - 1) / P.BN), (unsigned)bs);
    core.y_elems = (long long)bs * n * m;
    core.rows_b = bs * m;
    const size_t wbytes = (size_t)bs * m * core.Ktot * 4;
    int rc = raise_smem_limit(ctx);
    if (rc == PETB200_OK && (core.whi.alloc(wbytes) != cudaSuccess || core.wlo.alloc(wbytes) != cudaSuccess))
        rc = fail(ctx, PETB200_ERR_NOMEM, "packed value allocation failed");
    if (rc == PETB200_OK)
        rc = core.encode_b();
    if (rc) {
        delete t;
        return rc;
    }
    *out = t;
    return PETB200_OK;
}
// runs a GBMML plan: `p` is the band, `y` the result (the values v were packed by tc_matmul_pack_b)
int tc_gbmml_run(void *h, const float *p, float *y, cudaStream_t s) {
    auto *t = (TcMatmul *)h;
    t->core.P.band_p = p;
    return t->core.launch(p, nullptr, nullptr, y, s); // (the activation map is encoded over p but never used by this mode)
}

void tc_matmul_set_prof(void *h, long long *p) { ((TcMatmul *)h)->core.prof = p; }
int tc_matmul_native_a(void *h) { return ((TcMatmul *)h)->native_a ? 1 : 0; }
void tc_matmul_destroy(void *h) { delete (TcMatmul *)h; }
int tc_matmul_pack_b(void *h, const float *b, cudaStream_t s) {
    auto *t = (TcMatmul *)h;
    TcCore &c = t->core;
    long long total = (long long)t->bs * t->n * c.Ktot;
    int blocks = (int)std::min<long long>((total + 255) / 256, (long long)c.ctx->sm_count * 16);
    if (c.bf16)
        launch_pdl(k_pack_mm_b<true>, blocks, 256, 0, s, b, c.whi.p, c.wlo.p, t->bs, t->n, t->k, (int)c.Ktot, t->transB, 0, t->st[2], t->st[3],
                   c.P.BC, c.P.spc * c.P.ke);
    else
        launch_pdl(k_pack_mm_b<false>, blocks, 256, 0, s, b, c.whi.p, c.wlo.p, t->bs, t->n, t->k, (int)c.Ktot, t->transB, c.single_pass,
                   t->st[2], t->st[3], c.P.BC, c.P.spc * c.P.ke);
    c.weights_ready = true;
    return launched(c.ctx, "k_pack_mm_b");
}
int tc_matmul_run(void *h, const float *a_t, const float *bias, const float *res, float *cmat, cudaStream_t s) {
    auto *t = (TcMatmul *)h;
    return t->core.launch(a_t, bias, res, cmat, s);
}

} // namespace petb200
