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
__global__ void __launch_bounds__(256) k_rowcopy_v4(const uint4 *__restrict__ in, uint4 *__restrict__ out, MapParams p) {
    // iteration space counted in uint4 units along the innermost digit; strides of outer digits are word
    // strides divisible by 4 (checked on the host).
    long long total4 = p.total >> 2;
    int inner4 = p.ext[p.nd - 1] >> 2;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total4;
         i += (long long)gridDim.x * blockDim.x) {
        long long rem = i / inner4;
        long long io = p.ibase + (long long)(i - rem * inner4) * 4;
        long long oo = p.obase + (long long)(i - rem * inner4) * 4;
#pragma unroll
        for (int d = kMaxDigits - 2; d >= 0; --d) {
            if (d < p.nd - 1) {
                long long q = rem / p.ext[d];
                int idx = (int)(rem - q * p.ext[d]);
                rem = q;
                io += idx * p.istr[d];
                oo += idx * p.ostr[d];
            }
        }
        out[oo >> 2] = __ldg(in + (io >> 2));
    }
}

__global__ void __launch_bounds__(256) k_gather(const uint32_t *__restrict__ in, uint32_t *__restrict__ out, MapParams p) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.total;
         i += (long long)gridDim.x * blockDim.x) {
        long long rem = i, io = p.ibase, oo = p.obase;
        bool inside = true;
#pragma unroll
        for (int d = kMaxDigits - 1; d >= 0; --d) {
            if (d < p.nd) {
                long long q = rem / p.ext[d];
                int idx = (int)(rem - q * p.ext[d]);
                rem = q;
                io += idx * p.istr[d];
                oo += idx * p.ostr[d];
                if (p.guarded && (idx < p.glo[d] || idx >= p.ghi[d]))
                    inside = false;
            }
        }
        out[oo] = inside ? __ldg(in + io) : 0u;
    }
}

struct TileParams {
    MapParams m;   // digits with the two tile digits REMOVED (batch digits), in the same order
    int ext_a, ext_z;           // extents of the input-contiguous digit (a) and the output-contiguous digit (z)
    long long istr_z, ostr_a;   // a has istr 1, z has ostr 1
    int ta, tz;                 // tile extents
    int tiles_a, tiles_z;
};

__global__ void __launch_bounds__(256) k_tile(const uint32_t *__restrict__ in, uint32_t *__restrict__ out, TileParams t) {
    extern __shared__ uint32_t tile[];
    const int pitch = t.ta | 1; // odd pitch: conflict-free column reads
    long long ntiles = (long long)t.tiles_a * t.tiles_z * t.m.total;
    for (long long blk = blockIdx.x; blk < ntiles; blk += gridDim.x) {
        long long rem = blk;
        int tzi = (int)(rem % t.tiles_z);
        rem /= t.tiles_z;
        int tai = (int)(rem % t.tiles_a);
        rem /= t.tiles_a;
        long long io = t.m.ibase, oo = t.m.obase;
#pragma unroll
        for (int d = kMaxDigits - 1; d >= 0; --d) {
            if (d < t.m.nd) {
                long long q = rem / t.m.ext[d];
                int idx = (int)(rem - q * t.m.ext[d]);
                rem = q;
                io += idx * t.m.istr[d];
                oo += idx * t.m.ostr[d];
            }
        }
        int a0 = tai * t.ta, z0 = tzi * t.tz;
        int na = min(t.ta, t.ext_a - a0), nz = min(t.tz, t.ext_z - z0);
        // read: a fastest (input-contiguous)
        for (int e = threadIdx.x; e < na * nz; e += blockDim.x) {
            int zz = e / na, aa = e - zz * na;
            tile[zz * pitch + aa] = __ldg(in + io + (a0 + aa) + (long long)(z0 + zz) * t.istr_z);
        }
        __syncthreads();
        // write: z fastest (output-contiguous)
        for (int e = threadIdx.x; e < na * nz; e += blockDim.x) {
            int aa = e / nz, zz = e - aa * nz;
            out[oo + (long long)(a0 + aa) * t.ostr_a + (z0 + zz)] = tile[zz * pitch + aa];
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
    MapParams mp{};
    TileParams tp{};
    int out_nd = 0;
    int out_dims[kMaxDigits * 2]{};
    long long in_words = 0, out_words = 0;
    int grid = 1;
    size_t smem = 0;
    DevBuf bin, bout; // scratch for timing only
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
        long long blocks = (m.total / 4 + 255) / 256;
        pl->grid = (int)std::min<long long>(blocks, (long long)sms * 16);
        return PETB200_OK;
    }
    // tile: output-contiguous digit z = last (ostr 1); input-contiguous digit a != z with istr 1
    int a = -1;
    if (!m.guarded && m.ostr[last] == 1 && m.istr[last] != 1)
        for (int i = 0; i < last; ++i)
            if (m.istr[i] == 1)
                a = i;
    if (a >= 0) {
        TileParams &t = pl->tp;
        t.ext_a = m.ext[a];
        t.ext_z = m.ext[last];
        t.istr_z = m.istr[last];
        t.ostr_a = m.ostr[a];
        // tile extents: up to 64 x 64 words, favouring whichever digit is short
        int ta = std::min(64, t.ext_a), tz = std::min(64, t.ext_z);
        while (ta * tz < 2048 && tz < t.ext_z && tz < 1024)
            tz = std::min(t.ext_z, tz * 2);
        while (ta * tz < 2048 && ta < t.ext_a && ta < 1024)
            ta = std::min(t.ext_a, ta * 2);
        t.ta = ta;
        t.tz = tz;
        t.tiles_a = ceil_div(t.ext_a, ta);
        t.tiles_z = ceil_div(t.ext_z, tz);
        t.m = m;
        int k = 0;
        t.m.total = 1;
        for (int i = 0; i < m.nd; ++i)
            if (i != a && i != last) {
                t.m.ext[k] = m.ext[i];
                t.m.istr[k] = m.istr[i];
                t.m.ostr[k] = m.ostr[i];
                t.m.total *= m.ext[i];
                ++k;
            }
        t.m.nd = k;
        pl->mode = 1;
        pl->kernel = "tile";
        pl->smem = (size_t)tz * (ta | 1) * 4;
        long long ntiles = (long long)t.tiles_a * t.tiles_z * t.m.total;
        pl->grid = (int)std::min<long long>(ntiles, (long long)sms * 8);
        if (pl->smem > 48 * 1024)
            return fail(ctx, PETB200_ERR_UNSUPPORTED, "tile too large");
        return PETB200_OK;
    }
    pl->mode = 2;
    pl->kernel = "gather";
    long long blocks = (m.total + 255) / 256;
    pl->grid = (int)std::min<long long>(blocks, (long long)sms * 16);
    return PETB200_OK;
}

static int layout_launch(LayoutPlan *pl, const void *in, void *out, cudaStream_t s) {
    if (pl->mp.total == 0)
        return PETB200_OK;
    if (pl->mode == 0) {
        if ((((uintptr_t)in) | ((uintptr_t)out)) & 15) { // unaligned caller buffers: fall back to the word kernel
            k_gather<<<pl->grid, 256, 0, s>>>((const uint32_t *)in, (uint32_t *)out, pl->mp);
            return launched(pl->ctx, "k_gather");
        }
        k_rowcopy_v4<<<pl->grid, 256, 0, s>>>((const uint4 *)in, (uint4 *)out, pl->mp);
        return launched(pl->ctx, "k_rowcopy_v4");
    }
    if (pl->mode == 1) {
        k_tile<<<pl->grid, 256, pl->smem, s>>>((const uint32_t *)in, (uint32_t *)out, pl->tp);
        return launched(pl->ctx, "k_tile");
    }
    k_gather<<<pl->grid, 256, 0, s>>>((const uint32_t *)in, (uint32_t *)out, pl->mp);
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
