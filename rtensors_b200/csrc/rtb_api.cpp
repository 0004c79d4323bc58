// C ABI v2 (`rtb_*`) compute entry points: argument checks, planning, dispatch to the kernels.
#include <vector>

#include "rtb_internal.h"

namespace rtb {

#define RTB_DECL_EW(S) int ew_dispatch_##S(Ctx *, const EwCall &, const rtb_plan &);
RTB_DECL_EW(u8) RTB_DECL_EW(i8) RTB_DECL_EW(u16) RTB_DECL_EW(i16) RTB_DECL_EW(u32) RTB_DECL_EW(u128) RTB_DECL_EW(i32)
RTB_DECL_EW(u64) RTB_DECL_EW(i64) RTB_DECL_EW(i128) RTB_DECL_EW(f32) RTB_DECL_EW(f64) RTB_DECL_EW(boolean)

int launch_elementwise(Ctx *ctx, const EwCall &c, const rtb_plan &plan) {
    if (plan.kernel == kNothing) return RTB_OK;
    switch (c.dtype) {
        case RTB_U8: return ew_dispatch_u8(ctx, c, plan);
        case RTB_I8: return ew_dispatch_i8(ctx, c, plan);
        case RTB_U16: return ew_dispatch_u16(ctx, c, plan);
        case RTB_I16: return ew_dispatch_i16(ctx, c, plan);
        case RTB_U32: return ew_dispatch_u32(ctx, c, plan);
        case RTB_U128: return ew_dispatch_u128(ctx, c, plan);
        case RTB_I32: return ew_dispatch_i32(ctx, c, plan);
        case RTB_U64: return ew_dispatch_u64(ctx, c, plan);
        case RTB_I64: return ew_dispatch_i64(ctx, c, plan);
        case RTB_I128: return ew_dispatch_i128(ctx, c, plan);
        case RTB_F32: return ew_dispatch_f32(ctx, c, plan);
        case RTB_F64: return ew_dispatch_f64(ctx, c, plan);
        case RTB_BOOL: return ew_dispatch_boolean(ctx, c, plan);
    }
    return fail(RTB_ERR_DTYPE, "unknown dtype %d", c.dtype);
}

static int n_inputs_of(int family) { return family == kFamBinary ? 2 : family == kFamFill ? 0 : 1; }

int run_elementwise(Ctx *ctx, const EwCall &call, size_t rank, const size_t *shape, const ptrdiff_t *sd, size_t od,
                    const ptrdiff_t *sl, size_t ol, const ptrdiff_t *sr, size_t orr) {
    const size_t es = dtype_size(call.dtype);
    if (!es) return fail(RTB_ERR_DTYPE, "unknown dtype %d", call.dtype);
    const int nin = n_inputs_of(call.family);
    ViewArg d{sd, od, (uintptr_t)call.d}, l{sl, ol, (uintptr_t)call.l}, r{sr, orr, (uintptr_t)call.r};
    rtb_plan plan;
    int rc = make_plan(es, nin, rank, shape, d, l, r, &plan);
    if (rc == RTB_OK) return launch_elementwise(ctx, call, plan);
    if (rc != RTB_ERR_TOO_LARGE || rank == 0) return rc;
    // More dims (or rows) than one launch takes: peel the outermost dim on the host.
    size_t k0 = 0;
    while (k0 < rank && shape[k0] == 1) ++k0;
    if (k0 == rank) return rc;
    std::vector<size_t> sub(shape, shape + rank);
    sub[k0] = 1;
    for (size_t i = 0; i < shape[k0]; ++i) {
        int64_t dd = (int64_t)od + (int64_t)i * sd[k0];
        int64_t dl = nin >= 1 ? (int64_t)ol + (int64_t)i * sl[k0] : 0;
        int64_t dr = nin >= 2 ? (int64_t)orr + (int64_t)i * sr[k0] : 0;
        rc = run_elementwise(ctx, call, rank, sub.data(), sd, (size_t)dd, sl, (size_t)dl, sr, (size_t)dr);
        if (rc != RTB_OK) return rc;
    }
    return RTB_OK;
}

static int check_view_args(rtb_ctx *c, const void *buf, size_t rank, const size_t *shape, const ptrdiff_t *strides) {
    if (!c) return fail(RTB_ERR_INVALID, "null ctx");
    if (!buf) return fail(RTB_ERR_INVALID, "null buffer");
    if (rank > RTB_MAX_RANK) return fail(RTB_ERR_DIM, "rank %zu exceeds %d", rank, RTB_MAX_RANK);
    if (rank && (!shape || !strides)) return fail(RTB_ERR_INVALID, "null shape or strides");
    return RTB_OK;
}

}  // namespace rtb

using namespace rtb;

static inline Ctx *C(rtb_ctx *c) { return reinterpret_cast<Ctx *>(c); }

RTB_API int rtb_scalar_op(rtb_ctx *c, int dtype, int binop, void *buf, const void *value, size_t rank,
                          const size_t *shape, const ptrdiff_t *strides, size_t offset) {
    int rc = check_view_args(c, buf, rank, shape, strides);
    if (rc) return rc;
    if (!value) return fail(RTB_ERR_INVALID, "null scalar value");
    size_t es = dtype_size(dtype);
    if (!es) return fail(RTB_ERR_DTYPE, "unknown dtype %d", dtype);
    if ((rc = use_device(C(c)))) return rc;
    EwCall call{};
    call.dtype = dtype; call.family = kFamScalar; call.op = binop;
    std::memcpy(call.value, value, es);
    call.d = buf; call.l = buf; call.r = nullptr;
    return run_elementwise(C(c), call, rank, shape, strides, offset, strides, offset, nullptr, 0);
}

RTB_API int rtb_unary_op(rtb_ctx *c, int dtype, int unop, void *buf, size_t rank, const size_t *shape,
                         const ptrdiff_t *strides, size_t offset) {
    int rc = check_view_args(c, buf, rank, shape, strides);
    if (rc) return rc;
    if ((rc = use_device(C(c)))) return rc;
    EwCall call{};
    call.dtype = dtype; call.family = kFamUnary; call.op = unop;
    call.d = buf; call.l = buf; call.r = nullptr;
    return run_elementwise(C(c), call, rank, shape, strides, offset, strides, offset, nullptr, 0);
}

RTB_API int rtb_fill(rtb_ctx *c, int dtype, void *buf, const void *value, size_t rank, const size_t *shape,
                     const ptrdiff_t *strides, size_t offset) {
    int rc = check_view_args(c, buf, rank, shape, strides);
    if (rc) return rc;
    if (!value) return fail(RTB_ERR_INVALID, "null fill value");
    size_t es = dtype_size(dtype);
    if (!es) return fail(RTB_ERR_DTYPE, "unknown dtype %d", dtype);
    if ((rc = use_device(C(c)))) return rc;
    EwCall call{};
    call.dtype = dtype; call.family = kFamFill; call.op = 0;
    std::memcpy(call.value, value, es);
    call.d = buf; call.l = nullptr; call.r = nullptr;
    return run_elementwise(C(c), call, rank, shape, strides, offset, nullptr, 0, nullptr, 0);
}

RTB_API int rtb_copy_view(rtb_ctx *c, int dtype, const void *src, size_t rank, const size_t *shape,
                          const ptrdiff_t *strides, size_t offset, void *dst) {
    int rc = check_view_args(c, src, rank, shape, strides);
    if (rc) return rc;
    if (!dst) return fail(RTB_ERR_INVALID, "null destination");
    if ((rc = use_device(C(c)))) return rc;
    std::vector<ptrdiff_t> dense(rank ? rank : 1);
    rtb_meta_contiguous_strides(rank, shape, dense.data());
    EwCall call{};
    call.dtype = dtype; call.family = kFamCopy; call.op = 0;
    call.d = dst; call.l = src; call.r = nullptr;
    return run_elementwise(C(c), call, rank, shape, dense.data(), 0, strides, offset, nullptr, 0);
}

RTB_API int rtb_grad_mask(rtb_ctx *c, int dtype, int kind, const void *value, const void *src, size_t rank,
                          const size_t *shape, const ptrdiff_t *strides, size_t offset, void *dst) {
    int rc = check_view_args(c, src, rank, shape, strides);
    if (rc) return rc;
    if (!dst) return fail(RTB_ERR_INVALID, "null destination");
    if (kind < RTB_MASK_RELU || kind > RTB_MASK_RECIPROCAL) return fail(RTB_ERR_INVALID, "unknown gradient map kind %d", kind);
    if (kind == RTB_MASK_LEAKY_RELU && !value) return fail(RTB_ERR_INVALID, "the leaky_relu map needs its slope");
    const size_t es = dtype_size(dtype);
    if (es == 0) return fail(RTB_ERR_DTYPE, "unknown dtype %d", dtype);
    if ((rc = use_device(C(c)))) return rc;
    std::vector<ptrdiff_t> dense(rank ? rank : 1);
    rtb_meta_contiguous_strides(rank, shape, dense.data());
    EwCall call{};
    call.dtype = dtype; call.family = kFamCopy; call.op = kind;
    if (kind == RTB_MASK_LEAKY_RELU) std::memcpy(call.value, value, es);
    call.d = dst; call.l = src; call.r = nullptr;
    return run_elementwise(C(c), call, rank, shape, dense.data(), 0, strides, offset, nullptr, 0);
}

namespace {

// Lowest and one-past-highest byte address a view touches; false for an empty view.
bool byte_extent(const void *base, size_t es, size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t offset,
                 uintptr_t *lo, uintptr_t *hi) {
    int64_t mn = (int64_t)offset, mx = (int64_t)offset;
    for (size_t k = 0; k < rank; ++k) {
        if (shape[k] == 0) return false;
        int64_t span = (int64_t)(shape[k] - 1) * (int64_t)strides[k];
        if (span < 0) mn += span; else mx += span;
    }
    *lo = (uintptr_t)base + (uintptr_t)(mn * (int64_t)es);
    *hi = (uintptr_t)base + (uintptr_t)((mx + 1) * (int64_t)es);
    return true;
}

// Same element for every coordinate: same first address and the same stride on every dim that is walked.
bool same_walk(const void *a, const ptrdiff_t *sa, size_t oa, const void *b, const ptrdiff_t *sb, size_t ob, size_t es,
               size_t rank, const size_t *shape) {
    if ((uintptr_t)a + oa * es != (uintptr_t)b + ob * es) return false;
    for (size_t k = 0; k < rank; ++k)
        if (shape[k] > 1 && sa[k] != sb[k]) return false;
    return true;
}

// An input whose bytes intersect dst's while it walks them differently (a += a.T, v += reversed v)
// would be read while other threads overwrite it.
bool clashes(const void *in, const ptrdiff_t *si, size_t oi, const void *dst, const ptrdiff_t *sd, size_t od, size_t es,
             size_t rank, const size_t *shape) {
    uintptr_t ilo, ihi, dlo, dhi;
    if (!byte_extent(in, es, rank, shape, si, oi, &ilo, &ihi) || !byte_extent(dst, es, rank, shape, sd, od, &dlo, &dhi))
        return false;
    if (ihi <= dlo || dhi <= ilo) return false;
    return !same_walk(in, si, oi, dst, sd, od, es, rank, shape);
}

}  // namespace

RTB_API int rtb_broadcast(rtb_ctx *c, int dtype, int binop, const void *left, const ptrdiff_t *sl, size_t ol,
                          const void *right, const ptrdiff_t *sr, size_t orr, void *dst, const ptrdiff_t *sd,
                          size_t od, size_t rank, const size_t *shape) {
    if (!c) return fail(RTB_ERR_INVALID, "null ctx");
    if (!left || !right || !dst) return fail(RTB_ERR_INVALID, "null operand");
    if (rank > RTB_MAX_RANK) return fail(RTB_ERR_DIM, "rank %zu exceeds %d", rank, RTB_MAX_RANK);
    if (rank && (!shape || !sl || !sr || !sd)) return fail(RTB_ERR_INVALID, "null shape or strides");
    if (binop < RTB_ADD || binop > RTB_DIV) return fail(RTB_ERR_INVALID, "unknown binary op %d", binop);
    const size_t es = dtype_size(dtype);
    if (!es) return fail(RTB_ERR_DTYPE, "unknown dtype %d", dtype);
    int rc = use_device(C(c));
    if (rc) return rc;
    EwCall call{};
    call.dtype = dtype; call.family = kFamBinary; call.op = binop;
    call.d = dst; call.l = left; call.r = right;
    // Operands that overlap dst under a different walk are copied out first (dense, row-major), so
    // every input element is read before any output element is written.
    const bool clash_l = clashes(left, sl, ol, dst, sd, od, es, rank, shape);
    const bool clash_r = clashes(right, sr, orr, dst, sd, od, es, rank, shape);
    if (!clash_l && !clash_r) return run_elementwise(C(c), call, rank, shape, sd, od, sl, ol, sr, orr);
    size_t total = 1;
    for (size_t k = 0; k < rank; ++k) total *= shape[k];
    std::vector<ptrdiff_t> dense(rank ? rank : 1);
    rtb_meta_contiguous_strides(rank, shape, dense.data());
    void *tl = nullptr, *tr = nullptr;
    if (clash_l) {
        if ((rc = rtb_alloc(c, total * es, &tl)) == RTB_OK) rc = rtb_copy_view(c, dtype, left, rank, shape, sl, ol, tl);
        if (rc == RTB_OK) { call.l = tl; sl = dense.data(); ol = 0; }
    }
    if (rc == RTB_OK && clash_r) {
        if ((rc = rtb_alloc(c, total * es, &tr)) == RTB_OK) rc = rtb_copy_view(c, dtype, right, rank, shape, sr, orr, tr);
        if (rc == RTB_OK) { call.r = tr; sr = dense.data(); orr = 0; }
    }
    if (rc == RTB_OK) rc = run_elementwise(C(c), call, rank, shape, sd, od, sl, ol, sr, orr);
    if (tl) rtb_free(c, tl);  // stream order keeps the blocks alive until the kernels above are done
    if (tr) rtb_free(c, tr);
    return rc;
}

RTB_API int rtb_reduce_flat(rtb_ctx *c, int dtype, int redop, const void *src, size_t start, size_t len, void *dst) {
    if (!c || !src || !dst) return fail(RTB_ERR_INVALID, "null argument");
    size_t es = dtype_size(dtype);
    if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_reduce_flat(C(c), dtype, redop, (const char *)src + start * es, len, dst);
}

RTB_API int rtb_reduce_axis(rtb_ctx *c, int dtype, int redop, const void *src, size_t offset, size_t outer, size_t r,
                            size_t inner, void *dst) {
    if (!c || !src || !dst) return fail(RTB_ERR_INVALID, "null argument");
    size_t es = dtype_size(dtype);
    if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
    if (outer == 0 || inner == 0) return RTB_OK;  // no outputs: nothing to launch
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_reduce_axis(C(c), dtype, redop, (const char *)src + offset * es, outer, r, inner, dst);
}

namespace {

// Collapses dims [lo, hi) of a view into one (extent, stride) if every neighbouring pair is walked
// as one run; size-1 dims are ignored.  An empty / all-ones group collapses to (1, 0).
bool collapse_group(const size_t *shape, const ptrdiff_t *strides, size_t lo, size_t hi, size_t *n, ptrdiff_t *st) {
    size_t extent = 1;
    ptrdiff_t stride = 0;
    bool have = false;
    for (size_t k = hi; k-- > lo;) {  // innermost first
        if (shape[k] == 1) continue;
        if (!have) {
            extent = shape[k]; stride = strides[k]; have = true;
        } else {
            if (strides[k] != stride * (ptrdiff_t)extent) return false;
            extent *= shape[k];
        }
    }
    *n = extent; *st = have ? stride : 0;
    return true;
}

}  // namespace

namespace {

inline bool is_ext(int redop) { return redop >= RTB_VARIANCE && redop <= RTB_ARGMIN; }
inline bool is_arg(int redop) { return redop == RTB_ARGMAX || redop == RTB_ARGMIN; }

// flat and [outer, R, inner] launches for any reduction code
int any_flat(Ctx *ctx, int dtype, int redop, const rtb_reduce_settings *set, const void *p, size_t n, void *dst) {
    if (is_ext(redop)) return launch_reduce_ext(ctx, dtype, redop, set, p, 1, n, 1, 0, 1, dst);
    return launch_reduce_flat(ctx, dtype, redop, p, n, dst);
}
int any_axis(Ctx *ctx, int dtype, int redop, const rtb_reduce_settings *set, const void *p, size_t outer, size_t r,
             size_t inner, ptrdiff_t so, ptrdiff_t sr, void *dst) {
    if (is_ext(redop)) return launch_reduce_ext(ctx, dtype, redop, set, p, outer, r, inner, so, sr, dst);
    return launch_reduce_axis_strided(ctx, dtype, redop, p, outer, r, inner, so, sr, dst);
}

int reduce_view_impl(rtb_ctx *c, int dtype, int redop, const rtb_reduce_settings *set, const void *src, size_t rank,
                     const size_t *shape, const ptrdiff_t *strides, size_t offset, ptrdiff_t axis, void *dst) {
    if (!c || !src || !dst) return fail(RTB_ERR_INVALID, "null argument");
    if (rank > RTB_MAX_RANK) return fail(RTB_ERR_DIM, "rank %zu exceeds %d", rank, RTB_MAX_RANK);
    if (rank && (!shape || !strides)) return fail(RTB_ERR_INVALID, "null shape or strides");
    if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
    if (axis >= (ptrdiff_t)rank) return fail(RTB_ERR_DIM, "axis %td out of range for rank %zu", axis, rank);
    const size_t es = dtype_size(dtype);
    Ctx *ctx = C(c);
    int rc = use_device(ctx);
    if (rc) return rc;
    size_t total = 1;
    for (size_t k = 0; k < rank; ++k) total *= shape[k];
    const char *base = (const char *)src;

    if (axis < 0 || rank <= 1) {
        // Full reduction.  One run (possibly walked backwards: the order of a max / min does not
        // matter and sums are tree-ordered anyway) goes straight to the flat kernel; a position
        // (argmax / argmin) is only meaningful walking forwards.
        size_t n = 1; ptrdiff_t st = 0;
        if (collapse_group(shape, strides, 0, rank, &n, &st) && (n == 1 || st == 1 || (st == -1 && !is_arg(redop)))) {
            ptrdiff_t first = (ptrdiff_t)offset + (st < 0 ? (ptrdiff_t)(n - 1) * st : 0);
            return any_flat(ctx, dtype, redop, set, base + first * (ptrdiff_t)es, n, dst);
        }
    } else {
        if (total == 0) return RTB_OK;
        size_t nA = 1, nB = 1;
        ptrdiff_t sA = 0, sB = 0;
        const size_t R = shape[axis];
        const ptrdiff_t sR = strides[axis];
        const bool okA = collapse_group(shape, strides, 0, (size_t)axis, &nA, &sA);
        const bool okB = collapse_group(shape, strides, (size_t)axis + 1, rank, &nB, &sB);
        const char *p0 = base + (ptrdiff_t)offset * (ptrdiff_t)es;
        if (okA && okB) {
            // output is row-major over (A, 1, B): dst[a*nB + b]
            if (nB > 1 && sB == 1)  // B contiguous: [outer = A, R, inner = B]
                return any_axis(ctx, dtype, redop, set, p0, nA, R, nB, sA, sR, dst);
            if (nB == 1 && (sR == 1 || nA == 1 || sA != 1))  // rows of R (contiguous or strided), one per a
                return any_axis(ctx, dtype, redop, set, p0, nA, R, 1, sA, sR, dst);
            // B absent and A contiguous (a transposed matrix reduced along its strided dim): the
            // roles swap -- [outer = 1, R, inner = A], dst[a]
            if (nB == 1 && sA == 1) return any_axis(ctx, dtype, redop, set, p0, 1, R, nA, 0, sR, dst);
            // R is the contiguous dim and the dims around it walk as one strided run (a transposed
            // matrix reduced along its contiguous dim, a permuted cube ...): rows of R with a pitch,
            // one per (a, b), and dst[a * nB + b] is the row-major output
            if (nB > 1 && sR == 1 && (nA == 1 || sA == sB * (ptrdiff_t)nB))
                return any_axis(ctx, dtype, redop, set, p0, nA * nB, R, 1, sB, sR, dst);
        }
    }
    // General view: materialise it row-major (strided copy kernel), then reduce the copy -- what the
    // reference always does for a non-contiguous tensor (src/ops/reduction/mod.rs:351-360).
    if (total == 0) {
        if (axis < 0 || rank <= 1) return any_flat(ctx, dtype, redop, set, src, 0, dst);
        return RTB_OK;
    }
    void *tmp = nullptr;
    rc = rtb_alloc(c, total * es, &tmp);
    if (rc != RTB_OK) return rc;
    rc = rtb_copy_view(c, dtype, src, rank, shape, strides, offset, tmp);
    if (rc == RTB_OK) {
        if (axis < 0 || rank <= 1) {
            rc = any_flat(ctx, dtype, redop, set, tmp, total, dst);
        } else {
            size_t outer = 1, inner = 1;
            for (size_t k = 0; k < (size_t)axis; ++k) outer *= shape[k];
            for (size_t k = (size_t)axis + 1; k < rank; ++k) inner *= shape[k];
            rc = any_axis(ctx, dtype, redop, set, tmp, outer, shape[axis], inner, (ptrdiff_t)(shape[axis] * inner), (ptrdiff_t)inner, dst);
        }
    }
    rtb_free(c, tmp);  // stream order keeps the block alive until the kernels above are done
    return rc;
}

}  // namespace

RTB_API int rtb_reduce_view(rtb_ctx *c, int dtype, int redop, const void *src, size_t rank, const size_t *shape,
                            const ptrdiff_t *strides, size_t offset, ptrdiff_t axis, void *dst) {
    if (redop < RTB_SUM || redop > RTB_MEAN) return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
    return reduce_view_impl(c, dtype, redop, nullptr, src, rank, shape, strides, offset, axis, dst);
}

RTB_API int rtb_reduce_view_ex(rtb_ctx *c, int dtype, int redop, const rtb_reduce_settings *settings, const void *src,
                               size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t offset, ptrdiff_t axis,
                               void *dst) {
    if (redop < RTB_SUM || redop > RTB_ARGMIN) return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
    return reduce_view_impl(c, dtype, redop, settings, src, rank, shape, strides, offset, axis, dst);
}

RTB_API int rtb_reduce_flat_ex(rtb_ctx *c, int dtype, int redop, const rtb_reduce_settings *settings, const void *src,
                               size_t start, size_t len, void *dst) {
    if (!is_ext(redop)) return rtb_reduce_flat(c, dtype, redop, src, start, len, dst);
    if (!c || !src || !dst) return fail(RTB_ERR_INVALID, "null argument");
    if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_reduce_ext(C(c), dtype, redop, settings, (const char *)src + start * dtype_size(dtype), 1, len, 1, 0, 1, dst);
}

RTB_API int rtb_reduce_axis_ex(rtb_ctx *c, int dtype, int redop, const rtb_reduce_settings *settings, const void *src,
                               size_t offset, size_t outer, size_t r, size_t inner, void *dst) {
    if (!is_ext(redop)) return rtb_reduce_axis(c, dtype, redop, src, offset, outer, r, inner, dst);
    if (!c || !src || !dst) return fail(RTB_ERR_INVALID, "null argument");
    if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
    if (outer == 0 || inner == 0) return RTB_OK;  // no outputs: nothing to launch
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_reduce_ext(C(c), dtype, redop, settings, (const char *)src + offset * dtype_size(dtype), outer, r, inner,
                             (ptrdiff_t)(r * inner), (ptrdiff_t)inner, dst);
}

RTB_API int rtb_broadcast_reduce(rtb_ctx *c, int dtype, int binop, int redop, const void *left, const ptrdiff_t *sl,
                                 size_t ol, const void *right, const ptrdiff_t *sr, size_t orr, size_t rank,
                                 const size_t *shape, size_t axis, void *dst) {
    if (!c || !left || !right || !dst) return fail(RTB_ERR_INVALID, "null argument");
    if (rank == 0 || rank > RTB_MAX_RANK) return fail(RTB_ERR_DIM, "rank %zu not in [1,%d]", rank, RTB_MAX_RANK);
    if (!shape || !sl || !sr) return fail(RTB_ERR_INVALID, "null shape or strides");
    if (axis >= rank) return fail(RTB_ERR_DIM, "axis %zu out of range for rank %zu", axis, rank);
    if (binop < RTB_ADD || binop > RTB_DIV) return fail(RTB_ERR_INVALID, "unknown binary op %d", binop);
    if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
    const size_t es = dtype_size(dtype);
    Ctx *ctx = C(c);
    int rc = use_device(ctx);
    if (rc) return rc;
    size_t total = 1;
    for (size_t k = 0; k < rank; ++k) total *= shape[k];
    if (total == 0) return RTB_OK;
    // both operands must walk the dims before the axis, and the dims after it, as one run each
    size_t nA = 1, nB = 1, nA2 = 1, nB2 = 1;
    ptrdiff_t lA = 0, lB = 0, rA = 0, rB = 0;
    const bool ok = collapse_group(shape, sl, 0, axis, &nA, &lA) && collapse_group(shape, sr, 0, axis, &nA2, &rA) &&
                    collapse_group(shape, sl, axis + 1, rank, &nB, &lB) && collapse_group(shape, sr, axis + 1, rank, &nB2, &rB);
    if (ok) {
        const ptrdiff_t s_l[3] = {lA, sl[axis], lB}, s_r[3] = {rA, sr[axis], rB};
        std::lock_guard<std::mutex> lock(ctx->ws_mu);
        return launch_bcast_reduce(ctx, dtype, binop, redop, (const char *)left + (ptrdiff_t)ol * (ptrdiff_t)es, s_l,
                                   (const char *)right + (ptrdiff_t)orr * (ptrdiff_t)es, s_r, nA, shape[axis], nB, dst);
    }
    // views that do not collapse: materialise the broadcast result, then reduce it
    void *tmp = nullptr;
    rc = rtb_alloc(c, total * es, &tmp);
    if (rc != RTB_OK) return rc;
    std::vector<ptrdiff_t> dense(rank);
    rtb_meta_contiguous_strides(rank, shape, dense.data());
    rc = rtb_broadcast(c, dtype, binop, left, sl, ol, right, sr, orr, tmp, dense.data(), 0, rank, shape);
    if (rc == RTB_OK) {
        size_t outer = 1, inner = 1;
        for (size_t k = 0; k < axis; ++k) outer *= shape[k];
        for (size_t k = axis + 1; k < rank; ++k) inner *= shape[k];
        rc = rank == 1 ? launch_reduce_flat(ctx, dtype, redop, tmp, total, dst)
                       : launch_reduce_axis(ctx, dtype, redop, tmp, outer, shape[axis], inner, dst);
    }
    rtb_free(c, tmp);
    return rc;
}

RTB_API int rtb_l1_loss(rtb_ctx *c, int dtype, const void *a, const void *b, size_t n, int reduction, void *loss,
                        void *grad_map) {
    if (!c || !a || !b || !loss) return fail(RTB_ERR_INVALID, "null argument");
    if (reduction != 0 && reduction != 1) return fail(RTB_ERR_INVALID, "reduction must be 0 (mean) or 1 (sum)");
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_l1(C(c), dtype, a, b, n, reduction, loss, grad_map);
}

RTB_API int rtb_reduce_to_shape(rtb_ctx *c, int dtype, const void *upstream, size_t rank, const size_t *shape,
                                const ptrdiff_t *operand_strides, void *out, size_t *out_shape) {
    if (!c || !upstream || !out || !out_shape) return fail(RTB_ERR_INVALID, "null argument");
    if (rank > RTB_MAX_RANK) return fail(RTB_ERR_DIM, "rank %zu exceeds %d", rank, RTB_MAX_RANK);
    size_t es = dtype_size(dtype);
    if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "reduce_to_shape is defined for f32 and f64 only");
    Ctx *ctx = C(c);
    int rc = use_device(ctx);
    if (rc) return rc;
    std::vector<size_t> cur(shape, shape + rank);
    size_t total = 1;
    for (size_t k = 0; k < rank; ++k) total *= shape[k];
    // Runs of adjacent broadcast dims are summed in one pass each; between passes the running
    // tensor lives in allocator blocks (the reduction workspace is busy inside a pass).
    std::vector<std::pair<size_t, size_t>> runs;  // [first, last] dims with operand stride 0
    for (size_t k = 0; k < rank; ++k) {
        if (operand_strides[k] != 0) continue;
        if (!runs.empty() && runs.back().second + 1 == k) runs.back().second = k;
        else runs.emplace_back(k, k);
    }
    for (size_t k = 0; k < rank; ++k) out_shape[k] = operand_strides[k] == 0 ? 1 : shape[k];
    if (total == 0) return RTB_OK;
    if (runs.empty()) return rtb_d2d(c, out, upstream, total * es);
    const void *src = upstream;
    void *tmp[2] = {nullptr, nullptr};
    int which = 0;
    rc = RTB_OK;
    for (size_t i = 0; i < runs.size() && rc == RTB_OK; ++i) {
        size_t outer = 1, r = 1, inner = 1;
        for (size_t k = 0; k < runs[i].first; ++k) outer *= cur[k];
        for (size_t k = runs[i].first; k <= runs[i].second; ++k) r *= cur[k];
        for (size_t k = runs[i].second + 1; k < rank; ++k) inner *= cur[k];
        void *dst = out;
        if (i + 1 < runs.size()) {
            if (tmp[which]) rtb_free(c, tmp[which]);
            tmp[which] = nullptr;
            rc = rtb_alloc(c, outer * inner * es, &tmp[which]);
            if (rc != RTB_OK) break;
            dst = tmp[which];
        }
        rc = launch_reduce_axis(ctx, dtype, RTB_SUM, src, outer, r, inner, dst);
        for (size_t k = runs[i].first; k <= runs[i].second; ++k) cur[k] = 1;
        src = dst;
        which ^= 1;
    }
    for (int k = 0; k < 2; ++k)
        if (tmp[k]) rtb_free(c, tmp[k]);
    return rc;
}

RTB_API int rtb_relu_mask_f32(rtb_ctx *c, float *x, float *mask, size_t n) {
    if (!c || !x || !mask) return fail(RTB_ERR_INVALID, "null argument");
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_relu_mask(C(c), x, mask, n);
}

RTB_API int rtb_bias_relu_mask(rtb_ctx *c, int dtype, void *z, const void *bias, void *mask, size_t rows, size_t cols) {
    if (!c || !z || !bias || !mask) return fail(RTB_ERR_INVALID, "null argument");
    if (z == mask) return fail(RTB_ERR_INVALID, "the mask must not share the activations' buffer");
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_bias_relu_mask(C(c), dtype, z, bias, mask, rows, cols);
}

RTB_API int rtb_sgd_update_f32(rtb_ctx *c, float *p, const float *g, float lr, size_t n) {
    if (!c || !p || !g) return fail(RTB_ERR_INVALID, "null argument");
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_sgd(C(c), p, g, lr, n);
}

RTB_API int rtb_relu_mask_f64(rtb_ctx *c, double *x, double *mask, size_t n) {
    if (!c || !x || !mask) return fail(RTB_ERR_INVALID, "null argument");
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_relu_mask_f64(C(c), x, mask, n);
}

RTB_API int rtb_sgd_update_f64(rtb_ctx *c, double *p, const double *g, double lr, size_t n) {
    if (!c || !p || !g) return fail(RTB_ERR_INVALID, "null argument");
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_sgd_f64(C(c), p, g, lr, n);
}

RTB_API int rtb_convert(rtb_ctx *c, int src_dtype, int dst_dtype, const void *src, void *dst, size_t n) {
    if (!c) return fail(RTB_ERR_INVALID, "null context");
    if (src_dtype < 0 || src_dtype > RTB_BOOL || dst_dtype < 0 || dst_dtype > RTB_BOOL)
        return fail(RTB_ERR_DTYPE, "convert: unknown dtype");
    if (n == 0) return RTB_OK;
    if (!src || !dst) return fail(RTB_ERR_INVALID, "null argument");
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_convert(C(c), src_dtype, dst_dtype, src, dst, n);
}

RTB_API int rtb_u8_to_f32_div(rtb_ctx *c, const uint8_t *src, float *dst, float divisor, size_t n) {
    if (!c || !src || !dst) return fail(RTB_ERR_INVALID, "null argument");
    int rc = use_device(C(c));
    if (rc) return rc;
    return launch_u8_f32(C(c), src, dst, divisor, n);
}
