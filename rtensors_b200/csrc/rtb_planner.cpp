// Host-side view arithmetic and the stride/broadcast launch planner.  No CUDA calls in this file.
//
// The planner turns (shape, three stride vectors, offsets) into the smallest equivalent loop
// nest: size-1 dims dropped, dims with a negative output stride walked backwards (so the output
// is always written in increasing address order), dims sorted by output stride, and adjacent dims
// merged whenever every operand steps through them as one run.  The kernel then sees at most
// eight dims, the last one being the fastest-varying in output memory.
#include <algorithm>
#include <cstdarg>
#include <cstdio>

#include "rtb_internal.h"

namespace rtb {

static thread_local std::string g_error;

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
    return code;
}

int cuda_fail(cudaError_t e, const char *what) {
    return fail(e == cudaErrorMemoryAllocation ? RTB_ERR_ALLOC : RTB_ERR_CUDA, "CUDA error %d (%s) in %s", (int)e,
                cudaGetErrorString(e), what);
}

const char *last_error() { return g_error.c_str(); }

size_t dtype_size(int dtype) {
    switch (dtype) {
        case RTB_U8: case RTB_I8: case RTB_BOOL: return 1;
        case RTB_U16: case RTB_I16: return 2;
        case RTB_U32: case RTB_I32: case RTB_F32: return 4;
        case RTB_U64: case RTB_I64: case RTB_F64: return 8;
        case RTB_U128: case RTB_I128: return 16;
        default: return 0;
    }
}

namespace {

struct Dim {
    uint64_t n;
    int64_t sd, sl, sr;
};

inline int pow2_ceil(uint64_t v, int cap) {
    int p = 1;
    while ((uint64_t)p < v && p < cap) p <<= 1;
    return p;
}

}  // namespace

int make_plan(size_t es, int n_inputs, size_t rank, const size_t *shape, const ViewArg &d, const ViewArg &l,
              const ViewArg &r, rtb_plan *out) {
    std::memset(out, 0, sizeof *out);
    out->vec = es >= 16 ? 1 : (int)(16 / es);
    for (size_t k = 0; k < rank; ++k) {
        if (shape[k] == 0) {
            out->kernel = kNothing;
            return RTB_OK;
        }
    }
    int64_t bd = (int64_t)d.offset, bl = n_inputs >= 1 ? (int64_t)l.offset : 0, br = n_inputs >= 2 ? (int64_t)r.offset : 0;
    std::vector<Dim> dims;
    dims.reserve(rank);
    for (size_t k = 0; k < rank; ++k) {
        if (shape[k] == 1) continue;
        Dim x;
        x.n = shape[k];
        x.sd = d.strides[k];
        x.sl = n_inputs >= 1 ? l.strides[k] : x.sd;  // an absent operand never blocks a merge
        x.sr = n_inputs >= 2 ? r.strides[k] : x.sd;
        if (x.sd == 0) return fail(RTB_ERR_INVALID, "output stride 0 on a dim of extent %zu", shape[k]);
        if (x.sd < 0) {  // walk this dim backwards for every operand
            int64_t last = (int64_t)x.n - 1;
            bd += last * x.sd; bl += last * x.sl; br += last * x.sr;
            x.sd = -x.sd; x.sl = -x.sl; x.sr = -x.sr;
        }
        dims.push_back(x);
    }
    std::stable_sort(dims.begin(), dims.end(), [](const Dim &a, const Dim &b) { return a.sd > b.sd; });
    // merge dim k into k+1 when every operand walks (k, k+1) as one run
    std::vector<Dim> m;
    for (const Dim &x : dims) {
        if (!m.empty()) {
            Dim &p = m.back();  // p is the outer neighbour of x
            if (p.sd == x.sd * (int64_t)x.n && p.sl == x.sl * (int64_t)x.n && p.sr == x.sr * (int64_t)x.n) {
                p.n *= x.n; p.sd = x.sd; p.sl = x.sl; p.sr = x.sr;
                continue;
            }
        }
        m.push_back(x);
    }
    if (m.empty()) m.push_back(Dim{1, 1, 1, 1});
    if ((int)m.size() > kMaxPlanRank) return fail(RTB_ERR_TOO_LARGE, "collapsed rank %zu exceeds %d", m.size(), kMaxPlanRank);
    out->rank = (int)m.size();
    for (int k = 0; k < out->rank; ++k) {
        out->shape[k] = m[k].n;
        out->stride_d[k] = m[k].sd;
        out->stride_l[k] = n_inputs >= 1 ? m[k].sl : 0;
        out->stride_r[k] = n_inputs >= 2 ? m[k].sr : 0;
    }
    out->base_d = bd; out->base_l = bl; out->base_r = br;

    const int R = out->rank;
    const Dim &in = m[R - 1];
    const uint64_t vec = (uint64_t)out->vec;
    auto addr = [&](const ViewArg &v, int64_t base) { return (uint64_t)v.ptr + (uint64_t)(base * (int64_t)es); };

    if (R == 1 && in.sd == 1 && (n_inputs < 1 || in.sl == 1) && (n_inputs < 2 || in.sr == 1)) {
        // one contiguous run for every operand: flat kernel if they share their 16-byte phase
        // (then a common scalar head makes all of them vector-aligned); otherwise the row kernel
        // below runs it as a single row with per-operand access modes
        uint64_t ad = addr(d, bd) & 15u;
        bool same = (n_inputs < 1 || (addr(l, bl) & 15u) == ad) && (n_inputs < 2 || (addr(r, br) & 15u) == ad);
        if (same) {
            out->kernel = kFlatVec;
            out->mode_d = out->mode_l = out->mode_r = kContigVec;
            out->n_rows = 1;
            out->tile_x = 256; out->tile_y = 1;
            uint64_t nv = in.n / vec + 2;
            out->n_col_chunks = (nv + 1023) / 1024;
            out->grid = out->n_col_chunks;
            return RTB_OK;
        }
    }

    out->kernel = kRows;
    auto outer_ok = [&](int which) {  // every outer stride keeps rows 16-byte aligned
        for (int k = 0; k + 1 < R; ++k) {
            int64_t s = which == 0 ? m[k].sd : which == 1 ? m[k].sl : m[k].sr;
            if ((uint64_t)(s < 0 ? -s : s) % vec != 0) return false;
        }
        return true;
    };
    auto mode_of = [&](int which, const ViewArg &v, int64_t base, int64_t s) {
        if (s == 0) return (int)kBroadcast;
        if (s == 1) return (addr(v, base) % 16 == 0 && outer_ok(which)) ? (int)kContigVec : (int)kContigScalar;
        if (s == -1) return (addr(v, base + 1) % 16 == 0 && outer_ok(which)) ? (int)kRevVec : (int)kRevScalar;
        return (int)kStrided;
    };
    out->mode_d = mode_of(0, d, bd, in.sd);
    out->mode_l = n_inputs >= 1 ? mode_of(1, l, bl, in.sl) : (int)kBroadcast;
    out->mode_r = n_inputs >= 2 ? mode_of(2, r, br, in.sr) : (int)kBroadcast;

    // lean form: every operand walks the inner dim as whole aligned vectors / reversed vectors / a
    // broadcast scalar, and the output is a vector store -> the kernel instantiation without
    // per-element paths, with four 128-bit columns per thread once a row holds >= 128 vectors
    auto lean = [](int mode) { return mode == kContigVec || mode == kRevVec || mode == kBroadcast; };
    const bool fast = out->mode_d == kContigVec && (n_inputs < 1 || lean(out->mode_l)) &&
                      (n_inputs < 2 || lean(out->mode_r)) && in.n % vec == 0 && in.n < (1ull << 31);
    uint64_t inner_vecs = (in.n + vec - 1) / vec;
    out->fast = fast ? 1 : 0;
    out->ux = (fast && inner_vecs >= 128) ? 4 : 1;
    out->tile_x = pow2_ceil((inner_vecs + out->ux - 1) / out->ux, 256);
    out->tile_y = 256 / out->tile_x;
    uint64_t rows = 1;
    for (int k = 0; k + 1 < R; ++k) {
        rows *= m[k].n;
        if (rows >= (1ull << 31)) return fail(RTB_ERR_TOO_LARGE, "more than 2^31 rows in one launch");
    }
    out->n_rows = rows;
    // the launcher lets a CTA walk several row tiles, so `grid` is the upper bound (one tile per CTA)
    out->n_col_chunks = (inner_vecs + (uint64_t)out->tile_x * out->ux - 1) / ((uint64_t)out->tile_x * out->ux);
    uint64_t row_tiles = (rows + (uint64_t)out->tile_y - 1) / (uint64_t)out->tile_y;
    out->grid = row_tiles * out->n_col_chunks;
    if (out->grid >= (1ull << 31)) return fail(RTB_ERR_TOO_LARGE, "grid too large for one launch");
    return RTB_OK;
}

}  // namespace rtb

// ------------------------------------------------------------------------------------------------
// C ABI: view arithmetic
// ------------------------------------------------------------------------------------------------
namespace rtb { const char *last_error(); }

RTB_API const char *rtb_last_error_string(void) { return rtb::last_error(); }

RTB_API void rtb_meta_contiguous_strides(size_t rank, const size_t *shape, ptrdiff_t *strides) {
    ptrdiff_t run = 1;
    for (size_t k = rank; k-- > 0;) {
        strides[k] = run;
        run *= (ptrdiff_t)shape[k];
    }
}

RTB_API int rtb_meta_is_contiguous(size_t rank, const size_t *shape, const ptrdiff_t *strides) {
    size_t dense = 1;
    for (size_t k = 0; k < rank; ++k)
        if (shape[k] == 0) return 1;
    for (size_t k = rank; k-- > 0;) {
        if (shape[k] == 1) continue;
        size_t mag = strides[k] < 0 ? (size_t)0 - (size_t)strides[k] : (size_t)strides[k];
        if (mag != dense) return 0;
        dense *= shape[k];
    }
    return 1;
}

RTB_API int rtb_meta_slice(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t offset, size_t dim,
                           int has_start, size_t start_in, int has_end, size_t end_in, ptrdiff_t step,
                           size_t *out_rank, size_t *out_shape, ptrdiff_t *out_strides, size_t *out_offset) {
    if (dim >= rank) return rtb::fail(RTB_ERR_DIM, "Dimension %zu out of bounds for shape with rank %zu", dim, rank);
    if (step == 0) return rtb::fail(RTB_ERR_SHAPE, "Slice step cannot be zero");
    const ptrdiff_t extent = (ptrdiff_t)shape[dim];
    const bool fwd = step > 0;
    const ptrdiff_t first = has_start ? (ptrdiff_t)start_in : (fwd ? 0 : extent - 1);
    const ptrdiff_t stop = has_end ? (ptrdiff_t)end_in : (fwd ? extent : -1);
    const bool first_ok = first >= 0 && first < extent;
    const bool stop_ok = fwd ? (stop >= 0 && stop <= extent) : (stop >= -1 && stop < extent);
    if (!first_ok || !stop_ok)
        return rtb::fail(RTB_ERR_BOUNDS, "Slice indices out of bounds for dimension %zu with size %zu: start %td, end %td",
                         dim, shape[dim], first, stop);
    size_t count = 0;
    if (fwd ? first < stop : first > stop) {
        size_t span = (size_t)(fwd ? stop - first : first - stop) - 1;
        count = span / (size_t)(fwd ? step : -step) + 1;
    }
    // the reference clamps a negative advance to zero (core/slice.rs:229,236)
    const ptrdiff_t advance = first * strides[dim];
    *out_offset = offset + (advance > 0 ? (size_t)advance : 0);
    size_t w = 0;
    for (size_t k = 0; k < rank; ++k) {
        if (k == dim) {
            if (count == 0) continue;  // an empty range removes the dim (integer indexing `i..i`)
            out_shape[w] = count;
            out_strides[w] = strides[k] * step;
        } else {
            out_shape[w] = shape[k];
            out_strides[w] = strides[k];
        }
        ++w;
    }
    *out_rank = w;
    return RTB_OK;
}

RTB_API int rtb_meta_permute(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t ndims,
                             const size_t *dims, size_t *out_shape, ptrdiff_t *out_strides) {
    if (ndims != rank)
        return rtb::fail(RTB_ERR_DIM, "Permutation dims length %zu does not match tensor rank %zu", ndims, rank);
    for (size_t k = 0; k < rank; ++k) {
        size_t src = dims[k];
        if (src >= rank) return rtb::fail(RTB_ERR_DIM, "Permutation dim %zu is out of bounds for tensor rank %zu", src, rank);
        out_shape[k] = shape[src];
        out_strides[k] = strides[src];
    }
    return RTB_OK;
}

RTB_API int rtb_meta_unsqueeze(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t dim,
                               size_t *out_shape, ptrdiff_t *out_strides) {
    if (dim > rank) return rtb::fail(RTB_ERR_DIM, "Unsqueeze dim %zu is out of bounds for tensor rank %zu", dim, rank);
    // the new dim's stride spans the dim it is inserted before (1 when appended)
    ptrdiff_t span = dim < rank ? strides[dim] * (ptrdiff_t)shape[dim] : 1;
    for (size_t k = rank; k > dim; --k) {
        out_shape[k] = shape[k - 1];
        out_strides[k] = strides[k - 1];
    }
    out_shape[dim] = 1;
    out_strides[dim] = span;
    for (size_t k = 0; k < dim; ++k) {
        out_shape[k] = shape[k];
        out_strides[k] = strides[k];
    }
    return RTB_OK;
}

RTB_API int rtb_meta_squeeze(size_t rank, const size_t *shape, const ptrdiff_t *strides, ptrdiff_t dim,
                             size_t *out_rank, size_t *out_shape, ptrdiff_t *out_strides) {
    if (dim >= 0 && (size_t)dim >= rank)
        return rtb::fail(RTB_ERR_DIM, "Dimension %td is out of bounds for tensor with rank %zu", dim, rank);
    if (dim >= 0 && shape[dim] != 1)
        return rtb::fail(RTB_ERR_DIM, "Cannot squeeze dimension %td with size %zu", dim, shape[dim]);
    size_t w = 0;
    for (size_t k = 0; k < rank; ++k) {
        bool drop = dim >= 0 ? (size_t)dim == k : shape[k] == 1;
        if (drop) continue;
        out_shape[w] = shape[k];
        out_strides[w] = strides[k];
        ++w;
    }
    *out_rank = w;
    return RTB_OK;
}

RTB_API int rtb_broadcast_params(size_t ra, const size_t *shape_a, const ptrdiff_t *strides_a, size_t rb,
                                 const size_t *shape_b, const ptrdiff_t *strides_b, size_t *out_rank,
                                 size_t *out_shape, ptrdiff_t *out_sa, ptrdiff_t *out_sb) {
    const size_t rank = std::max(ra, rb);
    if (rank > RTB_MAX_RANK) return rtb::fail(RTB_ERR_DIM, "rank %zu exceeds %d", rank, RTB_MAX_RANK);
    // right-align: dim k of the output is dim k-(rank-ra) of a, absent dims act as extent 1 / stride 0
    for (size_t k = 0; k < rank; ++k) {
        const bool has_a = k + ra >= rank, has_b = k + rb >= rank;
        const size_t na = has_a ? shape_a[k + ra - rank] : 1, nb = has_b ? shape_b[k + rb - rank] : 1;
        const ptrdiff_t sa = has_a ? strides_a[k + ra - rank] : 0, sb = has_b ? strides_b[k + rb - rank] : 0;
        if (na != nb && na != 1 && nb != 1)
            return rtb::fail(RTB_ERR_BROADCAST, "Shapes are not broadcastable at dim %zu: %zu vs %zu", k, na, nb);
        const size_t n = na == 1 ? nb : na;
        out_shape[k] = n;
        out_sa[k] = (na == 1 && n > 1) ? 0 : sa;
        out_sb[k] = (nb == 1 && n > 1) ? 0 : sb;
    }
    *out_rank = rank;
    return RTB_OK;
}

RTB_API int rtb_meta_check_extent(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t offset,
                                  size_t buf_len) {
    __int128 lo = (__int128)offset, hi = (__int128)offset;
    for (size_t k = 0; k < rank; ++k) {
        if (shape[k] == 0) return RTB_OK;
        __int128 reach = (__int128)(shape[k] - 1) * (__int128)strides[k];
        if (reach < 0) lo += reach; else hi += reach;
    }
    if (lo < 0 || hi >= (__int128)buf_len)
        return rtb::fail(RTB_ERR_BOUNDS, "view addresses elements outside a buffer of %zu elements", buf_len);
    return RTB_OK;
}

RTB_API int rtb_plan_elementwise(int dtype, int n_inputs, size_t rank, const size_t *shape, const ptrdiff_t *sd,
                                 size_t od, uintptr_t pd, const ptrdiff_t *sl, size_t ol, uintptr_t pl,
                                 const ptrdiff_t *sr, size_t orr, uintptr_t pr, rtb_plan *out) {
    size_t es = rtb::dtype_size(dtype);
    if (!es) return rtb::fail(RTB_ERR_DTYPE, "unknown dtype %d", dtype);
    if (rank > RTB_MAX_RANK) return rtb::fail(RTB_ERR_DIM, "rank %zu exceeds %d", rank, RTB_MAX_RANK);
    rtb::ViewArg d{sd, od, pd}, l{sl, ol, pl}, r{sr, orr, pr};
    return rtb::make_plan(es, n_inputs, rank, shape, d, l, r, out);
}

RTB_API void rtb_shard_range(size_t extent, size_t parts, size_t part, size_t *begin, size_t *end) {
    if (parts == 0) parts = 1;
    size_t q = extent / parts, rem = extent % parts;
    size_t b = part * q + (part < rem ? part : rem);
    *begin = b;
    *end = b + q + (part < rem ? 1 : 0);
}

RTB_API int rtb_shard_pick_dim(size_t rank, const size_t *shape, size_t parts) {
    for (size_t k = 0; k < rank; ++k)
        if (shape[k] >= parts) return (int)k;
    return -1;
}

// This rank's slab of a broadcast binary op: the outermost output dim with extent >= parts is cut;
// an operand that is broadcast along it (stride 0) is replicated, any other operand's offset moves
// to the slab.  Returns the cut dim, or -1 when no dim is wide enough (part 0 then owns everything
// and the other parts get an empty slab on dim 0).
RTB_API int rtb_mg_slab(size_t rank, const size_t *shape, const ptrdiff_t *stride_l, size_t off_l, const ptrdiff_t *stride_r,
                        size_t off_r, size_t parts, size_t part, size_t *slab_shape, size_t *begin, size_t *end,
                        size_t *slab_off_l, size_t *slab_off_r) {
    for (size_t k = 0; k < rank; ++k) slab_shape[k] = shape[k];
    *slab_off_l = off_l;
    *slab_off_r = off_r;
    if (parts == 0) parts = 1;
    int dim = parts > 1 ? rtb_shard_pick_dim(rank, shape, parts) : -1;
    if (dim < 0) {
        *begin = 0;
        *end = rank ? shape[0] : 1;
        if (parts > 1 && part > 0) {
            *end = 0;
            if (rank) slab_shape[0] = 0;
        }
        return -1;
    }
    rtb_shard_range(shape[dim], parts, part, begin, end);
    slab_shape[dim] = *end - *begin;
    *slab_off_l = (size_t)((ptrdiff_t)off_l + (ptrdiff_t)*begin * stride_l[dim]);
    *slab_off_r = (size_t)((ptrdiff_t)off_r + (ptrdiff_t)*begin * stride_r[dim]);
    return dim;
}

// Which dim of `shape` to cut for an axis reduction over `axis`: a kept dim (outermost first) with
// extent >= parts gives every rank its own outputs and needs no exchange; only when there is none is
// the reduced dim itself cut (partial results are then combined across ranks).  -1: nothing to cut.
RTB_API int rtb_mg_pick_reduce_dim(size_t rank, const size_t *shape, size_t axis, size_t parts) {
    for (size_t k = 0; k < rank; ++k)
        if (k != axis && shape[k] >= parts) return (int)k;
    if (axis < rank && shape[axis] >= parts) return (int)axis;
    return -1;
}
