// Elementwise engine for ONE dtype: compiled once per dtype with -DRTB_EW_DTYPE=<rtb_dtype code>.
//
// Three kernels serve every elementwise family (broadcast binary, scalar op, unary op, fill, copy):
//
//   flat_kernel       one contiguous run per operand, all operands in the same 16-byte phase.
//                     A scalar head brings the pointers to a 16-byte boundary, the body moves
//                     128-bit vectors (every thread issues all its loads before its first store),
//                     a scalar tail finishes.  HBM-bound: 2*s bytes per element in place, 3*s for
//                     a same-shape binary op.
//   rows_lean_kernel  views (after the planner collapsed them to <= 8 dims) whose inner dim every
//                     operand walks as whole aligned vectors, reversed vectors or one broadcast
//                     scalar, with rows of at least 128 vectors.  A CTA owns a tile of (rows x
//                     4 x 128-bit columns per thread) and walks up to four row tiles: the row index
//                     is decoded once per CTA with multiply-shift division and then advanced by
//                     adds, never per element; operands that do not move from row to row stay in
//                     registers.
//   rows_kernel       every other view: each operand's walk along the inner dim is one of
//                     contiguous (vector or scalar), reversed (vector load at the mirrored address
//                     + lane reversal), broadcast (one load, splat) or strided, with partial
//                     vectors at the row ends.
//
// Arithmetic follows the reference CPU backend (src/backend/cpu.rs:549-557, 632-657, 679-696;
// src/ops/base.rs:29-36; src/core/value.rs:515-548, 708-764): integers wrap, boolean + - * are
// OR XOR AND, relu is `x > 0 ? x : 0`, sign(0) = 0.  Built with --fmad=false and precise division
// so each float op is the single IEEE operation the CPU performs.
#include "rtb_internal.h"

#ifndef RTB_EW_DTYPE
#error "compile with -DRTB_EW_DTYPE=<code>"
#endif

namespace rtb {
namespace {

#if RTB_EW_DTYPE == 0
using T = uint8_t; using UT = uint8_t;
#define RTB_KIND 0 /* unsigned */
#define RTB_SUFFIX u8
#elif RTB_EW_DTYPE == 1
using T = int8_t; using UT = uint8_t;
#define RTB_KIND 1 /* signed */
#define RTB_SUFFIX i8
#elif RTB_EW_DTYPE == 2
using T = uint16_t; using UT = uint16_t;
#define RTB_KIND 0
#define RTB_SUFFIX u16
#elif RTB_EW_DTYPE == 3
using T = int16_t; using UT = uint16_t;
#define RTB_KIND 1
#define RTB_SUFFIX i16
#elif RTB_EW_DTYPE == 4
using T = uint32_t; using UT = uint32_t;
#define RTB_KIND 0
#define RTB_SUFFIX u32
#elif RTB_EW_DTYPE == 5
using T = unsigned __int128; using UT = unsigned __int128;
#define RTB_KIND 0
#define RTB_SUFFIX u128
#elif RTB_EW_DTYPE == 6
using T = int32_t; using UT = uint32_t;
#define RTB_KIND 1
#define RTB_SUFFIX i32
#elif RTB_EW_DTYPE == 7
using T = uint64_t; using UT = uint64_t;
#define RTB_KIND 0
#define RTB_SUFFIX u64
#elif RTB_EW_DTYPE == 8
using T = int64_t; using UT = uint64_t;
#define RTB_KIND 1
#define RTB_SUFFIX i64
#elif RTB_EW_DTYPE == 9
using T = __int128; using UT = unsigned __int128;
#define RTB_KIND 1
#define RTB_SUFFIX i128
#elif RTB_EW_DTYPE == 10
using T = float; using UT = float;
#define RTB_KIND 2 /* float */
#define RTB_SUFFIX f32
#elif RTB_EW_DTYPE == 11
using T = double; using UT = double;
#define RTB_KIND 2
#define RTB_SUFFIX f64
#elif RTB_EW_DTYPE == 12
using T = uint8_t; using UT = uint8_t;
#define RTB_KIND 3 /* boolean, stored as one byte 0/1 */
#define RTB_SUFFIX boolean
#else
#error "unknown dtype code"
#endif

constexpr int VEC = sizeof(T) >= 16 ? 1 : 16 / (int)sizeof(T);

union Vec {
    uint4 q;
    T e[VEC];
};

// ---- arithmetic --------------------------------------------------------------------------------
template <int OP>
__device__ __forceinline__ T bin(T a, T b) {
#if RTB_KIND == 3
    if (OP == RTB_ADD) return (T)((a != 0) | (b != 0));
    if (OP == RTB_SUB) return (T)((a != 0) ^ (b != 0));
    return (T)((a != 0) & (b != 0));
#elif RTB_KIND == 2
    if (OP == RTB_ADD) return a + b;
    if (OP == RTB_SUB) return a - b;
    if (OP == RTB_MUL) return a * b;
    return a / b;
#else
    if (OP == RTB_ADD) return (T)((UT)a + (UT)b);
    if (OP == RTB_SUB) return (T)((UT)a - (UT)b);
    if (OP == RTB_MUL) return (T)((UT)a * (UT)b);
    return b == (T)0 ? (T)0 : (T)(a / b);  // the reference panics on /0; here the result is 0
#endif
}

template <int OP>
__device__ __forceinline__ T una(T x) {
#if RTB_KIND == 2
    if (OP == RTB_NEG) return -x;
    if (OP == RTB_RELU) return x > (T)0 ? x : (T)0;
    if (OP == RTB_ABS) return sizeof(T) == 4 ? (T)fabsf((float)x) : (T)fabs((double)x);
    return x < (T)0 ? (T)-1 : (x > (T)0 ? (T)1 : (T)0);
#elif RTB_KIND == 1
    if (OP == RTB_NEG) return (T)((UT)0 - (UT)x);
    if (OP == RTB_RELU) return x > (T)0 ? x : (T)0;
    if (OP == RTB_ABS) return x < (T)0 ? (T)((UT)0 - (UT)x) : x;
    return x < (T)0 ? (T)-1 : (x > (T)0 ? (T)1 : (T)0);
#else
    if (OP == RTB_SIGN) return x > (T)0 ? (T)1 : (T)0;
    return x;  // relu / abs of an unsigned or boolean value is the value
#endif
}

// family functors: f(left, right) -> out
template <int OP> struct FBinary { __device__ __forceinline__ T operator()(T a, T b) const { return bin<OP>(a, b); } };
template <int OP> struct FScalar { T v; __device__ __forceinline__ T operator()(T a, T) const { return bin<OP>(a, v); } };
template <int OP> struct FUnary { __device__ __forceinline__ T operator()(T a, T) const { return una<OP>(a); } };
struct FFill { T v; __device__ __forceinline__ T operator()(T, T) const { return v; } };
struct FCopy { __device__ __forceinline__ T operator()(T a, T) const { return a; } };
// Gradient maps the reference builds with one host get + one host set per element
// (src/ops/unary/mod.rs:213-252): relu -> (x > 0 ? 1 : 0); abs -> (x > 0 ? 1 : -1), so 0 and NaN map
// to -1 exactly as the `if val > T::ZERO` there does.  Out of place: src view -> dense map.
struct FMaskRelu { __device__ __forceinline__ T operator()(T a, T) const { return a > (T)0 ? (T)1 : (T)0; } };
#if RTB_KIND == 1 || RTB_KIND == 2
struct FMaskAbs { __device__ __forceinline__ T operator()(T a, T) const { return a > (T)0 ? (T)1 : (T)-1; } };
#endif
// leaky_relu's map: x > 0 ? 1 : slope (src/ops/scalar/mod.rs:149-166); and the element-wise reciprocal
// 1 / x the backward of a broadcast division stores (src/ops/broadcast/div.rs:583-587)
struct FMaskLeaky { T v; __device__ __forceinline__ T operator()(T a, T) const { return a > (T)0 ? (T)1 : v; } };
#if RTB_KIND != 3
struct FRecip { __device__ __forceinline__ T operator()(T a, T) const { return bin<RTB_DIV>((T)1, a); } };
#endif

// Extended families with a run-time op code (one instantiation each; the switch is noise next to
// the transcendental it selects).  Formulas are the reference CPU backend's, not libm shortcuts
// (src/backend/cpu.rs:485-724): tanh / sinh / cosh from exp(x) and exp(-x), asinh / acosh / atanh
// from ln and sqrt, sigmoid = 1 / (1 + exp(-x)), silu = x * sigmoid(x), cube = (x*x)*x,
// log(base) = ln(x) / ln(base), log1p(base) = ln_1p(x) / ln(base), elu = x >= 0 ? x : alpha * expm1(x),
// leaky_relu = x > 0 ? x : x * slope.
#if RTB_KIND == 2
__device__ __forceinline__ T una_ext(int op, T x) {
    const T one = (T)1;
    switch (op) {
        case RTB_SIGMOID: return one / (one + exp(-x));
        case RTB_SILU: return x * (one / (one + exp(-x)));
        case RTB_TANH: { T a = exp(x), b = exp(-x); return (a - b) / (a + b); }
        case RTB_SINH: { T a = exp(x), b = exp(-x); return (a - b) / (one + one); }
        case RTB_COSH: { T a = exp(x), b = exp(-x); return (a + b) / (one + one); }
        case RTB_ASINH: return log(x + sqrt(x * x + one));
        case RTB_ACOSH: return log(x + sqrt(x * x - one));
        case RTB_ATANH: return log((one + x) / (one - x)) / (one + one);
        case RTB_SQRT: return sqrt(x);
        case RTB_RSQRT: return one / sqrt(x);
        case RTB_RECIPROCAL: return one / x;
        case RTB_SQUARE: return x * x;
        case RTB_CUBE: return x * x * x;
        case RTB_EXP: return exp(x);
        case RTB_EXPM1: return expm1(x);
        case RTB_LN: return log(x);
        case RTB_LN1P: return log1p(x);
        case RTB_SIN: return sin(x);
        case RTB_COS: return cos(x);
        case RTB_TAN: return tan(x);
        case RTB_ASIN: return asin(x);
        case RTB_ACOS: return acos(x);
        case RTB_ATAN: return atan(x);
        case RTB_FLOOR: return floor(x);
        case RTB_CEIL: return ceil(x);
        case RTB_ROUND: return round(x);  // half away from zero, as Rust's f32::round
        case RTB_TRUNC: return trunc(x);
    }
    return x;
}
struct FUnaryRt { int op; __device__ __forceinline__ T operator()(T a, T) const { return una_ext(op, a); } };
#endif

struct FScalarRt {
    int op;
    T v;
    __device__ __forceinline__ T operator()(T x, T) const {
#if RTB_KIND == 2
        if (op == RTB_LOG) return log(x) / log(v);
        if (op == RTB_LOG1P) return log1p(x) / log(v);
        if (op == RTB_ELU) return x >= (T)0 ? x : v * expm1(x);
#endif
        return x > (T)0 ? x : bin<RTB_MUL>(x, v);  // leaky_relu
    }
};

// ---- flat kernel -------------------------------------------------------------------------------
constexpr int kBlock = 256;  // row kernels

// CTA shape of the flat kernel per operand count, from a sweep on B200 over (vectors per thread,
// threads per CTA) with 2^28 f32 elements: read-modify-write 6.80 TB/s at (4, 256), 6.97 at
// (2, 1024), 7.03 at (2, 768); a + b -> c 6.98 at (4, 256), 7.18 at (1, 1024); a pure fill runs at
// 7.47 TB/s whatever the shape.  Large CTAs issue their loads together and then their stores
// together, which keeps reads and writes apart in time at the memory controller.
template <int NIN> struct FlatShape { static constexpr int kThreads = 256, kVecs = 4; };
template <> struct FlatShape<1> { static constexpr int kThreads = 768, kVecs = 2; };
template <> struct FlatShape<2> { static constexpr int kThreads = 1024, kVecs = 1; };

template <typename F, int NIN>
__global__ void __launch_bounds__(FlatShape<NIN>::kThreads) flat_kernel(T *d, const T *l, const T *r, size_t n, F f) {
    grid_dep_sync();
    constexpr int BS = FlatShape<NIN>::kThreads, U = FlatShape<NIN>::kVecs;
    // head = elements before the first 16-byte boundary of d (l and r share d's phase)
    size_t head = ((16u - (unsigned)((uintptr_t)d & 15u)) & 15u) / sizeof(T);
    if (head > n) head = n;
    const size_t nvec = (n - head) / VEC;
    const size_t tail0 = head + nvec * VEC;
    if (blockIdx.x == 0) {
        size_t t = threadIdx.x;
        if (t < head) d[t] = f(NIN >= 1 ? l[t] : T(), NIN >= 2 ? r[t] : T());
        size_t k = tail0 + t;
        if (k < n) d[k] = f(NIN >= 1 ? l[k] : T(), NIN >= 2 ? r[k] : T());
    }
    uint4 *dv = reinterpret_cast<uint4 *>(d + head);
    const uint4 *lv = reinterpret_cast<const uint4 *>(l + head);
    const uint4 *rv = reinterpret_cast<const uint4 *>(r + head);
    const size_t base = (size_t)blockIdx.x * (BS * U) + threadIdx.x;
    Vec a[U], b[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        size_t i = base + (size_t)u * BS;
        if (i < nvec) {
            if (NIN >= 1) a[u].q = lv[i];
            if (NIN >= 2) b[u].q = rv[i];
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        size_t i = base + (size_t)u * BS;
        if (i < nvec) {
            Vec o;
#pragma unroll
            for (int j = 0; j < VEC; ++j) o.e[j] = f(NIN >= 1 ? a[u].e[j] : T(), NIN >= 2 ? b[u].e[j] : T());
            dv[i] = o.q;
        }
    }
}

// ---- rows kernel -------------------------------------------------------------------------------
struct FastDiv {
    uint32_t d, m, s;
};
// valid for n < 2^31
__device__ __forceinline__ uint32_t fdiv(uint32_t n, FastDiv f) { return (__umulhi(n, f.m) + n) >> f.s; }

struct RowParams {
    int rank;         // >= 1; dims 0..rank-2 are row dims, dim rank-1 is the inner dim
    int tx_log2;      // tile_x = 1 << tx_log2 threads along the inner dim, tile_y = 256 / tile_x
    int iters;        // rows each thread walks (row loop length); a CTA covers tile_y * iters rows
    int mode_d, mode_l, mode_r;
    uint32_t n_col_chunks;
    uint32_t n_rows;
    uint32_t n_last;  // extent of the innermost row dim (dim rank-2), 1 when rank == 1
    uint64_t inner;
    FastDiv div[kMaxPlanRank - 1];
    int64_t sd[kMaxPlanRank], sl[kMaxPlanRank], sr[kMaxPlanRank];
};

// General operand walk: any mode, partial vectors allowed.
__device__ __forceinline__ void load_operand(const T *row, int mode, int64_t stride, uint64_t col, int cnt, Vec &out) {
    if (mode == kContigVec && cnt == VEC) {
        out.q = *reinterpret_cast<const uint4 *>(row + col);
    } else if (mode == kRevVec && cnt == VEC) {
        Vec t;
        t.q = *reinterpret_cast<const uint4 *>(row - (int64_t)col - (VEC - 1));
#pragma unroll
        for (int j = 0; j < VEC; ++j) out.e[j] = t.e[VEC - 1 - j];
    } else if (mode == kBroadcast) {
        T x = row[0];
#pragma unroll
        for (int j = 0; j < VEC; ++j) out.e[j] = x;
    } else {
        int64_t s = (mode == kContigVec || mode == kContigScalar) ? 1 : (mode == kRevVec || mode == kRevScalar) ? -1 : stride;
#pragma unroll
        for (int j = 0; j < VEC; ++j)
            if (j < cnt) out.e[j] = row[(int64_t)(col + j) * s];
    }
}

// Lean operand walk (whole aligned vectors, reversed vectors or a broadcast scalar).
__device__ __forceinline__ void load_operand_fast(const T *row, int mode, uint32_t col, Vec &out) {
    if (mode == kBroadcast) {
        T x = row[0];
#pragma unroll
        for (int j = 0; j < VEC; ++j) out.e[j] = x;
    } else {
        const bool rev = mode == kRevVec;
        Vec t;
        t.q = *reinterpret_cast<const uint4 *>(rev ? row - (int64_t)col - (VEC - 1) : row + col);
#pragma unroll
        for (int j = 0; j < VEC; ++j) out.e[j] = rev ? t.e[VEC - 1 - j] : t.e[j];
    }
}

// Row cursor of one thread: linear row index, its coordinate in the innermost row dim and the
// three row pointers.  Stepping to the thread's next row is a handful of adds unless the
// innermost row dim wraps; then the row index is decoded again (multiply-shift division).
template <int NIN>
struct RowCursor {
    uint32_t row, c_last;
    T *pd;
    const T *pl;
    const T *pr;
    __device__ __forceinline__ void decode(const RowParams &p, T *d, const T *l, const T *r) {
        uint32_t rem = row;
        int64_t xd = 0, xl = 0, xr = 0;
        uint32_t c = 0;
        c_last = 0;
        for (int k = p.rank - 2; k >= 0; --k) {
            if (k > 0) {
                uint32_t q = fdiv(rem, p.div[k]);
                c = rem - q * p.div[k].d;
                rem = q;
            } else {
                c = rem;
            }
            if (k == p.rank - 2) c_last = c;
            xd += (int64_t)c * p.sd[k];
            if (NIN >= 1) xl += (int64_t)c * p.sl[k];
            if (NIN >= 2) xr += (int64_t)c * p.sr[k];
        }
        pd = d + xd; pl = l + xl; pr = r + xr;
    }
    // returns true when the row pointers were recomputed from scratch
    __device__ __forceinline__ bool advance(const RowParams &p, uint32_t step, int64_t step_d, int64_t step_l,
                                            int64_t step_r, T *d, const T *l, const T *r) {
        row += step;
        c_last += step;
        if (row >= p.n_rows) return false;
        if (c_last < p.n_last) {
            pd += step_d;
            if (NIN >= 1) pl += step_l;
            if (NIN >= 2) pr += step_r;
            return false;
        }
        decode(p, d, l, r);
        return true;
    }
};

// UX = 128-bit columns per thread per row.  FAST: every operand is in a lean mode, the inner
// extent is a whole number of vectors below 2^31 and the output is a vector store.  Operands
// that do not move between consecutive rows of the thread (zero stride along the innermost row
// dim: a broadcast row or column) stay in registers until that dim wraps.
template <typename F, int NIN, bool FAST, int UX>
__global__ void __launch_bounds__(kBlock, (UX == 4 && sizeof(T) == 4) ? 4 : 1) rows_kernel(T *d, const T *l, const T *r, const __grid_constant__ RowParams p, F f) {
    grid_dep_sync();
    const uint32_t chunk = blockIdx.x % p.n_col_chunks;
    const uint32_t row_block = blockIdx.x / p.n_col_chunks;
    const uint32_t tx = threadIdx.x & ((1u << p.tx_log2) - 1u);
    const uint32_t ty = threadIdx.x >> p.tx_log2;
    const uint32_t tile_y = kBlock >> p.tx_log2;
    const int last = p.rank - 2;
    const int64_t step_d = last >= 0 ? (int64_t)tile_y * p.sd[last] : 0;
    const int64_t step_l = last >= 0 ? (int64_t)tile_y * p.sl[last] : 0;
    const int64_t step_r = last >= 0 ? (int64_t)tile_y * p.sr[last] : 0;
    const int64_t sdi = p.sd[p.rank - 1], sli = p.sl[p.rank - 1], sri = p.sr[p.rank - 1];

    uint64_t col[UX];
    int cnt[UX];
#pragma unroll
    for (int u = 0; u < UX; ++u) {
        col[u] = (((uint64_t)chunk * UX + u) * (1u << p.tx_log2) + tx) * VEC;
        cnt[u] = col[u] < p.inner ? (p.inner - col[u] < (uint64_t)VEC ? (int)(p.inner - col[u]) : VEC) : 0;
    }
    if (cnt[0] == 0) return;

    RowCursor<NIN> cur;
    const uint64_t first = (uint64_t)row_block * tile_y * (uint32_t)p.iters + ty;
    if (first >= p.n_rows) return;
    cur.row = (uint32_t)first;
    cur.decode(p, d, l, r);

    Vec a[UX], b[UX];
    bool fresh = true;
#pragma unroll 1
    for (int it = 0; it < p.iters; ++it) {
        if (NIN >= 1 && (fresh || step_l != 0)) {
#pragma unroll
            for (int u = 0; u < UX; ++u)
                if (cnt[u] > 0) {
                    if (FAST) load_operand_fast(cur.pl, p.mode_l, (uint32_t)col[u], a[u]);
                    else load_operand(cur.pl, p.mode_l, sli, col[u], cnt[u], a[u]);
                }
        }
        if (NIN >= 2 && (fresh || step_r != 0)) {
#pragma unroll
            for (int u = 0; u < UX; ++u)
                if (cnt[u] > 0) {
                    if (FAST) load_operand_fast(cur.pr, p.mode_r, (uint32_t)col[u], b[u]);
                    else load_operand(cur.pr, p.mode_r, sri, col[u], cnt[u], b[u]);
                }
        }
#pragma unroll
        for (int u = 0; u < UX; ++u) {
            if (cnt[u] == 0) continue;
            Vec o;
#pragma unroll
            for (int j = 0; j < VEC; ++j) o.e[j] = f(NIN >= 1 ? a[u].e[j] : T(), NIN >= 2 ? b[u].e[j] : T());
            if (FAST || (p.mode_d == kContigVec && cnt[u] == VEC)) {
                *reinterpret_cast<uint4 *>(cur.pd + col[u]) = o.q;
            } else {
#pragma unroll
                for (int j = 0; j < VEC; ++j)
                    if (j < cnt[u]) cur.pd[(int64_t)(col[u] + j) * sdi] = o.e[j];
            }
        }
        fresh = cur.advance(p, tile_y, step_d, step_l, step_r, d, l, r);
        if (cur.row >= p.n_rows) break;
    }
}

// Lean form of the row kernel for the FAST conditions with four columns per thread (any operand
// count; the binary broadcast path first of all).  Column offsets are 32-bit, a ragged last column
// tile costs one loop-invariant compare per column, and a broadcast operand (LB / RB) is ONE
// scalar per row that feeds the functor directly.  Counters of the general kernel on the strided /
// negative-step broadcast showed ~50 warp instructions per 512-byte store, most of them
// predicates, scalar splats and 64-bit column arithmetic; this loop needs ~8.
template <typename F, int NIN, bool LB, bool RB>
__global__ void __launch_bounds__(kBlock, sizeof(T) == 4 ? 4 : 1) rows_lean_kernel(T *d, const T *l, const T *r,
                                                                                 const __grid_constant__ RowParams p, F f) {
    grid_dep_sync();
    constexpr int UX = 4;
    const uint32_t chunk = blockIdx.x % p.n_col_chunks;
    const uint32_t row_block = blockIdx.x / p.n_col_chunks;
    const uint32_t tx = threadIdx.x & ((1u << p.tx_log2) - 1u);
    const uint32_t ty = threadIdx.x >> p.tx_log2;
    const uint32_t tile_y = kBlock >> p.tx_log2;
    const int last = p.rank - 2;
    const int64_t step_d = last >= 0 ? (int64_t)tile_y * p.sd[last] : 0;
    const int64_t step_l = last >= 0 ? (int64_t)tile_y * p.sl[last] : 0;
    const int64_t step_r = last >= 0 ? (int64_t)tile_y * p.sr[last] : 0;
    const uint32_t ustride = (uint32_t)VEC << p.tx_log2;                   // elements between a thread's columns
    const uint32_t col0 = ((chunk * UX) << p.tx_log2) * VEC + tx * VEC;     // < 2^31 (FAST)
    const bool lrev = p.mode_l == kRevVec, rrev = p.mode_r == kRevVec;
    // columns of this thread inside the row (all four except in a ragged last column tile); they
    // are a prefix, so one loop-invariant compare per column is all the predication there is
    int nu = 0;
#pragma unroll
    for (int u = 0; u < UX; ++u)
        if ((uint64_t)col0 + (uint64_t)u * ustride < p.inner) nu = u + 1;
    if (nu == 0) return;

    RowCursor<NIN> cur;
    const uint64_t first = (uint64_t)row_block * tile_y * (uint32_t)p.iters + ty;
    if (first >= p.n_rows) return;
    cur.row = (uint32_t)first;
    cur.decode(p, d, l, r);
    // column u of a forward operand sits at base + u*ustride, of a reversed one at base - u*ustride
    auto place = [&](const T *row, bool bcast, bool rev) {
        return bcast ? row : rev ? row - (int64_t)col0 - (VEC - 1) : row + col0;
    };
    auto fetch = [&](const T *q, bool rev, Vec (&v)[UX]) {
#pragma unroll
        for (int u = 0; u < UX; ++u) {
            if (u >= nu) continue;
            Vec t;
            t.q = *reinterpret_cast<const uint4 *>(rev ? q - (int64_t)(u * ustride) : q + u * ustride);
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[u].e[j] = rev ? t.e[VEC - 1 - j] : t.e[j];
        }
    };
    T *pd = cur.pd + col0;
    const T *pl = place(cur.pl, LB, lrev);
    const T *pr = place(cur.pr, RB, rrev);
    Vec a[UX], b[UX];  // unused (and removed by the compiler) for a broadcast operand
    T as = T(), bs = T();
    bool fresh = true;
#pragma unroll 1
    for (int it = 0; it < p.iters; ++it) {
        if (NIN >= 1 && (fresh || step_l != 0)) {
            if constexpr (LB) as = *pl;
            else fetch(pl, lrev, a);
        }
        if (NIN >= 2 && (fresh || step_r != 0)) {
            if constexpr (RB) bs = *pr;
            else fetch(pr, rrev, b);
        }
#pragma unroll
        for (int u = 0; u < UX; ++u) {
            if (u >= nu) continue;
            Vec o;
#pragma unroll
            for (int j = 0; j < VEC; ++j) o.e[j] = f(NIN >= 1 ? (LB ? as : a[u].e[j]) : T(), NIN >= 2 ? (RB ? bs : b[u].e[j]) : T());
            *reinterpret_cast<uint4 *>(pd + u * ustride) = o.q;
        }
        cur.row += tile_y;
        cur.c_last += tile_y;
        if (cur.row >= p.n_rows) break;
        if (cur.c_last < p.n_last) {
            pd += step_d; pl += step_l; pr += step_r;
            fresh = false;
        } else {
            cur.decode(p, d, l, r);
            pd = cur.pd + col0;
            pl = place(cur.pl, LB, lrev);
            pr = place(cur.pr, RB, rrev);
            fresh = true;
        }
    }
}

// ---- host launch -------------------------------------------------------------------------------
FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    f.d = d;
    uint32_t s = 0;
    while (s < 32 && (1ull << s) < d) ++s;
    f.s = s;
    f.m = (uint32_t)(((1ull << 32) * ((1ull << s) - d)) / d + 1);
    return f;
}

int ilog2(uint64_t v) {
    int k = 0;
    while ((1ull << k) < v) ++k;
    return k;
}

// ---- transposing tiles -----------------------------------------------------------------------------
// For a call whose output is dense along its inner dim X while an input is strided along X but dense
// along another dim Y (a transposed matrix, a permuted cube being made contiguous or added to a
// row-major tensor).  The row kernels read such an input one 4-byte element per 32-byte sector; here
// a CTA owns a tile of TrRows x 32 elements of (X, Y): the transposed input is read along Y (dense), parked in
// shared memory, and read back along X, so both sides of the tile move whole sectors.  Inputs that
// are dense or broadcast along X are read directly.
constexpr int kTrTile = 32;  // tile extent along Y (one warp of 4..16-byte loads)
// Tile extent along X.  One input (a strided copy): as many rows as keep the staging array within
// 17 KB, so that a thread has up to 16 loads in flight -- a transposed 8192 x 8192 f32 copy runs at
// 4.6 TB/s against 2.7 with 32 rows (and 1.9 on the row kernel).  Two inputs: 32 rows measured best
// (a.T + b: 3.1 TB/s against 2.3 with 128 rows and 2.6 on the row kernel).
template <int NIN> struct TrRows { static constexpr int value = NIN >= 2 ? 32 : (sizeof(T) <= 4 ? 128 : (sizeof(T) == 8 ? 64 : 32)); };

struct TrParams {
    int rank;            // collapsed rank of the plan, >= 2
    int ydim;            // the row dim the transposed input is dense along
    int stage_l, stage_r;  // read that input through shared memory
    uint32_t tiles_x, tiles_y;
    uint32_t extent[kMaxPlanRank];
    int64_t sd[kMaxPlanRank], sl[kMaxPlanRank], sr[kMaxPlanRank];
};

template <typename F, int NIN>
__global__ void __launch_bounds__(kBlock) transpose_tiles_kernel(T *d, const T *l, const T *r, const __grid_constant__ TrParams p, F f) {
    grid_dep_sync();
    constexpr int kTrRows = TrRows<NIN>::value;
    __shared__ T tile_l[kTrRows][kTrTile + 1];
    __shared__ T tile_r[NIN >= 2 ? kTrRows : 1][kTrTile + 1];
    const int X = p.rank - 1, Y = p.ydim;
    uint32_t id = blockIdx.x;
    const uint32_t bx = id % p.tiles_x; id /= p.tiles_x;
    const uint32_t by = id % p.tiles_y; id /= p.tiles_y;
    int64_t od = 0, ol = 0, orr = 0;
    for (int k = p.rank - 2; k >= 0; --k) {  // the dims other than X and Y
        if (k == Y) continue;
        const uint32_t c = id % p.extent[k];
        id /= p.extent[k];
        od += (int64_t)c * p.sd[k];
        if (NIN >= 1) ol += (int64_t)c * p.sl[k];
        if (NIN >= 2) orr += (int64_t)c * p.sr[k];
    }
    const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;  // 32 x 8 threads
    const uint32_t x0 = bx * kTrRows, y0 = by * kTrTile;
    const uint32_t nx = p.extent[X], ny = p.extent[Y];
    // Two inputs (32-row tiles): the elements this thread reads directly (lanes along X) are
    // requested first, so that they are in flight with the staged loads; left to the store loop they
    // would each wait behind the previous store
    constexpr int NJ = kTrTile / 8;
    T pre_l[NJ], pre_r[NJ];
    if (NIN >= 2) {
        const uint32_t x = x0 + tx;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const uint32_t y = y0 + ty + 8 * j;
            if (x < nx && y < ny) {
                if (!p.stage_l) pre_l[j] = l[ol + (int64_t)x * p.sl[X] + (int64_t)y * p.sl[Y]];
                if (!p.stage_r) pre_r[j] = r[orr + (int64_t)x * p.sr[X] + (int64_t)y * p.sr[Y]];
            }
        }
    }
    // stage: lanes run along Y
    if (NIN >= 1 && (p.stage_l || (NIN >= 2 && p.stage_r))) {
        const uint32_t y = y0 + tx;
#pragma unroll
        for (int j = 0; j < kTrRows / 8; ++j) {
            const uint32_t xl = ty + 8 * j, x = x0 + xl;
            if (x < nx && y < ny) {
                if (p.stage_l) tile_l[xl][tx] = l[ol + (int64_t)x * p.sl[X] + (int64_t)y * p.sl[Y]];
                if (NIN >= 2 && p.stage_r) tile_r[xl][tx] = r[orr + (int64_t)x * p.sr[X] + (int64_t)y * p.sr[Y]];
            }
        }
        __syncthreads();
    }
    // compute and store: lanes run along X
#pragma unroll
    for (int h = 0; h < kTrRows / 32; ++h) {
        const uint32_t xl = tx + 32 * h, x = x0 + xl;
        if (x >= nx) break;
#pragma unroll
        for (int j = 0; j < kTrTile / 8; ++j) {
            const uint32_t yl = ty + 8 * j, y = y0 + yl;
            if (y >= ny) break;
            T a = T(), b = T();
            if (NIN >= 2) {  // kTrRows == 32 here, so h == 0
                a = p.stage_l ? tile_l[xl][yl] : pre_l[j];
                b = p.stage_r ? tile_r[xl][yl] : pre_r[j];
            } else if (NIN >= 1) {
                a = p.stage_l ? tile_l[xl][yl] : l[ol + (int64_t)x * p.sl[X] + (int64_t)y * p.sl[Y]];
            }
            d[od + (int64_t)x * p.sd[X] + (int64_t)y * p.sd[Y]] = f(a, b);
        }
    }
}

// The same tiles with 16-byte accesses on BOTH sides, for 4- and 8-byte elements whose views are
// vector-aligned (the common case: a transposed matrix or a permuted cube of f32 / f64 / i32 / i64).
// V = elements per 16 bytes.  A CTA owns 128 (X) x 8V (Y) elements (twice that along Y for a one-input copy).  Staging: a thread loads four
// vectors of V consecutive Y-elements (8 lanes cover 128 contiguous bytes of one X-row, a warp four
// X-rows) -- all four in flight before the first shared-memory store -- and parks them element by
// element in a tile whose pitch is one element more than its width, which makes the scattered stores
// and the gathering loads below bank-conflict free.  Output: a thread gathers V consecutive
// X-elements at one Y from the tile and writes one vector (8 lanes cover 128 contiguous bytes of an
// output row).  An input that is dense along X is fetched as vectors straight into registers before
// the staging loads are issued.  Measured against the element-wise tiles above (every global access
// one element): transposed 8192 x 8192 f32 copy and a.T + b, see the kernel table of the design notes.
constexpr int kTvX = 128;
// YT = number of 8V-wide Y sub-tiles a CTA owns: 1 for two inputs, 2 for a plain strided copy (one
// input), where twice the staged vectors in flight per thread is what the kernel is short of.
template <int NIN> struct TvYT { static constexpr int value = NIN >= 2 ? 1 : 2; };
template <typename F, int NIN>
__global__ void __launch_bounds__(kBlock) transpose_vec_kernel(T *d, const T *l, const T *r, const __grid_constant__ TrParams p, F f) {
    grid_dep_sync();
    constexpr int V = 16 / (int)sizeof(T), TY = 8 * V, NY = 2 * V, YT = TvYT<NIN>::value;
    union Vec {
        uint4 q;
        T e[V];
    };
    __shared__ T tile[kTvX][YT * TY + 1];
    const int X = p.rank - 1, Y = p.ydim;
    uint32_t id = blockIdx.x;
    const uint32_t bx = id % p.tiles_x; id /= p.tiles_x;
    const uint32_t by = id % p.tiles_y; id /= p.tiles_y;
    int64_t od = 0, ol = 0, orr = 0;
    for (int k = p.rank - 2; k >= 0; --k) {  // the dims other than X and Y
        if (k == Y) continue;
        const uint32_t c = id % p.extent[k];
        id /= p.extent[k];
        od += (int64_t)c * p.sd[k];
        ol += (int64_t)c * p.sl[k];
        if (NIN >= 2) orr += (int64_t)c * p.sr[k];
    }
    const uint32_t lane = threadIdx.x & 31u, w = threadIdx.x >> 5, l8 = lane & 7u, h4 = lane >> 3;
    const uint32_t x0 = bx * kTvX, y0 = by * (YT * TY);
    const uint32_t nx = p.extent[X], ny = p.extent[Y];
    const bool staged_is_l = p.stage_l != 0;
    const T *sp = staged_is_l ? l + ol : r + orr;                     // staged input: dense along Y
    const int64_t ssx = staged_is_l ? p.sl[X] : p.sr[X];
    const T *dp = staged_is_l ? r + orr : l + ol;                     // direct input (NIN == 2): dense along X
    const int64_t dsy = staged_is_l ? p.sr[Y] : p.sl[Y];
    Vec pre[4], st[YT][4];
    if (NIN >= 2) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t q = w + 8u * j, yg = q % NY, xg = q / NY;
            const uint32_t x = x0 + 8u * V * xg + V * l8, y = y0 + 4u * yg + h4;
            if (x < nx && y < ny) pre[j].q = *reinterpret_cast<const uint4 *>(dp + (int64_t)x + (int64_t)y * dsy);
        }
    }
#pragma unroll
    for (int t = 0; t < YT; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t x = x0 + 4u * (w + 8u * j) + h4, y = y0 + t * TY + V * l8;
            if (x < nx && y < ny) st[t][j].q = *reinterpret_cast<const uint4 *>(sp + (int64_t)x * ssx + (int64_t)y);
        }
#pragma unroll
    for (int t = 0; t < YT; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t xr = 4u * (w + 8u * j) + h4;
#pragma unroll
            for (int e = 0; e < V; ++e) tile[xr][t * TY + V * l8 + e] = st[t][j].e[e];
        }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < YT; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t q = w + 8u * j, yg = q % NY, xg = q / NY;
            const uint32_t xl = 8u * V * xg + V * l8, yl = t * TY + 4u * yg + h4;
            const uint32_t x = x0 + xl, y = y0 + yl;
            if (x < nx && y < ny) {
                Vec o;
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const T a = tile[xl + i][yl];
                    if (NIN >= 2) o.e[i] = staged_is_l ? f(a, pre[j].e[i]) : f(pre[j].e[i], a);
                    else o.e[i] = f(a, T());
                }
                *reinterpret_cast<uint4 *>(d + od + (int64_t)x + (int64_t)y * p.sd[Y]) = o.q;
            }
        }
}

// Can the planned transposing call run on the vector tiles?  (fills the tile counts of `p` if so)
template <int NIN>
bool vector_tiles_ok(const T *d, const T *l, const T *r, TrParams *p) {
    if (sizeof(T) != 4 && sizeof(T) != 8) return false;
    constexpr int64_t V = 16 / (int64_t)sizeof(T);
    const int X = p->rank - 1, Y = p->ydim;
    if (NIN >= 2 && p->stage_l && p->stage_r) return false;           // one staged input only
    if (p->extent[X] % V || p->extent[Y] % V) return false;
    auto al = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (!al(d) || !al(l) || (NIN >= 2 && !al(r))) return false;
    const int64_t *ss = p->stage_l ? p->sl : p->sr, *ds = p->stage_l ? p->sr : p->sl;
    for (int k = 0; k < p->rank; ++k) {
        if (k != X && p->sd[k] % V) return false;
        if (k != Y && ss[k] % V) return false;
        if (NIN >= 2 && k != X && ds[k] % V) return false;
    }
    if (p->sd[X] != 1 || ss[Y] != 1) return false;
    if (NIN >= 2 && ds[X] != 1) return false;
    p->tiles_x = (p->extent[X] + kTvX - 1) / kTvX;
    const uint32_t tile_y = 8 * (uint32_t)V * (uint32_t)TvYT<NIN>::value;
    p->tiles_y = (p->extent[Y] + tile_y - 1) / tile_y;
    uint64_t blocks = (uint64_t)p->tiles_x * p->tiles_y;
    for (int k = 0; k < p->rank - 1; ++k)
        if (k != Y) blocks *= p->extent[k];
    return blocks < (1ull << 31);
}

// Host-side choice: returns true and fills `p` when the call should run on transposing tiles.
template <int NIN>
bool plan_transpose(const EwCall &c, const rtb_plan &plan, TrParams *p) {
    const int R = plan.rank;
    if (NIN < 1 || R < 2 || plan.stride_d[R - 1] != 1) return false;
    if (plan.shape[R - 1] < 16) return false;
    auto dense_dim = [&](const int64_t *st) {  // strided along X, dense along some row dim with room for a tile
        const int64_t sx = st[R - 1];
        if (sx == 0 || sx == 1 || sx == -1) return -1;
        for (int k = R - 2; k >= 0; --k)
            if (st[k] == 1 && plan.shape[k] >= 16) return k;
        return -1;
    };
    const int yl = dense_dim(plan.stride_l), yr = NIN >= 2 ? dense_dim(plan.stride_r) : -1;
    // an input that shares the output's buffer is read where it is written only if it is not staged
    if (yl >= 0 && c.l == c.d) return false;
    if (yr >= 0 && c.r == c.d) return false;
    const int y = yl >= 0 ? yl : yr;
    if (y < 0) return false;
    std::memset(p, 0, sizeof *p);
    p->rank = R;
    p->ydim = y;
    p->stage_l = yl == y;
    p->stage_r = yr == y;
    uint64_t blocks = 1;
    for (int k = 0; k < R; ++k) {
        if (plan.shape[k] >= (1ull << 32)) return false;
        p->extent[k] = (uint32_t)plan.shape[k];
        p->sd[k] = plan.stride_d[k]; p->sl[k] = plan.stride_l[k]; p->sr[k] = plan.stride_r[k];
        if (k != y && k != R - 1) blocks *= plan.shape[k];
    }
    p->tiles_x = (uint32_t)((plan.shape[R - 1] + TrRows<NIN>::value - 1) / TrRows<NIN>::value);
    p->tiles_y = (uint32_t)((plan.shape[y] + kTrTile - 1) / kTrTile);
    blocks *= (uint64_t)p->tiles_x * p->tiles_y;
    return blocks < (1ull << 31);
}

template <typename F, int NIN>
int launch(Ctx *ctx, const EwCall &c, const rtb_plan &plan, F f) {
    T *d = reinterpret_cast<T *>(c.d) + plan.base_d;
    const T *l = NIN >= 1 ? reinterpret_cast<const T *>(c.l) + plan.base_l : reinterpret_cast<const T *>(d);
    const T *r = NIN >= 2 ? reinterpret_cast<const T *>(c.r) + plan.base_r : reinterpret_cast<const T *>(d);
    if (plan.kernel == kFlatVec) {
        size_t n = (size_t)plan.shape[0];
        size_t nvec = n / VEC + 1;
        constexpr size_t per_cta = (size_t)FlatShape<NIN>::kThreads * FlatShape<NIN>::kVecs;
        size_t blocks = (nvec + per_cta - 1) / per_cta;
        if (blocks >= (size_t(1) << 31)) return fail(RTB_ERR_TOO_LARGE, "flat launch too large");
        launch_dep(ctx, (unsigned)blocks, FlatShape<NIN>::kThreads, flat_kernel<F, NIN>, d, l, r, n, f);
        return check_launch(ctx, "flat_kernel");
    }
    if constexpr (NIN >= 1) {
        TrParams tp;
        if (plan_transpose<NIN>(c, plan, &tp)) {
            TrParams tv = tp;
            const bool vec = vector_tiles_ok<NIN>(d, l, r, &tv);
            const TrParams &use = vec ? tv : tp;
            uint64_t blocks = (uint64_t)use.tiles_x * use.tiles_y;
            for (int k = 0; k < use.rank - 1; ++k)
                if (k != use.ydim) blocks *= use.extent[k];
            if (vec) {
                if constexpr (sizeof(T) == 4 || sizeof(T) == 8) {
                    launch_dep(ctx, (unsigned)blocks, kBlock, transpose_vec_kernel<F, NIN>, d, l, r, tv, f);
                    return check_launch(ctx, "transpose_vec_kernel");
                }
            }
            launch_dep(ctx, (unsigned)blocks, kBlock, transpose_tiles_kernel<F, NIN>, d, l, r, tp, f);
            return check_launch(ctx, "transpose_tiles_kernel");
        }
    }
    RowParams p;
    std::memset(&p, 0, sizeof p);
    p.rank = plan.rank;
    p.tx_log2 = ilog2((uint64_t)plan.tile_x);
    const int R = plan.rank;
    p.mode_d = plan.mode_d; p.mode_l = plan.mode_l; p.mode_r = plan.mode_r;
    p.n_rows = (uint32_t)plan.n_rows;
    p.n_last = R >= 2 ? (uint32_t)plan.shape[R - 2] : 1u;
    p.inner = plan.shape[R - 1];
    for (int k = 0; k < R; ++k) {
        p.sd[k] = plan.stride_d[k]; p.sl[k] = plan.stride_l[k]; p.sr[k] = plan.stride_r[k];
        if (k < R - 1) p.div[k] = make_fastdiv((uint32_t)plan.shape[k]);
    }
    const bool fast = plan.fast != 0;
    const int ux = plan.ux;
    const uint64_t chunks = plan.n_col_chunks;
    p.n_col_chunks = (uint32_t)chunks;
    // A CTA walks `iters` consecutive row tiles, so the row decode and any broadcast operand held in
    // registers are paid once per CTA.  Small CTAs balance better than long loops: measured on B200
    // with the (16,64,1024,1024) strided / negative-step broadcast add, at most 1 / 2 / 3 / 4 / 8 / 64
    // tiles per CTA give 5.26 / 6.84 / 7.43 / 7.41 / 7.29 / 6.84 TB/s.  So: up to 4 tiles, fewer when
    // that would leave under 8 CTAs per SM.
    const uint64_t row_tiles = (plan.n_rows + (uint64_t)plan.tile_y - 1) / (uint64_t)plan.tile_y;
    uint64_t iters = (row_tiles * chunks) / ((uint64_t)ctx->sm_count * 8);
    if (iters < 1) iters = 1;
    if (iters > 4) iters = 4;
    p.iters = (int)iters;
    const uint64_t grid = ((row_tiles + iters - 1) / iters) * chunks;
    if (grid >= (1ull << 31)) return fail(RTB_ERR_TOO_LARGE, "grid too large for one launch");
    if (fast && ux == 4) {
        const bool lb = NIN >= 1 && plan.mode_l == kBroadcast, rb = NIN >= 2 && plan.mode_r == kBroadcast;
        const unsigned g = (unsigned)grid;
        if constexpr (NIN == 2) {
            if (lb && rb) launch_dep(ctx, g, kBlock, rows_lean_kernel<F, 2, true, true>, d, l, r, p, f);
            else if (lb) launch_dep(ctx, g, kBlock, rows_lean_kernel<F, 2, true, false>, d, l, r, p, f);
            else if (rb) launch_dep(ctx, g, kBlock, rows_lean_kernel<F, 2, false, true>, d, l, r, p, f);
            else launch_dep(ctx, g, kBlock, rows_lean_kernel<F, 2, false, false>, d, l, r, p, f);
        } else if constexpr (NIN == 1) {
            if (lb) launch_dep(ctx, g, kBlock, rows_lean_kernel<F, 1, true, false>, d, l, r, p, f);
            else launch_dep(ctx, g, kBlock, rows_lean_kernel<F, 1, false, false>, d, l, r, p, f);
        } else {
            launch_dep(ctx, g, kBlock, rows_lean_kernel<F, 0, false, false>, d, l, r, p, f);
        }
        return check_launch(ctx, "rows_lean_kernel");
    }
    if (fast)
        launch_dep(ctx, (unsigned)grid, kBlock, rows_kernel<F, NIN, true, 1>, d, l, r, p, f);
    else
        launch_dep(ctx, (unsigned)grid, kBlock, rows_kernel<F, NIN, false, 1>, d, l, r, p, f);
    return check_launch(ctx, "rows_kernel");
}

template <template <int> class Fam, int NIN>
int launch_by_binop(Ctx *ctx, const EwCall &c, const rtb_plan &plan, T v) {
    (void)v;
    switch (c.op) {
        case RTB_ADD: { Fam<RTB_ADD> f{}; return launch<Fam<RTB_ADD>, NIN>(ctx, c, plan, f); }
        case RTB_SUB: { Fam<RTB_SUB> f{}; return launch<Fam<RTB_SUB>, NIN>(ctx, c, plan, f); }
        case RTB_MUL: { Fam<RTB_MUL> f{}; return launch<Fam<RTB_MUL>, NIN>(ctx, c, plan, f); }
        case RTB_DIV:
#if RTB_KIND == 3
            return fail(RTB_ERR_DTYPE, "division is not defined for boolean tensors");
#else
            { Fam<RTB_DIV> f{}; return launch<Fam<RTB_DIV>, NIN>(ctx, c, plan, f); }
#endif
    }
    return fail(RTB_ERR_INVALID, "unknown binary op %d", c.op);
}

int launch_scalar(Ctx *ctx, const EwCall &c, const rtb_plan &plan, T v) {
    switch (c.op) {
        case RTB_ADD: return launch<FScalar<RTB_ADD>, 1>(ctx, c, plan, FScalar<RTB_ADD>{v});
        case RTB_SUB: return launch<FScalar<RTB_SUB>, 1>(ctx, c, plan, FScalar<RTB_SUB>{v});
        case RTB_MUL: return launch<FScalar<RTB_MUL>, 1>(ctx, c, plan, FScalar<RTB_MUL>{v});
        case RTB_DIV:
#if RTB_KIND == 3
            return fail(RTB_ERR_DTYPE, "division is not defined for boolean tensors");
#else
            return launch<FScalar<RTB_DIV>, 1>(ctx, c, plan, FScalar<RTB_DIV>{v});
#endif
        case RTB_LEAKY_RELU: return launch<FScalarRt, 1>(ctx, c, plan, FScalarRt{c.op, v});
        case RTB_LOG: case RTB_LOG1P: case RTB_ELU:
#if RTB_KIND == 2
            return launch<FScalarRt, 1>(ctx, c, plan, FScalarRt{c.op, v});
#else
            return fail(RTB_ERR_DTYPE, "log / log1p / elu are defined for f32 and f64 only");
#endif
    }
    return fail(RTB_ERR_INVALID, "unknown scalar op %d", c.op);
}

int launch_unary(Ctx *ctx, const EwCall &c, const rtb_plan &plan) {
    switch (c.op) {
        case RTB_NEG:
#if RTB_KIND == 0 || RTB_KIND == 3
            return fail(RTB_ERR_DTYPE, "negation is not defined for unsigned or boolean tensors");
#else
            return launch<FUnary<RTB_NEG>, 1>(ctx, c, plan, FUnary<RTB_NEG>{});
#endif
        case RTB_RELU: return launch<FUnary<RTB_RELU>, 1>(ctx, c, plan, FUnary<RTB_RELU>{});
        case RTB_ABS: return launch<FUnary<RTB_ABS>, 1>(ctx, c, plan, FUnary<RTB_ABS>{});
        case RTB_SIGN:
#if RTB_KIND == 3
            return fail(RTB_ERR_DTYPE, "sign is not defined for boolean tensors");
#else
            return launch<FUnary<RTB_SIGN>, 1>(ctx, c, plan, FUnary<RTB_SIGN>{});
#endif
    }
    if (c.op >= RTB_SIGMOID && c.op <= RTB_SILU) {
#if RTB_KIND == 2
        return launch<FUnaryRt, 1>(ctx, c, plan, FUnaryRt{c.op});
#else
        return fail(RTB_ERR_DTYPE, "unary op %d is defined for f32 and f64 only", c.op);
#endif
    }
    return fail(RTB_ERR_INVALID, "unknown unary op %d", c.op);
}

}  // namespace

#define RTB_CAT2(a, b) a##b
#define RTB_CAT(a, b) RTB_CAT2(a, b)

int RTB_CAT(ew_dispatch_, RTB_SUFFIX)(Ctx *ctx, const EwCall &c, const rtb_plan &plan) {
    T v;
    std::memcpy(&v, c.value, sizeof v);
#if RTB_KIND == 3
    v = v != 0 ? 1 : 0;
#endif
    switch (c.family) {
        case kFamBinary: return launch_by_binop<FBinary, 2>(ctx, c, plan, v);
        case kFamScalar: return launch_scalar(ctx, c, plan, v);
        case kFamUnary: return launch_unary(ctx, c, plan);
        case kFamFill: return launch<FFill, 0>(ctx, c, plan, FFill{v});
        case kFamCopy:
            if (c.op == 0) return launch<FCopy, 1>(ctx, c, plan, FCopy{});
            if (c.op == 1) return launch<FMaskRelu, 1>(ctx, c, plan, FMaskRelu{});
#if RTB_KIND == 1 || RTB_KIND == 2
            if (c.op == 2) return launch<FMaskAbs, 1>(ctx, c, plan, FMaskAbs{});
#endif
            if (c.op == 2) return fail(RTB_ERR_DTYPE, "abs gradient map needs a signed element type");
            if (c.op == 3) return launch<FMaskLeaky, 1>(ctx, c, plan, FMaskLeaky{v});
#if RTB_KIND != 3
            if (c.op == 4) return launch<FRecip, 1>(ctx, c, plan, FRecip{});
#endif
            return fail(RTB_ERR_DTYPE, "the reciprocal map is not defined for boolean");
    }
    return fail(RTB_ERR_INVALID, "unknown elementwise family %d", c.family);
}

}  // namespace rtb
