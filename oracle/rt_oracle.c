/*
 * rt_oracle.c -- CPU restatement of the rtensors CPU backend for the tensor hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is compared
 * against.  It is never linked into, loaded by, or called from the product library;
 * only the test-suite, the smoke check and the bench's CPU-baseline leg may use it.
 *
 * Parity status: PINNED by the reference's own known-answer tests (broadcast values,
 * negative-step broadcasts, scalar ops on slices, reductions on the (4,2) f64 matrix,
 * unary fixtures) transcribed under tests/golden/.  NOT pinned by any reference test:
 * mean_l1_loss values, gradient values, reduce-to-shape output, SGD update values
 * (the reference only asserts "loss decreased") -- for those, parity is defined by
 * this restatement alone.
 *
 * Every function cites the reference file:line it follows (paths relative to
 * libs/rtensors/src/ of aheschl1/rtensors).  Float semantics: IEEE binary32/64,
 * round-to-nearest-even, no FMA contraction and no reassociation -- build with
 * -ffp-contract=off -fno-fast-math.  Integer + - * wrap (two's complement), integer
 * division truncates, boolean + is OR, - is XOR, * is AND (core/value.rs:708-764).
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#include <math.h>

#define ORC_API __attribute__((visibility("default")))

/* dtype codes = DType discriminants, core/value.rs:567-581 */
enum { ORC_U8 = 0, ORC_I8 = 1, ORC_U16 = 2, ORC_I16 = 3, ORC_U32 = 4, ORC_U128 = 5, ORC_I32 = 6,
       ORC_U64 = 7, ORC_I64 = 8, ORC_I128 = 9, ORC_F32 = 10, ORC_F64 = 11, ORC_BOOL = 12 };
/* BinaryOpType, ops/base.rs:7-12; 4..7 = the other scalar families of the Backend trait
 * (backend/mod.rs:339-346), scalar-op form only */
enum { ORC_ADD = 0, ORC_SUB = 1, ORC_MUL = 2, ORC_DIV = 3, ORC_LOG = 4, ORC_LOG1P = 5, ORC_LEAKY_RELU = 6, ORC_ELU = 7 };
/* unary functor ids (same numbering as the CUDA library's rtb_unop) */
enum { ORC_NEG = 0, ORC_RELU = 1, ORC_ABS = 2, ORC_SIGN = 3,
       ORC_SIGMOID = 4, ORC_TANH = 5, ORC_SQRT = 6, ORC_SIN = 7, ORC_COS = 8, ORC_TAN = 9, ORC_ASIN = 10, ORC_ACOS = 11,
       ORC_ATAN = 12, ORC_SINH = 13, ORC_COSH = 14, ORC_ASINH = 15, ORC_ACOSH = 16, ORC_ATANH = 17, ORC_RSQRT = 18,
       ORC_RECIPROCAL = 19, ORC_SQUARE = 20, ORC_CUBE = 21, ORC_EXP = 22, ORC_LN = 23, ORC_LN1P = 24, ORC_FLOOR = 25,
       ORC_CEIL = 26, ORC_ROUND = 27, ORC_TRUNC = 28, ORC_EXPM1 = 29, ORC_SILU = 30 };
/* ReductionOpTypes::get_code, ops/reduction/mod.rs:161-175 */
enum { ORC_SUM = 1, ORC_PROD = 2, ORC_MAX = 3, ORC_MIN = 4, ORC_MEAN = 5 };

enum { ORC_OK = 0, ORC_ERR_DIM = -1, ORC_ERR_BOUNDS = -2, ORC_ERR_SHAPE = -3, ORC_ERR_BROADCAST = -4,
       ORC_ERR_DTYPE = -5, ORC_ERR_OP = -6, ORC_ERR_NONCONTIG = -7 };

#define ORC_MAX_RANK 128

/* ------------------------------------------------------------------------------------------
 * Meta / view arithmetic
 * ---------------------------------------------------------------------------------------- */

/* shape_to_stride, core/meta.rs:495-503 */
ORC_API void orc_shape_to_stride(size_t rank, const size_t *shape, ptrdiff_t *strides) {
    for (size_t k = rank; k-- > 0;) {
        strides[k] = (k + 1 < rank) ? strides[k + 1] * (ptrdiff_t)shape[k + 1] : 1;
    }
}

/* is_contiguous_relaxed, core/meta.rs:526-541: compares |stride|, skips size-1 dims,
 * empty shape and any zero extent are "contiguous". */
ORC_API int orc_is_contiguous(size_t rank, const size_t *shape, const ptrdiff_t *strides) {
    if (rank == 0) return 1;
    for (size_t k = 0; k < rank; ++k) if (shape[k] == 0) return 1;
    size_t expected = 1;
    for (size_t k = rank; k-- > 0;) {
        if (shape[k] != 1) {
            size_t a = strides[k] < 0 ? (size_t)(-strides[k]) : (size_t)strides[k];
            if (a != expected) return 0;
            expected *= shape[k];
        }
    }
    return 1;
}

static size_t meta_size(size_t rank, const size_t *shape) {
    size_t n = 1;
    for (size_t k = 0; k < rank; ++k) n *= shape[k];
    return n;
}

/* compute_sliced_parameters, core/slice.rs:145-239.  has_start/has_end = Option is Some.
 * A zero-length result removes the dimension (this is how an integer index `i..i` works). */
ORC_API int orc_slice(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t offset,
                      size_t dim, int has_start, size_t start_u, int has_end, size_t end_u,
                      ptrdiff_t step, size_t *out_rank, size_t *out_shape, ptrdiff_t *out_strides,
                      size_t *out_offset) {
    if (dim >= rank) return ORC_ERR_DIM;
    if (step == 0) return ORC_ERR_SHAPE;
    ptrdiff_t n = (ptrdiff_t)shape[dim];
    ptrdiff_t start = has_start ? (ptrdiff_t)start_u : (step > 0 ? 0 : n - 1);
    ptrdiff_t end = has_end ? (ptrdiff_t)end_u : (step > 0 ? n : -1);
    if (step > 0 && (start < 0 || start >= n || end < 0 || end > n)) return ORC_ERR_BOUNDS;
    if (step < 0 && (start < 0 || start >= n || end < -1 || end >= n)) return ORC_ERR_BOUNDS;
    size_t len;
    if ((step > 0 && start >= end) || (step < 0 && start <= end)) {
        len = 0;
    } else {
        ptrdiff_t dist = (start > end ? start - end : end - start) - 1;
        size_t astep = step < 0 ? (size_t)(-step) : (size_t)step;
        len = (size_t)dist / astep + 1;
    }
    ptrdiff_t adv = start * strides[dim];
    size_t new_offset = offset + (size_t)(adv > 0 ? adv : 0);
    if (len == 0) {
        size_t o = 0;
        for (size_t k = 0; k < rank; ++k) {
            if (k == dim) continue;
            out_shape[o] = shape[k];
            out_strides[o] = strides[k];
            ++o;
        }
        *out_rank = rank - 1;
        *out_offset = new_offset;
        return ORC_OK;
    }
    for (size_t k = 0; k < rank; ++k) {
        out_shape[k] = shape[k];
        out_strides[k] = strides[k];
    }
    out_shape[dim] = len;
    out_strides[dim] = strides[dim] * step;
    *out_rank = rank;
    *out_offset = new_offset;
    return ORC_OK;
}

/* compute_permuted_parameters, core/tensor.rs:909-941: new[i] = old[dims[i]] */
ORC_API int orc_permute(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t ndims,
                        const size_t *dims, size_t *out_shape, ptrdiff_t *out_strides) {
    if (ndims != rank) return ORC_ERR_DIM;
    for (size_t k = 0; k < rank; ++k) {
        if (dims[k] >= rank) return ORC_ERR_DIM;
        out_shape[k] = shape[dims[k]];
        out_strides[k] = strides[dims[k]];
    }
    return ORC_OK;
}

/* compute_unsqueezed_parameters, core/tensor.rs:973-990 */
ORC_API int orc_unsqueeze(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t dim,
                          size_t *out_shape, ptrdiff_t *out_strides) {
    if (dim > rank) return ORC_ERR_DIM;
    ptrdiff_t lstr = dim < rank ? strides[dim] : 1;
    ptrdiff_t lsh = dim < rank ? (ptrdiff_t)shape[dim] : 1;
    size_t o = 0;
    for (size_t k = 0; k <= rank; ++k) {
        if (k == dim) {
            out_shape[o] = 1;
            out_strides[o] = lstr * lsh;
            ++o;
        }
        if (k < rank) {
            out_shape[o] = shape[k];
            out_strides[o] = strides[k];
            ++o;
        }
    }
    return ORC_OK;
}

/* compute_squeezed_parameters, core/tensor.rs:992-1027.  dim < 0 means "all size-1 dims". */
ORC_API int orc_squeeze(size_t rank, const size_t *shape, const ptrdiff_t *strides, ptrdiff_t dim,
                        size_t *out_rank, size_t *out_shape, ptrdiff_t *out_strides) {
    if (dim >= 0 && (size_t)dim >= rank) return ORC_ERR_DIM;
    size_t o = 0;
    for (size_t k = 0; k < rank; ++k) {
        int squeeze = dim < 0 ? (shape[k] == 1) : ((size_t)dim == k);
        if (squeeze) {
            if (shape[k] != 1) return ORC_ERR_DIM;
            continue;
        }
        out_shape[o] = shape[k];
        out_strides[o] = strides[k];
        ++o;
    }
    *out_rank = o;
    return ORC_OK;
}

/* compute_broadcasted_params, ops/broadcast/mod.rs:13-55 */
ORC_API int orc_broadcast_params(size_t ra, const size_t *sha, const ptrdiff_t *stra, size_t rb,
                                 const size_t *shb, const ptrdiff_t *strb, size_t *out_rank,
                                 size_t *out_shape, ptrdiff_t *out_stra, ptrdiff_t *out_strb) {
    size_t r = ra > rb ? ra : rb;
    if (r > ORC_MAX_RANK) return ORC_ERR_DIM;
    size_t pa = r - ra, pb = r - rb;
    for (size_t k = 0; k < r; ++k) {
        size_t a = k < pa ? 1 : sha[k - pa];
        size_t b = k < pb ? 1 : shb[k - pb];
        ptrdiff_t sa = k < pa ? 0 : stra[k - pa];
        ptrdiff_t sb = k < pb ? 0 : strb[k - pb];
        size_t out;
        if (a == b) out = a;
        else if (a == 1) out = b;
        else if (b == 1) out = a;
        else return ORC_ERR_BROADCAST;
        out_shape[k] = out;
        out_stra[k] = (a == 1 && out > 1) ? 0 : sa;
        out_strb[k] = (b == 1 && out > 1) ? 0 : sb;
    }
    *out_rank = r;
    return ORC_OK;
}

/* reduction_output_meta, ops/reduction/mod.rs:512-538: reduced dim kept as size 1 */
ORC_API void orc_reduction_output_shape(size_t rank, const size_t *shape, size_t axis,
                                        size_t *out_shape, ptrdiff_t *out_strides) {
    for (size_t k = 0; k < rank; ++k) out_shape[k] = (k == axis) ? 1 : shape[k];
    orc_shape_to_stride(rank, out_shape, out_strides);
}

/* non_singleton_dims, core/meta.rs:618-625: returns count and the last seen (size, stride) */
static size_t non_singleton(size_t rank, const size_t *shape, const ptrdiff_t *strides,
                            size_t *dsize, ptrdiff_t *dstride) {
    size_t c = 0;
    for (size_t k = 0; k < rank; ++k) {
        if (shape[k] > 1) {
            if (c == 0) { *dsize = shape[k]; *dstride = strides[k]; }
            ++c;
        }
    }
    return c;
}

/* Layout class chosen by the 3-way dispatcher, backend/mod.rs:15-213:
 * 0 = contiguous(start=offset,len=size) 1 = 1-D strided 2 = N-d */
ORC_API int orc_layout_class(size_t rank, const size_t *shape, const ptrdiff_t *strides) {
    if (orc_is_contiguous(rank, shape, strides)) return 0;
    size_t ds; ptrdiff_t dst;
    if (non_singleton(rank, shape, strides, &ds, &dst) == 1) return 1;
    return 2;
}

/* TensorOffsetIterator, core/meta.rs:368-431: row-major odometer over the view. */
typedef struct { size_t rank; const size_t *shape; const ptrdiff_t *strides; size_t idx[ORC_MAX_RANK];
                 ptrdiff_t off; int done; } off_iter;

static void it_init(off_iter *it, size_t rank, const size_t *shape, const ptrdiff_t *strides,
                    size_t offset) {
    it->rank = rank; it->shape = shape; it->strides = strides; it->off = (ptrdiff_t)offset;
    it->done = 0;
    memset(it->idx, 0, sizeof(size_t) * (rank ? rank : 1));
    for (size_t k = 0; k < rank; ++k) if (shape[k] == 0) it->done = 1;
}
static inline void it_next(off_iter *it) {
    for (size_t d = it->rank; d-- > 0;) {
        it->idx[d] += 1;
        it->off += it->strides[d];
        if (it->idx[d] < it->shape[d]) return;
        it->off -= (ptrdiff_t)it->shape[d] * it->strides[d];
        it->idx[d] = 0;
    }
    it->done = 1;
}

/* ------------------------------------------------------------------------------------------
 * Typed element arithmetic.  Functors: backend/cpu.rs:549-557 (sign), :632-657 (abs, neg,
 * relu), :679-696 (scalar add/sub/mul/div); BinaryOpType::apply ops/base.rs:29-36;
 * Absolute core/value.rs:515-548 (unsigned/boolean: identity; signed: wrapping abs).
 * ---------------------------------------------------------------------------------------- */
typedef unsigned __int128 u128_t;
typedef __int128 i128_t;

#define DEF_INT_OPS(S, T, UT, SIGNED)                                                        \
    static inline T bin_##S(int op, T a, T b) {                                              \
        switch (op) {                                                                        \
            case ORC_ADD: return (T)((UT)a + (UT)b);                                         \
            case ORC_SUB: return (T)((UT)a - (UT)b);                                         \
            case ORC_MUL: return (T)((UT)a * (UT)b);                                         \
            case ORC_LEAKY_RELU: return a > (T)0 ? a : (T)((UT)a * (UT)b);                   \
            default: return (T)(a / b);                                                      \
        }                                                                                    \
    }                                                                                        \
    static inline T un_##S(int op, T x) {                                                    \
        switch (op) {                                                                        \
            case ORC_NEG: return (T)((UT)0 - (UT)x);                                         \
            case ORC_RELU: return x > (T)0 ? x : (T)0;                                       \
            case ORC_ABS: return (SIGNED && x < (T)0) ? (T)((UT)0 - (UT)x) : x;              \
            default: return x < (T)0 ? (T)((UT)0 - (UT)1) : (x > (T)0 ? (T)1 : (T)0);        \
        }                                                                                    \
    }

/* Remaining float unary families with the CPU backend's own formulas (backend/cpu.rs:485-724,
 * core/primops/exp.rs, core/value.rs:62-140): exp-based tanh/sinh/cosh, ln/sqrt-based inverse
 * hyperbolics, sigmoid = 1/(1+exp(-x)), silu = x*sigmoid(x), round = half away from zero.
 * Scalar families: log(base) = ln(x)/ln(base) (Rust f32::log), log1p(base) = ln_1p(x)/ln(base),
 * leaky_relu = x>0 ? x : x*slope, elu = x>=0 ? x : alpha*expm1(x) (backend/cpu.rs:699-724). */
#define DEF_FLOAT_OPS(S, T, SFX)                                                             \
    static inline T ext_##S(int op, T x) {                                                   \
        const T one = (T)1;                                                                  \
        switch (op) {                                                                        \
            case ORC_SIGMOID: return one / (one + exp##SFX(-x));                             \
            case ORC_SILU: return x * (one / (one + exp##SFX(-x)));                          \
            case ORC_TANH: { T a = exp##SFX(x), b = exp##SFX(-x); return (a - b) / (a + b); } \
            case ORC_SINH: { T a = exp##SFX(x), b = exp##SFX(-x); return (a - b) / (one + one); } \
            case ORC_COSH: { T a = exp##SFX(x), b = exp##SFX(-x); return (a + b) / (one + one); } \
            case ORC_ASINH: return log##SFX(x + sqrt##SFX(x * x + one));                     \
            case ORC_ACOSH: return log##SFX(x + sqrt##SFX(x * x - one));                     \
            case ORC_ATANH: return log##SFX((one + x) / (one - x)) / (one + one);            \
            case ORC_SQRT: return sqrt##SFX(x);                                              \
            case ORC_RSQRT: return one / sqrt##SFX(x);                                       \
            case ORC_RECIPROCAL: return one / x;                                             \
            case ORC_SQUARE: return x * x;                                                   \
            case ORC_CUBE: return x * x * x;                                                 \
            case ORC_EXP: return exp##SFX(x);                                                \
            case ORC_EXPM1: return expm1##SFX(x);                                            \
            case ORC_LN: return log##SFX(x);                                                 \
            case ORC_LN1P: return log1p##SFX(x);                                             \
            case ORC_SIN: return sin##SFX(x);                                                \
            case ORC_COS: return cos##SFX(x);                                                \
            case ORC_TAN: return tan##SFX(x);                                                \
            case ORC_ASIN: return asin##SFX(x);                                              \
            case ORC_ACOS: return acos##SFX(x);                                              \
            case ORC_ATAN: return atan##SFX(x);                                              \
            case ORC_FLOOR: return floor##SFX(x);                                            \
            case ORC_CEIL: return ceil##SFX(x);                                              \
            case ORC_ROUND: return round##SFX(x);                                            \
            case ORC_TRUNC: return trunc##SFX(x);                                            \
        }                                                                                    \
        return x;                                                                            \
    }                                                                                        \
    static inline T bin_##S(int op, T a, T b) {                                              \
        switch (op) {                                                                        \
            case ORC_ADD: return a + b;                                                      \
            case ORC_SUB: return a - b;                                                      \
            case ORC_MUL: return a * b;                                                      \
            case ORC_DIV: return a / b;                                                      \
            case ORC_LOG: return log##SFX(a) / log##SFX(b);                                  \
            case ORC_LOG1P: return log1p##SFX(a) / log##SFX(b);                              \
            case ORC_LEAKY_RELU: return a > (T)0 ? a : a * b;                                \
            default: return a >= (T)0 ? a : b * expm1##SFX(a); /* ELU */                     \
        }                                                                                    \
    }                                                                                        \
    static inline T un_##S(int op, T x) {                                                    \
        switch (op) {                                                                        \
            case ORC_NEG: return -x;                                                         \
            case ORC_RELU: return x > (T)0 ? x : (T)0;                                       \
            case ORC_ABS: return sizeof(T) == 4 ? (T)fabsf((float)x) : (T)fabs((double)x);   \
            case ORC_SIGN: return x < (T)0 ? (T)-1 : (x > (T)0 ? (T)1 : (T)0);               \
            default: return ext_##S(op, x);                                                  \
        }                                                                                    \
    }

DEF_INT_OPS(u8, uint8_t, uint8_t, 0)
DEF_INT_OPS(i8, int8_t, uint8_t, 1)
DEF_INT_OPS(u16, uint16_t, uint16_t, 0)
DEF_INT_OPS(i16, int16_t, uint16_t, 1)
DEF_INT_OPS(u32, uint32_t, uint32_t, 0)
DEF_INT_OPS(i32, int32_t, uint32_t, 1)
DEF_INT_OPS(u64, uint64_t, uint64_t, 0)
DEF_INT_OPS(i64, int64_t, uint64_t, 1)
DEF_INT_OPS(u128, u128_t, u128_t, 0)
DEF_INT_OPS(i128, i128_t, u128_t, 1)
DEF_FLOAT_OPS(f32, float, f)
DEF_FLOAT_OPS(f64, double, )

/* boolean: + OR, - XOR, * AND, / unimplemented in the reference (core/value.rs:708-764) */
static inline uint8_t bin_boolean(int op, uint8_t a, uint8_t b) {
    switch (op) {
        case ORC_ADD: return (uint8_t)((a != 0) || (b != 0));
        case ORC_SUB: return (uint8_t)((a != 0) != (b != 0));
        case ORC_LEAKY_RELU: return a; /* x > false ? x : x AND slope == x */
        default: return (uint8_t)((a != 0) && (b != 0));
    }
}
static inline uint8_t un_boolean(int op, uint8_t x) {
    switch (op) {
        case ORC_RELU: return x; /* x > false ? x : false */
        default: return x;       /* abs: identity */
    }
}

#define FOR_ALL_TYPES(X)                                                                     \
    X(u8, uint8_t, ORC_U8) X(i8, int8_t, ORC_I8) X(u16, uint16_t, ORC_U16)                   \
    X(i16, int16_t, ORC_I16) X(u32, uint32_t, ORC_U32) X(u128, u128_t, ORC_U128)             \
    X(i32, int32_t, ORC_I32) X(u64, uint64_t, ORC_U64) X(i64, int64_t, ORC_I64)              \
    X(i128, i128_t, ORC_I128) X(f32, float, ORC_F32) X(f64, double, ORC_F64)                 \
    X(boolean, uint8_t, ORC_BOOL)

/* ------------------------------------------------------------------------------------------
 * Elementwise loops: three loop shapes of backend/cpu.rs:10-42, selected by the dispatcher of
 * backend/mod.rs:146-177.  kind 0 = scalar op (value used), kind 1 = unary, kind 2 = fill
 * (backend/cpu.rs:245-289).
 * ---------------------------------------------------------------------------------------- */
#define DEF_ELEMWISE(S, T, CODE)                                                             \
    static void ew_##S(T *buf, int kind, int op, T v, size_t rank, const size_t *shape,      \
                       const ptrdiff_t *strides, size_t offset) {                            \
        size_t n = meta_size(rank, shape);                                                   \
        if (orc_is_contiguous(rank, shape, strides)) {                                       \
            /* elemwise_contiguous_loop: buf[start .. start+len], start = meta.offset */     \
            T *p = buf + offset;                                                             \
            if (kind == 0) { for (size_t i = 0; i < n; ++i) p[i] = bin_##S(op, p[i], v); }   \
            else if (kind == 1) { for (size_t i = 0; i < n; ++i) p[i] = un_##S(op, p[i]); }  \
            else { for (size_t i = 0; i < n; ++i) p[i] = v; }                                \
            return;                                                                          \
        }                                                                                    \
        size_t ds = 0; ptrdiff_t dst = 0;                                                    \
        if (non_singleton(rank, shape, strides, &ds, &dst) == 1) {                           \
            /* elemwise_1d_strided_loop */                                                   \
            ptrdiff_t idx = (ptrdiff_t)offset;                                               \
            for (size_t i = 0; i < ds; ++i) {                                                \
                T *x = buf + idx;                                                            \
                *x = kind == 0 ? bin_##S(op, *x, v) : (kind == 1 ? un_##S(op, *x) : v);      \
                idx += dst;                                                                  \
            }                                                                                \
            return;                                                                          \
        }                                                                                    \
        /* elemwise_nd_loop over TensorOffsetIterator */                                     \
        off_iter it;                                                                         \
        it_init(&it, rank, shape, strides, offset);                                          \
        while (!it.done) {                                                                   \
            T *x = buf + it.off;                                                             \
            *x = kind == 0 ? bin_##S(op, *x, v) : (kind == 1 ? un_##S(op, *x) : v);          \
            it_next(&it);                                                                    \
        }                                                                                    \
    }
FOR_ALL_TYPES(DEF_ELEMWISE)

/* kind: 0 scalar op (value -> *value), 1 unary, 2 fill.  In place over the view. */
ORC_API int orc_elementwise(int dtype, void *buf, int kind, int op, const void *value, size_t rank,
                            const size_t *shape, const ptrdiff_t *strides, size_t offset) {
    if (rank > ORC_MAX_RANK) return ORC_ERR_DIM;
    if (dtype == ORC_BOOL && kind == 0 && op == ORC_DIV) return ORC_ERR_OP;
    if (dtype != ORC_F32 && dtype != ORC_F64) {
        if (kind == 1 && op > ORC_SIGN) return ORC_ERR_DTYPE;
        if (kind == 0 && (op == ORC_LOG || op == ORC_LOG1P || op == ORC_ELU)) return ORC_ERR_DTYPE;
    }
    switch (dtype) {
#define CASE_EW(S, T, CODE)                                                                  \
    case CODE: {                                                                             \
        T v; memset(&v, 0, sizeof v);                                                        \
        if (value) memcpy(&v, value, sizeof v);                                              \
        ew_##S((T *)buf, kind, op, v, rank, shape, strides, offset);                         \
        return ORC_OK;                                                                       \
    }
        FOR_ALL_TYPES(CASE_EW)
    }
    return ORC_ERR_DTYPE;
}

/* ------------------------------------------------------------------------------------------
 * Broadcast: Cpu::broadcast, backend/cpu.rs:292-352.  All three metas carry the OUTPUT shape;
 * operands are pre-broadcast by stride 0.  Output coordinates are visited in row-major order,
 * which defines the result when dst aliases left (in-place form).
 * ---------------------------------------------------------------------------------------- */
#define DEF_BROADCAST(S, T, CODE)                                                            \
    static void bc_##S(const T *l, const T *r, T *d, int op, size_t rank, const size_t *shape,\
                       const ptrdiff_t *ls, size_t lo, const ptrdiff_t *rs, size_t ro,       \
                       const ptrdiff_t *ds, size_t doff) {                                   \
        size_t idx[ORC_MAX_RANK];                                                            \
        memset(idx, 0, sizeof idx);                                                          \
        size_t n = meta_size(rank, shape);                                                   \
        ptrdiff_t ol = (ptrdiff_t)lo, orr = (ptrdiff_t)ro, od = (ptrdiff_t)doff;             \
        for (size_t e = 0; e < n; ++e) {                                                     \
            d[od] = bin_##S(op, l[ol], r[orr]);                                              \
            for (size_t k = rank; k-- > 0;) {                                                \
                idx[k] += 1; ol += ls[k]; orr += rs[k]; od += ds[k];                         \
                if (idx[k] < shape[k]) break;                                                \
                ol -= (ptrdiff_t)shape[k] * ls[k]; orr -= (ptrdiff_t)shape[k] * rs[k];       \
                od -= (ptrdiff_t)shape[k] * ds[k]; idx[k] = 0;                               \
            }                                                                                \
        }                                                                                    \
    }
FOR_ALL_TYPES(DEF_BROADCAST)

ORC_API int orc_broadcast(int dtype, const void *l, const void *r, void *d, int op, size_t rank,
                          const size_t *shape, const ptrdiff_t *ls, size_t lo, const ptrdiff_t *rs,
                          size_t ro, const ptrdiff_t *ds, size_t doff) {
    if (rank > ORC_MAX_RANK) return ORC_ERR_DIM;
    if (dtype == ORC_BOOL && op == ORC_DIV) return ORC_ERR_OP;
    switch (dtype) {
#define CASE_BC(S, T, CODE)                                                                  \
    case CODE: bc_##S((const T *)l, (const T *)r, (T *)d, op, rank, shape, ls, lo, rs, ro, ds, doff); \
        return ORC_OK;
        FOR_ALL_TYPES(CASE_BC)
    }
    return ORC_ERR_DTYPE;
}

/* ------------------------------------------------------------------------------------------
 * Reductions (f32 / f64 only, as in the reference: T: WeightValue).
 * Accumulators ops/reduction/mod.rs:9-137: sum from 0 with +=; max from T::MIN (lowest finite)
 * with `if v > acc`; min from T::MAX with `if v < acc`; prod from 1; mean = sum / from_usize(n)
 * where from_usize goes through f32 (core/value.rs:54-56).
 * ---------------------------------------------------------------------------------------- */
#define DEF_REDUCE(S, T, TMIN, TMAX)                                                         \
    typedef struct { T acc; int op; } acc_##S;                                               \
    static inline void acc_init_##S(acc_##S *a, int op) {                                    \
        a->op = op;                                                                          \
        a->acc = op == ORC_PROD ? (T)1 : op == ORC_MAX ? (T)TMIN : op == ORC_MIN ? (T)TMAX : (T)0; \
    }                                                                                        \
    static inline void acc_add_##S(acc_##S *a, T v) {                                        \
        switch (a->op) {                                                                     \
            case ORC_PROD: a->acc *= v; break;                                               \
            case ORC_MAX: if (v > a->acc) a->acc = v; break;                                 \
            case ORC_MIN: if (v < a->acc) a->acc = v; break;                                 \
            default: a->acc += v; break;                                                     \
        }                                                                                    \
    }                                                                                        \
    static inline T acc_fin_##S(const acc_##S *a, size_t count) {                            \
        if (a->op == ORC_MEAN) return a->acc / (T)(float)count;                              \
        return a->acc;                                                                       \
    }                                                                                        \
    /* apply_reduce_contiguous_flat, backend/cpu.rs:397-411 */                               \
    static void red_flat_##S(const T *src, size_t start, size_t len, int op, T *dst) {       \
        acc_##S a; acc_init_##S(&a, op);                                                     \
        if (op == ORC_SUM || op == ORC_MEAN) {                                               \
            T s = 0; for (size_t i = 0; i < len; ++i) s += src[start + i]; a.acc = s;        \
        } else {                                                                             \
            for (size_t i = 0; i < len; ++i) acc_add_##S(&a, src[start + i]);                \
        }                                                                                    \
        dst[0] = acc_fin_##S(&a, len);                                                       \
    }                                                                                        \
    /* apply_reduce_contiguous_nd, backend/cpu.rs:413-449: base = o*R*inner + i (meta.offset \
     * is ignored by the reference CPU backend), element base + k*stride[dim], out o*inner+i */ \
    static void red_nd_##S(const T *src, size_t outer, size_t r, size_t inner,               \
                           size_t r_stride, int op, T *dst) {                                \
        size_t left = r * inner;                                                             \
        for (size_t i = 0; i < inner; ++i) {                                                 \
            for (size_t o = 0; o < outer; ++o) {                                             \
                size_t base = o * left + i;                                                  \
                acc_##S a; acc_init_##S(&a, op);                                             \
                for (size_t k = 0; k < r; ++k) acc_add_##S(&a, src[base + k * r_stride]);    \
                dst[o * inner + i] = acc_fin_##S(&a, r);                                     \
            }                                                                                \
        }                                                                                    \
    }
DEF_REDUCE(f32, float, -FLT_MAX, FLT_MAX)
DEF_REDUCE(f64, double, -DBL_MAX, DBL_MAX)

ORC_API int orc_reduce_flat(int dtype, const void *src, size_t start, size_t len, int op, void *dst) {
    if (op < ORC_SUM || op > ORC_MEAN) return ORC_ERR_OP;
    if (dtype == ORC_F32) { red_flat_f32((const float *)src, start, len, op, (float *)dst); return ORC_OK; }
    if (dtype == ORC_F64) { red_flat_f64((const double *)src, start, len, op, (double *)dst); return ORC_OK; }
    return ORC_ERR_DTYPE;
}

/* inner_dimensions / outer_dimensions, core/meta.rs:209-235 */
static void outer_r_inner(size_t rank, const size_t *shape, size_t dim, size_t *outer, size_t *r,
                          size_t *inner) {
    size_t o = 1, in = 1;
    for (size_t k = 0; k < dim; ++k) o *= shape[k];
    for (size_t k = dim + 1; k < rank; ++k) in *= shape[k];
    *outer = o; *r = shape[dim]; *inner = in > 1 ? in : 1;
}

/* Backend::apply_reduce, backend/mod.rs:375-409: contiguity is required; rank-1 input goes to
 * the flat routine (start = meta.offset), everything else to the N-d routine. */
ORC_API int orc_reduce_axis(int dtype, const void *src, size_t rank, const size_t *shape,
                            const ptrdiff_t *strides, size_t offset, size_t dim, int op, void *dst) {
    if (op < ORC_SUM || op > ORC_MEAN) return ORC_ERR_OP;
    if (dtype != ORC_F32 && dtype != ORC_F64) return ORC_ERR_DTYPE;
    if (!orc_is_contiguous(rank, shape, strides)) return ORC_ERR_NONCONTIG;
    if (rank == 1) return orc_reduce_flat(dtype, src, offset, shape[0], op, dst);
    if (dim >= rank) return ORC_ERR_DIM;
    size_t outer, r, inner;
    outer_r_inner(rank, shape, dim, &outer, &r, &inner);
    size_t r_stride = (size_t)strides[dim];
    if (dtype == ORC_F32) red_nd_f32((const float *)src, outer, r, inner, r_stride, op, (float *)dst);
    else red_nd_f64((const double *)src, outer, r, inner, r_stride, op, (double *)dst);
    return ORC_OK;
}

/* Same N-d routine with (outer, R, inner) given directly -- the form the CUDA launcher takes. */
ORC_API int orc_reduce_ori(int dtype, const void *src, size_t outer, size_t r, size_t inner, int op,
                           void *dst) {
    if (op < ORC_SUM || op > ORC_MEAN) return ORC_ERR_OP;
    if (dtype == ORC_F32) { red_nd_f32((const float *)src, outer, r, inner, inner, op, (float *)dst); return ORC_OK; }
    if (dtype == ORC_F64) { red_nd_f64((const double *)src, outer, r, inner, inner, op, (double *)dst); return ORC_OK; }
    return ORC_ERR_DTYPE;
}

/* ------------------------------------------------------------------------------------------
 * Reductions that only the reference's CUDA backend implements: variance / standard deviation,
 * L1 / L2 norm, logsumexp, argmax / argmin.  Its CPU backend has no accumulator for them
 * (get_accumulator panics, ops/reduction/mod.rs:187-197; apply_argmax_* is todo!(),
 * backend/cpu.rs:452-482), so this is a sequential restatement of the device algorithm in
 * cuda/kernels/reduction/reduce.cu, element by element in increasing k:
 *   variance  welford_update (reduce.cu:182-192); result m2 / (n-1) (unbiased) or m2 / n, with
 *             a denominator of 1 when that would be <= 0, square-rooted for the std form
 *             (reduce.cu:619-637; the flat form returns 0 for n <= 1, reduce.cu:344-357);
 *   norm      type 1: acc + |x| (L1SumOp, reduce.cu:66-75); type 2: sqrt(sum x*x)
 *             (SquareUnaryOp + PostSqrt, reduce.cu:77-86,143-152);
 *   logsumexp lse_combine(state, {x, 1}) then m + log(s) (reduce.cu:641-716).  The reference's
 *             FLAT dispatcher has no logsumexp case and leaves the output untouched
 *             (reduce.cu:795-843); here the flat form is the same formula over one row;
 *   argmax    strict `cur > best` from lowest() / `cur < best` from max(), so the FIRST index of
 *             the extreme value (reduce.cu:897-905; the flat form is cub ArgMax / ArgMin, which
 *             also returns the lowest index).  Indices are positions along the reduced axis.
 * Pinned by the expected values of the reference's CUDA tests (backend/cuda.rs:2320-2590).
 * ---------------------------------------------------------------------------------------- */
enum { ORC_VARIANCE = 6, ORC_LOGSUMEXP = 7, ORC_NORM = 8, ORC_ARGMAX = 9, ORC_ARGMIN = 10 };

#define DEF_REDUCE_EXT(S, T, TMIN, TMAX, SQRT, EXP, LOG, FABS)                               \
    static T ext_one_##S(const T *p, size_t r, size_t stride, int op, int unbiased,          \
                         int is_std, int norm_type) {                                        \
        if (op == ORC_VARIANCE) {                                                            \
            T mean = 0, m2 = 0; long count = 0;                                              \
            for (size_t k = 0; k < r; ++k) {                                                 \
                T x = p[k * stride];                                                         \
                count += 1;                                                                  \
                T delta = x - mean;                                                          \
                mean += delta / (T)count;                                                    \
                T delta2 = x - mean;                                                         \
                m2 += delta * delta2;                                                        \
            }                                                                                \
            T denom = unbiased ? (count > 1 ? (T)(count - 1) : (T)1) : (count > 0 ? (T)count : (T)1); \
            T v = m2 / denom;                                                                \
            return is_std ? SQRT(v) : v;                                                     \
        }                                                                                    \
        if (op == ORC_NORM) {                                                                \
            T acc = 0;                                                                       \
            if (norm_type == 1) { for (size_t k = 0; k < r; ++k) acc = acc + FABS(p[k * stride]); return acc; } \
            for (size_t k = 0; k < r; ++k) { T x = p[k * stride]; acc = acc + x * x; }       \
            return SQRT(acc);                                                                \
        }                                                                                    \
        /* logsumexp */                                                                      \
        T m = -(T)INFINITY, s = 0;                                                           \
        for (size_t k = 0; k < r; ++k) {                                                     \
            T x = p[k * stride];                                                             \
            if (s == (T)0) { m = x; s = (T)1; continue; }                                    \
            T mm = m > x ? m : x;                                                            \
            s = s * EXP(m - mm) + (T)1 * EXP(x - mm);                                        \
            m = mm;                                                                          \
        }                                                                                    \
        return r == 0 ? -(T)INFINITY : m + LOG(s);                                           \
    }                                                                                        \
    static uint64_t arg_one_##S(const T *p, size_t r, size_t stride, int op) {               \
        T best = op == ORC_ARGMAX ? (T)TMIN : (T)TMAX;                                       \
        uint64_t idx = 0;                                                                    \
        for (size_t k = 0; k < r; ++k) {                                                     \
            T x = p[k * stride];                                                             \
            if (op == ORC_ARGMAX ? x > best : x < best) { best = x; idx = (uint64_t)k; }     \
        }                                                                                    \
        return idx;                                                                          \
    }
DEF_REDUCE_EXT(f32, float, -FLT_MAX, FLT_MAX, sqrtf, expf, logf, fabsf)
DEF_REDUCE_EXT(f64, double, -DBL_MAX, DBL_MAX, sqrt, exp, log, fabs)

/* (outer, R, inner) form of launch_nd_reduce_contiguous_* for codes 6..8; flat = (1, len, 1). */
ORC_API int orc_reduce_ext_ori(int dtype, const void *src, size_t outer, size_t r, size_t inner, int op,
                               int unbiased, int is_std, int norm_type, void *dst) {
    if (op < ORC_VARIANCE || op > ORC_NORM) return ORC_ERR_OP;
    if (op == ORC_NORM && norm_type != 1 && norm_type != 2) return ORC_ERR_OP;
    if (dtype != ORC_F32 && dtype != ORC_F64) return ORC_ERR_DTYPE;
    for (size_t o = 0; o < outer; ++o)
        for (size_t i = 0; i < inner; ++i) {
            size_t base = o * r * inner + i;
            if (dtype == ORC_F32)
                ((float *)dst)[o * inner + i] = ext_one_f32((const float *)src + base, r, inner, op, unbiased, is_std, norm_type);
            else
                ((double *)dst)[o * inner + i] = ext_one_f64((const double *)src + base, r, inner, op, unbiased, is_std, norm_type);
        }
    return ORC_OK;
}

/* launch_nd_argmax_contiguous_* / launch_flat_contiguous_argmax_*: u64 positions along the axis */
ORC_API int orc_argreduce_ori(int dtype, const void *src, size_t outer, size_t r, size_t inner, int op,
                              uint64_t *dst) {
    if (op != ORC_ARGMAX && op != ORC_ARGMIN) return ORC_ERR_OP;
    if (dtype != ORC_F32 && dtype != ORC_F64) return ORC_ERR_DTYPE;
    for (size_t o = 0; o < outer; ++o)
        for (size_t i = 0; i < inner; ++i) {
            size_t base = o * r * inner + i;
            dst[o * inner + i] = dtype == ORC_F32 ? arg_one_f32((const float *)src + base, r, inner, op)
                                                  : arg_one_f64((const double *)src + base, r, inner, op);
        }
    return ORC_OK;
}

/* ------------------------------------------------------------------------------------------
 * L1 loss on two same-shape contiguous tensors: L1::l1 + attach_l1_grad,
 * ops/broadcast/l1.rs:16-77.  diff = a - b; g = sign(diff); diff = |diff|;
 * reduction 0 = mean (sum / from_usize(n)), 1 = sum.  grad_map (optional) = sign(g), divided
 * by from_usize(n) for the mean form.  Unpinned by reference tests.
 * ---------------------------------------------------------------------------------------- */
#define DEF_L1(S, T)                                                                         \
    static void l1_##S(const T *a, const T *b, size_t n, int reduction, T *loss, T *gmap) {  \
        T s = 0;                                                                             \
        T cnt = (T)(float)n;                                                                 \
        for (size_t i = 0; i < n; ++i) {                                                     \
            T d = a[i] - b[i];                                                               \
            T g = un_##S(ORC_SIGN, d);                                                       \
            d = un_##S(ORC_ABS, d);                                                          \
            s += d;                                                                          \
            if (gmap) { g = un_##S(ORC_SIGN, g); gmap[i] = reduction == 0 ? g / cnt : g; }   \
        }                                                                                    \
        loss[0] = reduction == 0 ? s / cnt : s;                                              \
    }
DEF_L1(f32, float)
DEF_L1(f64, double)

ORC_API int orc_l1_loss(int dtype, const void *a, const void *b, size_t n, int reduction, void *loss,
                        void *grad_map) {
    if (dtype == ORC_F32) { l1_f32((const float *)a, (const float *)b, n, reduction, (float *)loss, (float *)grad_map); return ORC_OK; }
    if (dtype == ORC_F64) { l1_f64((const double *)a, (const double *)b, n, reduction, (double *)loss, (double *)grad_map); return ORC_OK; }
    return ORC_ERR_DTYPE;
}

/* ------------------------------------------------------------------------------------------
 * Reduce-to-shape (broadcast gradient): inverse_broadcast_gradient, grad/backwards.rs:512-538.
 * For every dim whose operand stride is 0, sum_at(dim) on the (contiguous) upstream, keeping
 * the dim as size 1.  intended = 1: the running tensor is replaced by each sum (what the
 * comment in the reference says it does).  intended = 0: the reference's observable behaviour:
 * only the meta of each sum is kept, so the result buffer is the upstream buffer and the
 * reduced tensor reads its leading prod(out_shape) elements.  `out` receives prod(out_shape)
 * elements; out_shape (rank entries, before any squeeze) is returned too.  f32/f64.
 * ---------------------------------------------------------------------------------------- */
ORC_API int orc_reduce_to_shape(int dtype, const void *upstream, size_t rank, const size_t *shape,
                                const ptrdiff_t *operand_strides, int intended, void *out,
                                size_t *out_shape) {
    if (dtype != ORC_F32 && dtype != ORC_F64) return ORC_ERR_DTYPE;
    size_t es = dtype == ORC_F32 ? 4 : 8;
    size_t n = meta_size(rank, shape);
    size_t cur_shape[ORC_MAX_RANK];
    for (size_t k = 0; k < rank; ++k) cur_shape[k] = shape[k];
    void *cur = malloc(n * es ? n * es : 1);
    void *tmp = malloc(n * es ? n * es : 1);
    memcpy(cur, upstream, n * es);
    for (size_t dim = 0; dim < rank; ++dim) {
        if (operand_strides[dim] != 0) continue;
        size_t outer, r, inner;
        outer_r_inner(rank, cur_shape, dim, &outer, &r, &inner);
        if (rank == 1) orc_reduce_flat(dtype, cur, 0, r, ORC_SUM, tmp);
        else orc_reduce_ori(dtype, cur, outer, r, inner, ORC_SUM, tmp);
        cur_shape[dim] = 1;
        if (intended) { void *t = cur; cur = tmp; tmp = t; }
    }
    size_t m = meta_size(rank, cur_shape);
    memcpy(out, cur, m * es);
    for (size_t k = 0; k < rank; ++k) out_shape[k] = cur_shape[k];
    free(cur); free(tmp);
    return ORC_OK;
}

/* ------------------------------------------------------------------------------------------
 * Pieces of the dense-MLP SGD step that are not GEMMs (all f32, contiguous):
 *  - relu with gradient mask: ops/unary/mod.rs:213-252 (mask = x > 0 ? 1 : 0 on the
 *    pre-activation), relu backend/cpu.rs:651-657
 *  - SGD update: grad/optim.rs:30-50: update = grad * lr (own rounding), then p -= update
 *  - u8 -> f32 conversion followed by x / 255 (examples/mnist/src/main.rs:108-111)
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_relu_mask_f32(float *x, float *mask, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float v = x[i];
        mask[i] = v > 0.0f ? 1.0f : 0.0f;
        x[i] = v > 0.0f ? v : 0.0f;
    }
}
ORC_API void orc_sgd_update_f32(float *p, const float *g, float lr, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float u = g[i] * lr;
        p[i] = p[i] - u;
    }
}
ORC_API void orc_relu_mask_f64(double *x, double *mask, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        double v = x[i];
        mask[i] = v > 0.0 ? 1.0 : 0.0;
        x[i] = v > 0.0 ? v : 0.0;
    }
}
ORC_API void orc_sgd_update_f64(double *p, const double *g, double lr, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        double u = g[i] * lr;
        p[i] = p[i] - u;
    }
}
ORC_API void orc_u8_to_f32_div(const uint8_t *src, float *dst, float divisor, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = (float)src[i] / divisor;
}

/* ------------------------------------------------------------------------------------------
 * The per-element maps the autograd builds on the host: a zeros tensor of the input's shape, then
 * for every coordinate (row-major)
 *   kind 1 relu        map = input > 0 ? 1 : 0            ops/unary/mod.rs:236-252
 *   kind 2 abs         map = input > 0 ? 1 : -1           ops/unary/mod.rs:213-235
 *   kind 3 leaky_relu  map = input > 0 ? 1 : slope        ops/scalar/mod.rs:149-166
 *   kind 4 reciprocal  map = 1 / input                    ops/broadcast/div.rs:583-587
 * Integer 1 / 0 panics in the reference; here it yields 0 (precondition, as for division).
 * ---------------------------------------------------------------------------------------- */
#define DEF_GRAD_MASK(S, T, CODE)                                                            \
    static void mask_##S(int kind, T slope, const T *src, size_t rank, const size_t *shape,  \
                         const ptrdiff_t *strides, size_t offset, T *dst) {                  \
        if (meta_size(rank, shape) == 0) return;                                             \
        off_iter it;                                                                         \
        it_init(&it, rank, shape, strides, offset);                                          \
        size_t i = 0;                                                                        \
        while (!it.done) {                                                                   \
            T v = src[it.off];                                                               \
            /* (T)0.5 == 0 tells an integer type from a float one */                         \
            if (kind == 4) dst[i++] = ((T)0.5 == (T)0 && v == (T)0) ? (T)0 : bin_##S(ORC_DIV, (T)1, v); \
            else dst[i++] = v > (T)0 ? (T)1 : (kind == 1 ? (T)0 : (kind == 2 ? (T)-1 : slope)); \
            it_next(&it);                                                                    \
        }                                                                                    \
    }
FOR_ALL_TYPES(DEF_GRAD_MASK)

ORC_API int orc_grad_mask(int dtype, int kind, const void *value, const void *src, size_t rank,
                          const size_t *shape, const ptrdiff_t *strides, size_t offset, void *dst) {
    if (rank > ORC_MAX_RANK) return ORC_ERR_DIM;
    if (kind < 1 || kind > 4 || (kind == 3 && !value)) return ORC_ERR_OP;
    /* -T::ONE needs a signed type; boolean has no division */
    if (kind == 2 && (dtype == ORC_U8 || dtype == ORC_U16 || dtype == ORC_U32 || dtype == ORC_U64 ||
                      dtype == ORC_U128 || dtype == ORC_BOOL))
        return ORC_ERR_DTYPE;
    if (kind == 4 && dtype == ORC_BOOL) return ORC_ERR_DTYPE;
    switch (dtype) {
#define CASE_MASK(S, T, CODE)                                                                \
    case CODE: {                                                                             \
        T v; memset(&v, 0, sizeof v);                                                        \
        if (value) memcpy(&v, value, sizeof v);                                              \
        mask_##S(kind, v, (const T *)src, rank, shape, strides, offset, (T *)dst);           \
        return ORC_OK;                                                                       \
    }
        FOR_ALL_TYPES(CASE_MASK)
    }
    return ORC_ERR_DTYPE;
}

/* ------------------------------------------------------------------------------------------
 * dtype conversion: Backend::convert (backend/cpu.rs:221-233) applies DTypeConversion::convert
 * (core/value.rs:270-290) per element.  The per-type rules (core/value.rs:333-395 floats,
 * 402-460 integers, 770-822 boolean) are Rust `as` casts:
 *   float -> int   : round() (half away from zero) then a saturating cast, NaN -> 0
 *   float -> float : nearest-even (f64 -> f32 may overflow to inf)
 *   int   -> int   : two's-complement truncation / sign extension
 *   int   -> float : nearest-even of the exact value
 *   any   -> bool  : value != 0 (NaN is true);  bool -> any : 0 or 1
 * Every source value is widened exactly (integers to 128 bits, f32 to f64) and cast from there,
 * which gives the same result as the direct cast.
 * ---------------------------------------------------------------------------------------- */
typedef struct { int kind; /* 0 unsigned, 1 signed, 2 float */ u128_t u; i128_t s; double f; } wide_t;

static wide_t cv_load(int dtype, const void *p, size_t i) {
    wide_t w = {0, 0, 0, 0.0};
    switch (dtype) {
        case ORC_U8: w.u = ((const uint8_t *)p)[i]; break;
        case ORC_U16: w.u = ((const uint16_t *)p)[i]; break;
        case ORC_U32: w.u = ((const uint32_t *)p)[i]; break;
        case ORC_U64: w.u = ((const uint64_t *)p)[i]; break;
        case ORC_U128: w.u = ((const u128_t *)p)[i]; break;
        case ORC_BOOL: w.u = ((const uint8_t *)p)[i] ? 1 : 0; break;
        case ORC_I8: w.kind = 1; w.s = ((const int8_t *)p)[i]; break;
        case ORC_I16: w.kind = 1; w.s = ((const int16_t *)p)[i]; break;
        case ORC_I32: w.kind = 1; w.s = ((const int32_t *)p)[i]; break;
        case ORC_I64: w.kind = 1; w.s = ((const int64_t *)p)[i]; break;
        case ORC_I128: w.kind = 1; w.s = ((const i128_t *)p)[i]; break;
        case ORC_F32: w.kind = 2; w.f = (double)((const float *)p)[i]; break;
        default: w.kind = 2; w.f = ((const double *)p)[i]; break;
    }
    return w;
}

/* saturating float -> integer of `bits` bits; the value is already integral */
static u128_t cv_sat_unsigned(double r, int bits) {
    if (!(r > 0.0)) return 0; /* negative, zero and NaN */
    if (r >= ldexp(1.0, bits)) return bits == 128 ? ~(u128_t)0 : (((u128_t)1 << bits) - 1);
    return (u128_t)r;
}
static i128_t cv_sat_signed(double r, int bits) {
    if (r != r) return 0;
    i128_t lo = -((i128_t)1 << (bits - 2)) * 2, hi = -(lo + 1);
    if (r >= ldexp(1.0, bits - 1)) return hi;
    if (r <= -ldexp(1.0, bits - 1)) return lo;
    return (i128_t)r;
}

#define CV_INT_DST(T, BITS, SIGNED)                                                          \
    {                                                                                        \
        T v;                                                                                 \
        if (w.kind == 0) v = (T)w.u;                                                         \
        else if (w.kind == 1) v = (T)w.s;                                                    \
        else if (SIGNED) v = (T)cv_sat_signed(round(w.f), BITS);                             \
        else v = (T)cv_sat_unsigned(round(w.f), BITS);                                       \
        ((T *)dst)[i] = v;                                                                   \
    }                                                                                        \
    break

ORC_API int orc_convert(int src_dtype, int dst_dtype, const void *src, void *dst, size_t n) {
    if (src_dtype < 0 || src_dtype > ORC_BOOL || dst_dtype < 0 || dst_dtype > ORC_BOOL) return ORC_ERR_DTYPE;
    for (size_t i = 0; i < n; ++i) {
        wide_t w = cv_load(src_dtype, src, i);
        switch (dst_dtype) {
            case ORC_U8: CV_INT_DST(uint8_t, 8, 0);
            case ORC_U16: CV_INT_DST(uint16_t, 16, 0);
            case ORC_U32: CV_INT_DST(uint32_t, 32, 0);
            case ORC_U64: CV_INT_DST(uint64_t, 64, 0);
            case ORC_U128: CV_INT_DST(u128_t, 128, 0);
            case ORC_I8: CV_INT_DST(int8_t, 8, 1);
            case ORC_I16: CV_INT_DST(int16_t, 16, 1);
            case ORC_I32: CV_INT_DST(int32_t, 32, 1);
            case ORC_I64: CV_INT_DST(int64_t, 64, 1);
            case ORC_I128: CV_INT_DST(i128_t, 128, 1);
            case ORC_F32:
                /* an f32 source round-trips through f64 unchanged */
                ((float *)dst)[i] = w.kind == 0 ? (float)w.u : (w.kind == 1 ? (float)w.s : (float)w.f);
                break;
            case ORC_F64:
                ((double *)dst)[i] = w.kind == 0 ? (double)w.u : (w.kind == 1 ? (double)w.s : w.f);
                break;
            default:
                ((uint8_t *)dst)[i] = w.kind == 0 ? (w.u != 0) : (w.kind == 1 ? (w.s != 0) : (w.f != 0.0));
                break;
        }
    }
    return ORC_OK;
}

/* Plain row-major GEMM with f64 accumulation, C[m,n] = A[m,k] * B[k,n]; ta/tb read the operand
 * transposed.  Stands in for OpenBLAS sgemm in the oracle's MLP step; tolerance-checked only. */
ORC_API void orc_gemm_f32(const float *a, const float *b, float *c, size_t m, size_t k, size_t n,
                          int ta, int tb) {
    for (size_t i = 0; i < m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            double s = 0.0;
            for (size_t p = 0; p < k; ++p) {
                float av = ta ? a[p * m + i] : a[i * k + p];
                float bv = tb ? b[j * k + p] : b[p * n + j];
                s += (double)av * (double)bv;
            }
            c[i * n + j] = (float)s;
        }
    }
}

/* f64 ground-truth helpers used by the tolerance tests */
ORC_API double orc_sum_f64_of_f32(const float *x, size_t n) {
    double s = 0.0;
    for (size_t i = 0; i < n; ++i) s += (double)x[i];
    return s;
}
ORC_API double orc_abs_sum_f64_of_f32(const float *x, size_t n) {
    double s = 0.0;
    for (size_t i = 0; i < n; ++i) s += fabs((double)x[i]);
    return s;
}
