// C ABI v1: the reference's `launch_*` symbols, implemented on the same planner and kernels as
// the v2 entry points.  Work goes to the legacy default stream of the current device, as the
// reference does; shape / stride arrays arrive in device memory and are copied back to plan.
#include <vector>

#include "rt_b200_v1.h"
#include "rtb_internal.h"

namespace {

using namespace rtb;

thread_local int g_alloc_failed = 0;

void note(int rc) {
    if (rc == RTB_ERR_ALLOC) g_alloc_failed = 1;
}

// device arrays of `rank` 64-bit entries -> host
bool fetch(const void *dev, size_t rank, std::vector<int64_t> &out) {
    out.assign(rank ? rank : 1, 0);
    if (rank == 0) return true;
    return cudaMemcpy(out.data(), dev, rank * sizeof(int64_t), cudaMemcpyDeviceToHost) == cudaSuccess;
}

void ew_view(int dtype, int family, int op, const void *value, size_t vsize, void *data, size_t offset, size_t rank,
             const size_t *shape, const ptrdiff_t *strides) {
    Ctx *ctx = default_ctx();
    if (!ctx) return;
    EwCall call{};
    call.dtype = dtype; call.family = family; call.op = op;
    if (value) std::memcpy(call.value, value, vsize);
    call.d = data; call.l = family == kFamFill ? nullptr : data; call.r = nullptr;
    const ptrdiff_t *sl = family == kFamFill ? nullptr : strides;
    note(run_elementwise(ctx, call, rank, shape, strides, offset, sl, offset, nullptr, 0));
}

void ew_contig(int dtype, int family, int op, const void *value, size_t vsize, void *data, size_t start, size_t n) {
    size_t shape[1] = {n};
    ptrdiff_t strides[1] = {1};
    ew_view(dtype, family, op, value, vsize, data, start, 1, shape, strides);
}

void ew_strided(int dtype, int family, int op, const void *value, size_t vsize, void *data, size_t start,
                ptrdiff_t stride, size_t len) {
    size_t shape[1] = {len};
    ptrdiff_t strides[1] = {stride};
    ew_view(dtype, family, op, value, vsize, data, start, 1, shape, strides);
}

void ew_nd(int dtype, int family, int op, const void *value, size_t vsize, void *data, size_t offset,
           const ptrdiff_t *stride_dev, const size_t *shape_dev, size_t rank) {
    if (rank > RTB_MAX_RANK) return;
    std::vector<int64_t> st, sh;
    if (!fetch(stride_dev, rank, st) || !fetch(shape_dev, rank, sh)) return;
    std::vector<size_t> shape(sh.begin(), sh.end());
    std::vector<ptrdiff_t> strides(st.begin(), st.end());
    ew_view(dtype, family, op, value, vsize, data, offset, rank, shape.data(), strides.data());
}

void broadcast_v1(int dtype, const void *l, const void *r, void *d, size_t loff, size_t roff, size_t doff,
                  size_t rank, const ptrdiff_t *ls_dev, const ptrdiff_t *rs_dev, const ptrdiff_t *ds_dev,
                  const size_t *shape_dev, uint8_t op) {
    Ctx *ctx = default_ctx();
    if (!ctx || rank > RTB_MAX_RANK) return;
    std::vector<int64_t> ls, rs, ds, sh;
    if (!fetch(ls_dev, rank, ls) || !fetch(rs_dev, rank, rs) || !fetch(ds_dev, rank, ds) || !fetch(shape_dev, rank, sh))
        return;
    std::vector<size_t> shape(sh.begin(), sh.end());
    std::vector<ptrdiff_t> sl(ls.begin(), ls.end()), sr(rs.begin(), rs.end()), sd(ds.begin(), ds.end());
    EwCall call{};
    call.dtype = dtype; call.family = kFamBinary; call.op = op;
    call.d = d; call.l = l; call.r = r;
    note(run_elementwise(ctx, call, rank, shape.data(), sd.data(), doff, sl.data(), loff, sr.data(), roff));
}

rtb_reduce_settings settings_of(const RtbV1ReductionSettings *s) {
    rtb_reduce_settings r{true, false, 2};
    if (s) { r.unbiased = s->unbiased; r.is_std = s->is_std; r.norm_type = s->norm_type; }
    return r;
}

// codes 1..5 and, for the flat form, 6 (variance) and 8 (norm) as dispatch_flat_contiguous_reduce
// has them (cuda/kernels/reduction/reduce.cu:795-843); code 7 (logsumexp) is computed too, where
// the reference's flat dispatcher silently leaves `out` untouched.
void reduce_flat_v1(int dtype, const void *data, void *out, size_t start, size_t len, uint8_t code,
                    const RtbV1ReductionSettings *settings) {
    Ctx *ctx = default_ctx();
    if (!ctx) return;
    const char *p = (const char *)data + start * dtype_size(dtype);
    if (code >= RTB_VARIANCE && code <= RTB_NORM) {
        rtb_reduce_settings st = settings_of(settings);
        note(launch_reduce_ext(ctx, dtype, code, &st, p, 1, len, 1, 0, 1, out));
        return;
    }
    note(launch_reduce_flat(ctx, dtype, code, p, len, out));
}

void reduce_nd_v1(int dtype, const void *data, void *out, size_t offset, size_t outer, size_t r, size_t inner,
                  uint8_t code, const RtbV1ReductionSettings *settings) {
    Ctx *ctx = default_ctx();
    if (!ctx || outer == 0 || inner == 0) return;
    const char *p = (const char *)data + offset * dtype_size(dtype);
    if (code >= RTB_VARIANCE && code <= RTB_NORM) {
        rtb_reduce_settings st = settings_of(settings);
        note(launch_reduce_ext(ctx, dtype, code, &st, p, outer, r, inner, (ptrdiff_t)(r * inner), (ptrdiff_t)inner, out));
        return;
    }
    note(launch_reduce_axis(ctx, dtype, code, p, outer, r, inner, out));
}

// launch_flat_contiguous_argmax_* / launch_nd_argmax_contiguous_* (reduce.cu:992-1008): codes 9, 10
void argreduce_v1(int dtype, const void *data, uint64_t *out, size_t offset, size_t outer, size_t r, size_t inner,
                  uint8_t code) {
    Ctx *ctx = default_ctx();
    if (!ctx || outer == 0 || inner == 0) return;
    if (code != RTB_ARGMAX && code != RTB_ARGMIN) return;  // the reference launches nothing for other codes
    note(launch_reduce_ext(ctx, dtype, code, nullptr, (const char *)data + offset * dtype_size(dtype), outer, r, inner,
                           (ptrdiff_t)(r * inner), (ptrdiff_t)inner, out));
}

}  // namespace

#define V1_SCALAR_IMPL(OPNAME, OPCODE, TYPE, S, DT)                                                               \
    RTB_API void launch_##OPNAME##_contiguous_##S(TYPE *data, size_t n, TYPE value, unsigned int) {               \
        ew_contig(DT, rtb::kFamScalar, OPCODE, &value, sizeof value, data, 0, n);                                 \
    }                                                                                                             \
    RTB_API void launch_##OPNAME##_strided_##S(TYPE *data, size_t start, ptrdiff_t stride, size_t len, TYPE value, \
                                               unsigned int) {                                                    \
        ew_strided(DT, rtb::kFamScalar, OPCODE, &value, sizeof value, data, start, stride, len);                  \
    }                                                                                                             \
    RTB_API void launch_##OPNAME##_nd_affine_##S(TYPE *data, size_t offset, const ptrdiff_t *stride,              \
                                                 const size_t *shape, size_t rank, size_t, TYPE value,            \
                                                 unsigned int) {                                                  \
        ew_nd(DT, rtb::kFamScalar, OPCODE, &value, sizeof value, data, offset, stride, shape, rank);              \
    }

#define V1_UNARY_IMPL(OPNAME, OPCODE, TYPE, S, DT)                                                                \
    RTB_API void launch_##OPNAME##_contiguous_##S(TYPE *data, size_t start, size_t len, unsigned int) {           \
        ew_contig(DT, rtb::kFamUnary, OPCODE, nullptr, 0, data, start, len);                                      \
    }                                                                                                             \
    RTB_API void launch_##OPNAME##_strided_##S(TYPE *data, size_t offset, ptrdiff_t stride, size_t len,           \
                                               unsigned int) {                                                    \
        ew_strided(DT, rtb::kFamUnary, OPCODE, nullptr, 0, data, offset, stride, len);                            \
    }                                                                                                             \
    RTB_API void launch_##OPNAME##_nd_affine_##S(TYPE *data, size_t offset, const ptrdiff_t *stride,              \
                                                 const size_t *shape, size_t rank, size_t, unsigned int) {        \
        ew_nd(DT, rtb::kFamUnary, OPCODE, nullptr, 0, data, offset, stride, shape, rank);                         \
    }

#define V1_FILL_IMPL(TYPE, S, DT)                                                                                 \
    RTB_API void launch_fill_contiguous_##S(TYPE *data, size_t n, TYPE value, unsigned int) {                     \
        ew_contig(DT, rtb::kFamFill, 0, &value, sizeof value, data, 0, n);                                        \
    }                                                                                                             \
    RTB_API void launch_fill_strided_##S(TYPE *data, size_t start, ptrdiff_t stride, size_t len, TYPE value,      \
                                         unsigned int) {                                                          \
        ew_strided(DT, rtb::kFamFill, 0, &value, sizeof value, data, start, stride, len);                         \
    }                                                                                                             \
    RTB_API void launch_fill_nd_affine_##S(TYPE *data, size_t offset, const ptrdiff_t *stride, const size_t *shape, \
                                           size_t rank, size_t, TYPE value, unsigned int) {                       \
        ew_nd(DT, rtb::kFamFill, 0, &value, sizeof value, data, offset, stride, shape, rank);                     \
    }

#define V1_BROADCAST_IMPL(TYPE, S, DT)                                                                            \
    RTB_API void launch_binary_broadcast_elementwise_##S(                                                         \
        const TYPE *lbuf, const TYPE *rbuf, TYPE *dbuf, size_t loff, size_t roff, size_t doff, size_t rank, size_t, \
        const ptrdiff_t *lstride, const ptrdiff_t *rstride, const ptrdiff_t *dstride, const size_t *shape,        \
        uint8_t op, unsigned int) {                                                                               \
        broadcast_v1(DT, lbuf, rbuf, dbuf, loff, roff, doff, rank, lstride, rstride, dstride, shape, op);         \
    }

#define V1_PER_TYPE(TYPE, S, DT)                                                                                  \
    V1_SCALAR_IMPL(add, RTB_ADD, TYPE, S, DT)                                                                     \
    V1_SCALAR_IMPL(sub, RTB_SUB, TYPE, S, DT)                                                                     \
    V1_SCALAR_IMPL(mul, RTB_MUL, TYPE, S, DT)                                                                     \
    V1_SCALAR_IMPL(div, RTB_DIV, TYPE, S, DT)                                                                     \
    V1_SCALAR_IMPL(leaky_relu, RTB_LEAKY_RELU, TYPE, S, DT)                                                       \
    V1_FILL_IMPL(TYPE, S, DT)                                                                                     \
    V1_BROADCAST_IMPL(TYPE, S, DT)

V1_PER_TYPE(float, f32, RTB_F32)
V1_PER_TYPE(double, f64, RTB_F64)
V1_PER_TYPE(uint8_t, u8, RTB_U8)
V1_PER_TYPE(uint16_t, u16, RTB_U16)
V1_PER_TYPE(uint32_t, u32, RTB_U32)
V1_PER_TYPE(uint64_t, u64, RTB_U64)
V1_PER_TYPE(__uint128_t, u128, RTB_U128)
V1_PER_TYPE(int8_t, i8, RTB_I8)
V1_PER_TYPE(int16_t, i16, RTB_I16)
V1_PER_TYPE(int32_t, i32, RTB_I32)
V1_PER_TYPE(int64_t, i64, RTB_I64)
V1_PER_TYPE(__int128_t, i128, RTB_I128)
V1_PER_TYPE(bool, boolean, RTB_BOOL)

#define V1_SIGNED(TYPE, S, DT)                                                                                    \
    V1_UNARY_IMPL(negate, RTB_NEG, TYPE, S, DT)                                                                   \
    V1_UNARY_IMPL(relu, RTB_RELU, TYPE, S, DT)
V1_SIGNED(float, f32, RTB_F32)
V1_SIGNED(double, f64, RTB_F64)
V1_SIGNED(int8_t, i8, RTB_I8)
V1_SIGNED(int16_t, i16, RTB_I16)
V1_SIGNED(int32_t, i32, RTB_I32)
V1_SIGNED(int64_t, i64, RTB_I64)
V1_SIGNED(__int128_t, i128, RTB_I128)
#define V1_FLOAT_UNARY(OPNAME, OPCODE)                                                                            \
    V1_UNARY_IMPL(OPNAME, OPCODE, float, f32, RTB_F32)                                                            \
    V1_UNARY_IMPL(OPNAME, OPCODE, double, f64, RTB_F64)
V1_FLOAT_UNARY(abs, RTB_ABS) V1_FLOAT_UNARY(sign, RTB_SIGN) V1_FLOAT_UNARY(sigmoid, RTB_SIGMOID)
V1_FLOAT_UNARY(tanh, RTB_TANH) V1_FLOAT_UNARY(sqrt, RTB_SQRT) V1_FLOAT_UNARY(sin, RTB_SIN) V1_FLOAT_UNARY(cos, RTB_COS)
V1_FLOAT_UNARY(tan, RTB_TAN) V1_FLOAT_UNARY(asin, RTB_ASIN) V1_FLOAT_UNARY(acos, RTB_ACOS) V1_FLOAT_UNARY(atan, RTB_ATAN)
V1_FLOAT_UNARY(sinh, RTB_SINH) V1_FLOAT_UNARY(cosh, RTB_COSH) V1_FLOAT_UNARY(asinh, RTB_ASINH)
V1_FLOAT_UNARY(acosh, RTB_ACOSH) V1_FLOAT_UNARY(atanh, RTB_ATANH) V1_FLOAT_UNARY(rsqrt, RTB_RSQRT)
V1_FLOAT_UNARY(reciprocal, RTB_RECIPROCAL) V1_FLOAT_UNARY(square, RTB_SQUARE) V1_FLOAT_UNARY(cube, RTB_CUBE)
V1_FLOAT_UNARY(exp, RTB_EXP) V1_FLOAT_UNARY(ln, RTB_LN) V1_FLOAT_UNARY(ln1p, RTB_LN1P) V1_FLOAT_UNARY(floor, RTB_FLOOR)
V1_FLOAT_UNARY(ceil, RTB_CEIL) V1_FLOAT_UNARY(round, RTB_ROUND) V1_FLOAT_UNARY(trunc, RTB_TRUNC)
V1_FLOAT_UNARY(expm1, RTB_EXPM1) V1_FLOAT_UNARY(silu, RTB_SILU)

V1_SCALAR_IMPL(log, RTB_LOG, float, f32, RTB_F32) V1_SCALAR_IMPL(log, RTB_LOG, double, f64, RTB_F64)
V1_SCALAR_IMPL(log1p, RTB_LOG1P, float, f32, RTB_F32) V1_SCALAR_IMPL(log1p, RTB_LOG1P, double, f64, RTB_F64)
V1_SCALAR_IMPL(elu, RTB_ELU, float, f32, RTB_F32) V1_SCALAR_IMPL(elu, RTB_ELU, double, f64, RTB_F64)

#define V1_REDUCE_IMPL(TYPE, S, DT)                                                                               \
    RTB_API void launch_flat_contiguous_reduce_##S(const TYPE *data, TYPE *out, size_t start, size_t len,         \
                                                   uint8_t code, const RtbV1ReductionSettings *st, unsigned int) { \
        reduce_flat_v1(DT, data, out, start, len, code, st);                                                      \
    }                                                                                                             \
    RTB_API void launch_nd_reduce_contiguous_##S(TYPE *data, TYPE *out, size_t offset, size_t outer, size_t r,    \
                                                 size_t inner, uint8_t code, const RtbV1ReductionSettings *st,    \
                                                 unsigned int) {                                                  \
        reduce_nd_v1(DT, data, out, offset, outer, r, inner, code, st);                                           \
    }                                                                                                             \
    RTB_API void launch_flat_contiguous_argmax_##S(const TYPE *data, uint64_t *out, size_t start, size_t len,     \
                                                   uint8_t code, const RtbV1ReductionSettings *, unsigned int) {  \
        argreduce_v1(DT, data, out, start, 1, len, 1, code);                                                      \
    }                                                                                                             \
    RTB_API void launch_nd_argmax_contiguous_##S(TYPE *data, uint64_t *out, size_t offset, size_t outer, size_t r, \
                                                 size_t inner, uint8_t code, const RtbV1ReductionSettings *,      \
                                                 unsigned int) {                                                  \
        argreduce_v1(DT, data, out, offset, outer, r, inner, code);                                               \
    }
V1_REDUCE_IMPL(float, f32, RTB_F32)
V1_REDUCE_IMPL(double, f64, RTB_F64)

RTB_API int rtensors_take_cuda_alloc_error(void) {
    int v = g_alloc_failed;
    g_alloc_failed = 0;
    return v;
}
