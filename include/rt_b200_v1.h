/*
 * rt_b200_v1.h -- the reference's own launcher symbols for the hot path, re-implemented.
 *
 * Each symbol below has the name and signature the reference declares in
 * libs/rtensors/cuda/include/{scalar,binary,fill}.h, so `libs/rtensors/src/backend/cuda.rs`
 * (which binds them through bindgen over cuda/include/kernels.h, build.rs:537-566) links
 * against librt_b200.so without source changes.  Conventions as in the reference: device
 * pointers; `*_DEV` arrays (shape, stride) are DEVICE memory holding u64 / i64 and are copied
 * back to plan the launch; work goes to the legacy default stream; no status is returned
 * (errors surface at the caller's next synchronisation), except the scratch-allocation flag.
 * `block_size` is accepted and ignored.
 *
 * Covered: every scalar family (add sub mul div log log1p leaky_relu elu, scalar.h:9-96), every
 * unary family (negate relu, scalar.h:99-148; the 29 float-only ones, scalar.h:150-211), fill
 * (fill.h:9-12), broadcast (binary.h:8-20), flat / N-d reductions for f32/f64 -- codes SUM PROD MAX
 * MIN MEAN VARIANCE LOGSUMEXP NORM with their ReductionSettings, and the argmax / argmin launchers
 * (scalar.h:213-228; cuda/kernels/reduction/reduce.cu:992-1026) -- and the allocation flag.
 * Not provided (outside the path): integer matmul; buffer_equal.
 */
#ifndef RT_B200_V1_H
#define RT_B200_V1_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cuda/include/common.h:13-17 and :19-30 -- same layout and numeric codes */
typedef struct RtbV1ReductionSettings { bool unbiased; bool is_std; int norm_type; } RtbV1ReductionSettings;

#define RTB_V1_SCALAR(OP, TYPE, S)                                                                              \
    void launch_##OP##_contiguous_##S(TYPE *data /* already advanced to the first element */, size_t n,         \
                                      TYPE value, unsigned int block_size);                                     \
    void launch_##OP##_strided_##S(TYPE *data, size_t start, ptrdiff_t stride, size_t len, TYPE value,          \
                                   unsigned int block_size);                                                    \
    void launch_##OP##_nd_affine_##S(TYPE *data, size_t offset, const ptrdiff_t *stride_DEV,                    \
                                     const size_t *shape_DEV, size_t rank, size_t size, TYPE value,             \
                                     unsigned int block_size);

#define RTB_V1_UNARY(OP, TYPE, S)                                                                               \
    void launch_##OP##_contiguous_##S(TYPE *data /* buffer base */, size_t start, size_t len,                   \
                                      unsigned int block_size);                                                 \
    void launch_##OP##_strided_##S(TYPE *data, size_t offset, ptrdiff_t stride, size_t len,                     \
                                   unsigned int block_size);                                                    \
    void launch_##OP##_nd_affine_##S(TYPE *data, size_t offset, const ptrdiff_t *stride_DEV,                    \
                                     const size_t *shape_DEV, size_t rank, size_t size, unsigned int block_size);

#define RTB_V1_FILL(TYPE, S)                                                                                    \
    void launch_fill_contiguous_##S(TYPE *data, size_t n, TYPE value, unsigned int block_size);                 \
    void launch_fill_strided_##S(TYPE *data, size_t start, ptrdiff_t stride, size_t len, TYPE value,            \
                                 unsigned int block_size);                                                      \
    void launch_fill_nd_affine_##S(TYPE *data, size_t offset, const ptrdiff_t *stride_DEV,                      \
                                   const size_t *shape_DEV, size_t rank, size_t size, TYPE value,               \
                                   unsigned int block_size);

#define RTB_V1_BROADCAST(TYPE, S)                                                                               \
    void launch_binary_broadcast_elementwise_##S(const TYPE *lbuf, const TYPE *rbuf, TYPE *dbuf, size_t loff,   \
                                                 size_t roff, size_t doff, size_t rank, size_t size,            \
                                                 const ptrdiff_t *lstride_DEV, const ptrdiff_t *rstride_DEV,    \
                                                 const ptrdiff_t *dstride_DEV, const size_t *shape_DEV,         \
                                                 uint8_t op, unsigned int block_size);

#define RTB_V1_REDUCE(TYPE, S)                                                                                  \
    void launch_flat_contiguous_reduce_##S(const TYPE *data, TYPE *out, size_t start, size_t len, uint8_t code, \
                                           const RtbV1ReductionSettings *settings_HOST, unsigned int block_size); \
    void launch_nd_reduce_contiguous_##S(TYPE *data, TYPE *out, size_t offset, size_t outer, size_t r,          \
                                         size_t inner, uint8_t code, const RtbV1ReductionSettings *settings_HOST, \
                                         unsigned int block_size);                                              \
    void launch_flat_contiguous_argmax_##S(const TYPE *data, uint64_t *out, size_t start, size_t len,           \
                                           uint8_t code, const RtbV1ReductionSettings *settings_HOST,           \
                                           unsigned int block_size);                                            \
    void launch_nd_argmax_contiguous_##S(TYPE *data, uint64_t *out, size_t offset, size_t outer, size_t r,      \
                                         size_t inner, uint8_t code, const RtbV1ReductionSettings *settings_HOST, \
                                         unsigned int block_size);

#define RTB_V1_ALL_TYPES(X, ...)                                                                                \
    X(__VA_ARGS__ float, f32) X(__VA_ARGS__ double, f64) X(__VA_ARGS__ uint8_t, u8) X(__VA_ARGS__ uint16_t, u16) \
    X(__VA_ARGS__ uint32_t, u32) X(__VA_ARGS__ uint64_t, u64) X(__VA_ARGS__ __uint128_t, u128)                  \
    X(__VA_ARGS__ int8_t, i8) X(__VA_ARGS__ int16_t, i16) X(__VA_ARGS__ int32_t, i32) X(__VA_ARGS__ int64_t, i64) \
    X(__VA_ARGS__ __int128_t, i128) X(__VA_ARGS__ bool, boolean)

#define RTB_V1_SIGNED_TYPES(X, ...)                                                                             \
    X(__VA_ARGS__ float, f32) X(__VA_ARGS__ double, f64) X(__VA_ARGS__ int8_t, i8) X(__VA_ARGS__ int16_t, i16)  \
    X(__VA_ARGS__ int32_t, i32) X(__VA_ARGS__ int64_t, i64) X(__VA_ARGS__ __int128_t, i128)

#define RTB_V1_COMMA ,
RTB_V1_ALL_TYPES(RTB_V1_SCALAR, add RTB_V1_COMMA)
RTB_V1_ALL_TYPES(RTB_V1_SCALAR, sub RTB_V1_COMMA)
RTB_V1_ALL_TYPES(RTB_V1_SCALAR, mul RTB_V1_COMMA)
RTB_V1_ALL_TYPES(RTB_V1_SCALAR, div RTB_V1_COMMA)
RTB_V1_SIGNED_TYPES(RTB_V1_UNARY, negate RTB_V1_COMMA)
RTB_V1_SIGNED_TYPES(RTB_V1_UNARY, relu RTB_V1_COMMA)
/* the 29 float-only unary families, scalar.h:150-211 */
#define RTB_V1_FLOAT_UNARY(OP) RTB_V1_UNARY(OP, float, f32) RTB_V1_UNARY(OP, double, f64)
RTB_V1_FLOAT_UNARY(abs) RTB_V1_FLOAT_UNARY(sign) RTB_V1_FLOAT_UNARY(sigmoid) RTB_V1_FLOAT_UNARY(tanh)
RTB_V1_FLOAT_UNARY(sqrt) RTB_V1_FLOAT_UNARY(sin) RTB_V1_FLOAT_UNARY(cos) RTB_V1_FLOAT_UNARY(tan)
RTB_V1_FLOAT_UNARY(asin) RTB_V1_FLOAT_UNARY(acos) RTB_V1_FLOAT_UNARY(atan) RTB_V1_FLOAT_UNARY(sinh)
RTB_V1_FLOAT_UNARY(cosh) RTB_V1_FLOAT_UNARY(asinh) RTB_V1_FLOAT_UNARY(acosh) RTB_V1_FLOAT_UNARY(atanh)
RTB_V1_FLOAT_UNARY(rsqrt) RTB_V1_FLOAT_UNARY(reciprocal) RTB_V1_FLOAT_UNARY(square) RTB_V1_FLOAT_UNARY(cube)
RTB_V1_FLOAT_UNARY(exp) RTB_V1_FLOAT_UNARY(ln) RTB_V1_FLOAT_UNARY(ln1p) RTB_V1_FLOAT_UNARY(floor)
RTB_V1_FLOAT_UNARY(ceil) RTB_V1_FLOAT_UNARY(round) RTB_V1_FLOAT_UNARY(trunc) RTB_V1_FLOAT_UNARY(expm1)
RTB_V1_FLOAT_UNARY(silu)
/* remaining scalar families, scalar.h:74-96: log / log1p / elu for f32, f64; leaky_relu for all */
RTB_V1_SCALAR(log, float, f32) RTB_V1_SCALAR(log, double, f64)
RTB_V1_SCALAR(log1p, float, f32) RTB_V1_SCALAR(log1p, double, f64)
RTB_V1_SCALAR(elu, float, f32) RTB_V1_SCALAR(elu, double, f64)
RTB_V1_ALL_TYPES(RTB_V1_SCALAR, leaky_relu RTB_V1_COMMA)
RTB_V1_ALL_TYPES(RTB_V1_FILL)
RTB_V1_ALL_TYPES(RTB_V1_BROADCAST)
RTB_V1_REDUCE(float, f32) RTB_V1_REDUCE(double, f64)

/* scalar.h:226-228: 1 (and clears) if a reduction launcher on this thread skipped its work
 * because its scratch allocation failed */
int rtensors_take_cuda_alloc_error(void);

#ifdef __cplusplus
}
#endif
#endif /* RT_B200_V1_H */
