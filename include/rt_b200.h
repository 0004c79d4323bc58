/*
 * rt_b200.h -- C ABI of librt_b200.so: the tensor hot path of rtensors (scalar elementwise ops,
 * N-d broadcast binary ops over strided / permuted / negative-step views, axis and full
 * reductions, mean_l1_loss, reduce-to-shape) as hand-written CUDA for sm_100a.
 *
 * Two layers:
 *   v1  the `launch_*` symbols of the reference's own kernel library, with identical
 *       signatures, so the reference's `backend/cuda.rs` (bindgen over cuda/include/kernels.h)
 *       links against this library unchanged.  Declared in rt_b200_v1.h.
 *   v2  `rtb_*`: status-returning, stream-aware, host-side shape/stride (no per-call device
 *       uploads), out-of-place and fused forms.  This is what new host glue should call.
 *
 * Conventions (both layers): every data pointer is a DEVICE pointer owned by the caller; the
 * library never frees or retains it.  Offsets, shapes and strides are in ELEMENTS; strides may
 * be zero (broadcast) or negative (reversed slice).  Work is enqueued on a stream and returns
 * before completion; the caller synchronises before reading results on the host.  Kernels are
 * launched with programmatic stream serialization and wait for their predecessor on the stream
 * before touching memory: stream order is exactly that of plain launches, consecutive library
 * kernels merely overlap their launch gaps.  After a first eager pass (workspace and allocator
 * blocks in place) a sequence of calls can be captured into a CUDA graph.  Citations
 * give the reference interface each entry point replaces (paths relative to libs/rtensors/ of
 * aheschl1/rtensors).
 */
#ifndef RT_B200_H
#define RT_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes = the reference's DType discriminants (src/core/value.rs:567-581) */
typedef enum {
    RTB_U8 = 0, RTB_I8 = 1, RTB_U16 = 2, RTB_I16 = 3, RTB_U32 = 4, RTB_U128 = 5, RTB_I32 = 6,
    RTB_U64 = 7, RTB_I64 = 8, RTB_I128 = 9, RTB_F32 = 10, RTB_F64 = 11, RTB_BOOL = 12
} rtb_dtype;

/* binary op codes = OpCode (cuda/include/common.h:6-11) = BinaryOpType (src/ops/base.rs:7-12).
 * Codes 4..7 exist for rtb_scalar_op only: the remaining scalar families of the Backend trait
 * (src/backend/mod.rs:339-346; log / log1p / elu are f32 / f64 only, leaky_relu any dtype). */
typedef enum {
    RTB_ADD = 0, RTB_SUB = 1, RTB_MUL = 2, RTB_DIV = 3,
    RTB_LOG = 4, RTB_LOG1P = 5, RTB_LEAKY_RELU = 6, RTB_ELU = 7
} rtb_binop;

/* unary ops (src/backend/mod.rs:311-368), computed with the CPU backend's formulae
 * (src/backend/cpu.rs:485-724).  0..3 are on the hot path and exist for integer types too;
 * 4..30 are the remaining float-only families. */
typedef enum {
    RTB_NEG = 0, RTB_RELU = 1, RTB_ABS = 2, RTB_SIGN = 3,
    RTB_SIGMOID = 4, RTB_TANH = 5, RTB_SQRT = 6, RTB_SIN = 7, RTB_COS = 8, RTB_TAN = 9, RTB_ASIN = 10,
    RTB_ACOS = 11, RTB_ATAN = 12, RTB_SINH = 13, RTB_COSH = 14, RTB_ASINH = 15, RTB_ACOSH = 16, RTB_ATANH = 17,
    RTB_RSQRT = 18, RTB_RECIPROCAL = 19, RTB_SQUARE = 20, RTB_CUBE = 21, RTB_EXP = 22, RTB_LN = 23, RTB_LN1P = 24,
    RTB_FLOOR = 25, RTB_CEIL = 26, RTB_ROUND = 27, RTB_TRUNC = 28, RTB_EXPM1 = 29, RTB_SILU = 30
} rtb_unop;

/* reduction codes = ReductionOpCode (cuda/include/common.h:19-30) */
typedef enum {
    RTB_SUM = 1, RTB_PROD = 2, RTB_MAX = 3, RTB_MIN = 4, RTB_MEAN = 5,
    /* accepted by the *_ex entry points only */
    RTB_VARIANCE = 6, RTB_LOGSUMEXP = 7, RTB_NORM = 8, RTB_ARGMAX = 9, RTB_ARGMIN = 10
} rtb_redop;

/* = ReductionSettings (cuda/include/common.h:13-17), the record the reference front end fills for
 * var / pop_var / std / norm (src/ops/reduction/mod.rs:413-510): variance and std divide by n-1
 * when `unbiased`; `is_std` takes the square root; norm_type 1 = sum |x|, 2 = sqrt(sum x^2).
 * A NULL settings pointer means {unbiased = true, is_std = false, norm_type = 2}. */
typedef struct rtb_reduce_settings {
    bool unbiased;
    bool is_std;
    int norm_type;
} rtb_reduce_settings;

/* status codes; rtb_last_error_string() gives the text for the calling thread's last failure */
typedef enum {
    RTB_OK = 0,
    RTB_ERR_INVALID = -1,     /* bad argument (null pointer, rank too large, unknown code)          */
    RTB_ERR_DTYPE = -2,       /* op not defined for this dtype (e.g. boolean division, int reduce)  */
    RTB_ERR_BROADCAST = -3,   /* shapes are not broadcastable (TensorError::BroadcastError)          */
    RTB_ERR_BOUNDS = -4,      /* slice / extent out of bounds (TensorError::IdxOutOfBounds)          */
    RTB_ERR_DIM = -5,         /* dimension out of range (TensorError::InvalidDim / WrongDims)        */
    RTB_ERR_SHAPE = -6,       /* invalid shape or zero step (TensorError::InvalidShape)              */
    RTB_ERR_NONCONTIG = -7,   /* reduction input must be contiguous (src/backend/mod.rs:385-389)     */
    RTB_ERR_CUDA = -8,        /* a CUDA runtime call failed (TensorError::CudaError)                 */
    RTB_ERR_ALLOC = -9,       /* device allocation failed                                            */
    RTB_ERR_TOO_LARGE = -10   /* size beyond a stated limit                                          */
} rtb_status;

#define RTB_MAX_RANK 128 /* rank cap of the reference (src/core/primitives.rs:377-383) */

typedef struct rtb_ctx rtb_ctx;

/* ---- context: one per device, created once (replaces the per-call CudaContext + cuBLAS handle
 *      churn of `CUDA_BACKENDS`, src/backend/cuda.rs:38-51,155-162) ------------------------- */
int rtb_ctx_create(int device, rtb_ctx **out);
void rtb_ctx_destroy(rtb_ctx *ctx);
/* stream all later calls on this ctx are enqueued on (a cudaStream_t; NULL = legacy default).
 * The context's scratch state (reduction workspace, allocator free list) is ordered by the stream
 * only, so a change of stream makes the new stream wait (event record + cudaStreamWaitEvent) for
 * everything this context has enqueued on the old one: calls through one context keep one total
 * order on the device whatever streams they were issued on.  Use one context per stream for work
 * that should overlap. */
int rtb_ctx_set_stream(rtb_ctx *ctx, void *stream);
void *rtb_ctx_get_stream(rtb_ctx *ctx);
int rtb_ctx_device(rtb_ctx *ctx);
int rtb_ctx_sm_count(rtb_ctx *ctx);
/* waits for the ctx stream (Cuda::sync, src/backend/cuda.rs:164-185) and for the transfer lanes of the
 * host-buffer operations, if any were used */
int rtb_ctx_sync(rtb_ctx *ctx);
/* number of kernels this ctx has launched since creation (bench bookkeeping) */
uint64_t rtb_ctx_launch_count(rtb_ctx *ctx);
/* CUDA graphs and the context's device memory.  A captured sequence of calls bakes in the address
 * of the reduction workspace and of the allocator blocks it used.  Rules that keep replays valid:
 *   - a workspace that is outgrown is retired, not freed (freed with the context), so an old graph
 *     never touches released memory;
 *   - during stream capture nothing is allocated or freed: a call that would have to grow the
 *     workspace, rtb_alloc without a cached block, and rtb_release_cached return an error instead
 *     (run the sequence once eagerly, or reserve the workspace, before capturing);
 *   - rtb_ctx_workspace_generation() changes whenever the workspace moved or cached blocks were
 *     released; a holder of a graph compares it with the value at capture time and records the
 *     graph again when it differs (an outdated graph is still safe for the workspace, but uses
 *     the old, smaller one and may hold released allocator blocks after rtb_release_cached). */
int rtb_ctx_reserve_workspace(rtb_ctx *ctx, size_t bytes);
uint64_t rtb_ctx_workspace_generation(rtb_ctx *ctx);
const char *rtb_last_error_string(void);

/* ---- device memory: caching allocator (Backend::alloc / alloc_from_slice / dump / copy,
 *      src/backend/cuda.rs:668-836).  rtb_alloc returns UNINITIALISED memory: out-of-place ops
 *      write every output element, so the zero-upload of `zeros_on`
 *      (src/core/primitives.rs:463-468) is not needed. ---------------------------------------- */
int rtb_alloc(rtb_ctx *ctx, size_t bytes, void **out);
int rtb_free(rtb_ctx *ctx, void *ptr);
int rtb_release_cached(rtb_ctx *ctx);
int rtb_h2d(rtb_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
int rtb_d2h(rtb_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes); /* synchronises */
int rtb_d2d(rtb_ctx *ctx, void *dst_dev, const void *src_dev, size_t bytes);

/* ---- host-buffer operations: inputs and results in HOST memory.  The reference moves whole tensors
 *      with one blocking copy each way (alloc_from_slice / dump, src/backend/cuda.rs:668-680, 770-788).
 *      Here the context owns an upload lane and a download lane (two more streams) and a pool of
 *      device blocks; uploads, kernels and copy-outs of independent work run concurrently and are
 *      ordered by events.  Every call below only enqueues, except rtb_host_wait and rtb_host_trim;
 *      rtb_ctx_sync also waits for the lanes.  Host memory should be page-locked (rtb_host_alloc, or
 *      rtb_host_pin for memory the caller already owns): a copy from pageable memory is staged by the
 *      driver and does not overlap.  None of these calls can be captured into a CUDA graph.
 *      The pool: a request takes a free block of its kind (upload target / result) that fits and is at
 *      most twice as large, preferring one whose last readers are done; while every candidate is still in
 *      use, up to three blocks per kind and size class are allocated rather than waited for (an upload, the
 *      kernels and a copy-out each hold one), after which the request shares a busy block and its first
 *      writer waits.  Blocks stay in the pool until rtb_host_trim or rtb_ctx_destroy; when the device has no
 *      room for a block that is needed, the pool's unused blocks are given back first.
 *
 *      rtb_host_stage_in    takes a block from the pool and starts host -> block on the upload lane.
 *                           The compute stream does NOT wait for it until rtb_host_ready(block): work
 *                           enqueued in between runs while the upload is in flight.
 *      rtb_host_scratch     a block of the pool for a result the compute stream will write.
 *      rtb_host_stage_out   device -> host on the download lane, after everything enqueued on the compute
 *                           stream so far; src may be any device address (a pool block, part of one, or
 *                           memory of rtb_alloc, which the caller then keeps alive until the copy is done).
 *      rtb_host_release     gives a block back.  Kernels and copy-outs already enqueued on it stay valid:
 *                           the block's next user waits for them.
 *      rtb_host_join        the compute stream waits for both lanes (stream-ordered completion).
 *      rtb_host_wait        the host waits for the compute stream and both lanes.
 *      rtb_host_trim        waits, then frees the pool's unused blocks.
 *
 *      rtb_host_reduce_view rtb_reduce_view_ex of a tensor whose buffer (src_len elements) is in host
 *                           memory; the result (one element, or the view's shape without `axis`; uint64_t
 *                           for argmax / argmin) is written to dst_host.
 *      rtb_host_broadcast   rtb_broadcast with operand BUFFERS (left_len / right_len elements) in host
 *                           memory and the result written row-major to dst_host, restricted to indices
 *                           [begin, end) of the outermost output dim (dst_host receives only that part: a
 *                           rank's share).  The output never exists as a whole on the device: it is
 *                           produced in stages of about 64 MiB (rtb_host_set_stage_bytes; a stage is
 *                           at least one index of the outermost dim) into a ring of three blocks, stage
 *                           k's copy-out running behind stage k+1's kernel. -------------------------- */
int rtb_host_alloc(size_t bytes, void **out);
int rtb_host_free(void *ptr);
int rtb_host_pin(void *ptr, size_t bytes);
int rtb_host_unpin(void *ptr);
int rtb_host_stage_in(rtb_ctx *ctx, const void *src_host, size_t bytes, void **dev_out);
int rtb_host_scratch(rtb_ctx *ctx, size_t bytes, void **dev_out);
int rtb_host_ready(rtb_ctx *ctx, const void *dev);
int rtb_host_stage_out(rtb_ctx *ctx, const void *src_dev, void *dst_host, size_t bytes);
int rtb_host_release(rtb_ctx *ctx, void *dev);
int rtb_host_join(rtb_ctx *ctx);
int rtb_host_wait(rtb_ctx *ctx);
int rtb_host_trim(rtb_ctx *ctx);
int rtb_host_set_stage_bytes(rtb_ctx *ctx, size_t bytes);
int rtb_host_reduce_view(rtb_ctx *ctx, int dtype, int redop, const rtb_reduce_settings *settings, const void *src_host,
                         size_t src_len, size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t offset,
                         ptrdiff_t axis, void *dst_host);
int rtb_host_broadcast(rtb_ctx *ctx, int dtype, int binop, const void *left_host, size_t left_len, const ptrdiff_t *stride_l,
                       size_t off_l, const void *right_host, size_t right_len, const ptrdiff_t *stride_r, size_t off_r,
                       void *dst_host, size_t rank, const size_t *shape, size_t begin, size_t end);

/* ---- view arithmetic (host only; no CUDA call).  out arrays need room for `rank` (+1 for
 *      unsqueeze) entries. --------------------------------------------------------------------- */
/* shape_to_stride, src/core/meta.rs:495-503 */
void rtb_meta_contiguous_strides(size_t rank, const size_t *shape, ptrdiff_t *strides);
/* is_contiguous_relaxed, src/core/meta.rs:526-541 (|stride| dense, size-1 dims ignored) */
int rtb_meta_is_contiguous(size_t rank, const size_t *shape, const ptrdiff_t *strides);
/* compute_sliced_parameters, src/core/slice.rs:145-239 */
int rtb_meta_slice(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t offset, size_t dim,
                   int has_start, size_t start, int has_end, size_t end, ptrdiff_t step, size_t *out_rank,
                   size_t *out_shape, ptrdiff_t *out_strides, size_t *out_offset);
/* compute_permuted_parameters, src/core/tensor.rs:909-941 */
int rtb_meta_permute(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t ndims,
                     const size_t *dims, size_t *out_shape, ptrdiff_t *out_strides);
/* compute_unsqueezed_parameters / compute_squeezed_parameters, src/core/tensor.rs:973-1027
 * (squeeze: dim < 0 removes every size-1 dim) */
int rtb_meta_unsqueeze(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t dim,
                       size_t *out_shape, ptrdiff_t *out_strides);
int rtb_meta_squeeze(size_t rank, const size_t *shape, const ptrdiff_t *strides, ptrdiff_t dim,
                     size_t *out_rank, size_t *out_shape, ptrdiff_t *out_strides);
/* compute_broadcasted_params, src/ops/broadcast/mod.rs:13-55 */
int rtb_broadcast_params(size_t ra, const size_t *shape_a, const ptrdiff_t *strides_a, size_t rb,
                         const size_t *shape_b, const ptrdiff_t *strides_b, size_t *out_rank,
                         size_t *out_shape, ptrdiff_t *out_strides_a, ptrdiff_t *out_strides_b);
/* check_extent, src/backend/remote/server.rs:241-270: every addressed element of the view lies
 * inside a buffer of buf_len elements */
int rtb_meta_check_extent(size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t offset,
                          size_t buf_len);

/* The launch plan the library derives for an elementwise / broadcast call: size-1 dims dropped,
 * negative output strides flipped, dims sorted by output stride, adjacent dims merged.  Exposed
 * so the planner can be tested without a GPU.  kernel: 0 = nothing to do, 1 = flat vectorised
 * (one contiguous run, operands share their 16-byte phase), 3 = tiled row kernel. */
typedef struct {
    int kernel;
    int rank;             /* collapsed rank, 1..8 */
    uint64_t shape[8];    /* shape[rank-1] is the inner (fastest) dim */
    int64_t stride_d[8], stride_l[8], stride_r[8];
    int64_t base_d, base_l, base_r; /* element offsets after flipping */
    int vec;              /* elements per 16-byte vector for this dtype */
    int mode_d, mode_l, mode_r; /* inner-dim access: 0 contig-vector 1 contig-scalar 2 reversed-vector
                                   3 reversed-scalar 4 broadcast(stride 0) 5 strided */
    int tile_x, tile_y;   /* thread tile of the row kernel */
    uint64_t n_rows, n_col_chunks, grid;
    int fast, ux;         /* row kernel: lean instantiation? 128-bit columns per thread per row (1 or 4) */
} rtb_plan;
int rtb_plan_elementwise(int dtype, int n_inputs, size_t rank, const size_t *shape, const ptrdiff_t *stride_d,
                         size_t off_d, uintptr_t ptr_d, const ptrdiff_t *stride_l, size_t off_l, uintptr_t ptr_l,
                         const ptrdiff_t *stride_r, size_t off_r, uintptr_t ptr_r, rtb_plan *out);

/* ---- elementwise, in place over a view (Backend::scalar_apply_{add,sub,mul,div},
 *      apply_{neg,relu,abs,sign}, fill: src/backend/mod.rs:146-177, 239-268; kernels
 *      cuda/kernels/elementwise/{scalar,unary,fill}.cu).  `value` points at one host element of
 *      the dtype.  The three layout classes of the reference dispatcher (contiguous, 1-D strided,
 *      N-d) are one call here; a view whose strides are dense up to sign is walked from its
 *      lowest address. --------------------------------------------------------------------------- */
int rtb_scalar_op(rtb_ctx *ctx, int dtype, int binop, void *buf, const void *value, size_t rank,
                  const size_t *shape, const ptrdiff_t *strides, size_t offset);
int rtb_unary_op(rtb_ctx *ctx, int dtype, int unop, void *buf, size_t rank, const size_t *shape,
                 const ptrdiff_t *strides, size_t offset);
int rtb_fill(rtb_ctx *ctx, int dtype, void *buf, const void *value, size_t rank, const size_t *shape,
             const ptrdiff_t *strides, size_t offset);
/* row-major copy of a view into contiguous memory (view_to_contiguous,
 * src/core/tensor.rs:299-325: one kernel instead of a memcpy per run / per element) */
int rtb_copy_view(rtb_ctx *ctx, int dtype, const void *src, size_t rank, const size_t *shape,
                  const ptrdiff_t *strides, size_t offset, void *dst);

/* ---- broadcast binary op (Backend::broadcast, src/backend/mod.rs:296-309; kernel
 *      cuda/kernels/elementwise/binary/broadcast.cu:3-109).  All three views carry the OUTPUT
 *      shape; operands are pre-broadcast by stride 0 on broadcast dims.  dst may alias left (or
 *      right) with the same strides and offset (in-place form).
 *      Overlap rule: an input whose bytes intersect dst's while it walks them differently
 *      (a += a.T, v += v reversed, a window shifted over itself) is first copied out by the
 *      strided copy kernel into a block of the context allocator, so EVERY INPUT ELEMENT IS READ
 *      BEFORE ANY OUTPUT ELEMENT IS WRITTEN.  The reference's CPU walk (src/backend/cpu.rs:292-352)
 *      reads such an operand while writing it, element by element in row-major order, so its result
 *      depends on that order; TensorBase cannot express the call (the right-hand view would borrow
 *      the tensor that `+=` borrows mutably), only the raw Backend::broadcast can, whose contract
 *      (src/backend/mod.rs:296-302) does not define it.  Views of one buffer that interleave without
 *      sharing an element take the same copy and give the same result as the reference. -------- */
int rtb_broadcast(rtb_ctx *ctx, int dtype, int binop, const void *left, const ptrdiff_t *stride_l, size_t off_l,
                  const void *right, const ptrdiff_t *stride_r, size_t off_r, void *dst,
                  const ptrdiff_t *stride_d, size_t off_d, size_t rank, const size_t *shape);

/* ---- reductions, f32 / f64 (Backend::apply_reduce_contiguous_flat / _nd,
 *      src/backend/mod.rs:357-409; kernels cuda/kernels/reduction/reduce.cu:239-274, 463-513).
 *      src is row-major contiguous; flat: src[start .. start+len] -> dst[0]; axis: src viewed as
 *      [outer, r, inner] from `offset` -> dst[outer*inner].  mean divides by (T)(float)count
 *      (src/core/value.rs:54-56).  max/min start from the lowest/highest finite value and use
 *      the CPU comparisons `v > acc` / `v < acc` (src/ops/reduction/mod.rs:43-120). ------------ */
int rtb_reduce_flat(rtb_ctx *ctx, int dtype, int redop, const void *src, size_t start, size_t len, void *dst);
int rtb_reduce_axis(rtb_ctx *ctx, int dtype, int redop, const void *src, size_t offset, size_t outer, size_t r,
                    size_t inner, void *dst);

/* ---- reduction over a VIEW (ReductionOp::*_at / TotalReductionOp on a non-contiguous tensor,
 *      src/ops/reduction/mod.rs:351-360, where the reference first copies the view with
 *      `contiguous()`).  axis < 0: full reduction into dst[0]; otherwise dst is row-major over the
 *      view's shape with dim `axis` kept as 1.  Views that are [outer, R, inner] with a contiguous
 *      inner run under arbitrary outer / R strides (slices, reversed or permuted outer dims,
 *      transposed matrices) are reduced in place with no copy; any other view is materialised by
 *      the strided copy kernel into a temporary from the context allocator first.  f32 / f64. ---- */
int rtb_reduce_view(rtb_ctx *ctx, int dtype, int redop, const void *src, size_t rank, const size_t *shape,
                    const ptrdiff_t *strides, size_t offset, ptrdiff_t axis, void *dst);

/* ---- every reduction code, 1..10 (launch_flat_contiguous_reduce_*, launch_nd_reduce_contiguous_*,
 *      launch_flat_contiguous_argmax_*, launch_nd_argmax_contiguous_*; cuda/kernels/reduction/
 *      reduce.cu:992-1026).  Codes 1..5 behave as in the entry points above.  Codes 6..10 exist only
 *      in the reference's CUDA backend -- its CPU backend panics for them
 *      (src/ops/reduction/mod.rs:187-197, src/backend/cpu.rs:452-482):
 *        VARIANCE   Welford states merged pairwise; m2 / (n-1) or m2 / n, denominator 1 when that
 *                   would be <= 0 (so one element gives 0), square root when is_std;
 *        LOGSUMEXP  max + log(sum exp(x - max)) in one pass.  The reference's FLAT launcher has no
 *                   logsumexp case and leaves its output untouched (reduce.cu:795-843); here the
 *                   flat form computes the same formula over the whole range;
 *        NORM       type 1 or 2;
 *        ARGMAX / ARGMIN  dst is uint64_t: the FIRST position along the reduced run of the largest
 *                   / smallest value, 0 if no element compares above lowest() / below max() (the
 *                   reference picks among equal values by thread order once the run is longer
 *                   than its block size, reduce.cu:897-926).
 *      f32 / f64.  The _view form follows rtb_reduce_view; argmax / argmin of a full reduction over
 *      a view count positions in the view's row-major order. ---------------------------------- */
int rtb_reduce_flat_ex(rtb_ctx *ctx, int dtype, int redop, const rtb_reduce_settings *settings, const void *src,
                       size_t start, size_t len, void *dst);
int rtb_reduce_axis_ex(rtb_ctx *ctx, int dtype, int redop, const rtb_reduce_settings *settings, const void *src,
                       size_t offset, size_t outer, size_t r, size_t inner, void *dst);
int rtb_reduce_view_ex(rtb_ctx *ctx, int dtype, int redop, const rtb_reduce_settings *settings, const void *src,
                       size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t offset, ptrdiff_t axis,
                       void *dst);

/* ---- fused broadcast binary op + axis reduction: dst = reduce_axis(left (op) right) without writing
 *      the broadcast result (the reference materialises it: Backend::broadcast into a fresh
 *      tensor, then `*_at(axis)`, src/ops/broadcast/add.rs:441-477 + src/ops/reduction/mod.rs:351-360).
 *      Both views carry the OUTPUT shape with stride 0 on broadcast dims; dst is row-major with
 *      dim `axis` kept as 1.  f32 / f64.  Views whose dims before / after the axis do not each
 *      collapse to one run fall back to materialise + reduce. ---------------------------------- */
int rtb_broadcast_reduce(rtb_ctx *ctx, int dtype, int binop, int redop, const void *left, const ptrdiff_t *stride_l,
                         size_t off_l, const void *right, const ptrdiff_t *stride_r, size_t off_r, size_t rank,
                         const size_t *shape, size_t axis, void *dst);

/* ---- full reduction without any device allocation.  NO COUNTERPART IN THE REFERENCE (its flat
 *      reduction allocates and frees CUB scratch on every call, cuda/kernels/reduction/reduce.cu:
 *      239-274).  For hosts that must not, or cannot, call cudaMalloc: all device memory already
 *      given to their own pool, a loop that may not take cudaMalloc's device-wide synchronisation,
 *      or a runtime that forbids allocations by foreign libraries.  Same result contract as
 *      rtb_reduce_flat (src[start .. start+len] -> dst[0], f32 / f64, SUM PROD MAX MIN MEAN), but
 *      the partial results live in a 64.25 KiB array inside the library image instead of the
 *      context workspace; it needs no rtb_ctx and runs on `stream` (a cudaStream_t, NULL = legacy
 *      default) of the CURRENT device.
 *      Limits and rules: len <= RTB_NOALLOC_MAX_LEN, larger is refused with RTB_ERR_TOO_LARGE;
 *      every GPU that loads the library holds the array until exit; all calls on a device share
 *      it, so calls whose kernels could overlap (other streams, other threads) race and must be
 *      ordered by the caller; the first call on each device looks up the array's device address
 *      and should be made outside any stream capture.  Calls no cudaMalloc / cudaFree. --------- */
#define RTB_NOALLOC_MAX_LEN ((size_t)1 << 29)
int rtb_reduce_flat_noalloc(int dtype, int redop, const void *src, size_t start, size_t len, void *dst,
                            void *stream);

/* ---- fused L1 loss of two same-length contiguous tensors (L1::l1 + attach_l1_grad,
 *      src/ops/broadcast/l1.rs:16-77: five launches and two temporaries in the reference).
 *      reduction: 0 mean, 1 sum.  grad_map (may be NULL) receives sign(a-b), divided by
 *      (T)(float)n for the mean form; sign(0) = 0 as on the CPU backend. ----------------------- */
int rtb_l1_loss(rtb_ctx *ctx, int dtype, const void *a, const void *b, size_t n, int reduction, void *loss,
                void *grad_map);

/* ---- reduce-to-shape for broadcast gradients (inverse_broadcast_gradient,
 *      src/grad/backwards.rs:512-538): sums the contiguous `upstream` of `shape` over every dim
 *      whose operand stride is 0; out receives prod(out_shape) elements, the reduced dims kept as
 *      size 1.  f32 / f64. ------------------------------------------------------------------------ */
int rtb_reduce_to_shape(rtb_ctx *ctx, int dtype, const void *upstream, size_t rank, const size_t *shape,
                        const ptrdiff_t *operand_strides, void *out, size_t *out_shape);

/* ---- fused pieces of the autograd MLP step (f32) --------------------------------------------
 * relu with its gradient mask in one pass (relu_inplace + the per-element mask loop of
 * src/ops/unary/mod.rs:213-252): x = x>0 ? x : 0, mask = x>0 ? 1 : 0 */
int rtb_relu_mask_f32(rtb_ctx *ctx, float *x, float *mask, size_t n);
/* One dense layer's `+ bias` (Backend::broadcast with the (1, cols) bias, src/ops/broadcast/add.rs:14-46),
 * relu_inplace and its gradient map (src/ops/unary/mod.rs:56-92, 234-252) in one pass over a dense
 * row-major (rows, cols) activation: z = relu(z + bias), mask = (z + bias) > 0 ? 1 : 0.  The bits equal
 * those of the three separate calls (one IEEE add, then `x > 0` tests).  f32 / f64. */
int rtb_bias_relu_mask(rtb_ctx *ctx, int dtype, void *z, const void *bias, void *mask, size_t rows, size_t cols);
/* The per-element maps the reference's autograd fills with one host get and one host set per
 * element, as one kernel each.  dst is a dense row-major tensor of the view's shape; src is any
 * view (strided, permuted, negative step); src and dst must not overlap.
 *   RTB_MASK_RELU        dst = src > 0 ? 1 : 0          any dtype        (src/ops/unary/mod.rs:236-252)
 *   RTB_MASK_ABS         dst = src > 0 ? 1 : -1         signed / float   (src/ops/unary/mod.rs:213-235;
 *                                                        0 and NaN give -1 as there)
 *   RTB_MASK_LEAKY_RELU  dst = src > 0 ? 1 : *value     any dtype        (src/ops/scalar/mod.rs:149-166)
 *   RTB_MASK_RECIPROCAL  dst = 1 / src                  all but boolean  (src/ops/broadcast/div.rs:583-587;
 *                                                        integer 1/0 gives 0 where the reference panics)
 * `value` points at one element of `dtype` (the slope) for RTB_MASK_LEAKY_RELU and is ignored
 * otherwise (may be NULL). */
enum { RTB_MASK_RELU = 1, RTB_MASK_ABS = 2, RTB_MASK_LEAKY_RELU = 3, RTB_MASK_RECIPROCAL = 4 };
int rtb_grad_mask(rtb_ctx *ctx, int dtype, int kind, const void *value, const void *src, size_t rank,
                  const size_t *shape, const ptrdiff_t *strides, size_t offset, void *dst);
/* SGD::step (src/grad/optim.rs:30-50): u = g*lr rounded, then p = p - u (no FMA) */
int rtb_sgd_update_f32(rtb_ctx *ctx, float *p, const float *g, float lr, size_t n);
/* the same two for f64 (the reference's relu map and SGD::step are generic over the float type) */
int rtb_relu_mask_f64(rtb_ctx *ctx, double *x, double *mask, size_t n);
int rtb_sgd_update_f64(rtb_ctx *ctx, double *p, const double *g, double lr, size_t n);
/* Backend::convert u8 -> f32 followed by `/ divisor` (src/backend/cuda.rs:790-812,
 * examples/mnist/src/main.rs:108-111) */
int rtb_u8_to_f32_div(rtb_ctx *ctx, const uint8_t *src, float *dst, float divisor, size_t n);
/* Backend::convert (src/backend/mod.rs:234; CPU loop src/backend/cpu.rs:221-233; the reference's
 * CUDA form is one host read + one host write per element, src/backend/cuda.rs:682-703): dst[i] =
 * src[i] converted by the rules of DTypeConversion (src/core/value.rs:270-290, 333-460, 770-822),
 * i.e. Rust `as` casts: float -> integer rounds half away from zero and saturates (NaN -> 0),
 * integer -> integer truncates, integer -> float and f64 -> f32 round to nearest even, anything
 * -> boolean is `!= 0`, boolean -> anything is 0 or 1.  Any pair of the 13 dtypes, equal ones
 * included.  Both buffers hold n elements, must not overlap, and must be aligned to their element
 * type (16 bytes for the 128-bit integers).  TensorBase::into_dtype (src/core/primitives.rs:527-538)
 * is alloc + this call. */
int rtb_convert(rtb_ctx *ctx, int src_dtype, int dst_dtype, const void *src, void *dst, size_t n);

/* ---- multi-GPU (new; the reference is single-device: `Cuda::new()` -> device 0 with
 *      `// TODO multiple devices`, src/backend/cuda.rs:155-162, 815-818).  One rank per GPU, one
 *      communicator per context.  The path shards by slabs with no data-path collective for
 *      elementwise and broadcast work; ranks exchange data only where a reduction runs across the
 *      cut dim.
 *
 *      Host-only partition arithmetic (no CUDA call, testable on a CPU): ------------------------- */
/* rank `part` of `parts` gets the half-open slab [*begin, *end) of an extent, earlier ranks taking
 * the remainder */
void rtb_shard_range(size_t extent, size_t parts, size_t part, size_t *begin, size_t *end);
/* the outermost dim of an output shape with extent >= parts (the slab dim); -1 if none */
int rtb_shard_pick_dim(size_t rank, const size_t *shape, size_t parts);
/* this rank's slab of a broadcast binary op whose operand views carry the output shape: the slab
 * shape, its range along the cut dim and both operands' offsets inside the slab (an operand with
 * stride 0 along the cut dim is replicated).  Returns the cut dim or -1 (no dim is wide enough:
 * part 0 owns everything, the others get an empty slab). */
int rtb_mg_slab(size_t rank, const size_t *shape, const ptrdiff_t *stride_l, size_t off_l, const ptrdiff_t *stride_r,
                size_t off_r, size_t parts, size_t part, size_t *slab_shape, size_t *begin, size_t *end,
                size_t *slab_off_l, size_t *slab_off_r);
/* which dim to cut for a reduction over `axis`: a kept dim with extent >= parts when there is one
 * (every rank owns its outputs, no exchange), else the reduced dim (partials are combined), else -1 */
int rtb_mg_pick_reduce_dim(size_t rank, const size_t *shape, size_t axis, size_t parts);

/*      Communicator.  rtb_mg_unique_id makes the 128-byte id on one rank; the host carries it to
 *      the others over whatever channel it has (a store, MPI, a file) and every rank calls
 *      rtb_mg_init with its own context (collective).  NCCL is bound at run time (libnccl.so.2,
 *      the copy already loaded in the process if there is one).  Besides the NCCL communicator the
 *      context gets a 4 MiB exchange buffer that every rank maps from every other rank (CUDA IPC):
 *      small results travel through it as plain stores over NVLink from inside the library's own
 *      kernels, with no collective launch (*peer_mapped of rtb_mg_info; when the mapping is not
 *      possible -- or RTB_MG_NO_PEER=1 is set in the environment of any rank -- everything falls
 *      back to NCCL).  All rtb_mg_* calls below are collective: every
 *      rank makes the same calls in the same order on its context's stream. ------------------------ */
#define RTB_MG_ID_BYTES 128
#define RTB_MG_MAX_RANKS 16
#define RTB_MG_SMALL_BYTES 65536 /* largest partial vector the peer exchange takes */
int rtb_mg_unique_id(void *id_out /* RTB_MG_ID_BYTES */);
int rtb_mg_init(rtb_ctx *ctx, int nranks, int rank, const void *id /* RTB_MG_ID_BYTES */);
int rtb_mg_finalize(rtb_ctx *ctx); /* collective; rtb_ctx_destroy releases without one */
int rtb_mg_info(rtb_ctx *ctx, int *nranks, int *rank, int *peer_mapped);
/* Failure detection.  Every wait inside an exchange kernel is bounded by this limit (default 2 s).
 * A wait that runs out does not trap or hang: the kernel sets status bit 0, writes NaN as the
 * result and returns.  rtb_mg_status synchronises the stream and returns the bits (bit 1: NCCL
 * reported an asynchronous error).  After a failure the ranks' exchange epochs may differ;
 * rtb_mg_realign (collective, NCCL) brings them back in step and clears the status. */
int rtb_mg_set_wait_ns(rtb_ctx *ctx, uint64_t ns);
int rtb_mg_status(rtb_ctx *ctx, unsigned int *bits);
int rtb_mg_realign(rtb_ctx *ctx);
/* in-place all-reduce of n elements with NCCL on the context's stream (SUM PROD MAX MIN, MEAN =
 * sum / (T)(float)mean_count for f32 / f64); u8 i8 i32 u32 i64 u64 f32 f64 */
int rtb_mg_allreduce(rtb_ctx *ctx, int dtype, int redop, void *buf, size_t n, size_t mean_count);
/* the same on the communicator's own side stream, ordered after the work enqueued so far:
 * _begin returns at once and later calls on the context overlap the transfer; _join makes the
 * context's stream wait for every transfer begun since the last join.  Capturable in a CUDA graph
 * (fork / join by events). */
int rtb_mg_allreduce_begin(rtb_ctx *ctx, int dtype, int redop, void *buf, size_t n, size_t mean_count);
int rtb_mg_allreduce_join(rtb_ctx *ctx);
/* in-place combine of a per-rank partial result: f32 / f64 buffers of up to RTB_MG_SMALL_BYTES go
 * through the peer exchange (folded in rank order, so every rank gets the same bits), anything
 * else through NCCL */
int rtb_mg_combine(rtb_ctx *ctx, int dtype, int redop, void *buf, size_t n, size_t mean_count);
/* full reduction of a tensor whose flat range is split across the ranks: src[start .. start +
 * local_len] is this rank's part of global_len elements; every rank gets the result in dst[0].
 * One launch: the last CTA of the local reduction exchanges the per-GPU totals through peer memory
 * (TotalReductionOp over the whole tensor, src/ops/reduction/mod.rs:208-257). */
int rtb_mg_reduce_flat(rtb_ctx *ctx, int dtype, int redop, const void *src, size_t start, size_t local_len,
                       size_t global_len, void *dst);
/* axis reduction whose REDUCED dim is split across the ranks: this rank holds r_local of the
 * global_r rows of [outer, r, inner] (element (o, k, i) at offset + o*outer_stride + k*row_stride + i);
 * dst receives the combined outer*inner results on every rank.  (When a kept dim is split instead,
 * rtb_reduce_axis / rtb_reduce_view on the slab needs no exchange.) */
int rtb_mg_reduce_axis(rtb_ctx *ctx, int dtype, int redop, const void *src, size_t offset, size_t outer, size_t r_local,
                       size_t inner, ptrdiff_t outer_stride, ptrdiff_t row_stride, size_t global_r, void *dst);
/* rtb_l1_loss over tensors split across the ranks: the loss is the global one on every rank and
 * the gradient map is scaled by the global element count */
int rtb_mg_l1_loss(rtb_ctx *ctx, int dtype, const void *a, const void *b, size_t local_n, size_t global_n,
                   int reduction, void *loss, void *grad_map);

#ifdef __cplusplus
}
#endif
#endif /* RT_B200_H */
