//! `rt_b200_sys` -- raw FFI declarations of librt_b200.so's v2 C ABI (`include/rt_b200.h`) for the Rust
//! host of rtensors: what `libs/rtensors/src/backend/cuda.rs` binds instead of the bindgen output of
//! `cuda/include/kernels.h` once it calls `rtb_*` instead of the `launch_*` launchers.
//!
//! NOT COMPILED where this repository is built (its image has no Rust toolchain): the file is text
//! that mirrors the C header one declaration per function.  `tests/test_rust_binding_text.py` checks
//! that every function declared in `include/rt_b200.h` appears here with the same name and parameter
//! count, and that every name here is exported by the shared library.
//!
//! Link with `println!("cargo:rustc-link-lib=dylib=rt_b200");` in `build.rs`.
//! `dtype` arguments are `T::DTYPE as c_int` (the crate's own `DType` discriminants,
//! src/core/value.rs:567-581), `binop` is `BinaryOpType::to_op_code()`, `redop` is
//! `ReductionOpTypes::get_code()`.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_int, c_uint, c_void};

/// Opaque library context: one per device, created once (replaces `CUDA_BACKENDS`' per-call contexts).
#[repr(C)]
pub struct rtb_ctx {
    _private: [u8; 0],
}

/// = `ReductionSettings` (cuda/include/common.h:13-17).
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rtb_reduce_settings {
    pub unbiased: bool,
    pub is_std: bool,
    pub norm_type: c_int,
}

/// The launch plan `rtb_plan_elementwise` reports (host-only; for tests and diagnostics).
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct rtb_plan {
    pub kernel: c_int,
    pub rank: c_int,
    pub shape: [u64; 8],
    pub stride_d: [i64; 8],
    pub stride_l: [i64; 8],
    pub stride_r: [i64; 8],
    pub base_d: i64,
    pub base_l: i64,
    pub base_r: i64,
    pub vec: c_int,
    pub mode_d: c_int,
    pub mode_l: c_int,
    pub mode_r: c_int,
    pub tile_x: c_int,
    pub tile_y: c_int,
    pub n_rows: u64,
    pub n_col_chunks: u64,
    pub grid: u64,
    pub fast: c_int,
    pub ux: c_int,
}

pub const RTB_OK: c_int = 0;
pub const RTB_ERR_INVALID: c_int = -1;
pub const RTB_ERR_DTYPE: c_int = -2;
pub const RTB_ERR_BROADCAST: c_int = -3;
pub const RTB_ERR_BOUNDS: c_int = -4;
pub const RTB_ERR_DIM: c_int = -5;
pub const RTB_ERR_SHAPE: c_int = -6;
pub const RTB_ERR_NONCONTIG: c_int = -7;
pub const RTB_ERR_CUDA: c_int = -8;
pub const RTB_ERR_ALLOC: c_int = -9;
pub const RTB_ERR_TOO_LARGE: c_int = -10;
pub const RTB_MAX_RANK: usize = 128;
pub const RTB_MG_ID_BYTES: usize = 128;
pub const RTB_MG_MAX_RANKS: usize = 16;
pub const RTB_MG_SMALL_BYTES: usize = 65536;
pub const RTB_NOALLOC_MAX_LEN: usize = 1 << 29;
pub const RTB_MASK_RELU: c_int = 1;
pub const RTB_MASK_ABS: c_int = 2;
pub const RTB_MASK_LEAKY_RELU: c_int = 3;
pub const RTB_MASK_RECIPROCAL: c_int = 4;

extern "C" {
    pub fn rtb_ctx_create(device: c_int, out: *mut *mut rtb_ctx) -> c_int;
    pub fn rtb_ctx_destroy(ctx: *mut rtb_ctx);
    pub fn rtb_ctx_set_stream(ctx: *mut rtb_ctx, stream: *mut c_void) -> c_int;
    pub fn rtb_ctx_get_stream(ctx: *mut rtb_ctx) -> *mut c_void;
    pub fn rtb_ctx_device(ctx: *mut rtb_ctx) -> c_int;
    pub fn rtb_ctx_sm_count(ctx: *mut rtb_ctx) -> c_int;
    pub fn rtb_ctx_sync(ctx: *mut rtb_ctx) -> c_int;
    pub fn rtb_ctx_launch_count(ctx: *mut rtb_ctx) -> u64;
    pub fn rtb_ctx_reserve_workspace(ctx: *mut rtb_ctx, bytes: usize) -> c_int;
    pub fn rtb_ctx_workspace_generation(ctx: *mut rtb_ctx) -> u64;
    pub fn rtb_last_error_string() -> *const c_char;
    pub fn rtb_alloc(ctx: *mut rtb_ctx, bytes: usize, out: *mut *mut c_void) -> c_int;
    pub fn rtb_free(ctx: *mut rtb_ctx, ptr: *mut c_void) -> c_int;
    pub fn rtb_release_cached(ctx: *mut rtb_ctx) -> c_int;
    pub fn rtb_h2d(ctx: *mut rtb_ctx, dst_dev: *mut c_void, src_host: *const c_void, bytes: usize) -> c_int;
    pub fn rtb_d2h(ctx: *mut rtb_ctx, dst_host: *mut c_void, src_dev: *const c_void, bytes: usize) -> c_int;
    pub fn rtb_d2d(ctx: *mut rtb_ctx, dst_dev: *mut c_void, src_dev: *const c_void, bytes: usize) -> c_int;
    pub fn rtb_meta_contiguous_strides(rank: usize, shape: *const usize, strides: *mut isize);
    pub fn rtb_meta_is_contiguous(rank: usize, shape: *const usize, strides: *const isize) -> c_int;
    pub fn rtb_meta_slice(rank: usize, shape: *const usize, strides: *const isize, offset: usize, dim: usize, has_start: c_int, start: usize, has_end: c_int, end: usize, step: isize, out_rank: *mut usize, out_shape: *mut usize, out_strides: *mut isize, out_offset: *mut usize) -> c_int;
    pub fn rtb_meta_permute(rank: usize, shape: *const usize, strides: *const isize, ndims: usize, dims: *const usize, out_shape: *mut usize, out_strides: *mut isize) -> c_int;
    pub fn rtb_meta_unsqueeze(rank: usize, shape: *const usize, strides: *const isize, dim: usize, out_shape: *mut usize, out_strides: *mut isize) -> c_int;
    pub fn rtb_meta_squeeze(rank: usize, shape: *const usize, strides: *const isize, dim: isize, out_rank: *mut usize, out_shape: *mut usize, out_strides: *mut isize) -> c_int;
    pub fn rtb_broadcast_params(ra: usize, shape_a: *const usize, strides_a: *const isize, rb: usize, shape_b: *const usize, strides_b: *const isize, out_rank: *mut usize, out_shape: *mut usize, out_strides_a: *mut isize, out_strides_b: *mut isize) -> c_int;
    pub fn rtb_meta_check_extent(rank: usize, shape: *const usize, strides: *const isize, offset: usize, buf_len: usize) -> c_int;
    pub fn rtb_plan_elementwise(dtype: c_int, n_inputs: c_int, rank: usize, shape: *const usize, stride_d: *const isize, off_d: usize, ptr_d: usize, stride_l: *const isize, off_l: usize, ptr_l: usize, stride_r: *const isize, off_r: usize, ptr_r: usize, out: *mut rtb_plan) -> c_int;
    pub fn rtb_scalar_op(ctx: *mut rtb_ctx, dtype: c_int, binop: c_int, buf: *mut c_void, value: *const c_void, rank: usize, shape: *const usize, strides: *const isize, offset: usize) -> c_int;
    pub fn rtb_unary_op(ctx: *mut rtb_ctx, dtype: c_int, unop: c_int, buf: *mut c_void, rank: usize, shape: *const usize, strides: *const isize, offset: usize) -> c_int;
    pub fn rtb_fill(ctx: *mut rtb_ctx, dtype: c_int, buf: *mut c_void, value: *const c_void, rank: usize, shape: *const usize, strides: *const isize, offset: usize) -> c_int;
    pub fn rtb_copy_view(ctx: *mut rtb_ctx, dtype: c_int, src: *const c_void, rank: usize, shape: *const usize, strides: *const isize, offset: usize, dst: *mut c_void) -> c_int;
    pub fn rtb_broadcast(ctx: *mut rtb_ctx, dtype: c_int, binop: c_int, left: *const c_void, stride_l: *const isize, off_l: usize, right: *const c_void, stride_r: *const isize, off_r: usize, dst: *mut c_void, stride_d: *const isize, off_d: usize, rank: usize, shape: *const usize) -> c_int;
    pub fn rtb_reduce_flat(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, src: *const c_void, start: usize, len: usize, dst: *mut c_void) -> c_int;
    pub fn rtb_reduce_axis(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, src: *const c_void, offset: usize, outer: usize, r: usize, inner: usize, dst: *mut c_void) -> c_int;
    pub fn rtb_reduce_view(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, src: *const c_void, rank: usize, shape: *const usize, strides: *const isize, offset: usize, axis: isize, dst: *mut c_void) -> c_int;
    pub fn rtb_reduce_flat_ex(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, settings: *const rtb_reduce_settings, src: *const c_void, start: usize, len: usize, dst: *mut c_void) -> c_int;
    pub fn rtb_reduce_axis_ex(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, settings: *const rtb_reduce_settings, src: *const c_void, offset: usize, outer: usize, r: usize, inner: usize, dst: *mut c_void) -> c_int;
    pub fn rtb_reduce_view_ex(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, settings: *const rtb_reduce_settings, src: *const c_void, rank: usize, shape: *const usize, strides: *const isize, offset: usize, axis: isize, dst: *mut c_void) -> c_int;
    pub fn rtb_broadcast_reduce(ctx: *mut rtb_ctx, dtype: c_int, binop: c_int, redop: c_int, left: *const c_void, stride_l: *const isize, off_l: usize, right: *const c_void, stride_r: *const isize, off_r: usize, rank: usize, shape: *const usize, axis: usize, dst: *mut c_void) -> c_int;
    pub fn rtb_reduce_flat_noalloc(dtype: c_int, redop: c_int, src: *const c_void, start: usize, len: usize, dst: *mut c_void, stream: *mut c_void) -> c_int;
    pub fn rtb_l1_loss(ctx: *mut rtb_ctx, dtype: c_int, a: *const c_void, b: *const c_void, n: usize, reduction: c_int, loss: *mut c_void, grad_map: *mut c_void) -> c_int;
    pub fn rtb_reduce_to_shape(ctx: *mut rtb_ctx, dtype: c_int, upstream: *const c_void, rank: usize, shape: *const usize, operand_strides: *const isize, out: *mut c_void, out_shape: *mut usize) -> c_int;
    pub fn rtb_relu_mask_f32(ctx: *mut rtb_ctx, x: *mut f32, mask: *mut f32, n: usize) -> c_int;
    pub fn rtb_bias_relu_mask(ctx: *mut rtb_ctx, dtype: c_int, z: *mut c_void, bias: *const c_void, mask: *mut c_void, rows: usize, cols: usize) -> c_int;
    pub fn rtb_grad_mask(ctx: *mut rtb_ctx, dtype: c_int, kind: c_int, value: *const c_void, src: *const c_void, rank: usize, shape: *const usize, strides: *const isize, offset: usize, dst: *mut c_void) -> c_int;
    pub fn rtb_sgd_update_f32(ctx: *mut rtb_ctx, p: *mut f32, g: *const f32, lr: f32, n: usize) -> c_int;
    pub fn rtb_relu_mask_f64(ctx: *mut rtb_ctx, x: *mut f64, mask: *mut f64, n: usize) -> c_int;
    pub fn rtb_sgd_update_f64(ctx: *mut rtb_ctx, p: *mut f64, g: *const f64, lr: f64, n: usize) -> c_int;
    pub fn rtb_u8_to_f32_div(ctx: *mut rtb_ctx, src: *const u8, dst: *mut f32, divisor: f32, n: usize) -> c_int;
    pub fn rtb_convert(ctx: *mut rtb_ctx, src_dtype: c_int, dst_dtype: c_int, src: *const c_void, dst: *mut c_void, n: usize) -> c_int;
    pub fn rtb_shard_range(extent: usize, parts: usize, part: usize, begin: *mut usize, end: *mut usize);
    pub fn rtb_shard_pick_dim(rank: usize, shape: *const usize, parts: usize) -> c_int;
    pub fn rtb_mg_slab(rank: usize, shape: *const usize, stride_l: *const isize, off_l: usize, stride_r: *const isize, off_r: usize, parts: usize, part: usize, slab_shape: *mut usize, begin: *mut usize, end: *mut usize, slab_off_l: *mut usize, slab_off_r: *mut usize) -> c_int;
    pub fn rtb_mg_pick_reduce_dim(rank: usize, shape: *const usize, axis: usize, parts: usize) -> c_int;
    pub fn rtb_mg_unique_id(id_out: *mut c_void) -> c_int;
    pub fn rtb_mg_init(ctx: *mut rtb_ctx, nranks: c_int, rank: c_int, id: *const c_void) -> c_int;
    pub fn rtb_mg_finalize(ctx: *mut rtb_ctx) -> c_int;
    pub fn rtb_mg_info(ctx: *mut rtb_ctx, nranks: *mut c_int, rank: *mut c_int, peer_mapped: *mut c_int) -> c_int;
    pub fn rtb_mg_set_wait_ns(ctx: *mut rtb_ctx, ns: u64) -> c_int;
    pub fn rtb_mg_status(ctx: *mut rtb_ctx, bits: *mut c_uint) -> c_int;
    pub fn rtb_mg_realign(ctx: *mut rtb_ctx) -> c_int;
    pub fn rtb_mg_allreduce(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, buf: *mut c_void, n: usize, mean_count: usize) -> c_int;
    pub fn rtb_mg_allreduce_begin(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, buf: *mut c_void, n: usize, mean_count: usize) -> c_int;
    pub fn rtb_mg_allreduce_join(ctx: *mut rtb_ctx) -> c_int;
    pub fn rtb_mg_combine(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, buf: *mut c_void, n: usize, mean_count: usize) -> c_int;
    pub fn rtb_mg_reduce_flat(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, src: *const c_void, start: usize, local_len: usize, global_len: usize, dst: *mut c_void) -> c_int;
    pub fn rtb_mg_reduce_axis(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, src: *const c_void, offset: usize, outer: usize, r_local: usize, inner: usize, outer_stride: isize, row_stride: isize, global_r: usize, dst: *mut c_void) -> c_int;
    pub fn rtb_mg_l1_loss(ctx: *mut rtb_ctx, dtype: c_int, a: *const c_void, b: *const c_void, local_n: usize, global_n: usize, reduction: c_int, loss: *mut c_void, grad_map: *mut c_void) -> c_int;


    // host-buffer operations: transfer lanes and the pool of device blocks
    pub fn rtb_host_alloc(bytes: usize, out: *mut *mut c_void) -> c_int;
    pub fn rtb_host_free(ptr: *mut c_void) -> c_int;
    pub fn rtb_host_pin(ptr: *mut c_void, bytes: usize) -> c_int;
    pub fn rtb_host_unpin(ptr: *mut c_void) -> c_int;
    pub fn rtb_host_stage_in(ctx: *mut rtb_ctx, src_host: *const c_void, bytes: usize, dev_out: *mut *mut c_void) -> c_int;
    pub fn rtb_host_scratch(ctx: *mut rtb_ctx, bytes: usize, dev_out: *mut *mut c_void) -> c_int;
    pub fn rtb_host_ready(ctx: *mut rtb_ctx, dev: *const c_void) -> c_int;
    pub fn rtb_host_stage_out(ctx: *mut rtb_ctx, src_dev: *const c_void, dst_host: *mut c_void, bytes: usize) -> c_int;
    pub fn rtb_host_release(ctx: *mut rtb_ctx, dev: *mut c_void) -> c_int;
    pub fn rtb_host_join(ctx: *mut rtb_ctx) -> c_int;
    pub fn rtb_host_wait(ctx: *mut rtb_ctx) -> c_int;
    pub fn rtb_host_trim(ctx: *mut rtb_ctx) -> c_int;
    pub fn rtb_host_set_stage_bytes(ctx: *mut rtb_ctx, bytes: usize) -> c_int;
    pub fn rtb_host_reduce_view(ctx: *mut rtb_ctx, dtype: c_int, redop: c_int, settings: *const rtb_reduce_settings, src_host: *const c_void, src_len: usize, rank: usize, shape: *const usize, strides: *const isize, offset: usize, axis: isize, dst_host: *mut c_void) -> c_int;
    pub fn rtb_host_broadcast(ctx: *mut rtb_ctx, dtype: c_int, binop: c_int, left_host: *const c_void, left_len: usize, stride_l: *const isize, off_l: usize, right_host: *const c_void, right_len: usize, stride_r: *const isize, off_r: usize, dst_host: *mut c_void, rank: usize, shape: *const usize, begin: usize, end: usize) -> c_int;
}

/// Maps a status code to the crate's error type the way `cuda.rs` would:
/// ```ignore
/// fn check(rc: c_int) -> Result<(), TensorError> {
///     if rc == RTB_OK { return Ok(()); }
///     let msg = unsafe { CStr::from_ptr(rtb_last_error_string()) }.to_string_lossy().into_owned();
///     Err(match rc {
///         RTB_ERR_BROADCAST => TensorError::BroadcastError(msg),
///         RTB_ERR_BOUNDS => TensorError::IdxOutOfBounds(msg),
///         RTB_ERR_DIM => TensorError::InvalidDim(msg),
///         RTB_ERR_SHAPE => TensorError::InvalidShape(msg),
///         RTB_ERR_NONCONTIG => TensorError::WrongDims(msg),
///         _ => TensorError::CudaError(msg),
///     })
/// }
/// ```
pub fn status_is_ok(rc: c_int) -> bool {
    rc == RTB_OK
}
