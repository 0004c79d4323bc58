//! `cuda_b200.rs` -- a `Backend` for rtensors whose every device operation is one call into
//! librt_b200.so (`include/rt_b200.h`, declared for Rust in `rt_b200_sys.rs`).  It is meant to sit at
//! `libs/rtensors/src/backend/cuda_b200.rs` next to `cuda.rs` and to be selected like it
//! (`pub type CudaTensor<T> = TensorBase<T, CudaB200>;`), or to replace the bodies of `cuda.rs`
//! method by method.
//!
//! NOT COMPILED where this repository is built (its image has no Rust toolchain).  It is written
//! against the trait as it stands in `src/backend/mod.rs:216-472`; what it shows is the shape of the
//! host side once the library is underneath:
//!   * one context per device, created once (`CONTEXTS`), instead of a `CudaContext` and a cuBLAS
//!     handle per tensor constructor (`src/backend/cuda.rs:38-51`);
//!   * no shape / stride uploads: the library takes them as host slices (`cuda.rs:1024-1173` allocates
//!     and uploads four index arrays per broadcast call);
//!   * the three layout entry points of every op family (`_contiguous`, `_1d_strided`, `_nd`) collapse
//!     into one call -- the library's planner picks the kernel;
//!   * buffers come from the library's caching allocator and are returned to it on drop.
//! `matmul` and `apply_conv_2d` are not on this path and keep their `cuda.rs` implementations
//! (cuBLAS; the slow convolution fallback).
#![allow(dead_code)]

use std::ffi::CStr;
use std::marker::PhantomData;
use std::os::raw::{c_int, c_void};
use std::ptr;
use std::sync::{Arc, LazyLock, Mutex};

use paste::paste;

use super::rt_b200_sys::*;
use crate::{
    backend::Backend,
    core::{
        primitives::DeviceType,
        tensor::TensorError,
        value::{TensorValue, WeightValue},
        Dim, MetaTensor,
    },
    ops::{
        base::BinaryOpType,
        reduction::{NormType, ReductionOpTypes},
    },
};

/// Codes of `rtb_unop` (include/rt_b200.h); the scalar families use `rtb_binop` codes 0..7.
mod unop {
    pub const NEG: i32 = 0;
    pub const RELU: i32 = 1;
    pub const ABS: i32 = 2;
    pub const SIGN: i32 = 3;
    pub const SIGMOID: i32 = 4;
    pub const TANH: i32 = 5;
    pub const SQRT: i32 = 6;
    pub const SIN: i32 = 7;
    pub const COS: i32 = 8;
    pub const TAN: i32 = 9;
    pub const ASIN: i32 = 10;
    pub const ACOS: i32 = 11;
    pub const ATAN: i32 = 12;
    pub const SINH: i32 = 13;
    pub const COSH: i32 = 14;
    pub const ASINH: i32 = 15;
    pub const ACOSH: i32 = 16;
    pub const ATANH: i32 = 17;
    pub const RSQRT: i32 = 18;
    pub const RECIPROCAL: i32 = 19;
    pub const SQUARE: i32 = 20;
    pub const CUBE: i32 = 21;
    pub const EXP: i32 = 22;
    pub const LN: i32 = 23;
    pub const LN1P: i32 = 24;
    pub const FLOOR: i32 = 25;
    pub const CEIL: i32 = 26;
    pub const ROUND: i32 = 27;
    pub const TRUNC: i32 = 28;
    pub const EXPM1: i32 = 29;
    pub const SILU: i32 = 30;
}
mod binop {
    pub const ADD: i32 = 0;
    pub const SUB: i32 = 1;
    pub const MUL: i32 = 2;
    pub const DIV: i32 = 3;
    pub const LOG: i32 = 4;
    pub const LOG1P: i32 = 5;
    pub const LEAKY_RELU: i32 = 6;
    pub const ELU: i32 = 7;
}

/// The library's per-thread error text becomes the `TensorError` variant the CPU backend returns for the
/// same mistake.
fn check(rc: c_int) -> Result<(), TensorError> {
    if rc == RTB_OK {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(rtb_last_error_string()) }.to_string_lossy().into_owned();
    Err(match rc {
        RTB_ERR_BOUNDS => TensorError::IdxOutOfBounds(msg),
        RTB_ERR_BROADCAST => TensorError::BroadcastError(msg),
        RTB_ERR_SHAPE => TensorError::InvalidShape(msg),
        RTB_ERR_DIM => TensorError::InvalidDim(msg),
        RTB_ERR_NONCONTIG => TensorError::WrongDims(msg),
        _ => TensorError::CudaError(msg),
    })
}

/// One library context per device for the life of the process.
struct Context(*mut rtb_ctx);
unsafe impl Send for Context {}
unsafe impl Sync for Context {}
impl Drop for Context {
    fn drop(&mut self) {
        unsafe { rtb_ctx_destroy(self.0) }
    }
}

static CONTEXTS: LazyLock<Mutex<Vec<Option<Arc<Context>>>>> = LazyLock::new(|| Mutex::new(Vec::new()));

fn context_of(device: usize) -> Arc<Context> {
    let mut all = CONTEXTS.lock().unwrap();
    if all.len() <= device {
        all.resize(device + 1, None);
    }
    if all[device].is_none() {
        let mut raw: *mut rtb_ctx = ptr::null_mut();
        check(unsafe { rtb_ctx_create(device as c_int, &mut raw) }).expect("rtb_ctx_create");
        all[device] = Some(Arc::new(Context(raw)));
    }
    all[device].as_ref().unwrap().clone()
}

#[derive(Clone)]
pub struct CudaB200 {
    ctx: Arc<Context>,
    device: usize,
}

impl std::fmt::Debug for CudaB200 {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "CudaB200(device {})", self.device)
    }
}

impl CudaB200 {
    pub fn on_device(device: usize) -> Self {
        Self { ctx: context_of(device), device }
    }
    #[inline]
    fn raw(&self) -> *mut rtb_ctx {
        self.ctx.0
    }
    /// `Cuda::sync` (`cuda.rs:164-185`): waits for everything enqueued on the context.
    pub fn sync(&self) -> Result<(), TensorError> {
        check(unsafe { rtb_ctx_sync(self.raw()) })
    }
}

/// Device memory from the library's caching allocator (`rtb_alloc` / `rtb_free`).
pub struct B200Buf<T: TensorValue> {
    ptr: *mut c_void,
    len: usize,
    ctx: Arc<Context>,
    _t: PhantomData<T>,
}
unsafe impl<T: TensorValue> Send for B200Buf<T> {}
unsafe impl<T: TensorValue> Sync for B200Buf<T> {}

impl<T: TensorValue> Drop for B200Buf<T> {
    fn drop(&mut self) {
        // stream-ordered: kernels already enqueued on the block finish before it is handed out again
        unsafe { rtb_free(self.ctx.0, self.ptr) };
    }
}
impl<T: TensorValue> std::fmt::Debug for B200Buf<T> {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result {
        write!(f, "B200Buf<{:?}>[{}]", T::DTYPE, self.len)
    }
}
impl<T: TensorValue> PartialEq for B200Buf<T> {
    /// Element-wise comparison through the host, as the tests use it (`CudaBuf::eq`, `cuda.rs:59-90`).
    fn eq(&self, other: &Self) -> bool {
        if self.len != other.len {
            return false;
        }
        let bytes = self.len * std::mem::size_of::<T>();
        let (mut a, mut b) = (vec![0u8; bytes], vec![0u8; bytes]);
        let ok = unsafe {
            rtb_d2h(self.ctx.0, a.as_mut_ptr().cast(), self.ptr, bytes) == RTB_OK
                && rtb_d2h(other.ctx.0, b.as_mut_ptr().cast(), other.ptr, bytes) == RTB_OK
        };
        ok && a == b
    }
}

#[inline]
fn dt<T: TensorValue>() -> c_int {
    T::DTYPE as c_int
}

/// (code, settings) of a reduction for the `_ex` entry points.
fn reduction_code(op: ReductionOpTypes) -> (c_int, rtb_reduce_settings) {
    let mut st = rtb_reduce_settings { unbiased: true, is_std: false, norm_type: 2 };
    match op {
        ReductionOpTypes::Variance { unbiased } => st.unbiased = unbiased,
        ReductionOpTypes::Stdev { unbiased } => {
            st.unbiased = unbiased;
            st.is_std = true;
        }
        ReductionOpTypes::Norm(NormType::L1) => st.norm_type = 1,
        _ => {}
    }
    (op.get_code() as c_int, st)
}

/// [outer, R, inner] of a contiguous tensor reduced along `dim`.
fn outer_r_inner(meta: &MetaTensor, dim: Dim) -> (usize, usize, usize) {
    let shape = meta.shape.as_slice();
    let outer: usize = shape[..dim].iter().product();
    let inner: usize = shape[dim + 1..].iter().product();
    (outer, shape[dim], inner.max(1))
}

impl CudaB200 {
    fn unary<T: TensorValue>(&self, buf: &mut B200Buf<T>, op: i32, shape: &[usize], strides: &[isize], offset: usize) -> Result<(), TensorError> {
        check(unsafe { rtb_unary_op(self.raw(), dt::<T>(), op, buf.ptr, shape.len(), shape.as_ptr(), strides.as_ptr(), offset) })
    }
    fn scalar<T: TensorValue>(&self, buf: &mut B200Buf<T>, op: i32, value: T, shape: &[usize], strides: &[isize], offset: usize) -> Result<(), TensorError> {
        check(unsafe {
            rtb_scalar_op(self.raw(), dt::<T>(), op, buf.ptr, (&value as *const T).cast(), shape.len(), shape.as_ptr(), strides.as_ptr(), offset)
        })
    }
}

/// The four methods of a unary family (`specify_trait_unary_cabal!`, `backend/mod.rs:95-139`): the view
/// form and the three layout forms are the same library call.
macro_rules! unary_family {
    ($name:ident, $code:expr $(, where $($extra:tt)+)?) => {
        paste! {
            fn [<apply_ $name>]<T: TensorValue>(&self, buf: &mut Self::Buf<T>, meta: &MetaTensor) -> Result<(), TensorError>
            $( where $($extra)+ )? {
                self.unary(buf, $code, meta.shape.as_slice(), meta.strides.as_ref(), meta.offset)
            }
            fn [<apply_ $name _nd>]<T: TensorValue>(&self, buf: &mut Self::Buf<T>, offset: usize, shape: &[usize], stride: &[isize]) -> Result<(), TensorError>
            $( where $($extra)+ )? {
                self.unary(buf, $code, shape, stride, offset)
            }
            fn [<apply_ $name _1d_strided>]<T: TensorValue>(&self, buf: &mut Self::Buf<T>, offset: usize, stride: isize, len: usize) -> Result<(), TensorError>
            $( where $($extra)+ )? {
                self.unary(buf, $code, &[len], &[stride], offset)
            }
            fn [<apply_ $name _contiguous>]<T: TensorValue>(&self, buf: &mut Self::Buf<T>, start: usize, len: usize) -> Result<(), TensorError>
            $( where $($extra)+ )? {
                self.unary(buf, $code, &[len], &[1], start)
            }
        }
    };
}

/// The four methods of a scalar family (`specify_trait_scalar_cabal!`, `backend/mod.rs:143-211`).
macro_rules! scalar_family {
    ($name:ident, $code:expr $(, where $($extra:tt)+)?) => {
        paste! {
            fn [<scalar_apply_ $name>]<T: TensorValue>(&self, buf: &mut Self::Buf<T>, value: T, meta: &MetaTensor) -> Result<(), TensorError>
            $( where $($extra)+ )? {
                self.scalar(buf, $code, value, meta.shape.as_slice(), meta.strides.as_ref(), meta.offset)
            }
            fn [<scalar_apply_ $name _nd>]<T: TensorValue>(&self, buf: &mut Self::Buf<T>, value: T, offset: usize, shape: &[usize], stride: &[isize]) -> Result<(), TensorError>
            $( where $($extra)+ )? {
                self.scalar(buf, $code, value, shape, stride, offset)
            }
            fn [<scalar_apply_ $name _1d_strided>]<T: TensorValue>(&self, buf: &mut Self::Buf<T>, value: T, offset: usize, stride: isize, len: usize) -> Result<(), TensorError>
            $( where $($extra)+ )? {
                self.scalar(buf, $code, value, &[len], &[stride], offset)
            }
            fn [<scalar_apply_ $name _contiguous>]<T: TensorValue>(&self, buf: &mut Self::Buf<T>, value: T, start: usize, len: usize) -> Result<(), TensorError>
            $( where $($extra)+ )? {
                self.scalar(buf, $code, value, &[len], &[1], start)
            }
        }
    };
}

impl Backend for CudaB200 {
    type Buf<T: TensorValue> = B200Buf<T>;

    fn device_type() -> DeviceType {
        DeviceType::Cuda(0)
    }
    fn device(&self) -> DeviceType {
        DeviceType::Cuda(self.device)
    }
    fn new() -> Self {
        Self::on_device(0)
    }

    // ---- buffers (`cuda.rs:668-836`) ------------------------------------------------------------
    fn alloc<T: TensorValue>(&self, len: usize) -> Result<Self::Buf<T>, TensorError> {
        // uninitialised: out-of-place ops write every output element, so the zero upload of `zeros_on` is not needed
        let mut p: *mut c_void = ptr::null_mut();
        check(unsafe { rtb_alloc(self.raw(), len * std::mem::size_of::<T>(), &mut p) })?;
        Ok(B200Buf { ptr: p, len, ctx: self.ctx.clone(), _t: PhantomData })
    }
    fn alloc_from_slice<T: TensorValue>(&self, src: Box<[T]>) -> Result<Self::Buf<T>, TensorError> {
        let buf = self.alloc::<T>(src.len())?;
        check(unsafe { rtb_h2d(self.raw(), buf.ptr, src.as_ptr().cast(), src.len() * std::mem::size_of::<T>()) })?;
        self.sync()?; // `src` is dropped when this returns
        Ok(buf)
    }
    fn copy_from_slice<T: TensorValue>(&self, dst: &mut Self::Buf<T>, src: &[T]) -> Result<(), TensorError> {
        if src.len() != dst.len {
            return Err(TensorError::SizeMismatch(format!("copy_from_slice: {} elements into a buffer of {}", src.len(), dst.len)));
        }
        check(unsafe { rtb_h2d(self.raw(), dst.ptr, src.as_ptr().cast(), src.len() * std::mem::size_of::<T>()) })?;
        self.sync()
    }
    fn copy_range_within<T: TensorValue>(&self, dst: &mut Self::Buf<T>, src: &Self::Buf<T>, dst_offset: usize, src_offset: usize, len: usize) -> Result<(), TensorError> {
        if dst_offset + len > dst.len || src_offset + len > src.len {
            return Err(TensorError::IdxOutOfBounds("copy_range_within: range exceeds a buffer".to_string()));
        }
        let es = std::mem::size_of::<T>();
        check(unsafe {
            rtb_d2d(self.raw(), (dst.ptr as *mut u8).add(dst_offset * es).cast(), (src.ptr as *const u8).add(src_offset * es).cast(), len * es)
        })
    }
    fn read<T: TensorValue>(&self, buf: &Self::Buf<T>, offset: usize) -> Result<T, TensorError> {
        if offset >= buf.len {
            return Err(TensorError::IdxOutOfBounds(format!("read at {} of {}", offset, buf.len)));
        }
        let mut v = std::mem::MaybeUninit::<T>::uninit();
        let es = std::mem::size_of::<T>();
        check(unsafe { rtb_d2h(self.raw(), v.as_mut_ptr().cast(), (buf.ptr as *const u8).add(offset * es).cast(), es) })?;
        Ok(unsafe { v.assume_init() })
    }
    fn write<T: TensorValue>(&self, buf: &mut Self::Buf<T>, offset: usize, value: T) -> Result<(), TensorError> {
        if offset >= buf.len {
            return Err(TensorError::IdxOutOfBounds(format!("write at {} of {}", offset, buf.len)));
        }
        let es = std::mem::size_of::<T>();
        check(unsafe { rtb_h2d(self.raw(), (buf.ptr as *mut u8).add(offset * es).cast(), (&value as *const T).cast(), es) })?;
        self.sync()
    }
    fn len<T: TensorValue>(&self, buf: &Self::Buf<T>) -> usize {
        buf.len
    }
    fn copy<T: TensorValue>(&self, src: &Self::Buf<T>) -> Result<Self::Buf<T>, TensorError> {
        let out = self.alloc::<T>(src.len)?;
        check(unsafe { rtb_d2d(self.raw(), out.ptr, src.ptr, src.len * std::mem::size_of::<T>()) })?;
        Ok(out)
    }
    fn dump<T: TensorValue>(&self, src: &Self::Buf<T>) -> Result<Box<[T]>, TensorError> {
        let mut out: Vec<T> = Vec::with_capacity(src.len);
        check(unsafe { rtb_d2h(self.raw(), out.as_mut_ptr().cast(), src.ptr, src.len * std::mem::size_of::<T>()) })?; // synchronises
        unsafe { out.set_len(src.len) };
        Ok(out.into_boxed_slice())
    }
    /// One kernel for any of the 13 x 13 dtype pairs (the reference reads and writes element by element
    /// through the host).
    fn convert<T: TensorValue, N: TensorValue>(&self, src: &Self::Buf<T>, dst: &mut Self::Buf<N>) -> Result<(), TensorError> {
        if src.len != dst.len {
            return Err(TensorError::SizeMismatch("Buffer size mismatch in convert".to_string()));
        }
        check(unsafe { rtb_convert(self.raw(), dt::<T>(), dt::<N>(), src.ptr, dst.ptr, src.len) })
    }

    // ---- fill ----------------------------------------------------------------------------------
    fn fill<T: TensorValue>(&self, buf: &mut Self::Buf<T>, value: T, meta: &MetaTensor) -> Result<(), TensorError> {
        self.fill_nd(buf, value, meta.offset, meta.shape.as_slice(), meta.strides.as_ref())
    }
    fn fill_nd<T: TensorValue>(&self, buf: &mut Self::Buf<T>, value: T, offset: usize, shape: &[usize], stride: &[isize]) -> Result<(), TensorError> {
        check(unsafe { rtb_fill(self.raw(), dt::<T>(), buf.ptr, (&value as *const T).cast(), shape.len(), shape.as_ptr(), stride.as_ptr(), offset) })
    }
    fn fill_1d_strided<T: TensorValue>(&self, buf: &mut Self::Buf<T>, value: T, offset: usize, stride: isize, len: usize) -> Result<(), TensorError> {
        self.fill_nd(buf, value, offset, &[len], &[stride])
    }
    fn fill_contiguous<T: TensorValue>(&self, buf: &mut Self::Buf<T>, value: T, start: usize, len: usize) -> Result<(), TensorError> {
        self.fill_nd(buf, value, start, &[len], &[1])
    }

    // ---- broadcast binary op: the three metas carry the output shape (`backend/mod.rs:296-309`) ------
    fn broadcast<T: TensorValue>(
        &self,
        left: (*const Self::Buf<T>, &MetaTensor),
        right: (*const Self::Buf<T>, &MetaTensor),
        dst: (*mut Self::Buf<T>, &MetaTensor),
        op: BinaryOpType,
    ) -> Result<(), TensorError> {
        let (l, lm) = left;
        let (r, rm) = right;
        let (d, dm) = dst;
        let (l, r, d) = unsafe { (&*l, &*r, &mut *d) };
        check(unsafe {
            rtb_broadcast(
                self.raw(), dt::<T>(), op.to_op_code() as c_int,
                l.ptr, lm.strides.as_ref().as_ptr(), lm.offset,
                r.ptr, rm.strides.as_ref().as_ptr(), rm.offset,
                d.ptr, dm.strides.as_ref().as_ptr(), dm.offset,
                dm.rank(), dm.shape.as_slice().as_ptr(),
            )
        })
    }

    // ---- unary and scalar families -----------------------------------------------------------------
    unary_family! {neg, unop::NEG, where T: std::ops::Neg<Output = T>}
    unary_family! {relu, unop::RELU}
    unary_family! {sigmoid, unop::SIGMOID, where T: crate::core::primops::InvExp}
    unary_family! {silu, unop::SILU, where T: crate::core::primops::InvExp}
    unary_family! {tanh, unop::TANH, where T: crate::core::primops::Exp + crate::core::primops::InvExp}
    unary_family! {abs, unop::ABS}
    unary_family! {sqrt, unop::SQRT, where T: crate::core::primops::SquareRoot}
    unary_family! {ln, unop::LN, where T: WeightValue}
    unary_family! {expm1, unop::EXPM1, where T: crate::core::primops::Exp}
    unary_family! {ln1p, unop::LN1P, where T: WeightValue}
    unary_family! {floor, unop::FLOOR, where T: WeightValue}
    unary_family! {ceil, unop::CEIL, where T: WeightValue}
    unary_family! {round, unop::ROUND, where T: WeightValue}
    unary_family! {trunc, unop::TRUNC, where T: WeightValue}

    scalar_family! {add, binop::ADD}
    scalar_family! {sub, binop::SUB}
    scalar_family! {mul, binop::MUL}
    scalar_family! {div, binop::DIV}
    scalar_family! {log, binop::LOG, where T: WeightValue}
    scalar_family! {log1p, binop::LOG1P, where T: WeightValue}
    scalar_family! {leaky_relu, binop::LEAKY_RELU}
    scalar_family! {elu, binop::ELU, where T: WeightValue}

    unary_family! {sin, unop::SIN, where T: WeightValue}
    unary_family! {cos, unop::COS, where T: WeightValue}
    unary_family! {tan, unop::TAN, where T: WeightValue}
    unary_family! {asin, unop::ASIN, where T: WeightValue}
    unary_family! {acos, unop::ACOS, where T: WeightValue}
    unary_family! {atan, unop::ATAN, where T: WeightValue}
    unary_family! {sinh, unop::SINH, where T: WeightValue}
    unary_family! {cosh, unop::COSH, where T: WeightValue}
    unary_family! {asinh, unop::ASINH, where T: WeightValue}
    unary_family! {acosh, unop::ACOSH, where T: WeightValue}
    unary_family! {atanh, unop::ATANH, where T: WeightValue}
    unary_family! {rsqrt, unop::RSQRT, where T: WeightValue}
    unary_family! {reciprocal, unop::RECIPROCAL, where T: WeightValue}
    unary_family! {square, unop::SQUARE, where T: WeightValue}
    unary_family! {cube, unop::CUBE, where T: WeightValue}
    unary_family! {exp, unop::EXP, where T: WeightValue}
    unary_family! {sign, unop::SIGN, where T: WeightValue}

    // ---- reductions (`backend/mod.rs:375-465`) ----------------------------------------------------------
    fn apply_reduce_contiguous_flat<T: WeightValue>(&self, src: &Self::Buf<T>, dst: &mut Self::Buf<T>, start: usize, len: usize, op: ReductionOpTypes) -> Result<(), TensorError> {
        if start + len > src.len {
            return Err(TensorError::IdxOutOfBounds("flat reduction range exceeds the buffer".to_string()));
        }
        let (code, st) = reduction_code(op);
        check(unsafe { rtb_reduce_flat_ex(self.raw(), dt::<T>(), code, &st, src.ptr, start, len, dst.ptr) })
    }
    fn apply_reduce_contiguous_nd<T: WeightValue>(&self, src: (&Self::Buf<T>, &MetaTensor), dst: (&mut Self::Buf<T>, &MetaTensor), dim: Dim, op: ReductionOpTypes) -> Result<(), TensorError> {
        let (sb, sm) = src;
        let (db, _) = dst;
        let (outer, r, inner) = outer_r_inner(sm, dim);
        let (code, st) = reduction_code(op);
        check(unsafe { rtb_reduce_axis_ex(self.raw(), dt::<T>(), code, &st, sb.ptr, sm.offset, outer, r, inner, db.ptr) })
    }
    /// A reduction over a VIEW needs no `contiguous()` copy here (`ops/reduction/mod.rs:351-360` makes one):
    /// slices, reversed or permuted outer dims and transposed matrices are reduced in place.
    fn apply_reduce<T: WeightValue>(&self, src: (&Self::Buf<T>, &MetaTensor), dst: (&mut Self::Buf<T>, &MetaTensor), dim: Dim, op: ReductionOpTypes) -> Result<(), TensorError> {
        let (sb, sm) = src;
        let (db, _) = dst;
        let (code, st) = reduction_code(op);
        let axis: isize = if sm.rank() == 1 { -1 } else { dim as isize };
        check(unsafe {
            rtb_reduce_view_ex(self.raw(), dt::<T>(), code, &st, sb.ptr, sm.rank(), sm.shape.as_slice().as_ptr(), sm.strides.as_ref().as_ptr(), sm.offset, axis, db.ptr)
        })
    }
    fn apply_argmax_contiguous_flat<T: WeightValue>(&self, src: &Self::Buf<T>, dst: &mut Self::Buf<u64>, start: usize, len: usize, op: ReductionOpTypes) -> Result<(), TensorError> {
        if start + len > src.len {
            return Err(TensorError::IdxOutOfBounds("flat reduction range exceeds the buffer".to_string()));
        }
        let (code, st) = reduction_code(op);
        check(unsafe { rtb_reduce_flat_ex(self.raw(), dt::<T>(), code, &st, src.ptr, start, len, dst.ptr) })
    }
    fn apply_argmax_contiguous_nd<T: WeightValue>(&self, src: (&Self::Buf<T>, &MetaTensor), dst: (&mut Self::Buf<u64>, &MetaTensor), dim: Dim, op: ReductionOpTypes) -> Result<(), TensorError> {
        let (sb, sm) = src;
        let (db, _) = dst;
        let (outer, r, inner) = outer_r_inner(sm, dim);
        let (code, st) = reduction_code(op);
        check(unsafe { rtb_reduce_axis_ex(self.raw(), dt::<T>(), code, &st, sb.ptr, sm.offset, outer, r, inner, db.ptr) })
    }

    fn apply_conv_2d<T: WeightValue>(
        &self,
        _input: (&Self::Buf<T>, &MetaTensor),
        _kernel: (&Self::Buf<T>, &MetaTensor),
        _output: &mut Self::Buf<T>,
        _config: &crate::ops::linalg::ConvConfig2D,
    ) -> Result<(), TensorError> {
        Err(TensorError::BackendError("convolution is not part of librt_b200: use the cuda.rs fallback".to_string()))
    }
}

// ---- what the trait does not have and the operator layer gains ------------------------------------------------
impl CudaB200 {
    /// `mean_l1_loss` with its gradient map in one launch (`ops/broadcast/l1.rs:16-84` runs a subtract, a
    /// sign, an abs, a mean and a scalar division).
    pub fn mean_l1_loss<T: WeightValue>(&self, a: &B200Buf<T>, b: &B200Buf<T>, n: usize, loss: &mut B200Buf<T>, grad_map: Option<&mut B200Buf<T>>) -> Result<(), TensorError> {
        let map = grad_map.map_or(ptr::null_mut(), |m| m.ptr);
        check(unsafe { rtb_l1_loss(self.raw(), dt::<T>(), a.ptr, b.ptr, n, 0, loss.ptr, map) })
    }
    /// `inverse_broadcast_gradient` (`grad/backwards.rs:512-538`) as one reduction of the upstream over the
    /// dims whose operand stride is 0.
    pub fn reduce_to_shape<T: WeightValue>(&self, upstream: &B200Buf<T>, shape: &[usize], operand_strides: &[isize], out: &mut B200Buf<T>) -> Result<Vec<usize>, TensorError> {
        let mut out_shape = vec![0usize; shape.len().max(1)];
        check(unsafe { rtb_reduce_to_shape(self.raw(), dt::<T>(), upstream.ptr, shape.len(), shape.as_ptr(), operand_strides.as_ptr(), out.ptr, out_shape.as_mut_ptr()) })?;
        out_shape.truncate(shape.len());
        Ok(out_shape)
    }
    /// `view_to_contiguous` (`core/tensor.rs:299-325`) as one strided-copy kernel.
    pub fn copy_view<T: TensorValue>(&self, src: &B200Buf<T>, meta: &MetaTensor, dst: &mut B200Buf<T>) -> Result<(), TensorError> {
        check(unsafe { rtb_copy_view(self.raw(), dt::<T>(), src.ptr, meta.rank(), meta.shape.as_slice().as_ptr(), meta.strides.as_ref().as_ptr(), meta.offset, dst.ptr) })
    }
}
