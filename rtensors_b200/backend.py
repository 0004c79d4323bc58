"""Host-side mirror of the reference's `Backend` trait for the hot path (src/backend/mod.rs:216-472)
on top of the C ABI.  Device memory and streams come from PyTorch; every computation is a call
into librt_b200.so.  Method names and argument meaning follow the trait: `scalar_apply_*`,
`apply_*`, `fill`, `broadcast`, `apply_reduce_contiguous_flat`, `apply_reduce` ...
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib as L
from ._lib import check, diffs, lib, sizes
from .meta import Meta, broadcast_params

TORCH_TO_CODE = {
    torch.uint8: L.U8, torch.int8: L.I8, torch.int16: L.I16, torch.int32: L.I32, torch.int64: L.I64,
    torch.float32: L.F32, torch.float64: L.F64, torch.bool: L.BOOL,
}
for _name, _code in (("uint16", L.U16), ("uint32", L.U32), ("uint64", L.U64)):
    if hasattr(torch, _name):
        TORCH_TO_CODE[getattr(torch, _name)] = _code
CODE_TO_TORCH = {v: k for k, v in TORCH_TO_CODE.items()}
CODE_TO_NP = {L.U8: np.uint8, L.I8: np.int8, L.U16: np.uint16, L.I16: np.int16, L.U32: np.uint32, L.I32: np.int32,
              L.U64: np.uint64, L.I64: np.int64, L.F32: np.float32, L.F64: np.float64, L.BOOL: np.bool_}


def dtype_code(t: torch.Tensor) -> int:
    return TORCH_TO_CODE[t.dtype]


def _scalar_bytes(code: int, value) -> bytes:
    """The operand in the element type's own representation (ctypes passes bytes as a pointer)."""
    return np.array(value, dtype=CODE_TO_NP[code]).tobytes()


_TYPESTR = {torch.float32: "<f4", torch.float64: "<f8", torch.int32: "<i4", torch.int64: "<i8", torch.int16: "<i2",
            torch.int8: "|i1", torch.uint8: "|u1", torch.bool: "|b1"}


class _DeviceBlock:
    """A raw device address as an object torch can wrap without copying (CUDA array interface)."""

    def __init__(self, ptr: int, n: int, dtype: torch.dtype):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": _TYPESTR[dtype], "data": (int(ptr), False), "version": 2}


class CudaB200:
    """One instance per device (`Cuda` of the reference, src/backend/cuda.rs:38-186): owns the
    library context (stream, workspace, allocator).  Calls are enqueued on torch's current
    stream of that device."""

    def __init__(self, device: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("CudaB200 needs a CUDA device; there is no CPU fallback")
        self.device = int(device)
        torch.cuda.set_device(self.device)
        self._ctx = C.c_void_p()
        check(lib().rtb_ctx_create(C.c_int(self.device), C.byref(self._ctx)))
        self._stream = None
        self.mg_world, self.mg_rank, self.mg_peer_mapped = 1, 0, False
        self.sync_stream()

    def close(self):
        if self._ctx:
            lib().rtb_ctx_destroy(self._ctx)
            self._ctx = C.c_void_p()
            self.mg_world = 1

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    # -- plumbing ---------------------------------------------------------------------------
    def sync_stream(self):
        """Binds the context to torch's current stream (call after switching streams)."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        if s != self._stream:
            check(lib().rtb_ctx_set_stream(self._ctx, C.c_void_p(s)))
            self._stream = s

    def sync(self):
        check(lib().rtb_ctx_sync(self._ctx))

    @property
    def launches(self) -> int:
        return int(lib().rtb_ctx_launch_count(self._ctx))

    @property
    def sm_count(self) -> int:
        return int(lib().rtb_ctx_sm_count(self._ctx))

    def alloc(self, n: int, dtype: torch.dtype) -> torch.Tensor:
        """Uninitialised device buffer (Backend::alloc)."""
        return torch.empty(int(n), dtype=dtype, device=f"cuda:{self.device}")

    def alloc_from_slice(self, host: np.ndarray) -> torch.Tensor:
        return torch.from_numpy(np.ascontiguousarray(host).reshape(-1)).to(f"cuda:{self.device}")

    def dump(self, buf: torch.Tensor) -> np.ndarray:
        return buf.detach().cpu().numpy()

    # buffer-level methods of the trait (src/backend/mod.rs:227-233), checks as in src/backend/cpu.rs:151-207
    def len(self, buf: torch.Tensor) -> int:
        return buf.numel()

    def copy(self, buf: torch.Tensor) -> torch.Tensor:
        out = self.alloc(max(buf.numel(), 1), buf.dtype)
        if buf.numel():
            check(lib().rtb_d2d(self._ctx, self._p(out), self._p(buf), C.c_size_t(buf.numel() * buf.element_size())))
        return out[: buf.numel()]

    def copy_from_slice(self, dst: torch.Tensor, src: np.ndarray):
        src = np.ascontiguousarray(src).reshape(-1)
        if dst.numel() != src.size:
            raise L.RtbError(L.ERR_SHAPE, f"Buffer size mismatch in copy_from_slice: dst size {dst.numel()}, src size {src.size}")
        if src.size:
            check(lib().rtb_h2d(self._ctx, self._p(dst), src.ctypes.data_as(C.c_void_p), C.c_size_t(src.nbytes)))
            self.sync()  # the host array may go away

    def copy_range_within(self, dst: torch.Tensor, src: torch.Tensor, dst_offset: int, src_offset: int, n: int):
        if dst_offset + n > dst.numel() or src_offset + n > src.numel():
            raise L.RtbError(L.ERR_BOUNDS, "Index out of bounds in copy_range_within")
        if n:
            es = dst.element_size()
            check(lib().rtb_d2d(self._ctx, C.c_void_p(dst.data_ptr() + dst_offset * es),
                                C.c_void_p(src.data_ptr() + src_offset * es), C.c_size_t(n * es)))

    def read(self, buf: torch.Tensor, offset: int):
        if not 0 <= offset < buf.numel():
            raise L.RtbError(L.ERR_BOUNDS, f"Index {offset} out of bounds for buffer of length {buf.numel()}")
        host = np.empty(1, dtype=CODE_TO_NP[dtype_code(buf)])
        check(lib().rtb_d2h(self._ctx, host.ctypes.data_as(C.c_void_p),
                            C.c_void_p(buf.data_ptr() + offset * buf.element_size()), C.c_size_t(host.nbytes)))
        return host[0]

    def write(self, buf: torch.Tensor, offset: int, value):
        if not 0 <= offset < buf.numel():
            raise L.RtbError(L.ERR_BOUNDS, f"Index {offset} out of bounds for buffer of length {buf.numel()}")
        host = np.array([value], dtype=CODE_TO_NP[dtype_code(buf)])
        check(lib().rtb_h2d(self._ctx, C.c_void_p(buf.data_ptr() + offset * buf.element_size()),
                            host.ctypes.data_as(C.c_void_p), C.c_size_t(host.nbytes)))
        self.sync()

    @staticmethod
    def _p(t: Optional[torch.Tensor]):
        return C.c_void_p(0 if t is None else t.data_ptr())

    # -- elementwise over a view --------------------------------------------------------------
    def scalar_apply(self, buf: torch.Tensor, op: int, value, meta: Meta, dtype: Optional[int] = None):
        code = dtype_code(buf) if dtype is None else dtype
        v = _scalar_bytes(code, value)
        meta.check_extent(buf.numel())
        check(lib().rtb_scalar_op(self._ctx, C.c_int(code), C.c_int(op), self._p(buf), v,
                                  C.c_size_t(meta.rank), meta.c_shape, meta.c_strides,
                                  C.c_size_t(meta.offset)))

    def scalar_apply_add(self, buf, value, meta): self.scalar_apply(buf, L.ADD, value, meta)
    def scalar_apply_sub(self, buf, value, meta): self.scalar_apply(buf, L.SUB, value, meta)
    def scalar_apply_mul(self, buf, value, meta): self.scalar_apply(buf, L.MUL, value, meta)
    def scalar_apply_div(self, buf, value, meta): self.scalar_apply(buf, L.DIV, value, meta)

    def apply_unary(self, buf: torch.Tensor, op: int, meta: Meta):
        meta.check_extent(buf.numel())
        check(lib().rtb_unary_op(self._ctx, C.c_int(dtype_code(buf)), C.c_int(op), self._p(buf), C.c_size_t(meta.rank),
                                 meta.c_shape, meta.c_strides, C.c_size_t(meta.offset)))

    def scalar_apply_log(self, buf, value, meta): self.scalar_apply(buf, L.LOG, value, meta)
    def scalar_apply_log1p(self, buf, value, meta): self.scalar_apply(buf, L.LOG1P, value, meta)
    def scalar_apply_leaky_relu(self, buf, value, meta): self.scalar_apply(buf, L.LEAKY_RELU, value, meta)
    def scalar_apply_elu(self, buf, value, meta): self.scalar_apply(buf, L.ELU, value, meta)

    def apply_neg(self, buf, meta): self.apply_unary(buf, L.NEG, meta)
    def apply_relu(self, buf, meta): self.apply_unary(buf, L.RELU, meta)
    def apply_abs(self, buf, meta): self.apply_unary(buf, L.ABS, meta)
    def apply_sign(self, buf, meta): self.apply_unary(buf, L.SIGN, meta)

    def __getattr__(self, name):
        # apply_sigmoid, apply_tanh, ... apply_silu: the remaining unary families of the trait
        if name.startswith("apply_") and hasattr(L, name[6:].upper()):
            code = getattr(L, name[6:].upper())
            return lambda buf, meta: self.apply_unary(buf, code, meta)
        raise AttributeError(name)

    def fill(self, buf: torch.Tensor, value, meta: Meta):
        code = dtype_code(buf)
        v = _scalar_bytes(code, value)
        meta.check_extent(buf.numel())
        check(lib().rtb_fill(self._ctx, C.c_int(code), self._p(buf), v,
                             C.c_size_t(meta.rank), meta.c_shape, meta.c_strides, C.c_size_t(meta.offset)))

    def contiguous(self, buf: torch.Tensor, meta: Meta) -> torch.Tensor:
        """Row-major copy of a view (view_to_contiguous, src/core/tensor.rs:299-325)."""
        out = self.alloc(max(meta.size, 1), buf.dtype)
        if meta.size:
            meta.check_extent(buf.numel())
            check(lib().rtb_copy_view(self._ctx, C.c_int(dtype_code(buf)), self._p(buf), C.c_size_t(meta.rank),
                                      meta.c_shape, meta.c_strides, C.c_size_t(meta.offset), self._p(out)))
        return out

    def grad_mask(self, buf: torch.Tensor, meta: Meta, kind: int, value=None) -> torch.Tensor:
        """Dense per-element map of a view in one kernel instead of the reference's get / set loops:
        L.MASK_RELU, L.MASK_ABS (src/ops/unary/mod.rs:213-252), L.MASK_LEAKY_RELU with its slope
        (src/ops/scalar/mod.rs:149-166), L.MASK_RECIPROCAL (src/ops/broadcast/div.rs:583-587)."""
        out = self.alloc(max(meta.size, 1), buf.dtype)
        if meta.size:
            meta.check_extent(buf.numel())
            code = dtype_code(buf)
            v = None if value is None else _scalar_bytes(code, value)
            check(lib().rtb_grad_mask(self._ctx, C.c_int(code), C.c_int(kind), v, self._p(buf), C.c_size_t(meta.rank),
                                      meta.c_shape, meta.c_strides, C.c_size_t(meta.offset), self._p(out)))
        return out

    # -- broadcast ----------------------------------------------------------------------------
    def broadcast(self, left: Tuple[torch.Tensor, Meta], right: Tuple[torch.Tensor, Meta],
                  dst: Tuple[torch.Tensor, Meta], op: int):
        """Backend::broadcast: the three metas carry the output shape; dst may be left."""
        (lb, lm), (rb, rm), (db, dm) = left, right, dst
        assert lm.shape == rm.shape == dm.shape
        lm.check_extent(lb.numel()); rm.check_extent(rb.numel()); dm.check_extent(db.numel())
        check(lib().rtb_broadcast(self._ctx, C.c_int(dtype_code(db)), C.c_int(op), self._p(lb), lm.c_strides,
                                  C.c_size_t(lm.offset), self._p(rb), rm.c_strides, C.c_size_t(rm.offset),
                                  self._p(db), dm.c_strides, C.c_size_t(dm.offset), C.c_size_t(dm.rank),
                                  dm.c_shape))

    def binary(self, a: torch.Tensor, am: Meta, b: torch.Tensor, bm: Meta, op: int):
        """`a op b` as the operator impls do it (src/ops/broadcast/add.rs:441-477), except that the
        output is allocated uninitialised instead of uploaded as zeros."""
        shape, sa, sb = broadcast_params(am, bm)
        dm = Meta.contiguous(shape)
        out = self.alloc(max(dm.size, 1), a.dtype)
        self.broadcast((a, Meta(shape, sa, am.offset)), (b, Meta(shape, sb, bm.offset)), (out, dm), op)
        return out, dm

    def binary_assign(self, a: torch.Tensor, am: Meta, b: torch.Tensor, bm: Meta, op: int):
        """`a op= b` (src/ops/broadcast/add.rs:14-46): the broadcast shape must be a's shape."""
        shape, sa, sb = broadcast_params(am, bm)
        if tuple(shape) != tuple(am.shape):
            raise ValueError(f"Incompatible shapes for in-place op: {bm.shape} does not broadcast to {am.shape}")
        ma = Meta(shape, sa, am.offset)
        self.broadcast((a, ma), (b, Meta(shape, sb, bm.offset)), (a, ma), op)

    # -- reductions ---------------------------------------------------------------------------
    def apply_reduce_contiguous_flat(self, src: torch.Tensor, dst: torch.Tensor, start: int, length: int, op: int):
        if start + length > src.numel():
            raise L.RtbError(-4, "flat reduction range exceeds the buffer")
        check(lib().rtb_reduce_flat(self._ctx, C.c_int(dtype_code(src)), C.c_int(op), self._p(src), C.c_size_t(start),
                                    C.c_size_t(length), self._p(dst)))

    def apply_reduce(self, src: Tuple[torch.Tensor, Meta], dst: torch.Tensor, dim: int, op: int):
        """Backend::apply_reduce (src/backend/mod.rs:375-409): contiguous input; rank 1 -> flat."""
        sb, sm = src
        if not sm.is_contiguous():
            raise L.RtbError(-7, "Reduction over non-contiguous tensors is not implemented yet.")
        if sm.rank == 1:
            return self.apply_reduce_contiguous_flat(sb, dst, sm.offset, sm.size, op)
        outer = int(np.prod(sm.shape[:dim], dtype=np.int64)) if dim > 0 else 1
        inner = max(int(np.prod(sm.shape[dim + 1:], dtype=np.int64)), 1)
        r = sm.shape[dim]
        if sm.offset + outer * r * inner > sb.numel():
            raise L.RtbError(-4, "axis reduction range exceeds the buffer")
        check(lib().rtb_reduce_axis(self._ctx, C.c_int(dtype_code(sb)), C.c_int(op), self._p(sb),
                                    C.c_size_t(sm.offset), C.c_size_t(outer), C.c_size_t(r), C.c_size_t(inner),
                                    self._p(dst)))

    def reduce_view(self, src: torch.Tensor, meta: Meta, axis: Optional[int], op: int,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Reduction over an arbitrary view without requiring contiguity (rtb_reduce_view); axis
        None = full reduction.  Returns the row-major result buffer (reduced dim kept as 1)."""
        meta.check_extent(src.numel())
        if axis is None:
            n_out = 1
        else:
            n_out = 1
            for k, s_ in enumerate(meta.shape):
                n_out *= 1 if k == axis else s_
        if out is None:
            out = self.alloc(max(n_out, 1), src.dtype)
        elif out.numel() < n_out or out.dtype != src.dtype:
            raise ValueError("reduce_view: the output buffer is too small or of another dtype")
        check(lib().rtb_reduce_view(self._ctx, C.c_int(dtype_code(src)), C.c_int(op), self._p(src), C.c_size_t(meta.rank),
                                    meta.c_shape, meta.c_strides, C.c_size_t(meta.offset),
                                    C.c_ssize_t(-1 if axis is None else axis), self._p(out)))
        return out

    def reduce_view_ex(self, src: torch.Tensor, meta: Meta, axis: Optional[int], op: int, unbiased: bool = True,
                       is_std: bool = False, norm_type: int = 2) -> torch.Tensor:
        """Any reduction code over a view (rtb_reduce_view_ex): also variance / std, logsumexp, norms and
        argmax / argmin (whose result buffer is int64 holding the u64 positions)."""
        meta.check_extent(src.numel())
        n_out = 1
        if axis is not None:
            for k, s_ in enumerate(meta.shape):
                n_out *= 1 if k == axis else s_
        out = self.alloc(max(n_out, 1), torch.int64 if op in (L.ARGMAX, L.ARGMIN) else src.dtype)
        st = L.ReduceSettings(bool(unbiased), bool(is_std), int(norm_type))
        check(lib().rtb_reduce_view_ex(self._ctx, C.c_int(dtype_code(src)), C.c_int(op), C.byref(st), self._p(src),
                                       C.c_size_t(meta.rank), meta.c_shape, meta.c_strides, C.c_size_t(meta.offset),
                                       C.c_ssize_t(-1 if axis is None else axis), self._p(out)))
        return out

    def apply_reduce_ex(self, src: Tuple[torch.Tensor, Meta], dst: torch.Tensor, dim: int, op: int, unbiased: bool = True,
                        is_std: bool = False, norm_type: int = 2):
        """Backend::apply_reduce / apply_argmax with the op's settings (src/backend/mod.rs:375-465): contiguous
        input; rank 1 goes to the flat launcher; dst is int64 (u64 positions) for ARGMAX / ARGMIN."""
        sb, sm = src
        if not sm.is_contiguous():
            raise L.RtbError(-7, "Reduction over non-contiguous tensors is not implemented yet.")
        st = L.ReduceSettings(bool(unbiased), bool(is_std), int(norm_type))
        if sm.rank == 1:
            if sm.offset + sm.size > sb.numel():
                raise L.RtbError(-4, "flat reduction range exceeds the buffer")
            return check(lib().rtb_reduce_flat_ex(self._ctx, C.c_int(dtype_code(sb)), C.c_int(op), C.byref(st), self._p(sb),
                                                  C.c_size_t(sm.offset), C.c_size_t(sm.size), self._p(dst)))
        outer = int(np.prod(sm.shape[:dim], dtype=np.int64)) if dim > 0 else 1
        inner = max(int(np.prod(sm.shape[dim + 1:], dtype=np.int64)), 1)
        r = sm.shape[dim]
        if sm.offset + outer * r * inner > sb.numel():
            raise L.RtbError(-4, "axis reduction range exceeds the buffer")
        check(lib().rtb_reduce_axis_ex(self._ctx, C.c_int(dtype_code(sb)), C.c_int(op), C.byref(st), self._p(sb),
                                       C.c_size_t(sm.offset), C.c_size_t(outer), C.c_size_t(r), C.c_size_t(inner),
                                       self._p(dst)))

    def broadcast_reduce(self, a: torch.Tensor, am: Meta, b: torch.Tensor, bm: Meta, binop: int, axis: int, redop: int):
        """`(a binop b).<redop>_at(axis)` in one kernel: the broadcast result is never written.
        -> (result buffer, result Meta with dim `axis` = 1)"""
        shape, sa, sb = broadcast_params(am, bm)
        Meta(shape, sa, am.offset).check_extent(a.numel()); Meta(shape, sb, bm.offset).check_extent(b.numel())
        om = Meta.contiguous(tuple(1 if k == axis else s_ for k, s_ in enumerate(shape)))
        out = self.alloc(max(om.size, 1), a.dtype)
        check(lib().rtb_broadcast_reduce(self._ctx, C.c_int(dtype_code(a)), C.c_int(binop), C.c_int(redop), self._p(a),
                                         diffs(sa), C.c_size_t(am.offset), self._p(b), diffs(sb), C.c_size_t(bm.offset),
                                         C.c_size_t(len(shape)), sizes(shape), C.c_size_t(axis), self._p(out)))
        return out, om

    def reduce_axis_ori(self, src: torch.Tensor, offset: int, outer: int, r: int, inner: int, op: int):
        out = self.alloc(max(outer * inner, 1), src.dtype)
        check(lib().rtb_reduce_axis(self._ctx, C.c_int(dtype_code(src)), C.c_int(op), self._p(src), C.c_size_t(offset),
                                    C.c_size_t(outer), C.c_size_t(r), C.c_size_t(inner), self._p(out)))
        return out

    def reduce_ext_ori(self, src: torch.Tensor, offset: int, outer: int, r: int, inner: int, op: int, unbiased: bool = True,
                       is_std: bool = False, norm_type: int = 2):
        """Codes 6..10 over a contiguous (outer, r, inner) block (rtb_reduce_axis_ex); int64 output for positions."""
        out = self.alloc(max(outer * inner, 1), torch.int64 if op in (L.ARGMAX, L.ARGMIN) else src.dtype)
        st = L.ReduceSettings(bool(unbiased), bool(is_std), int(norm_type))
        check(lib().rtb_reduce_axis_ex(self._ctx, C.c_int(dtype_code(src)), C.c_int(op), C.byref(st), self._p(src),
                                       C.c_size_t(offset), C.c_size_t(outer), C.c_size_t(r), C.c_size_t(inner), self._p(out)))
        return out

    def l1_loss(self, a: torch.Tensor, b: torch.Tensor, reduction: int = 0, with_grad: bool = False):
        assert a.numel() == b.numel() and a.dtype == b.dtype
        loss = self.alloc(1, a.dtype)
        g = self.alloc(a.numel(), a.dtype) if with_grad else None
        check(lib().rtb_l1_loss(self._ctx, C.c_int(dtype_code(a)), self._p(a), self._p(b), C.c_size_t(a.numel()),
                                C.c_int(reduction), self._p(loss), self._p(g)))
        return loss, g

    def reduce_to_shape(self, upstream: torch.Tensor, shape: Sequence[int], operand_strides: Sequence[int],
                        out: Optional[torch.Tensor] = None):
        r = len(shape)
        oshape = tuple(1 if s == 0 else n for n, s in zip(shape, operand_strides))
        n_out = int(np.prod(oshape, dtype=np.int64)) if r else 1
        if out is None:
            out = self.alloc(max(n_out, 1), upstream.dtype)
        elif out.numel() < n_out or out.dtype != upstream.dtype:
            raise ValueError("reduce_to_shape: the output buffer is too small or of another dtype")
        osh = (C.c_size_t * max(r, 1))()
        check(lib().rtb_reduce_to_shape(self._ctx, C.c_int(dtype_code(upstream)), self._p(upstream), C.c_size_t(r),
                                        sizes(shape), diffs(operand_strides), self._p(out), osh))
        assert tuple(osh[:r]) == oshape
        return out, oshape

    # -- fused MLP pieces ---------------------------------------------------------------------
    def relu_mask(self, x: torch.Tensor) -> torch.Tensor:
        mask = torch.empty_like(x)
        fn = lib().rtb_relu_mask_f64 if x.dtype == torch.float64 else lib().rtb_relu_mask_f32
        check(fn(self._ctx, self._p(x), self._p(mask), C.c_size_t(x.numel())))
        return mask

    def bias_relu_mask(self, z: torch.Tensor, bias: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
        """z = relu(z + bias) in place over a dense (rows, cols) activation; returns the gradient mask."""
        mask = torch.empty_like(z)
        check(lib().rtb_bias_relu_mask(self._ctx, C.c_int(dtype_code(z)), self._p(z), self._p(bias), self._p(mask),
                                       C.c_size_t(rows), C.c_size_t(cols)))
        return mask

    def sgd_update(self, p: torch.Tensor, g: torch.Tensor, lr: float):
        if p.dtype == torch.float64:
            check(lib().rtb_sgd_update_f64(self._ctx, self._p(p), self._p(g), C.c_double(lr), C.c_size_t(p.numel())))
        else:
            check(lib().rtb_sgd_update_f32(self._ctx, self._p(p), self._p(g), C.c_float(lr), C.c_size_t(p.numel())))

    def convert(self, src: torch.Tensor, dst_dtype: torch.dtype, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`convert::<T, N>` (src/backend/mod.rs:234) into `out`, or into a fresh buffer: every element
        cast by the reference's DTypeConversion rules (src/core/value.rs:270-290)."""
        if out is None:
            out = self.alloc(max(src.numel(), 1), dst_dtype)
        elif out.dtype != dst_dtype or out.numel() < src.numel():
            raise ValueError("Buffer size mismatch in convert")
        check(lib().rtb_convert(self._ctx, C.c_int(dtype_code(src)), C.c_int(TORCH_TO_CODE[dst_dtype]), self._p(src),
                                self._p(out), C.c_size_t(src.numel())))
        return out

    def convert_raw(self, src: torch.Tensor, src_code: int, dst_code: int) -> torch.Tensor:
        """convert over raw byte buffers (torch.uint8), for the 128-bit integer types torch lacks."""
        n = src.numel() // L.DTYPE_SIZE[src_code]
        out = self.alloc(max(n, 1) * L.DTYPE_SIZE[dst_code], torch.uint8)
        check(lib().rtb_convert(self._ctx, C.c_int(src_code), C.c_int(dst_code), self._p(src), self._p(out), C.c_size_t(n)))
        return out

    def u8_to_f32_div(self, src: torch.Tensor, divisor: float = 255.0) -> torch.Tensor:
        out = self.alloc(src.numel(), torch.float32)
        check(lib().rtb_u8_to_f32_div(self._ctx, self._p(src), self._p(out), C.c_float(divisor),
                                      C.c_size_t(src.numel())))
        return out

    # -- multi-GPU (rtb_mg_*): one rank per GPU, the communicator lives in the library context -----
    @staticmethod
    def mg_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check(lib().rtb_mg_unique_id(buf))
        return buf.raw

    def mg_init(self, nranks: int, rank: int, unique_id: bytes):
        """Collective: every rank passes the id made by rank 0's mg_unique_id()."""
        check(lib().rtb_mg_init(self._ctx, C.c_int(nranks), C.c_int(rank), C.c_char_p(unique_id)))
        n, r, m = C.c_int(), C.c_int(), C.c_int()
        check(lib().rtb_mg_info(self._ctx, C.byref(n), C.byref(r), C.byref(m)))
        self.mg_world, self.mg_rank, self.mg_peer_mapped = n.value, r.value, bool(m.value)

    def mg_finalize(self):
        check(lib().rtb_mg_finalize(self._ctx))
        self.mg_world, self.mg_rank, self.mg_peer_mapped = 1, 0, False

    def mg_set_wait_ns(self, ns: int):
        check(lib().rtb_mg_set_wait_ns(self._ctx, C.c_uint64(ns)))

    def mg_status(self) -> int:
        bits = C.c_uint()
        check(lib().rtb_mg_status(self._ctx, C.byref(bits)))
        return bits.value

    def mg_realign(self):
        check(lib().rtb_mg_realign(self._ctx))

    def mg_allreduce(self, buf: torch.Tensor, op: int = L.SUM, mean_count: int = 0, overlap: bool = False):
        fn = lib().rtb_mg_allreduce_begin if overlap else lib().rtb_mg_allreduce
        check(fn(self._ctx, C.c_int(dtype_code(buf)), C.c_int(op), self._p(buf), C.c_size_t(buf.numel()),
                 C.c_size_t(mean_count)))

    def mg_allreduce_join(self):
        check(lib().rtb_mg_allreduce_join(self._ctx))

    # -- host-buffer operations (rtb_host_*): two transfer lanes and a pool of device blocks inside the library --
    def _pool_tensor(self, ptr: int, n: int, dtype: torch.dtype) -> torch.Tensor:
        """A torch view of a block of the library's pool (no copy; valid until host_release)."""
        return torch.as_tensor(_DeviceBlock(ptr, int(n), dtype), device=f"cuda:{self.device}")

    def host_stage_in(self, host: torch.Tensor) -> torch.Tensor:
        """Starts the upload of a (pinned) host tensor; the compute stream waits only at host_ready."""
        out = C.c_void_p()
        check(lib().rtb_host_stage_in(self._ctx, C.c_void_p(host.data_ptr()), C.c_size_t(host.numel() * host.element_size()),
                                      C.byref(out)))
        return self._pool_tensor(out.value, max(host.numel(), 1), host.dtype)

    def host_scratch(self, n: int, dtype: torch.dtype) -> torch.Tensor:
        out = C.c_void_p()
        check(lib().rtb_host_scratch(self._ctx, C.c_size_t(int(n) * torch.empty(0, dtype=dtype).element_size()), C.byref(out)))
        return self._pool_tensor(out.value, max(int(n), 1), dtype)

    def host_ready(self, dev: torch.Tensor):
        check(lib().rtb_host_ready(self._ctx, self._p(dev)))

    def host_stage_out(self, dev: torch.Tensor, host: torch.Tensor):
        if host.numel() * host.element_size() > dev.numel() * dev.element_size():
            raise L.RtbError(-4, "host_stage_out: the host tensor is larger than the device block")
        check(lib().rtb_host_stage_out(self._ctx, self._p(dev), C.c_void_p(host.data_ptr()),
                                       C.c_size_t(host.numel() * host.element_size())))

    def host_release(self, dev: torch.Tensor):
        check(lib().rtb_host_release(self._ctx, self._p(dev)))

    def host_join(self):
        check(lib().rtb_host_join(self._ctx))

    def host_wait(self):
        check(lib().rtb_host_wait(self._ctx))

    def host_trim(self):
        check(lib().rtb_host_trim(self._ctx))

    def host_set_stage_bytes(self, n: int):
        check(lib().rtb_host_set_stage_bytes(self._ctx, C.c_size_t(int(n))))

    def host_reduce_view(self, host: torch.Tensor, meta: Meta, axis: Optional[int], op: int, host_out: torch.Tensor,
                         unbiased: bool = True, is_std: bool = False, norm_type: int = 2):
        """Reduction of a tensor whose buffer is in host memory; the result goes to host_out (enqueues only)."""
        st = L.ReduceSettings(bool(unbiased), bool(is_std), int(norm_type))
        check(lib().rtb_host_reduce_view(self._ctx, C.c_int(dtype_code(host)), C.c_int(op), C.byref(st), C.c_void_p(host.data_ptr()),
                                         C.c_size_t(host.numel()), C.c_size_t(meta.rank), meta.c_shape, meta.c_strides,
                                         C.c_size_t(meta.offset), C.c_ssize_t(-1 if axis is None else axis),
                                         C.c_void_p(host_out.data_ptr())))

    def host_broadcast(self, a_host: torch.Tensor, am: Meta, b_host: torch.Tensor, bm: Meta, op: int, out_host: torch.Tensor,
                       dim_range: Optional[Tuple[int, int]] = None):
        """`a op b` with operand buffers in host memory, the result written row-major to out_host (this
        call's range of the outermost output dim only).  Enqueues only."""
        shape, sa, sb = broadcast_params(am, bm)
        lo, hi = dim_range if dim_range is not None else (0, shape[0] if shape else 1)
        per = 1
        for n in shape[1:]:
            per *= n
        if out_host.numel() < (hi - lo) * per or out_host.dtype != a_host.dtype:
            raise ValueError("host_broadcast: the output tensor is too small or of another dtype")
        check(lib().rtb_host_broadcast(self._ctx, C.c_int(dtype_code(a_host)), C.c_int(op), C.c_void_p(a_host.data_ptr()),
                                       C.c_size_t(a_host.numel()), diffs(sa), C.c_size_t(am.offset), C.c_void_p(b_host.data_ptr()),
                                       C.c_size_t(b_host.numel()), diffs(sb), C.c_size_t(bm.offset), C.c_void_p(out_host.data_ptr()),
                                       C.c_size_t(len(shape)), sizes(shape), C.c_size_t(lo), C.c_size_t(hi)))

    def mg_combine(self, buf: torch.Tensor, op: int = L.SUM, mean_count: int = 0):
        check(lib().rtb_mg_combine(self._ctx, C.c_int(dtype_code(buf)), C.c_int(op), self._p(buf), C.c_size_t(buf.numel()),
                                   C.c_size_t(mean_count)))

    def mg_reduce_flat(self, src: torch.Tensor, start: int, local_len: int, global_len: int, op: int,
                       dst: Optional[torch.Tensor] = None) -> torch.Tensor:
        if start + local_len > src.numel():
            raise L.RtbError(-4, "flat reduction range exceeds the buffer")
        dst = self.alloc(1, src.dtype) if dst is None else dst
        check(lib().rtb_mg_reduce_flat(self._ctx, C.c_int(dtype_code(src)), C.c_int(op), self._p(src), C.c_size_t(start),
                                       C.c_size_t(local_len), C.c_size_t(global_len), self._p(dst)))
        return dst

    def mg_reduce_axis(self, src: torch.Tensor, offset: int, outer: int, r_local: int, inner: int, global_r: int, op: int,
                       outer_stride: Optional[int] = None, row_stride: Optional[int] = None,
                       dst: Optional[torch.Tensor] = None) -> torch.Tensor:
        dst = self.alloc(max(outer * inner, 1), src.dtype) if dst is None else dst
        so = r_local * inner if outer_stride is None else outer_stride
        sr = inner if row_stride is None else row_stride
        check(lib().rtb_mg_reduce_axis(self._ctx, C.c_int(dtype_code(src)), C.c_int(op), self._p(src), C.c_size_t(offset),
                                       C.c_size_t(outer), C.c_size_t(r_local), C.c_size_t(inner), C.c_ssize_t(so),
                                       C.c_ssize_t(sr), C.c_size_t(global_r), self._p(dst)))
        return dst

    def mg_l1_loss(self, a: torch.Tensor, b: torch.Tensor, global_n: int, reduction: int = 0, with_grad: bool = False):
        assert a.numel() == b.numel() and a.dtype == b.dtype
        loss = self.alloc(1, a.dtype)
        g = self.alloc(a.numel(), a.dtype) if with_grad else None
        check(lib().rtb_mg_l1_loss(self._ctx, C.c_int(dtype_code(a)), self._p(a), self._p(b), C.c_size_t(a.numel()),
                                   C.c_size_t(global_n), C.c_int(reduction), self._p(loss), self._p(g)))
        return loss, g
