"""CPU oracle for the tensor hot path -- TEST INFRASTRUCTURE, not product code.

ctypes front-end over ``rt_oracle.c`` (a C restatement of the rtensors CPU backend).  Only the
test-suite, the smoke check and the bench's CPU-baseline leg may import this package; the
product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

# dtype codes = DType discriminants of the reference (core/value.rs:567-581)
U8, I8, U16, I16, U32, U128, I32, U64, I64, I128, F32, F64, BOOL = range(13)
ADD, SUB, MUL, DIV, LOG, LOG1P, LEAKY_RELU, ELU = range(8)
(NEG, RELU, ABS, SIGN, SIGMOID, TANH, SQRT, SIN, COS, TAN, ASIN, ACOS, ATAN, SINH, COSH, ASINH, ACOSH, ATANH, RSQRT,
 RECIPROCAL, SQUARE, CUBE, EXP, LN, LN1P, FLOOR, CEIL, ROUND, TRUNC, EXPM1, SILU) = range(31)
SUM, PROD, MAX, MIN, MEAN = 1, 2, 3, 4, 5
VARIANCE, LOGSUMEXP, NORM, ARGMAX, ARGMIN = 6, 7, 8, 9, 10   # ReductionOpTypes::get_code, ops/reduction/mod.rs:160-175

NP_TO_CODE = {
    np.dtype(np.uint8): U8, np.dtype(np.int8): I8, np.dtype(np.uint16): U16, np.dtype(np.int16): I16,
    np.dtype(np.uint32): U32, np.dtype(np.int32): I32, np.dtype(np.uint64): U64, np.dtype(np.int64): I64,
    np.dtype(np.float32): F32, np.dtype(np.float64): F64, np.dtype(np.bool_): BOOL,
}


def build(force: bool = False) -> None:
    """Compile liboracle.so / liboracle_fast.so with gcc if missing or older than the source."""
    src = os.path.join(_HERE, "rt_oracle.c")
    outs = [os.path.join(_HERE, "liboracle.so"), os.path.join(_HERE, "liboracle_fast.so")]
    stale = force or any((not os.path.exists(o)) or os.path.getmtime(o) < os.path.getmtime(src) for o in outs)
    if stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)


def _sizes(xs: Sequence[int]):
    return (C.c_size_t * max(len(xs), 1))(*[int(x) for x in xs])


def _diffs(xs: Sequence[int]):
    return (C.c_ssize_t * max(len(xs), 1))(*[int(x) for x in xs])


class _Lib:
    def __init__(self, fast: bool):
        build()
        self.lib = C.CDLL(os.path.join(_HERE, "liboracle_fast.so" if fast else "liboracle.so"))
        self.lib.orc_sum_f64_of_f32.restype = C.c_double
        self.lib.orc_abs_sum_f64_of_f32.restype = C.c_double


_LIBS = {}


def lib(fast: bool = False) -> C.CDLL:
    if fast not in _LIBS:
        _LIBS[fast] = _Lib(fast)
    return _LIBS[fast].lib


class OracleError(Exception):
    def __init__(self, code: int):
        super().__init__(f"oracle error {code}")
        self.code = code


def _chk(rc: int) -> None:
    if rc != 0:
        raise OracleError(rc)


@dataclass(frozen=True)
class Meta:
    """(shape, strides, offset) in elements, as MetaTensor of the reference (core/meta.rs:155-159)."""
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    offset: int = 0

    @staticmethod
    def contiguous(shape: Sequence[int]) -> "Meta":
        shape = tuple(int(s) for s in shape)
        out = (C.c_ssize_t * max(len(shape), 1))()
        lib().orc_shape_to_stride(C.c_size_t(len(shape)), _sizes(shape), out)
        return Meta(shape, tuple(out[: len(shape)]), 0)

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def is_contiguous(self) -> bool:
        return bool(lib().orc_is_contiguous(C.c_size_t(self.rank), _sizes(self.shape), _diffs(self.strides)))

    def layout_class(self) -> int:
        return int(lib().orc_layout_class(C.c_size_t(self.rank), _sizes(self.shape), _diffs(self.strides)))

    def slice(self, dim: int, start: Optional[int] = None, end: Optional[int] = None, step: int = 1) -> "Meta":
        r = self.rank
        osh = (C.c_size_t * max(r, 1))()
        ost = (C.c_ssize_t * max(r, 1))()
        orank = C.c_size_t()
        ooff = C.c_size_t()
        _chk(lib().orc_slice(C.c_size_t(r), _sizes(self.shape), _diffs(self.strides), C.c_size_t(self.offset),
                             C.c_size_t(dim), C.c_int(start is not None), C.c_size_t(start or 0),
                             C.c_int(end is not None), C.c_size_t(end or 0), C.c_ssize_t(step),
                             C.byref(orank), osh, ost, C.byref(ooff)))
        k = orank.value
        return Meta(tuple(osh[:k]), tuple(ost[:k]), ooff.value)

    def index(self, dim: int, i: int) -> "Meta":
        """`slice(dim, i..i)`: removes the dimension (core/slice.rs:107-115, 213-223)."""
        return self.slice(dim, i, i, 1)

    def permute(self, dims: Sequence[int]) -> "Meta":
        r = self.rank
        osh = (C.c_size_t * max(r, 1))()
        ost = (C.c_ssize_t * max(r, 1))()
        _chk(lib().orc_permute(C.c_size_t(r), _sizes(self.shape), _diffs(self.strides), C.c_size_t(len(dims)),
                               _sizes(dims), osh, ost))
        return Meta(tuple(osh[:r]), tuple(ost[:r]), self.offset)

    def unsqueeze(self, dim: int) -> "Meta":
        r = self.rank
        osh = (C.c_size_t * (r + 1))()
        ost = (C.c_ssize_t * (r + 1))()
        _chk(lib().orc_unsqueeze(C.c_size_t(r), _sizes(self.shape), _diffs(self.strides), C.c_size_t(dim), osh, ost))
        return Meta(tuple(osh[: r + 1]), tuple(ost[: r + 1]), self.offset)

    def squeeze(self, dim: Optional[int] = None) -> "Meta":
        r = self.rank
        osh = (C.c_size_t * max(r, 1))()
        ost = (C.c_ssize_t * max(r, 1))()
        orank = C.c_size_t()
        _chk(lib().orc_squeeze(C.c_size_t(r), _sizes(self.shape), _diffs(self.strides),
                               C.c_ssize_t(-1 if dim is None else dim), C.byref(orank), osh, ost))
        k = orank.value
        return Meta(tuple(osh[:k]), tuple(ost[:k]), self.offset)

    def view_as(self, shape: Sequence[int]) -> "Meta":
        """Re-label a contiguous tensor with another shape of the same size, same offset."""
        m = Meta.contiguous(shape)
        if m.size != self.size or not self.is_contiguous():
            raise OracleError(-3)
        return Meta(m.shape, m.strides, self.offset)


def broadcast_params(a: Meta, b: Meta) -> Tuple[Tuple[int, ...], Tuple[int, ...], Tuple[int, ...]]:
    r = max(a.rank, b.rank)
    osh = (C.c_size_t * max(r, 1))()
    osa = (C.c_ssize_t * max(r, 1))()
    osb = (C.c_ssize_t * max(r, 1))()
    orank = C.c_size_t()
    _chk(lib().orc_broadcast_params(C.c_size_t(a.rank), _sizes(a.shape), _diffs(a.strides), C.c_size_t(b.rank),
                                    _sizes(b.shape), _diffs(b.strides), C.byref(orank), osh, osa, osb))
    return tuple(osh[:r]), tuple(osa[:r]), tuple(osb[:r])


def _code(arr: np.ndarray) -> int:
    return NP_TO_CODE[arr.dtype]


def _ptr(arr: np.ndarray):
    return arr.ctypes.data_as(C.c_void_p)


def elementwise(buf: np.ndarray, kind: int, op: int, value, meta: Meta, fast: bool = False) -> None:
    """In-place scalar op (kind 0), unary op (kind 1) or fill (kind 2) over the view `meta` of `buf`."""
    assert buf.flags.c_contiguous and buf.ndim == 1
    if meta.is_contiguous() and meta.offset + meta.size > buf.size:
        # A view whose strides are dense up to sign counts as "contiguous" in the reference
        # (core/meta.rs:526-541) and is then walked FORWARD from its offset: the Rust slice index
        # `buf[start..start+len]` panics.  Refuse here instead of writing past the numpy buffer.
        raise OracleError(-2)
    v = np.array([0 if value is None else value], dtype=buf.dtype)
    _chk(lib(fast).orc_elementwise(C.c_int(_code(buf)), _ptr(buf), C.c_int(kind), C.c_int(op), _ptr(v),
                                   C.c_size_t(meta.rank), _sizes(meta.shape), _diffs(meta.strides),
                                   C.c_size_t(meta.offset)))


MASK_RELU, MASK_ABS, MASK_LEAKY_RELU, MASK_RECIPROCAL = 1, 2, 3, 4


def grad_mask(buf: np.ndarray, kind: int, meta: Meta, value=None, fast: bool = False) -> np.ndarray:
    """The relu / abs / leaky_relu gradient map or the reciprocal map of the view `meta` of `buf` as a
    dense array (ops/unary/mod.rs:213-252, ops/scalar/mod.rs:149-166, ops/broadcast/div.rs:583-587)."""
    assert buf.flags.c_contiguous and buf.ndim == 1
    out = np.zeros(max(meta.size, 1), dtype=buf.dtype)
    v = None if value is None else np.array([value], dtype=buf.dtype)
    _chk(lib(fast).orc_grad_mask(C.c_int(_code(buf)), C.c_int(kind), None if v is None else _ptr(v), _ptr(buf),
                                 C.c_size_t(meta.rank), _sizes(meta.shape), _diffs(meta.strides), C.c_size_t(meta.offset),
                                 _ptr(out)))
    return out[: meta.size]


def scalar_op(buf, op, value, meta, fast=False):
    elementwise(buf, 0, op, value, meta, fast)


def unary_op(buf, op, meta, fast=False):
    elementwise(buf, 1, op, None, meta, fast)


def fill(buf, value, meta, fast=False):
    elementwise(buf, 2, 0, value, meta, fast)


def broadcast(l: np.ndarray, lmeta: Meta, r: np.ndarray, rmeta: Meta, d: np.ndarray, dmeta: Meta, op: int,
              fast: bool = False) -> None:
    """Backend::broadcast: all metas carry the output shape; d may be the same array as l."""
    assert lmeta.shape == rmeta.shape == dmeta.shape
    _chk(lib(fast).orc_broadcast(C.c_int(_code(d)), _ptr(l), _ptr(r), _ptr(d), C.c_int(op), C.c_size_t(dmeta.rank),
                                 _sizes(dmeta.shape), _diffs(lmeta.strides), C.c_size_t(lmeta.offset),
                                 _diffs(rmeta.strides), C.c_size_t(rmeta.offset), _diffs(dmeta.strides),
                                 C.c_size_t(dmeta.offset)))


def binary(a: np.ndarray, ameta: Meta, b: np.ndarray, bmeta: Meta, op: int, fast: bool = False):
    """Out-of-place `a op b` as the operator impls do it (ops/broadcast/add.rs:441-477):
    broadcast params, fresh row-major output."""
    shape, sa, sb = broadcast_params(ameta, bmeta)
    dm = Meta.contiguous(shape)
    out = np.zeros(dm.size, dtype=a.dtype)
    broadcast(a, Meta(shape, sa, ameta.offset), b, Meta(shape, sb, bmeta.offset), out, dm, op, fast)
    return out, dm


def reduce_flat(src: np.ndarray, start: int, length: int, op: int, fast: bool = False):
    out = np.zeros(1, dtype=src.dtype)
    _chk(lib(fast).orc_reduce_flat(C.c_int(_code(src)), _ptr(src), C.c_size_t(start), C.c_size_t(length),
                                   C.c_int(op), _ptr(out)))
    return out


def reduce_axis(src: np.ndarray, meta: Meta, axis: int, op: int, fast: bool = False):
    """`<op>_at(axis)` on a contiguous tensor: output keeps the reduced dim as size 1."""
    oshape = tuple(1 if k == axis else s for k, s in enumerate(meta.shape))
    om = Meta.contiguous(oshape)
    out = np.zeros(max(om.size, 1), dtype=src.dtype)
    _chk(lib(fast).orc_reduce_axis(C.c_int(_code(src)), _ptr(src), C.c_size_t(meta.rank), _sizes(meta.shape),
                                   _diffs(meta.strides), C.c_size_t(meta.offset), C.c_size_t(axis), C.c_int(op),
                                   _ptr(out)))
    return out, om


def reduce_ori(src: np.ndarray, outer: int, r: int, inner: int, op: int, fast: bool = False):
    out = np.zeros(max(outer * inner, 1), dtype=src.dtype)
    _chk(lib(fast).orc_reduce_ori(C.c_int(_code(src)), _ptr(src), C.c_size_t(outer), C.c_size_t(r),
                                  C.c_size_t(inner), C.c_int(op), _ptr(out)))
    return out


def reduce_ext_ori(src: np.ndarray, outer: int, r: int, inner: int, op: int, unbiased: bool = True, is_std: bool = False,
                   norm_type: int = 2, fast: bool = False):
    """variance / std / norm / logsumexp of a contiguous (outer, R, inner) block over R; flat = (1, n, 1)."""
    out = np.zeros(max(outer * inner, 1), dtype=src.dtype)
    _chk(lib(fast).orc_reduce_ext_ori(C.c_int(_code(src)), _ptr(src), C.c_size_t(outer), C.c_size_t(r), C.c_size_t(inner),
                                      C.c_int(op), C.c_int(bool(unbiased)), C.c_int(bool(is_std)), C.c_int(norm_type),
                                      _ptr(out)))
    return out


def argreduce_ori(src: np.ndarray, outer: int, r: int, inner: int, op: int, fast: bool = False):
    """argmax / argmin positions (u64) along R of a contiguous (outer, R, inner) block."""
    out = np.zeros(max(outer * inner, 1), dtype=np.uint64)
    _chk(lib(fast).orc_argreduce_ori(C.c_int(_code(src)), _ptr(src), C.c_size_t(outer), C.c_size_t(r), C.c_size_t(inner),
                                     C.c_int(op), _ptr(out)))
    return out


def l1_loss(a: np.ndarray, b: np.ndarray, reduction: int = 0, with_grad: bool = False, fast: bool = False):
    loss = np.zeros(1, dtype=a.dtype)
    g = np.zeros(a.size, dtype=a.dtype) if with_grad else None
    _chk(lib(fast).orc_l1_loss(C.c_int(_code(a)), _ptr(a), _ptr(b), C.c_size_t(a.size), C.c_int(reduction),
                               _ptr(loss), _ptr(g) if with_grad else None))
    return loss, g


def reduce_to_shape(upstream: np.ndarray, shape: Sequence[int], operand_strides: Sequence[int],
                    intended: bool = True):
    r = len(shape)
    out = np.zeros(upstream.size, dtype=upstream.dtype)
    osh = (C.c_size_t * max(r, 1))()
    _chk(lib().orc_reduce_to_shape(C.c_int(_code(upstream)), _ptr(upstream), C.c_size_t(r), _sizes(shape),
                                   _diffs(operand_strides), C.c_int(1 if intended else 0), _ptr(out), osh))
    oshape = tuple(osh[:r])
    n = 1
    for s in oshape:
        n *= s
    return out[:n].copy(), oshape


def relu_mask(x: np.ndarray):
    mask = np.zeros_like(x)
    if x.dtype == np.float64:
        lib().orc_relu_mask_f64(_ptr(x), _ptr(mask), C.c_size_t(x.size))
    else:
        lib().orc_relu_mask_f32(_ptr(x), _ptr(mask), C.c_size_t(x.size))
    return mask


def sgd_update(p: np.ndarray, g: np.ndarray, lr: float) -> None:
    if p.dtype == np.float64:
        lib().orc_sgd_update_f64(_ptr(p), _ptr(g), C.c_double(lr), C.c_size_t(p.size))
    else:
        lib().orc_sgd_update_f32(_ptr(p), _ptr(g), C.c_float(lr), C.c_size_t(p.size))


def u8_to_f32_div(src: np.ndarray, divisor: float = 255.0) -> np.ndarray:
    out = np.zeros(src.size, dtype=np.float32)
    lib().orc_u8_to_f32_div(_ptr(src), _ptr(out), C.c_float(divisor), C.c_size_t(src.size))
    return out


DTYPE_SIZE = {U8: 1, I8: 1, U16: 2, I16: 2, U32: 4, U128: 16, I32: 4, U64: 8, I64: 8, I128: 16, F32: 4, F64: 8, BOOL: 1}


def convert(src_bytes: bytes, src_dtype: int, dst_dtype: int, fast: bool = False) -> bytes:
    """Backend::convert over raw little-endian element bytes (so that the 128-bit types, which numpy
    lacks, go through the same door).  Returns the destination buffer's bytes."""
    if src_dtype not in DTYPE_SIZE or dst_dtype not in DTYPE_SIZE:
        raise OracleError(-5)
    n, rem = divmod(len(src_bytes), DTYPE_SIZE[src_dtype])
    assert rem == 0
    src = np.frombuffer(bytes(src_bytes), dtype=np.uint8).copy() if n else np.zeros(1, np.uint8)
    out = np.zeros(max(n * DTYPE_SIZE[dst_dtype], 1), dtype=np.uint8)
    rc = lib(fast).orc_convert(C.c_int(src_dtype), C.c_int(dst_dtype), _ptr(src), _ptr(out), C.c_size_t(n))
    if rc != 0:
        raise OracleError(rc)
    return out[: n * DTYPE_SIZE[dst_dtype]].tobytes()


def gemm(a: np.ndarray, b: np.ndarray, m: int, k: int, n: int, ta: bool = False, tb: bool = False) -> np.ndarray:
    c = np.zeros(m * n, dtype=np.float32)
    lib(True).orc_gemm_f32(_ptr(a), _ptr(b), _ptr(c), C.c_size_t(m), C.c_size_t(k), C.c_size_t(n),
                           C.c_int(ta), C.c_int(tb))
    return c


def sum_f64(x: np.ndarray) -> float:
    return float(lib(True).orc_sum_f64_of_f32(_ptr(x), C.c_size_t(x.size)))


def abs_sum_f64(x: np.ndarray) -> float:
    return float(lib(True).orc_abs_sum_f64_of_f32(_ptr(x), C.c_size_t(x.size)))
