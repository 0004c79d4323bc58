"""`Tensor`: the host mirror of the reference's `TensorBase<T, B>` / `TensorView` API surface that
the hot path exercises (src/core/primitives.rs:367-484, src/core/tensor.rs:66-105, 418-524,
src/ops/{scalar,unary,broadcast,reduction}).  A Tensor is (backend, flat device buffer, Meta);
views share the buffer.  Semantics follow the reference operators: `a + 3` copies then works in
place, `a += b` requires b to broadcast to a's shape, `sum_at(k)` keeps dim k as size 1 and first
copies a non-contiguous view, full reductions return a rank-0 tensor.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib as L
from . import grad as _grad
from .backend import CODE_TO_NP, CudaB200, dtype_code
from .meta import Meta

_NP_TO_TORCH = {np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64,
                np.dtype(np.int8): torch.int8, np.dtype(np.int16): torch.int16, np.dtype(np.int32): torch.int32,
                np.dtype(np.int64): torch.int64, np.dtype(np.uint8): torch.uint8, np.dtype(np.bool_): torch.bool}
for _n in ("uint16", "uint32", "uint64"):
    if hasattr(torch, _n):
        _NP_TO_TORCH[np.dtype(getattr(np, _n))] = getattr(torch, _n)

_default_backend: Optional[CudaB200] = None


def default_backend() -> CudaB200:
    global _default_backend
    if _default_backend is None:
        _default_backend = CudaB200(torch.cuda.current_device() if torch.cuda.is_available() else 0)
    return _default_backend


class Tensor:
    def __init__(self, backend: CudaB200, buf: torch.Tensor, meta: Meta):
        self.backend, self.buf, self.meta = backend, buf, meta
        self.op = None      # key of the tape node that produced this tensor (rtensors_b200.grad)
        self.grad = None    # GradHolder of a leaf (set by param())

    @property
    def np_dtype(self):
        return CODE_TO_NP[dtype_code(self.buf)]

    def param(self) -> "Tensor":
        """Marks the tensor as a trainable leaf of the current grad context (TensorBase::param)."""
        _grad.make_leaf(self)
        return self

    # ---- constructors -----------------------------------------------------------------------
    @staticmethod
    def from_buf(data, shape: Sequence[int], dtype=np.float32, backend: Optional[CudaB200] = None) -> "Tensor":
        b = backend or default_backend()
        host = np.ascontiguousarray(np.asarray(data, dtype=dtype).reshape(-1))
        meta = Meta.contiguous(shape)
        if host.size != meta.size:
            raise ValueError(f"Element count mismatch: shape {tuple(shape)} vs buffer of {host.size}")
        return Tensor(b, b.alloc_from_slice(host), meta)

    @staticmethod
    def full(shape, value, dtype=np.float32, backend=None) -> "Tensor":
        b = backend or default_backend()
        meta = Meta.contiguous(shape)
        t = Tensor(b, b.alloc(max(meta.size, 1), _NP_TO_TORCH[np.dtype(dtype)]), meta)
        b.fill(t.buf, value, meta)
        return t

    @staticmethod
    def zeros(shape, dtype=np.float32, backend=None): return Tensor.full(shape, 0, dtype, backend)

    @staticmethod
    def ones(shape, dtype=np.float32, backend=None): return Tensor.full(shape, 1, dtype, backend)

    @staticmethod
    def scalar(value, dtype=np.float32, backend=None): return Tensor.from_buf([value], (), dtype, backend)

    @staticmethod
    def column(values, dtype=np.float32, backend=None):  # shape (n,), src/core/primitives.rs:428-432
        return Tensor.from_buf(values, (len(values),), dtype, backend)

    @staticmethod
    def row(values, dtype=np.float32, backend=None):  # shape (1, n), src/core/primitives.rs:440-444
        return Tensor.from_buf(values, (1, len(values)), dtype, backend)

    # ---- meta -------------------------------------------------------------------------------
    @property
    def shape(self): return self.meta.shape
    @property
    def strides(self): return self.meta.strides
    @property
    def offset(self): return self.meta.offset
    @property
    def size(self): return self.meta.size
    @property
    def rank(self): return self.meta.rank
    def is_contiguous(self): return self.meta.is_contiguous()

    def _view(self, meta: Meta) -> "Tensor": return Tensor(self.backend, self.buf, meta)

    def view(self):
        v = self._view(self.meta)
        v.op, v.grad = self.op, self.grad
        return v

    def slice(self, dim, start=None, end=None, step=1): return self._view(self.meta.slice(dim, start, end, step))
    def index(self, dim, i): return self._view(self.meta.index(dim, i))

    def permute(self, dims):
        v = self._view(self.meta.permute(dims))
        _grad.attach_unary("Permute", v, self, dims=tuple(dims))
        return v

    def transpose(self): return self.permute(tuple(reversed(range(self.rank))))

    def squeeze(self, dim=None):
        v = self._view(self.meta.squeeze(dim))
        _grad.attach_unary("Squeeze", v, self, original_shape=tuple(self.shape))
        return v

    def unsqueeze(self, dim):
        v = self._view(self.meta.unsqueeze(dim))
        _grad.attach_unary("Unsqueeze", v, self, dim=dim)
        return v

    def view_as(self, shape): return self._view(self.meta.view_as(shape))

    def contiguous(self) -> "Tensor":
        return Tensor(self.backend, self.backend.contiguous(self.buf, self.meta), Meta.contiguous(self.shape))

    owned = contiguous

    def reshape(self, shape) -> "Tensor":
        """contiguous() then view_as: always a fresh buffer (src/core/tensor.rs:238-243)."""
        c = self.contiguous()
        out = Tensor(c.backend, c.buf, c.meta.view_as(shape))
        _grad.attach_unary("Reshape", out, self, original_shape=tuple(self.shape))
        return out

    def into_dtype(self, dtype) -> "Tensor":
        """A tensor of the same meta over a converted copy of the whole buffer
        (src/core/primitives.rs:527-538: alloc + Backend::convert, meta cloned)."""
        out = self.backend.convert(self.buf, _NP_TO_TORCH[np.dtype(dtype)])
        return Tensor(self.backend, out, self.meta)

    # ---- host access ------------------------------------------------------------------------
    def cpu(self) -> np.ndarray:
        flat = self.backend.dump(self.contiguous().buf)[: max(self.size, 1) if self.rank == 0 else self.size]
        return flat.reshape(self.shape)

    def item(self):
        if self.size != 1:
            raise ValueError("item() needs a single-element tensor")
        return self.cpu().reshape(-1)[0]

    def get(self, coord):
        return self.backend.dump(self.buf[self.offset + sum(c * s for c, s in zip(coord, self.strides))].reshape(1))[0]

    def set(self, coord, value):
        self.buf[self.offset + sum(c * s for c, s in zip(coord, self.strides))] = value

    def fill(self, value): self.backend.fill(self.buf, value, self.meta)

    # ---- scalar / tensor operators ----------------------------------------------------------
    def _binary(self, other, op: int) -> "Tensor":
        if isinstance(other, Tensor):
            out, dm = self.backend.binary(self.buf, self.meta, other.buf, other.meta, op)
            res = Tensor(self.backend, out, dm)
            if op in _BROADCAST_NODE:
                _grad.attach_broadcast(_BROADCAST_NODE[op], res, self, other)
            return res
        t = self.owned()
        t.backend.scalar_apply(t.buf, op, other, t.meta)
        if op == L.ADD or op == L.SUB:
            _grad.attach_unary("AddScalar", t, self)
        elif op == L.MUL:
            _grad.attach_unary("MulScalar", t, self, scalar=other)
        elif op == L.DIV:
            _grad.attach_unary("DivScalar", t, self, scalar=other)
        return t

    def matmul(self, other: "Tensor") -> "Tensor":
        """2-D matrix product on cuBLAS (matmul stays a library GEMM by design; the reference calls
        cuBLAS too, src/backend/cuda.rs:2139-2280).  Operands may be transposed / strided views."""
        if self.rank != 2 or other.rank != 2 or self.shape[1] != other.shape[0]:
            raise ValueError(f"matmul needs (m,k) x (k,n), got {self.shape} x {other.shape}")

        def as_torch(t):
            if any(st < 0 for st in t.strides):
                t = t.contiguous()
            return torch.as_strided(t.buf, t.shape, t.strides, t.offset)
        out = torch.matmul(as_torch(self), as_torch(other))
        res = Tensor(self.backend, out.reshape(-1), Meta.contiguous((self.shape[0], other.shape[1])))
        _grad.attach_matmul(res, self, other)
        return res

    def _assign(self, other, op: int) -> "Tensor":
        if isinstance(other, Tensor):
            self.backend.binary_assign(self.buf, self.meta, other.buf, other.meta, op)
        else:
            self.backend.scalar_apply(self.buf, op, other, self.meta)
        return self

    def __add__(self, o): return self._binary(o, L.ADD)
    def __sub__(self, o): return self._binary(o, L.SUB)
    def __mul__(self, o): return self._binary(o, L.MUL)
    def __truediv__(self, o): return self._binary(o, L.DIV)
    def __iadd__(self, o): return self._assign(o, L.ADD)
    def __isub__(self, o): return self._assign(o, L.SUB)
    def __imul__(self, o): return self._assign(o, L.MUL)
    def __itruediv__(self, o): return self._assign(o, L.DIV)

    # ---- unary ------------------------------------------------------------------------------
    def _unary_inplace(self, op):
        self.backend.apply_unary(self.buf, op, self.meta)
        return self

    def relu_inplace(self): return self._unary_inplace(L.RELU)
    def abs_inplace(self): return self._unary_inplace(L.ABS)
    def sign_inplace(self): return self._unary_inplace(L.SIGN)
    def neg_inplace(self): return self._unary_inplace(L.NEG)
    def relu(self):
        out = self.owned().relu_inplace()
        if _grad.is_enabled():   # the map of the pre-activation, one kernel (the reference: a get/set loop)
            _grad.attach_unary("ReLU", out, self, grad_map=self.relu_grad_map())
        return out

    def abs(self):
        out = self.owned().abs_inplace()
        if _grad.is_enabled():
            _grad.attach_unary("Abs", out, self, grad_map=self.abs_grad_map())
        return out

    def sign(self): return self.owned().sign_inplace()

    def neg(self):
        out = self.owned().neg_inplace()
        _grad.attach_unary("Negate", out, self)
        return out

    def __neg__(self): return self.neg()

    # gradient maps the reference's autograd stores for relu and abs (src/ops/unary/mod.rs:213-252)
    def relu_grad_map(self) -> "Tensor":
        return Tensor(self.backend, self.backend.grad_mask(self.buf, self.meta, L.MASK_RELU), Meta.contiguous(self.shape))

    def abs_grad_map(self) -> "Tensor":
        return Tensor(self.backend, self.backend.grad_mask(self.buf, self.meta, L.MASK_ABS), Meta.contiguous(self.shape))

    def leaky_relu_grad_map(self, slope) -> "Tensor":  # src/ops/scalar/mod.rs:149-166
        return Tensor(self.backend, self.backend.grad_mask(self.buf, self.meta, L.MASK_LEAKY_RELU, slope),
                      Meta.contiguous(self.shape))

    def reciprocal_map(self) -> "Tensor":  # 1 / x, src/ops/broadcast/div.rs:583-587
        return Tensor(self.backend, self.backend.grad_mask(self.buf, self.meta, L.MASK_RECIPROCAL), Meta.contiguous(self.shape))

    # ---- reductions -------------------------------------------------------------------------
    def _reduce(self, op: int, axis: Optional[int]) -> "Tensor":
        # The reference copies a non-contiguous view first (`contiguous()`); here the library reduces
        # the view in place where its layout allows and copies only otherwise -- same result.
        b = self.backend
        if axis is None:
            return Tensor(b, b.reduce_view(self.buf, self.meta, None, op), Meta.contiguous(()))
        if not 0 <= axis < self.rank:
            raise L.RtbError(-5, f"axis {axis} out of range for rank {self.rank}")
        om = Meta.contiguous(tuple(1 if k == axis else s for k, s in enumerate(self.shape)))
        return Tensor(b, b.reduce_view(self.buf, self.meta, axis, op), om)

    def sum(self): return self._reduce(L.SUM, None)
    def mean(self): return self._reduce(L.MEAN, None)
    def max(self): return self._reduce(L.MAX, None)
    def min(self): return self._reduce(L.MIN, None)
    def prod(self): return self._reduce(L.PROD, None)
    def sum_at(self, axis): return self._reduce(L.SUM, axis)
    def mean_at(self, axis): return self._reduce(L.MEAN, axis)
    def max_at(self, axis): return self._reduce(L.MAX, axis)
    def min_at(self, axis): return self._reduce(L.MIN, axis)
    def prod_at(self, axis): return self._reduce(L.PROD, axis)

    # The reductions only the reference's CUDA backend implements (ReductionOp, src/ops/reduction/mod.rs:413-510).
    def _reduce_ex(self, op: int, axis: Optional[int], unbiased=True, is_std=False, norm_type=2) -> "Tensor":
        b = self.backend
        if axis is not None and not 0 <= axis < self.rank:
            raise ValueError(f"axis {axis} out of range for rank {self.rank}")
        out = b.reduce_view_ex(self.buf, self.meta, axis, op, unbiased, is_std, norm_type)
        shape = () if axis is None else tuple(1 if k == axis else s for k, s in enumerate(self.shape))
        return Tensor(b, out, Meta.contiguous(shape))

    def var_at(self, axis): return self._reduce_ex(L.VARIANCE, axis, True)
    def pop_var_at(self, axis): return self._reduce_ex(L.VARIANCE, axis, False)
    def std_at(self, axis, unbiased=True): return self._reduce_ex(L.VARIANCE, axis, unbiased, True)
    def norm_at(self, axis, norm_type=2): return self._reduce_ex(L.NORM, axis, norm_type=norm_type)
    def l1_norm_at(self, axis): return self.norm_at(axis, 1)
    def l2_norm_at(self, axis): return self.norm_at(axis, 2)
    def logsumexp_at(self, axis): return self._reduce_ex(L.LOGSUMEXP, axis)
    def argmax_at(self, axis): return self._reduce_ex(L.ARGMAX, axis)
    def argmin_at(self, axis): return self._reduce_ex(L.ARGMIN, axis)
    def var(self): return self.var_at(None)
    def pop_var(self): return self.pop_var_at(None)
    def std(self, unbiased=True): return self.std_at(None, unbiased)
    def norm(self, norm_type=2): return self.norm_at(None, norm_type)
    def l1_norm(self): return self.norm_at(None, 1)
    def l2_norm(self): return self.norm_at(None, 2)
    def logsumexp(self): return self.logsumexp_at(None)
    def argmax(self): return self.argmax_at(None)
    def argmin(self): return self.argmin_at(None)


def mean_l1_loss(a: Tensor, b: Tensor, with_grad: bool = False):
    """mean(|a - b|) as a rank-0 tensor (src/ops/broadcast/l1.rs:79-84); with_grad also returns the
    gradient map sign(a - b) / N the reference stores on the tape."""
    if a.shape != b.shape:
        raise ValueError("mean_l1_loss needs equal shapes")
    ca = a if a.is_contiguous() else a.contiguous()
    cb = b if b.is_contiguous() else b.contiguous()
    n = a.size
    loss, g = a.backend.l1_loss(ca.buf[ca.offset: ca.offset + n], cb.buf[cb.offset: cb.offset + n], 0, with_grad)
    lt = Tensor(a.backend, loss, Meta.contiguous(()))
    if with_grad:
        return lt, Tensor(a.backend, g, Meta.contiguous(a.shape))
    return lt


_BROADCAST_NODE = {L.ADD: "BroadcastAdd", L.SUB: "BroadcastSub", L.MUL: "BroadcastMul", L.DIV: "BroadcastDiv"}

# The float-only unary families (src/ops/unary/mod.rs): `t.sigmoid()` copies then works in place, as the
# reference's owned forms do; under a grad context each attaches its node with the tensor its backward
# function needs -- the input, the result, or (ln) the reciprocal of the input.
_UNARY_NODES = {"sigmoid": (L.SIGMOID, "Sigmoid", "result"), "tanh": (L.TANH, "Tanh", "result"), "sqrt": (L.SQRT, "Sqrt", "result"),
                "exp": (L.EXP, "Exp", "result"), "reciprocal": (L.RECIPROCAL, "Reciprocal", "result"),
                "rsqrt": (L.RSQRT, "Rsqrt", "result"), "ln": (L.LN, "Ln", "x_reciprocal"), "sin": (L.SIN, "Sin", "input"),
                "cos": (L.COS, "Cos", "input"), "tan": (L.TAN, "Tan", "input"), "square": (L.SQUARE, "Square", "input"),
                "cube": (L.CUBE, "Cube", "input"), "sinh": (L.SINH, "Sinh", "input"), "cosh": (L.COSH, "Cosh", "input"),
                "expm1": (L.EXPM1, "ExpM1", "input"), "ln1p": (L.LN1P, "Ln1p", "input")}


def _make_unary(name, code, node, saves):
    def inplace(self):
        return self._unary_inplace(code)

    def owned(self):
        out = self.owned()._unary_inplace(code)
        if _grad.is_enabled():
            if saves == "result":
                _grad.attach_unary(node, out, self, result=out)
            elif saves == "input":
                _grad.attach_unary(node, out, self, input=self)
            else:
                _grad.attach_unary(node, out, self, x_reciprocal=self.reciprocal_map())
        return out
    inplace.__name__, owned.__name__ = name + "_inplace", name
    setattr(Tensor, name + "_inplace", inplace)
    setattr(Tensor, name, owned)


for _name, (_code, _node, _saves) in _UNARY_NODES.items():
    _make_unary(_name, _code, _node, _saves)


def mean_l1_loss_tracked(a: Tensor, b: Tensor) -> Tensor:
    """mean_l1_loss under a grad context: the loss and the gradient map sign(a - b) / N come out of one
    fused kernel and an L1 node goes on the tape (attach_l1_grad, src/ops/broadcast/l1.rs:16-46)."""
    if not _grad.is_enabled():
        return mean_l1_loss(a, b)
    loss, gmap = mean_l1_loss(a, b, with_grad=True)
    _grad.attach_l1(loss, a, b, gmap)
    return loss
