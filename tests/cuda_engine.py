"""Adapter: the CUDA library (through the C ABI) behind the engine interface of golden_runner."""
import numpy as np
import torch

import rtensors_b200 as rt
from rtensors_b200.backend import CudaB200
from rtensors_b200.meta import Meta, broadcast_params

_backend = None


def backend() -> CudaB200:
    global _backend
    if _backend is None:
        _backend = CudaB200(0)
    return _backend


def to_dev(a: np.ndarray) -> torch.Tensor:
    return backend().alloc_from_slice(a)


def to_host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


class CudaEngine:
    Meta = Meta
    tree_sums = True  # float sums are tree-ordered on the GPU (sequential on the CPU backend)

    def __init__(self):
        self.b = backend()

    def broadcast_params(self, a, b):
        return broadcast_params(a, b)

    @staticmethod
    def error_kind(e):
        return {-4: "bounds", -6: "shape", -5: "dim"}.get(getattr(e, "code", None))

    def scalar_assign(self, buf, meta, op, value):
        d = to_dev(buf)
        self.b.scalar_apply(d, op, value, meta)
        return to_host(d)

    def unary_assign(self, buf, meta, op):
        d = to_dev(buf)
        self.b.apply_unary(d, op, meta)
        return to_host(d)

    def fill(self, buf, meta, value):
        d = to_dev(buf)
        self.b.fill(d, value, meta)
        return to_host(d)

    def owned(self, buf, meta):
        return to_host(self.b.contiguous(to_dev(buf), meta))

    def scalar_out(self, buf, meta, op, value):
        d = to_dev(buf)
        out = self.b.contiguous(d, meta)
        m = Meta.contiguous(meta.shape)
        self.b.scalar_apply(out, op, value, m)
        buf[...] = to_host(d)  # the source must be left unchanged: hand it back for the caller's check
        return to_host(out), meta.shape

    def binary(self, a, am, b, bm, op):
        out, dm = self.b.binary(to_dev(a), am, to_dev(b), bm, op)
        return to_host(out), dm.shape

    def binary_assign(self, a, am, b, bm, op):
        d = to_dev(a)
        self.b.binary_assign(d, am, to_dev(b), bm, op)
        return to_host(d)

    def reduce_total(self, a, am, op):
        d = to_dev(a)
        out = self.b.alloc(1, d.dtype)
        self.b.apply_reduce_contiguous_flat(d, out, am.offset, am.size, op)
        return to_host(out)[0]

    def reduce_ext(self, a, am, axis, code, unbiased, is_std, norm_type):
        import torch
        d = to_dev(a)
        if axis is None:
            # Idx::Item goes to the flat launcher over [offset, offset + size) (ops/reduction/mod.rs:262-279)
            flat = self.Meta.contiguous((am.size,))
            flat = type(flat)(flat.shape, flat.strides, am.offset)
            shape, src = (), (d, flat)
        else:
            shape, src = tuple(1 if k == axis else s for k, s in enumerate(am.shape)), (d, am)
        n = max(int(np.prod(shape)), 1)
        out = self.b.alloc(n, torch.int64 if code >= 9 else d.dtype)
        self.b.apply_reduce_ex(src, out, 0 if axis is None else axis, code, unbiased, is_std, norm_type)
        h = to_host(out)
        return (h.view(np.uint64) if code >= 9 else h), shape

    def reduce_axis(self, a, am, axis, op):
        d = to_dev(a)
        oshape = tuple(1 if k == axis else s for k, s in enumerate(am.shape))
        out = self.b.alloc(max(int(np.prod(oshape)), 1), d.dtype)
        self.b.apply_reduce((d, am), out, axis, op)
        return to_host(out), oshape
