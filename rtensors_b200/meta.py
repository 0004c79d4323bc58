"""View metadata (shape, strides, offset in elements) -- the host mirror of the reference's
MetaTensor (src/core/meta.rs:155-159); every computation is done by the library's C++ planner."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from functools import cached_property, lru_cache
from typing import Optional, Sequence, Tuple

from ._lib import Plan, check, diffs, lib, sizes


@dataclass(frozen=True)
class Meta:
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    offset: int = 0

    @staticmethod
    def contiguous(shape: Sequence[int]) -> "Meta":
        return _contiguous(tuple(int(s) for s in shape))

    @property
    def rank(self) -> int:
        return len(self.shape)

    # the ctypes arrays every launch passes; built once per Meta (instances are immutable)
    @cached_property
    def c_shape(self):
        return sizes(self.shape)

    @cached_property
    def c_strides(self):
        return diffs(self.strides)

    @property
    def size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def is_contiguous(self) -> bool:
        return bool(lib().rtb_meta_is_contiguous(C.c_size_t(self.rank), sizes(self.shape), diffs(self.strides)))

    def slice(self, dim: int, start: Optional[int] = None, end: Optional[int] = None, step: int = 1) -> "Meta":
        r = self.rank
        osh = (C.c_size_t * max(r, 1))()
        ost = (C.c_ssize_t * max(r, 1))()
        orank, ooff = C.c_size_t(), C.c_size_t()
        check(lib().rtb_meta_slice(C.c_size_t(r), sizes(self.shape), diffs(self.strides), C.c_size_t(self.offset),
                                   C.c_size_t(dim), C.c_int(start is not None), C.c_size_t(start or 0),
                                   C.c_int(end is not None), C.c_size_t(end or 0), C.c_ssize_t(step),
                                   C.byref(orank), osh, ost, C.byref(ooff)))
        k = orank.value
        return Meta(tuple(osh[:k]), tuple(ost[:k]), ooff.value)

    def index(self, dim: int, i: int) -> "Meta":
        return self.slice(dim, i, i, 1)

    def permute(self, dims: Sequence[int]) -> "Meta":
        r = self.rank
        osh = (C.c_size_t * max(r, 1))()
        ost = (C.c_ssize_t * max(r, 1))()
        check(lib().rtb_meta_permute(C.c_size_t(r), sizes(self.shape), diffs(self.strides), C.c_size_t(len(dims)),
                                     sizes(dims), osh, ost))
        return Meta(tuple(osh[:r]), tuple(ost[:r]), self.offset)

    def transpose(self) -> "Meta":
        return self.permute(tuple(reversed(range(self.rank))))

    def unsqueeze(self, dim: int) -> "Meta":
        r = self.rank
        osh = (C.c_size_t * (r + 1))()
        ost = (C.c_ssize_t * (r + 1))()
        check(lib().rtb_meta_unsqueeze(C.c_size_t(r), sizes(self.shape), diffs(self.strides), C.c_size_t(dim), osh, ost))
        return Meta(tuple(osh[: r + 1]), tuple(ost[: r + 1]), self.offset)

    def squeeze(self, dim: Optional[int] = None) -> "Meta":
        r = self.rank
        osh = (C.c_size_t * max(r, 1))()
        ost = (C.c_ssize_t * max(r, 1))()
        orank = C.c_size_t()
        check(lib().rtb_meta_squeeze(C.c_size_t(r), sizes(self.shape), diffs(self.strides),
                                     C.c_ssize_t(-1 if dim is None else dim), C.byref(orank), osh, ost))
        k = orank.value
        return Meta(tuple(osh[:k]), tuple(ost[:k]), self.offset)

    def view_as(self, shape: Sequence[int]) -> "Meta":
        m = Meta.contiguous(shape)
        if m.size != self.size or not self.is_contiguous():
            raise ValueError("view_as needs a contiguous tensor and an equal element count")
        return Meta(m.shape, m.strides, self.offset)

    def check_extent(self, buf_len: int) -> None:
        # a view that fits a buffer of n elements fits every longer one: remember the shortest seen
        ok = self.__dict__.get("_fits")
        if ok is not None and buf_len >= ok:
            return
        check(lib().rtb_meta_check_extent(C.c_size_t(self.rank), self.c_shape, self.c_strides,
                                          C.c_size_t(self.offset), C.c_size_t(buf_len)))
        self.__dict__["_fits"] = buf_len if ok is None else min(ok, buf_len)


@lru_cache(maxsize=4096)
def _contiguous(shape: Tuple[int, ...]) -> Meta:
    out = (C.c_ssize_t * max(len(shape), 1))()
    lib().rtb_meta_contiguous_strides(C.c_size_t(len(shape)), sizes(shape), out)
    return Meta(shape, tuple(out[: len(shape)]), 0)


def broadcast_params(a: Meta, b: Meta):
    """-> (out_shape, strides_a, strides_b), compute_broadcasted_params of the reference."""
    r = max(a.rank, b.rank)
    osh = (C.c_size_t * max(r, 1))()
    osa = (C.c_ssize_t * max(r, 1))()
    osb = (C.c_ssize_t * max(r, 1))()
    orank = C.c_size_t()
    check(lib().rtb_broadcast_params(C.c_size_t(a.rank), sizes(a.shape), diffs(a.strides), C.c_size_t(b.rank),
                                     sizes(b.shape), diffs(b.strides), C.byref(orank), osh, osa, osb))
    return tuple(osh[:r]), tuple(osa[:r]), tuple(osb[:r])


def plan_elementwise(dtype: int, n_inputs: int, shape, d: Meta, l: Optional[Meta] = None, r: Optional[Meta] = None,
                     ptr_d: int = 0, ptr_l: int = 0, ptr_r: int = 0) -> Plan:
    """The launch plan the library would use (host only; for tests and diagnostics)."""
    p = Plan()
    l = l or d
    r = r or d
    check(lib().rtb_plan_elementwise(C.c_int(dtype), C.c_int(n_inputs), C.c_size_t(len(shape)), sizes(shape),
                                     diffs(d.strides), C.c_size_t(d.offset), C.c_size_t(ptr_d),
                                     diffs(l.strides), C.c_size_t(l.offset), C.c_size_t(ptr_l),
                                     diffs(r.strides), C.c_size_t(r.offset), C.c_size_t(ptr_r), C.byref(p)))
    return p


def shard_range(extent: int, parts: int, part: int):
    b, e = C.c_size_t(), C.c_size_t()
    lib().rtb_shard_range(C.c_size_t(extent), C.c_size_t(parts), C.c_size_t(part), C.byref(b), C.byref(e))
    return b.value, e.value
