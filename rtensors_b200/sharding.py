"""Multi-GPU layer (new: the reference is single-device, `Cuda::new()` -> device 0,
src/backend/cuda.rs:155-162, 815-818).  One process per GPU; the path shards by outer-dimension
slabs with NO data-path collective for elementwise / broadcast work.  Ranks exchange data only where
the path has a real exchange: a reduction over the cut dim combines per-GPU partials.

This module is a binding over the library's `rtb_mg_*` entry points: the partition arithmetic
(`rtb_mg_slab`, `rtb_mg_pick_reduce_dim`, `rtb_shard_range`) is host-only C and runs without a GPU;
with an engine that owns a communicator (`CudaB200.mg_init`) the combines run inside the library --
fused peer-memory exchange for small results, NCCL for large buffers.  An engine without one (the
CPU engine of the gloo tests) combines through `torch.distributed`, so the same host logic is
testable on CPU.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from . import _lib as L
from ._lib import diffs, lib, sizes
from .meta import Meta, broadcast_params, shard_range


def world_info() -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


def init_communicator(be) -> None:
    """Gives the engine's library context its communicator (collective over torch.distributed's
    default group, which only carries the 128-byte id from rank 0 to the others)."""
    world, rank = world_info()
    if world == 1 or getattr(be, "mg_world", 1) == world:
        return
    box = [be.mg_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    be.mg_init(world, rank, box[0])


def _in_library(engine) -> bool:
    return getattr(engine, "mg_world", 1) > 1


def pick_shard_dim(shape, parts: int) -> Optional[int]:
    """Outermost dim with extent >= parts (the slab dim), or None if the tensor is too small."""
    d = lib().rtb_shard_pick_dim(C.c_size_t(len(shape)), sizes(shape), C.c_size_t(parts))
    return None if d < 0 else d


def pick_reduce_dim(shape, axis: int, parts: int) -> Optional[int]:
    """Dim to cut for a reduction over `axis`: a kept dim when one is wide enough (no exchange), else
    the reduced dim, else None."""
    d = lib().rtb_mg_pick_reduce_dim(C.c_size_t(len(shape)), sizes(shape), C.c_size_t(axis), C.c_size_t(parts))
    return None if d < 0 else d


@dataclass(frozen=True)
class BinarySlab:
    """This rank's part of `a op b`: the output slab [begin, end) along `dim` and the operand views
    restricted to it (a broadcast operand keeps stride 0 there and is simply replicated)."""
    full_shape: Tuple[int, ...]
    dim: Optional[int]
    begin: int
    end: int
    shape: Tuple[int, ...]
    left: Meta
    right: Meta


def binary_slab(am: Meta, bm: Meta, world: int, rank: int) -> BinarySlab:
    shape, sa, sb = broadcast_params(am, bm)
    r = len(shape)
    if r == 0:
        sa, sb = (0,), (0,)
    osh = (C.c_size_t * max(r, 1))()
    b, e, ol, orr = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t()
    dim = lib().rtb_mg_slab(C.c_size_t(r), sizes(shape), diffs(sa), C.c_size_t(am.offset), diffs(sb), C.c_size_t(bm.offset),
                            C.c_size_t(world), C.c_size_t(rank), osh, C.byref(b), C.byref(e), C.byref(ol), C.byref(orr))
    sshape = tuple(osh[:r]) if r else ((0,) if e.value == 0 else ())
    if r == 0 and e.value == 0:
        return BinarySlab((), None, 0, 0, (0,), Meta((0,), (0,), am.offset), Meta((0,), (0,), bm.offset))
    return BinarySlab(tuple(shape), None if dim < 0 else dim, b.value, e.value, sshape,
                      Meta(sshape, tuple(sa[:r]), ol.value), Meta(sshape, tuple(sb[:r]), orr.value))


def sharded_binary(engine, a, am: Meta, b, bm: Meta, op: int, world: Optional[int] = None, rank: Optional[int] = None):
    """Computes this rank's slab of the out-of-place broadcast op.  -> (slab buffer, slab Meta, BinarySlab)"""
    if world is None:
        world, rank = world_info()
    slab = binary_slab(am, bm, world, rank)
    dm = Meta.contiguous(slab.shape)
    out = engine.alloc(max(dm.size, 1), a.dtype)
    if dm.size:
        engine.broadcast((a, slab.left), (b, slab.right), (out, dm), op)
    return out, dm, slab


def scalar_slab(n: int, world: int, rank: int) -> Tuple[int, int]:
    """Flat range [begin, end) of a contiguous tensor of n elements owned by this rank."""
    return shard_range(n, world, rank)


_RED = {L.SUM: "sum", L.MEAN: "sum", L.MAX: "max", L.MIN: "min", L.PROD: "prod"}


def _all_reduce(t: torch.Tensor, kind: str, group=None):
    op = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN,
          "prod": dist.ReduceOp.PRODUCT}[kind]
    dist.all_reduce(t, op=op, group=group)


def _as_torch(x):
    return x if isinstance(x, torch.Tensor) else torch.from_numpy(x)


def finish_mean(total: torch.Tensor, count: int) -> torch.Tensor:
    """mean = sum / (T)(float)count, the reference's `from_usize` (src/core/value.rs:54-56)."""
    div = torch.tensor(float(np.float32(count)), dtype=total.dtype, device=total.device)
    return total / div


def sharded_reduce_flat(engine, local, local_len: int, global_len: int, op: int, group=None):
    """Full reduction of a tensor whose flat range is split across ranks: per-GPU partial (one
    launch) + one all-reduce of a single element.  `local` holds this rank's elements."""
    world, _ = world_info()
    if _in_library(engine):   # one launch: local reduction + peer exchange in its last CTA
        return engine.mg_reduce_flat(local, 0, local_len, global_len, op)
    part = engine.alloc(1, local.dtype)
    engine.apply_reduce_contiguous_flat(local, part, 0, local_len, L.SUM if op == L.MEAN else op)
    t = _as_torch(part)
    if world > 1:
        _all_reduce(t, _RED[op], group)
    return finish_mean(t, global_len) if op == L.MEAN else t


def sharded_reduce_axis(engine, local, outer: int, r: int, inner: int, op: int, sharded: str, global_r: int,
                        group=None):
    """Axis reduction of the local [outer, r, inner] block.  sharded = "outer": ranks own disjoint
    outputs, no communication.  sharded = "r": the reduced dim is split, so the partial vectors are
    combined with one all-reduce of outer*inner elements."""
    world, _ = world_info()
    if sharded == "outer" or world == 1:
        return _as_torch(engine.reduce_axis_ori(local, 0, outer, r, inner, op))
    if _in_library(engine):
        return engine.mg_reduce_axis(local, 0, outer, r, inner, global_r, op)
    part = _as_torch(engine.reduce_axis_ori(local, 0, outer, r, inner, L.SUM if op == L.MEAN else op))
    _all_reduce(part, _RED[op], group)
    return finish_mean(part, global_r) if op == L.MEAN else part


def _all_gather(t: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """[world, *t.shape]: every rank's copy of a small partial tensor."""
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.stack(parts)


def sharded_reduce_ex(engine, local, outer: int, r: int, inner: int, op: int, sharded: str, global_r: int, r_begin: int = 0,
                      unbiased: bool = True, is_std: bool = False, norm_type: int = 2, group=None):
    """variance / std, norm, logsumexp, argmax / argmin of the local [outer, r, inner] block over r.
    sharded = "outer": disjoint outputs, no communication.  sharded = "r": this rank holds rows
    [r_begin, r_begin + r) of global_r; every rank reduces its slab with the library and the small
    per-rank results (outer*inner values each) are combined after ONE all-gather (norms: one
    all-reduce): variance from (n, mean, M2) per rank with Chan's formula, logsumexp as the
    logsumexp of the per-rank values, argmax / argmin as the best (value, global position) with
    ties to the lower position."""
    world, _ = world_info()

    def run(code, *args):
        return _as_torch(engine.reduce_ext_ori(local, 0, outer, r, inner, code, *args))

    if sharded == "outer" or world == 1:
        return run(op, unbiased, is_std, norm_type)
    if op == L.NORM:
        part = run(op, True, False, norm_type)
        if norm_type == 2:
            part = part * part
        _all_reduce(part, "sum", group)
        return torch.sqrt(part) if norm_type == 2 else part
    if op == L.LOGSUMEXP:
        g = _all_gather(run(op, True, False, 2), world, group)
        m = g.max(dim=0).values
        return m + torch.log(torch.exp(g - m).sum(dim=0))
    if op == L.VARIANCE:
        mean = _as_torch(engine.reduce_axis_ori(local, 0, outer, r, inner, L.MEAN)).double()
        m2 = run(op, False, False, 2).double() * r                 # population variance * n = M2
        n = torch.full_like(mean, float(r))
        g = _all_gather(torch.stack([n, mean, m2]), world, group)  # [world, 3, outputs]
        ns, means, m2s = g[:, 0], g[:, 1], g[:, 2]
        total = ns.sum(dim=0)
        gmean = (ns * means).sum(dim=0) / total
        gm2 = m2s.sum(dim=0) + (ns * (means - gmean) ** 2).sum(dim=0)
        den = torch.clamp(total - 1, min=1) if unbiased else torch.clamp(total, min=1)
        v = gm2 / den
        dt = _as_torch(local).dtype
        return (torch.sqrt(v) if is_std else v).to(dt)
    if op in (L.ARGMAX, L.ARGMIN):
        vals = _as_torch(engine.reduce_axis_ori(local, 0, outer, r, inner, L.MAX if op == L.ARGMAX else L.MIN))
        pos = run(op, True, False, 2).to(torch.int64) + int(r_begin)
        gv = _all_gather(vals, world, group)
        gp = _all_gather(pos, world, group)
        best = gv.max(dim=0).values if op == L.ARGMAX else gv.min(dim=0).values
        cand = torch.where(gv == best, gp, torch.full_like(gp, torch.iinfo(torch.int64).max))
        return cand.min(dim=0).values
    raise ValueError(f"unsupported reduction code {op}")


def sharded_mean_l1_loss(engine, a_local, b_local, global_n: int, group=None):
    """mean(|a-b|) over tensors split across ranks: local sum of |a-b| -> all-reduce -> / (T)(float)N."""
    world, _ = world_info()
    if _in_library(engine):
        return engine.mg_l1_loss(a_local, b_local, global_n, 0, False)[0]
    loss, _ = engine.l1_loss(a_local, b_local, 1, False)  # reduction 1 = sum
    t = _as_torch(loss)
    if world > 1:
        _all_reduce(t, "sum", group)
    return finish_mean(t, global_n)


def sharded_reduce_view(engine, buf, meta: Meta, axis: int, op: int, world: Optional[int] = None, rank: Optional[int] = None):
    """`t.<op>_at(axis)` of a GLOBAL tensor every rank can address (buf, meta), each rank computing its
    share.  A kept dim with extent >= world is cut when there is one: the rank reduces its slab view in
    place (a strided window for an inner dim) and owns the outputs [begin, end) along that dim -- no
    exchange at all.  Otherwise the reduced dim is cut and the partial results are combined, every
    rank ending with the full result.  -> (result, cut dim or None, begin, end)"""
    if world is None:
        world, rank = world_info()
    dim = pick_reduce_dim(meta.shape, axis, world) if world > 1 else None
    if dim is None:
        return _as_torch(engine.reduce_view(buf, meta, axis, op)), None, 0, meta.shape[axis] if meta.shape else 1
    b, e = shard_range(meta.shape[dim], world, rank)
    slab = meta.slice(dim, b, e, 1)
    if dim != axis:
        return _as_torch(engine.reduce_view(buf, slab, axis, op)), dim, b, e
    part = _as_torch(engine.reduce_view(buf, slab, axis, L.SUM if op == L.MEAN else op))
    if _in_library(engine):
        engine.mg_combine(part, op, meta.shape[axis])
        return part, dim, b, e
    _all_reduce(part, _RED[op])
    return (finish_mean(part, meta.shape[axis]) if op == L.MEAN else part), dim, b, e
