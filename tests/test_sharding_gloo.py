"""World-size-2 checks of the multi-GPU host logic on CPU (gloo): slab arithmetic, replicated
broadcast operands, and the all-reduce combine of partial reductions.  The compute engine here is
the CPU oracle behind the Backend-mirror method names; the product's CUDA engine plugs into the
same functions on GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from rtensors_b200 import _lib as L
from rtensors_b200 import sharding
from rtensors_b200.meta import Meta


class OracleBackendMirror:
    """numpy buffers + the oracle, exposing the method names sharding.py calls."""

    def alloc(self, n, dtype):
        return np.zeros(int(n), dtype=dtype)

    @staticmethod
    def _m(m):
        return O.Meta(tuple(m.shape), tuple(m.strides), m.offset)

    def broadcast(self, left, right, dst, op):
        (lb, lm), (rb, rm), (db, dm) = left, right, dst
        O.broadcast(lb, self._m(lm), rb, self._m(rm), db, self._m(dm), op)

    def apply_reduce_contiguous_flat(self, src, dst, start, length, op):
        dst[0] = O.reduce_flat(src, start, length, op)[0]

    def reduce_axis_ori(self, src, offset, outer, r, inner, op):
        return O.reduce_ori(np.ascontiguousarray(src[offset:offset + outer * r * inner]), outer, r, inner, op)

    def l1_loss(self, a, b, reduction, with_grad):
        return O.l1_loss(a, b, reduction, with_grad)

    def reduce_view(self, src, meta, axis, op):
        """What the reference does for a non-contiguous tensor: copy the view row-major, then reduce."""
        from golden_runner import gather_view
        dense = gather_view(src, meta)
        if axis is None:
            return O.reduce_flat(dense, 0, dense.size, op)
        return O.reduce_axis(dense, O.Meta.contiguous(meta.shape), axis, op)[0]

    def reduce_ext_ori(self, src, offset, outer, r, inner, op, unbiased=True, is_std=False, norm_type=2):
        blk = np.ascontiguousarray(src[offset:offset + outer * r * inner])
        if op in (O.ARGMAX, O.ARGMIN):
            return O.argreduce_ori(blk, outer, r, inner, op).astype(np.int64)
        return O.reduce_ext_ori(blk, outer, r, inner, op, unbiased, is_std, norm_type)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        eng = OracleBackendMirror()
        rng = np.random.default_rng(42)  # same data on every rank
        # 1. strided / negative-step broadcast, sharded on the outermost output dim
        bufa = rng.uniform(-1, 1, 40 * 16).astype(np.float32)
        bufb = rng.uniform(-1, 1, 6 * 24).astype(np.float32)
        A = Meta.contiguous((40, 16, 1, 1)).view_as((1, 40, 16, 1)).permute((2, 0, 1, 3))
        B = Meta.contiguous((1, 6, 1, 24)).slice(3, None, None, -1)
        out, dm, slab = sharding.sharded_binary(eng, bufa, A, bufb, B, L.ADD)
        assert slab.dim == 0 and slab.end - slab.begin == 8
        full, fm = O.binary(bufa, O.Meta(A.shape, A.strides, A.offset), bufb, O.Meta(B.shape, B.strides, B.offset), O.ADD)
        per = full.size // 16
        assert out.tobytes() == full[slab.begin * per: slab.end * per].tobytes()
        # 2. outer product where the LEFT operand is the one sliced and the right one replicated
        a = rng.uniform(-1, 1, 10).astype(np.float32)
        b = rng.uniform(-1, 1, 7).astype(np.float32)
        out, dm, slab = sharding.sharded_binary(eng, a, Meta.contiguous((10, 1)), b, Meta.contiguous((1, 7)), L.MUL)
        full, _ = O.binary(a, O.Meta.contiguous((10, 1)), b, O.Meta.contiguous((1, 7)), O.MUL)
        assert out.tobytes() == full[slab.begin * 7: slab.end * 7].tobytes()
        # leading dim of extent 1: the slab dim moves inwards
        out, dm, slab = sharding.sharded_binary(eng, a, Meta.contiguous((1, 10)), b[:1], Meta.contiguous((1, 1)), L.ADD)
        assert slab.dim == 1
        # 3. full reductions: partial per rank + all-reduce
        x = rng.standard_normal(10001).astype(np.float32)
        lo, hi = sharding.scalar_slab(x.size, world, rank)
        local = np.ascontiguousarray(x[lo:hi])
        for op in (L.SUM, L.MEAN, L.MAX, L.MIN):
            got = sharding.sharded_reduce_flat(eng, local, hi - lo, x.size, op).numpy()[0]
            want = O.reduce_flat(x, 0, x.size, op)[0]
            if op in (L.MAX, L.MIN):
                assert got == want
            else:
                assert abs(float(got) - float(want)) <= 1e-5 * 14 * float(np.abs(x).sum()) / (x.size if op == L.MEAN else 1)
        # 4. axis reduction with the reduced dim sharded -> all-reduce of the partial vectors
        y = rng.standard_normal((3, 50, 8)).astype(np.float32)
        lo, hi = sharding.scalar_slab(50, world, rank)
        local = np.ascontiguousarray(y[:, lo:hi, :]).reshape(-1)
        for op in (L.SUM, L.MEAN, L.MAX):
            got = sharding.sharded_reduce_axis(eng, local, 3, hi - lo, 8, op, "r", 50).numpy()
            want = O.reduce_ori(y.reshape(-1), 3, 50, 8, op)
            assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
        # sharded on the outer dim: disjoint outputs, no collective
        lo, hi = sharding.scalar_slab(3, world, rank)
        local = np.ascontiguousarray(y[lo:hi]).reshape(-1)
        got = sharding.sharded_reduce_axis(eng, local, hi - lo, 50, 8, L.SUM, "outer", 50).numpy()
        want = O.reduce_ori(y.reshape(-1), 3, 50, 8, O.SUM).reshape(3, 8)[lo:hi].reshape(-1)
        assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
        # 4b. variance / std / norm / logsumexp / argmax with the reduced dim sharded: per-rank results
        # combined after one all-gather; ties in argmax resolve to the lowest GLOBAL position
        z = (rng.standard_normal((3, 50, 8)) * 2 + 1).astype(np.float32)
        z[1, 7, 3] = z[1, 40, 3] = 99.0   # the same maximum in both ranks' slabs
        lo, hi = sharding.scalar_slab(50, world, rank)
        local = np.ascontiguousarray(z[:, lo:hi, :]).reshape(-1)
        for op, args in ((L.VARIANCE, (True, False, 2)), (L.VARIANCE, (False, True, 2)), (L.NORM, (True, False, 1)),
                         (L.NORM, (True, False, 2)), (L.LOGSUMEXP, (True, False, 2))):
            got = sharding.sharded_reduce_ex(eng, local, 3, hi - lo, 8, op, "r", 50, lo, *args).numpy()
            want = O.reduce_ext_ori(z.reshape(-1), 3, 50, 8, op, *args)
            assert np.allclose(got, want, rtol=2e-5, atol=1e-6), (op, args)
        for op in (L.ARGMAX, L.ARGMIN):
            got = sharding.sharded_reduce_ex(eng, local, 3, hi - lo, 8, op, "r", 50, lo).numpy()
            want = O.argreduce_ori(z.reshape(-1), 3, 50, 8, op).astype(np.int64)
            assert np.array_equal(got, want), (op, got, want)
        assert sharding.sharded_reduce_ex(eng, local, 3, hi - lo, 8, L.ARGMAX, "r", 50, lo).numpy().reshape(3, 8)[1, 3] == 7
        # 4c. the partitioner prefers a kept dim: sum_at(0) of a matrix cuts the COLUMNS (each rank reduces a
        # strided window and owns its outputs, no exchange); only a tensor with no wide kept dim cuts the
        # reduced dim and combines
        mat = rng.standard_normal((30, 12)).astype(np.float32)
        mm = Meta.contiguous((30, 12))
        for axis in (0, 1):
            got, dim, b, e = sharding.sharded_reduce_view(eng, mat.reshape(-1), mm, axis, L.SUM)
            assert dim == 1 - axis and (b, e) == sharding.scalar_slab(mat.shape[dim], world, rank)
            want = mat.sum(axis=axis, dtype=np.float64)[b:e]
            assert np.allclose(got.numpy().reshape(-1), want, rtol=1e-5, atol=1e-5)
        tall = rng.standard_normal((40, 1)).astype(np.float32)
        for op, ref in ((L.SUM, tall.sum(dtype=np.float64)), (L.MEAN, tall.mean(dtype=np.float64)), (L.MAX, tall.max())):
            got, dim, b, e = sharding.sharded_reduce_view(eng, tall.reshape(-1), Meta.contiguous((40, 1)), 0, op)
            assert dim == 0 and abs(float(got.numpy().reshape(-1)[0]) - float(ref)) <= 1e-5 * 40
        # 5. mean_l1_loss over sharded tensors
        p, q = rng.standard_normal(4000).astype(np.float32), rng.standard_normal(4000).astype(np.float32)
        lo, hi = sharding.scalar_slab(4000, world, rank)
        got = sharding.sharded_mean_l1_loss(eng, np.ascontiguousarray(p[lo:hi]), np.ascontiguousarray(q[lo:hi]), 4000)
        want = O.l1_loss(p, q, 0, False)[0][0]
        assert abs(float(got[0]) - float(want)) <= 1e-5 * 12 * float(np.abs(p - q).mean())
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_sharding_world_size_2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_binary_slab_covers_output_exactly():
    am, bm = Meta.contiguous((4096, 1)), Meta.contiguous((1, 4096))
    for world in (1, 2, 3, 4, 8):
        slabs = [sharding.binary_slab(am, bm, world, r) for r in range(world)]
        assert slabs[0].begin == 0 and slabs[-1].end == 4096
        for s0, s1 in zip(slabs, slabs[1:]):
            assert s0.end == s1.begin
        for s in slabs:
            assert s.left.offset == s.begin and s.right.offset == 0  # left sliced, right replicated
    assert sharding.pick_reduce_dim((8192, 8192), 0, 8) == 1 and sharding.pick_reduce_dim((8192, 8192), 1, 8) == 0
    assert sharding.pick_reduce_dim((64, 4096, 1024), 1, 8) == 0 and sharding.pick_reduce_dim((4, 4096, 2), 1, 8) == 1
    assert sharding.pick_reduce_dim((4, 4, 2), 1, 8) is None
    # too small to shard: rank 0 owns everything
    s0 = sharding.binary_slab(Meta.contiguous((3,)), Meta.contiguous((3,)), 8, 0)
    s1 = sharding.binary_slab(Meta.contiguous((3,)), Meta.contiguous((3,)), 8, 5)
    assert s0.shape == (3,) and s1.shape == (0,)
