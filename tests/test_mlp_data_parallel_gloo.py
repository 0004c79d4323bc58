"""The data-parallel MLP step's host logic at world size 2 on CPU (gloo): `DenseMlp.step` -- the product's
own step function -- runs unchanged over an engine made of the CPU oracle's pieces, with the library's
collective entry points stood in by gloo all-reduces.  Two ranks with half the batch each must reproduce
the single-rank step (loss, updated W / b within 1e-4 of max|.| per tensor) in both modes: seed 1 and
batch-sum bias gradient; seed = the loss value and bias "gradient" = global row 0 (src/grad/mod.rs:441-447,
src/grad/backwards.rs:512-538, src/grad/optim.rs:30-50)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from rtensors_b200 import _lib as L


class OracleMlpEngine:
    """CPU torch tensors (sharing memory with numpy) + the oracle, behind the method names DenseMlp calls."""
    torch_device = "cpu"
    device = 0

    def __init__(self, world=1, rank=0):
        self.mg_world, self.mg_rank = world, rank

    @staticmethod
    def _m(m):
        return O.Meta(tuple(m.shape), tuple(m.strides), m.offset)

    def u8_to_f32_div(self, src, divisor):
        return torch.from_numpy(O.u8_to_f32_div(src.numpy().reshape(-1), divisor))

    def binary_assign(self, a, am, b, bm, op):
        shape, sa, sb = O.broadcast_params(self._m(am), self._m(bm))
        ma = O.Meta(shape, sa, am.offset)
        O.broadcast(a.numpy(), ma, b.numpy(), O.Meta(shape, sb, bm.offset), a.numpy(), ma, op)

    def bias_relu_mask(self, z, bias, rows, cols):
        from rtensors_b200.meta import Meta
        self.binary_assign(z, Meta.contiguous((rows, cols)), bias, Meta.contiguous((1, cols)), L.ADD)
        return torch.from_numpy(O.relu_mask(z.numpy()))

    def broadcast(self, left, right, dst, op):
        (lb, lm), (rb, rm), (db, dm) = left, right, dst
        O.broadcast(lb.numpy(), self._m(lm), rb.numpy(), self._m(rm), db.numpy(), self._m(dm), op)

    def l1_loss(self, a, b, reduction=0, with_grad=False):
        loss, g = O.l1_loss(np.ascontiguousarray(a.numpy()), np.ascontiguousarray(b.numpy()), reduction, with_grad)
        return torch.from_numpy(loss), (torch.from_numpy(g) if g is not None else None)

    def mg_l1_loss(self, a, b, global_n, reduction=0, with_grad=False):
        """rtb_mg_l1_loss: local sum of |a - b|, combined across ranks, / (f32)N; map = sign / (f32)N."""
        an, bn = np.ascontiguousarray(a.numpy()), np.ascontiguousarray(b.numpy())
        lsum, g = O.l1_loss(an, bn, 1, with_grad)          # reduction 1 = sum, map = sign
        t = torch.from_numpy(lsum)
        dist.all_reduce(t)
        div = np.float32(np.float32(global_n))
        if reduction == 0:
            t = t / float(div)
            if g is not None:
                g = (g / div).astype(np.float32)
        return t, (torch.from_numpy(g) if g is not None else None)

    def reduce_to_shape(self, upstream, shape, operand_strides, out=None):
        red, oshape = O.reduce_to_shape(np.ascontiguousarray(upstream.numpy()), shape, operand_strides, intended=True)
        if out is None:
            return torch.from_numpy(red), oshape
        out[: red.size] = torch.from_numpy(red)
        return out, oshape

    def mg_allreduce(self, buf, op=L.SUM, mean_count=0, overlap=False):
        dist.all_reduce(buf)

    def mg_allreduce_join(self):
        pass

    def sgd_update(self, p, g, lr):
        O.sgd_update(p.numpy(), g.numpy(), lr)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _batch(n, seed=77):
    rng = np.random.default_rng(seed)
    img = rng.integers(0, 256, (n, 784), dtype=np.uint8)
    tgt = np.zeros((n, 10), dtype=np.float32)
    tgt[np.arange(n), rng.integers(0, 10, n)] = 1.0
    return torch.from_numpy(img), torch.from_numpy(tgt)


def _worker(rank, world, port, out_dir):
    from rtensors_b200.mlp import DenseMlp
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gbatch, sizes = 64, (784, 48, 32, 10)
        img, tgt = _batch(gbatch)
        per = gbatch // world
        for quirks in (False, True):
            solo = DenseMlp(OracleMlpEngine(1, 0), sizes, lr=0.01, ref_quirks=quirks)
            dp = DenseMlp(OracleMlpEngine(world, rank), sizes, lr=0.01, ref_quirks=quirks)
            host = solo.host_params()
            host[1][:] = np.linspace(-0.05, 0.05, host[1].size, dtype=np.float32).reshape(host[1].shape)
            solo.load_params(host)
            dp.load_params(host)
            for step in range(3):
                l1 = solo.step(img, tgt, gbatch)
                l2 = dp.step(img[rank * per:(rank + 1) * per], tgt[rank * per:(rank + 1) * per], gbatch)
                assert abs(float(l1.item()) - float(l2.item())) <= 1e-5 * abs(float(l1.item())) + 1e-7, (quirks, step)
            for a, b in zip(solo.host_params(), dp.host_params()):
                assert np.max(np.abs(a - b)) <= 1e-4 * max(float(np.max(np.abs(a))), 1e-6), quirks
            # every rank holds the same parameters afterwards
            flat = dp.params.clone()
            other = [torch.zeros_like(flat) for _ in range(world)]
            dist.all_gather(other, flat)
            assert all(torch.equal(o, other[0]) for o in other), quirks
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_data_parallel_mlp_step_world_size_2(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()


def test_single_rank_step_on_the_cpu_engine_equals_the_oracle_step():
    """The engine above is faithful: DenseMlp.step over it reproduces tests/mlp_oracle.py (which uses the
    oracle's f64-accumulating GEMM where this uses torch's CPU GEMM) within the GEMM tolerance."""
    from mlp_oracle import mlp_step
    from rtensors_b200.mlp import DenseMlp
    sizes = (784, 48, 32, 10)
    img, tgt = _batch(32, seed=5)
    for quirks in (False, True):
        model = DenseMlp(OracleMlpEngine(), sizes, lr=0.01, ref_quirks=quirks)
        params = model.host_params()
        loss = model.step(img, tgt)
        l_ref, new_params, _ = mlp_step(params, sizes, img.numpy(), tgt.numpy(), 0.01, quirks)
        assert abs(float(loss.item()) - l_ref) <= 1e-4 * abs(l_ref)
        for a, r in zip(model.host_params(), new_params):
            assert np.max(np.abs(a - r)) <= 1e-4 * max(float(np.max(np.abs(r))), 1e-6)
