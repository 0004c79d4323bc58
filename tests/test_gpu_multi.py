"""Two-GPU checks of the multi-GPU layer with the CUDA engine (skipped on a 1-GPU box): slab-sharded
broadcast add with no collective; full reductions, partial vectors and L1 loss combined inside the
library (peer-memory exchange) against the NCCL path and the CPU oracle; the partitioner's kept-dim
cut; a wait that runs out because one rank skipped its call (made on the host, nothing faults); the
data-parallel MLP step against the single-rank step; two contexts on two devices in one process."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    import oracle as O
    from rtensors_b200 import _lib as L
    from rtensors_b200 import sharding
    from rtensors_b200.backend import CudaB200
    from rtensors_b200.meta import Meta
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    try:
        be = CudaB200(rank)
        sharding.init_communicator(be)      # rtb_mg_init: NCCL communicator + peer-mapped exchange buffers
        assert be.mg_world == world and be.mg_rank == rank
        mapped = be.mg_peer_mapped
        rng = np.random.default_rng(7)
        bufa = rng.uniform(-1, 1, 64 * 16).astype(np.float32)
        bufb = rng.uniform(-1, 1, 8 * 256).astype(np.float32)
        A = Meta.contiguous((64, 16, 1, 1)).view_as((1, 64, 16, 1)).permute((2, 0, 1, 3))
        B = Meta.contiguous((1, 8, 1, 256)).slice(3, None, None, -1)
        out, dm, slab = sharding.sharded_binary(be, be.alloc_from_slice(bufa), A, be.alloc_from_slice(bufb), B, L.ADD)
        full, _ = O.binary(bufa, O.Meta(A.shape, A.strides, A.offset), bufb, O.Meta(B.shape, B.strides, B.offset), O.ADD)
        per = full.size // 16
        assert out.cpu().numpy().tobytes() == full[slab.begin * per: slab.end * per].tobytes()
        x = rng.standard_normal(1 << 20).astype(np.float32)
        lo, hi = sharding.scalar_slab(x.size, world, rank)
        local = be.alloc_from_slice(x[lo:hi])
        for op in (L.SUM, L.MEAN, L.MAX, L.MIN):
            got = float(sharding.sharded_reduce_flat(be, local, hi - lo, x.size, op).item())
            want = float(O.reduce_flat(x, 0, x.size, op)[0])
            if op in (L.MAX, L.MIN):
                assert got == want
            else:
                assert abs(got - want) <= 1e-5 * 20 * float(np.abs(x).sum()) / (x.size if op == L.MEAN else 1)
        # state-merging reductions with the reduced dim split across the two GPUs
        z = (rng.standard_normal((5, 600, 64)) * 2 + 1).astype(np.float32)
        z[2, 11, 9] = z[2, 500, 9] = 99.0
        lo, hi = sharding.scalar_slab(600, world, rank)
        zl = be.alloc_from_slice(np.ascontiguousarray(z[:, lo:hi, :]).reshape(-1))
        for op, args in ((L.VARIANCE, (True, False, 2)), (L.VARIANCE, (False, True, 2)), (L.NORM, (True, False, 2)),
                         (L.LOGSUMEXP, (True, False, 2))):
            got = sharding.sharded_reduce_ex(be, zl, 5, hi - lo, 64, op, "r", 600, lo, *args).cpu().numpy()
            want = O.reduce_ext_ori(z.reshape(-1), 5, 600, 64, op, *args)
            assert np.allclose(got, want, rtol=1e-4, atol=1e-6), (op, args)
        got = sharding.sharded_reduce_ex(be, zl, 5, hi - lo, 64, L.ARGMAX, "r", 600, lo).cpu().numpy()
        assert np.array_equal(got, O.argreduce_ori(z.reshape(-1), 5, 600, 64, O.ARGMAX).astype(np.int64))
        _library_combines(be, rank, world, rng)
        _wait_that_runs_out(be, rank, world)
        _mlp_data_parallel(be, rank, world)
        torch.cuda.synchronize()
        be.mg_finalize()
        open(os.path.join(out_dir, f"ok{rank}"), "w").write(f"ok peer_mapped={mapped}")
    finally:
        dist.destroy_process_group()


def _library_combines(be, rank, world, rng):
    """rtb_mg_reduce_flat / rtb_mg_reduce_axis / rtb_mg_l1_loss / rtb_mg_combine against the NCCL
    all-reduce of the same partials (max / min bit for bit, sums within the float-sum tolerance) and
    against the oracle on the global data; every rank must hold the same bits."""
    import torch.distributed as dist

    import oracle as O
    from rtensors_b200 import _lib as L
    from rtensors_b200 import sharding
    from rtensors_b200.meta import Meta
    # 6.3 M elements per rank at world 2: the size range where the flat kernel runs one CTA per 32 KiB block
    x = rng.standard_normal((12 << 20) + 10).astype(np.float32)
    lo, hi = sharding.scalar_slab(x.size, world, rank)
    local = be.alloc_from_slice(x[lo:hi])
    for rep in range(3):                       # repeated: the two epoch-parity buffers are reused
        for op in (L.SUM, L.MEAN, L.MAX, L.MIN):
            got = be.mg_reduce_flat(local, 0, hi - lo, x.size, op)
            part = be.alloc(1, torch.float32)
            be.apply_reduce_contiguous_flat(local, part, 0, hi - lo, L.SUM if op == L.MEAN else op)
            dist.all_reduce(part, op={L.SUM: dist.ReduceOp.SUM, L.MEAN: dist.ReduceOp.SUM, L.MAX: dist.ReduceOp.MAX,
                                      L.MIN: dist.ReduceOp.MIN}[op])
            nccl = float(part.item()) / (float(np.float32(x.size)) if op == L.MEAN else 1.0)
            g = float(got.item())
            want = float(O.reduce_flat(x, 0, x.size, op)[0])
            if op in (L.MAX, L.MIN):
                assert g == nccl == want
            else:
                tol = 1e-5 * 24 * float(np.abs(x).sum()) / (x.size if op == L.MEAN else 1)
                assert abs(g - nccl) <= tol and abs(g - want) <= tol
            same = [torch.zeros(1, device=got.device) for _ in range(world)]
            dist.all_gather(same, got)
            assert all(t.cpu().numpy().tobytes() == same[0].cpu().numpy().tobytes() for t in same)
    # partial vectors (the reduced dim is the cut one): f32 and f64, 32 KiB and a ragged length
    for dt, tdt, cols in ((np.float32, torch.float32, 8192), (np.float64, torch.float64, 1000)):
        y = rng.standard_normal((600, cols)).astype(dt)
        lo, hi = sharding.scalar_slab(600, world, rank)
        yl = be.alloc_from_slice(np.ascontiguousarray(y[lo:hi]).reshape(-1))
        for op in (L.SUM, L.MEAN, L.MAX, L.MIN):
            got = be.mg_reduce_axis(yl, 0, 1, hi - lo, cols, 600, op).cpu().numpy()
            want = O.reduce_ori(y.reshape(-1), 1, 600, cols, op)
            if op in (L.MAX, L.MIN):
                assert got.tobytes() == want.tobytes()
            else:
                scale = np.abs(y).sum(axis=0, dtype=np.float64) / (600 if op == L.MEAN else 1)
                assert np.all(np.abs(got.astype(np.float64) - want.astype(np.float64)) <= 1e-5 * 10 * scale)
    # a buffer beyond the peer exchange's size goes through NCCL inside the same entry point
    big = torch.full((40000,), float(rank + 1), device=f"cuda:{be.device}")
    be.mg_combine(big, L.SUM)
    assert float(big[0]) == float(big[-1]) == sum(range(1, world + 1))
    ints = torch.full((5,), rank + 1, device=f"cuda:{be.device}", dtype=torch.int32)
    be.mg_allreduce(ints, L.MAX)
    assert int(ints[0]) == world
    # L1 loss over tensors split across the ranks, with the gradient map scaled by the global count
    p, q = rng.standard_normal(40000).astype(np.float32), rng.standard_normal(40000).astype(np.float32)
    q[::97] = p[::97]
    lo, hi = sharding.scalar_slab(40000, world, rank)
    loss, gmap = be.mg_l1_loss(be.alloc_from_slice(p[lo:hi]), be.alloc_from_slice(q[lo:hi]), 40000, 0, True)
    wl, wg = O.l1_loss(p, q, 0, True)
    assert abs(float(loss.item()) - float(wl[0])) <= 1e-5 * 16 * float(np.abs(p - q).mean())
    assert gmap.cpu().numpy().tobytes() == wg[lo:hi].tobytes()
    # the partitioner cuts a kept dim when it can: sum_at(0) of a matrix = each rank's own columns
    m = rng.standard_normal((512, 2048)).astype(np.float32)
    dm = be.alloc_from_slice(m.reshape(-1))
    for axis in (0, 1):
        got, dim, b, e = sharding.sharded_reduce_view(be, dm, Meta.contiguous(m.shape), axis, L.SUM, world, rank)
        assert dim == 1 - axis
        want = m.sum(axis=axis, dtype=np.float64)[b:e]
        assert np.allclose(got.cpu().numpy().reshape(-1), want, rtol=1e-4, atol=1e-3)


def _wait_that_runs_out(be, rank, world):
    """A failure made on the host: rank 1 does not enqueue one collective call.  Rank 0's exchange
    waits for a packet that never comes, gives up after the limit, reports status bit 0 and NaN, and
    its context stays usable; rtb_mg_realign then brings the epochs back in step."""
    import math

    from rtensors_b200 import _lib as L
    if not be.mg_peer_mapped:
        return
    v = torch.full((4096,), float(rank + 1), device=f"cuda:{be.device}")
    be.mg_set_wait_ns(150_000_000)
    if rank != 1:
        got = be.mg_reduce_flat(v, 0, 4096, 4096 * world, L.SUM)
        assert be.mg_status() & 1
        assert math.isnan(float(got.item()))
    else:
        assert be.mg_status() == 0
    be.mg_realign()
    assert be.mg_status() == 0
    be.mg_set_wait_ns(2_000_000_000)
    got = be.mg_reduce_flat(v, 0, 4096, 4096 * world, L.SUM)
    assert float(got.item()) == 4096.0 * sum(range(1, world + 1))
    part = torch.full((300,), float(rank + 1), device=f"cuda:{be.device}")
    be.mg_combine(part, L.MAX)
    assert float(part.max()) == float(part.min()) == float(world)
    assert be.mg_status() == 0


def _mlp_data_parallel(be, rank, world):
    """Two ranks with half the batch each must reproduce the single-rank step: same loss, same updated
    parameters within 1e-4 of max|.| per tensor, in both modes (seed = 1 and batch-sum bias gradient;
    seed = loss value and bias "gradient" = global row 0, src/grad/mod.rs:441-447,
    src/grad/backwards.rs:512-538)."""
    from rtensors_b200.backend import CudaB200
    from rtensors_b200.mlp import DenseMlp, synthetic_batch
    torch.backends.cuda.matmul.allow_tf32 = False
    dev = f"cuda:{be.device}"
    gbatch = 256
    img, tgt, _, _ = synthetic_batch(gbatch, dev)          # the same global batch on every rank
    per = gbatch // world
    for quirks in (False, True):
        solo_be = CudaB200(be.device)                        # no communicator: the single-rank step
        solo = DenseMlp(solo_be, (784, 96, 64, 10), lr=0.01, ref_quirks=quirks)
        dp = DenseMlp(be, (784, 96, 64, 10), lr=0.01, ref_quirks=quirks)
        dp.load_params(solo.host_params())
        for step in range(3):
            l1 = solo.step(img, tgt, gbatch)
            l2 = dp.step(img[rank * per:(rank + 1) * per], tgt[rank * per:(rank + 1) * per], gbatch)
            assert abs(float(l1.item()) - float(l2.item())) <= 1e-5 * abs(float(l1.item())) + 1e-7, (quirks, step)
        for a, b in zip(solo.host_params(), dp.host_params()):
            assert np.max(np.abs(a - b)) <= 1e-4 * max(np.max(np.abs(a)), 1e-6), quirks
        # the graph-replayed multi-rank step equals the eager one
        l3 = dp.step_graphed(img[rank * per:(rank + 1) * per], tgt[rank * per:(rank + 1) * per], gbatch)
        l3 = dp.step_graphed(img[rank * per:(rank + 1) * per], tgt[rank * per:(rank + 1) * per], gbatch)
        for _ in range(2):
            l1 = solo.step(img, tgt, gbatch)
        assert abs(float(l1.item()) - float(l3.item())) <= 1e-5 * abs(float(l1.item())) + 1e-7, quirks
        for a, b in zip(solo.host_params(), dp.host_params()):
            assert np.max(np.abs(a - b)) <= 1e-4 * max(np.max(np.abs(a)), 1e-6), quirks
        torch.cuda.synchronize()
        solo_be.close()


def test_two_gpu_sharding(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
    assert "peer_mapped=True" in (tmp_path / "ok0").read_text()


def test_two_gpu_sharding_without_peer_mapping(tmp_path, monkeypatch):
    """The same checks with the peer-memory path switched off: every combine goes through NCCL."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    monkeypatch.setenv("RTB_MG_NO_PEER", "1")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert "peer_mapped=False" in (tmp_path / "ok0").read_text()


def test_two_contexts_on_two_devices_in_one_process():
    """Allocation, copies and kernels go to the context's own device whichever device is current."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import ctypes as C

    from rtensors_b200 import _lib as L
    from rtensors_b200.backend import CudaB200
    from rtensors_b200.meta import Meta
    lib = L.lib()
    b0, b1 = CudaB200(0), CudaB200(1)
    try:
        torch.cuda.set_device(0)
        p = C.c_void_p()
        L.check(lib.rtb_alloc(b1._ctx, C.c_size_t(1 << 20), C.byref(p)))

        class Attr(C.Structure):
            _fields_ = [("type", C.c_int), ("device", C.c_int), ("devicePointer", C.c_void_p), ("hostPointer", C.c_void_p)]
        rt = C.CDLL("libcudart.so.12")
        a = Attr()
        assert rt.cudaPointerGetAttributes(C.byref(a), p) == 0
        assert a.device == 1
        host = np.arange(1024, dtype=np.float32)
        back = np.zeros_like(host)
        torch.cuda.set_device(0)
        L.check(lib.rtb_h2d(b1._ctx, p, host.ctypes.data_as(C.c_void_p), C.c_size_t(host.nbytes)))
        m = Meta.contiguous((1024,))
        v = np.array(2.0, dtype=np.float32).tobytes()
        L.check(lib.rtb_scalar_op(b1._ctx, C.c_int(L.F32), C.c_int(L.MUL), p, v, C.c_size_t(1), m.c_shape, m.c_strides, C.c_size_t(0)))
        torch.cuda.set_device(0)
        L.check(lib.rtb_d2h(b1._ctx, back.ctypes.data_as(C.c_void_p), p, C.c_size_t(host.nbytes)))
        assert np.array_equal(back, host * 2)
        L.check(lib.rtb_free(b1._ctx, p))
    finally:
        torch.cuda.set_device(0)
        b1.close()
        b0.close()
