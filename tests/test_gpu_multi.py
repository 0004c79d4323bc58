"""Two-GPU check of the sharding layer with the CUDA engine and NCCL (skipped on a 1-GPU box):
slab-sharded broadcast add with no collective, full sum as per-GPU partials + all-reduce."""
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
        torch.cuda.synchronize()
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharding(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
