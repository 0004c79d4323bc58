"""The library's host-buffer operations (rtb_host_*): work whose inputs and results live in pinned host
memory, moved on the context's transfer lanes.  Broadcast results must equal the CPU oracle bit for bit;
reductions must equal the device-resident call on the same data bit for bit (that call is checked against
the oracle elsewhere) -- the transfer path may not change a single bit."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle as O
from golden_runner import gather_view

pytestmark = pytest.mark.gpu


def _b():
    from cuda_engine import backend
    return backend()


def _meta(m):
    from rtensors_b200.meta import Meta
    return Meta(m.shape, m.strides, m.offset)


def _pin(a):
    return torch.from_numpy(np.ascontiguousarray(a).reshape(-1)).pin_memory()


@pytest.mark.parametrize("dt", [np.float32, np.int32, np.float64, np.uint8], ids=lambda d: np.dtype(d).name)
def test_host_broadcast_matches_oracle_over_views_and_stage_counts(dt):
    """Strided, negative-step, permuted and stride-0 operands; one stage, a partial ring, and a ring that is
    reused several times (stage size lowered so that small tensors give many stages); sub-ranges of the
    outermost dim."""
    be = _b()
    rng = np.random.default_rng(5)
    base_a = O.Meta.contiguous((13, 24, 40))
    base_b = O.Meta.contiguous((24, 80))
    if np.dtype(dt).kind == "f":
        a = rng.uniform(-2, 2, base_a.size).astype(dt)
        b = rng.uniform(-2, 2, base_b.size).astype(dt)
    else:
        a = rng.integers(0, 100, base_a.size).astype(dt)
        b = rng.integers(1, 100, base_b.size).astype(dt)
    cases = [
        (base_a, base_b.slice(1, None, None, 2)),                                    # (13,24,40) op (24,40 strided)
        (base_a.slice(0, None, None, -1), base_b.slice(1, None, None, -2)),            # reversed outer, negative-step inner
        (base_a.slice(1, 2, 22, 3).permute((1, 0, 2)), base_b.slice(1, 0, 40, 1).slice(0, 0, 1, 1)),   # permuted; (1,40) row
        (base_a.index(0, 4), base_b.slice(1, 40, 80, 1)),                            # rank 2
    ]
    es = np.dtype(dt).itemsize
    ha, hb = _pin(a), _pin(b)
    try:
        for stage_bytes in (64 << 20, 24 * 40 * es * 2, 40 * es):   # 1 stage; 2 indices per stage; 1 index per stage
            be.host_set_stage_bytes(stage_bytes)
            for op in (O.ADD, O.MUL):
                for ma, mb in cases:
                    want, wm = O.binary(a, ma, b, mb, op)
                    n0 = wm.shape[0]
                    per = wm.size // n0
                    for lo, hi in ((0, n0), (1, n0 - 1), (n0 - 1, n0), (2, 2)):
                        out = torch.zeros((hi - lo) * per + 3, dtype=ha.dtype).pin_memory()
                        be.host_broadcast(ha, _meta(ma), hb, _meta(mb), op, out, (lo, hi))
                        be.host_wait()
                        got = out.numpy()
                        assert got[: (hi - lo) * per].tobytes() == want[lo * per:hi * per].tobytes(), (stage_bytes, op, ma, lo, hi)
                        assert not got[(hi - lo) * per:].any()       # nothing written past the range
    finally:
        be.host_set_stage_bytes(64 << 20)


def test_host_broadcast_rejects_bad_arguments():
    from rtensors_b200 import _lib as L
    be = _b()
    m = _meta(O.Meta.contiguous((4, 8)))
    a, b = _pin(np.zeros(32, np.float32)), _pin(np.zeros(16, np.float32))      # b too small for its view
    out = torch.zeros(96).pin_memory()
    with pytest.raises(L.RtbError):
        be.host_broadcast(a, m, b, m, O.ADD, out)
    with pytest.raises(L.RtbError):
        be.host_broadcast(a, m, a, m, O.ADD, out, (3, 9))                      # range past the outermost dim


def test_host_reduce_view_equals_the_resident_call():
    be = _b()
    rng = np.random.default_rng(6)
    base = O.Meta.contiguous((12, 40, 64))
    x = rng.standard_normal(base.size).astype(np.float32)
    hx = _pin(x)
    dx = be.alloc_from_slice(x)
    views = [base, base.slice(0, 2, 11, 3), base.slice(1, None, None, -1), base.permute((2, 0, 1)), base.slice(2, None, None, 2)]
    for m in views:
        for axis in [None] + list(range(3)):
            for op in (O.SUM, O.MAX, O.MEAN, O.VARIANCE, O.LOGSUMEXP, O.ARGMAX):
                want = be.reduce_view_ex(dx, _meta(m), axis, op).cpu().numpy()
                n_out = 1 if axis is None else m.size // m.shape[axis]
                got = torch.zeros(n_out, dtype=torch.int64 if op == O.ARGMAX else torch.float32).pin_memory()
                be.host_reduce_view(hx, _meta(m), axis, op, got)
                be.host_wait()
                assert got.numpy().tobytes() == want[:n_out].tobytes(), (m, axis, op)
    # and against the oracle once, on the dense gather of a view
    m = views[3]
    dense = gather_view(x, m)
    want, _ = O.reduce_axis(dense, O.Meta.contiguous(m.shape), 1, O.MAX)
    got = torch.zeros(want.size).pin_memory()
    be.host_reduce_view(hx, _meta(m), 1, O.MAX, got)
    be.sync()                                                   # rtb_ctx_sync waits for the lanes too
    assert got.numpy().tobytes() == want.tobytes()


def test_pool_blocks_are_reused_without_stale_data_and_without_waiting_for_unused_uploads():
    """stage_in / ready / kernels / stage_out / release over several rounds with different data: a block
    that comes back from the pool must never show the previous round's content, results must not be
    overwritten before their copy-out ran, and trim leaves taken blocks alone."""
    from rtensors_b200.meta import Meta
    be = _b()
    n = 300_001
    mc = Meta.contiguous((n,))
    rng = np.random.default_rng(7)
    outs, wants, pinned = [], [], []                          # pinned inputs stay alive until their uploads ran
    for r in range(6):
        x = rng.standard_normal(n).astype(np.float32)
        y = rng.standard_normal(n).astype(np.float32)
        pinned += [_pin(x), _pin(y)]
        bx, by = be.host_stage_in(pinned[-2]), be.host_stage_in(pinned[-1])
        res = be.host_scratch(n, torch.float32)
        be.host_ready(bx)
        be.scalar_apply(bx, O.MUL, 2.0, mc)                 # runs while y may still be uploading
        be.host_ready(by)
        be.broadcast((bx, mc), (by, mc), (res, mc), O.ADD)
        out = torch.zeros(n).pin_memory()
        be.host_stage_out(res, out)
        for blk in (bx, by, res):
            be.host_release(blk)
        outs.append(out)
        wants.append(x * np.float32(2.0) + y)
    pinned.append(_pin(np.arange(16, dtype=np.float32)))
    kept = be.host_stage_in(pinned[-1])
    be.host_trim()                                          # waits, frees the unused blocks, keeps `kept`
    for out, want in zip(outs, wants):
        assert out.numpy().tobytes() == want.tobytes()
    be.host_ready(kept)
    back = torch.zeros(16).pin_memory()
    be.host_stage_out(kept, back)
    be.host_join()
    torch.cuda.current_stream().synchronize()               # join made the compute stream wait for the lanes
    assert back.numpy().tolist() == list(range(16))
    be.host_release(kept)
    from rtensors_b200 import _lib as L
    with pytest.raises(L.RtbError):
        be.host_release(kept)                               # not taken any more
    with pytest.raises(L.RtbError):
        be.host_ready(torch.empty(4, device="cuda"))        # not a pool block
    small = be.host_scratch(16, torch.float32)
    rc = L.lib().rtb_host_stage_out(be._ctx, C.c_void_p(small.data_ptr()), C.c_void_p(back.data_ptr()), C.c_size_t(1 << 20))
    assert rc == L.ERR_BOUNDS                               # a copy-out may not run past the end of its block
    be.host_release(small)


def test_host_operations_are_refused_during_capture():
    from rtensors_b200 import _lib as L
    from rtensors_b200.backend import CudaB200
    be = CudaB200(0)
    try:
        h = _pin(np.zeros(8, np.float32))
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        refused = False
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                be.sync_stream()
                try:
                    be.host_stage_in(h)
                except L.RtbError as e:
                    refused = "graph" in str(e)
            side.synchronize()
        torch.cuda.current_stream().wait_stream(side)
        assert refused
    finally:
        torch.cuda.synchronize()
        be.close()


def test_pinning_caller_memory():
    lib = __import__("rtensors_b200")._lib.lib()
    p = C.c_void_p()
    assert lib.rtb_host_alloc(C.c_size_t(4096), C.byref(p)) == 0 and p.value
    assert lib.rtb_host_free(p) == 0
    buf = np.zeros(1 << 16, np.float32)
    assert lib.rtb_host_pin(C.c_void_p(buf.ctypes.data), C.c_size_t(buf.nbytes)) == 0
    assert lib.rtb_host_unpin(C.c_void_p(buf.ctypes.data)) == 0
    assert lib.rtb_host_pin(C.c_void_p(0), C.c_size_t(16)) != 0
