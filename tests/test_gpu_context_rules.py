"""Rules of the library context that the parity of single calls does not show: operands that overlap
the destination, one context driven from two streams, captured graphs while the workspace grows --
and the scalar chain / i32 add at the benchmark's own size, bit for bit against the CPU oracle.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def _b():
    from cuda_engine import backend
    return backend()


def _dev(a):
    return _b().alloc_from_slice(a)


def _host(t):
    return t.detach().cpu().numpy()


def _m(m):
    from rtensors_b200.meta import Meta
    return Meta(m.shape, m.strides, m.offset)


# ----------------------------------------------------------------------------- operand overlap
def _inplace_read_all_first(buf, am, bm, op):
    """`a op= b` where b is a view of a's own buffer, with every input read before any output is
    written: the CPU walk (src/backend/cpu.rs:292-352) over a private copy of the right operand."""
    shape, sa, sb = O.broadcast_params(am, bm)
    ref = buf.copy()
    frozen = buf.copy()
    ma = O.Meta(shape, sa, am.offset)
    O.broadcast(ref, ma, frozen, O.Meta(shape, sb, bm.offset), ref, ma, op)
    return ref


@pytest.mark.parametrize("dt", [np.float32, np.int32, np.float64, np.uint8], ids=lambda d: np.dtype(d).name)
def test_right_operand_overlapping_dst_is_read_before_dst_is_written(dt):
    rng = np.random.default_rng(77)
    n = 192
    base = O.Meta.contiguous((n, n))
    cases = [
        (base, base.permute((1, 0))),                                   # a += a.T
        (base, base.slice(1, None, None, -1)),                          # rows += their own reverse
        (base, base.slice(0, None, None, -1).slice(1, None, None, -1)),  # a += a rotated by 180 degrees
        (base.slice(0, 0, n - 1, 1), base.slice(0, 1, n, 1)),           # a window shifted over itself by one row
        (base, base.slice(0, 0, 1, 1)),                                 # a += a[0:1, :] broadcast over the rows
    ]
    for am, bm in cases:
        buf = (rng.integers(0, 50, n * n) if np.dtype(dt).kind == "u" else rng.integers(-50, 50, n * n)).astype(dt)
        want = _inplace_read_all_first(buf, am, bm, O.ADD)
        d = _dev(buf)
        _b().binary_assign(d, _m(am), d, _m(bm), O.ADD)
        assert _host(d).tobytes() == want.tobytes(), (am, bm)


def test_views_of_one_buffer_that_share_no_element_match_the_cpu_walk():
    """even columns += odd columns of the same buffer: the byte ranges intersect, the elements do
    not, so the reference's row-major walk and read-all-first agree."""
    rng = np.random.default_rng(78)
    base = O.Meta.contiguous((64, 256))
    even, odd = base.slice(1, 0, 256, 2), base.slice(1, 1, 256, 2)
    buf = rng.uniform(-1, 1, base.size).astype(np.float32)
    ref = buf.copy()
    shape, sa, sb = O.broadcast_params(even, odd)
    ma = O.Meta(shape, sa, even.offset)
    O.broadcast(ref, ma, ref, O.Meta(shape, sb, odd.offset), ref, ma, O.MUL)   # the true aliased CPU walk
    d = _dev(buf)
    _b().binary_assign(d, _m(even), d, _m(odd), O.MUL)
    assert _host(d).tobytes() == ref.tobytes()


def test_out_of_place_with_dst_inside_an_operand_buffer():
    """dst is a dense block at the front of the buffer both operands are views of."""
    from rtensors_b200.meta import Meta
    rng = np.random.default_rng(79)
    n = 96
    buf = rng.uniform(-1, 1, 2 * n * n).astype(np.float32)
    base = O.Meta.contiguous((n, n))
    lm = base.permute((1, 0))                 # left = block 0 transposed (overlaps dst = block 0)
    rm = O.Meta((n, n), (n, 1), n * n)        # right = block 1 (disjoint)
    want = (buf[:n * n].reshape(n, n).T + buf[n * n:].reshape(n, n)).astype(np.float32)
    d = _dev(buf)
    _b().broadcast((d, _m(lm)), (d, _m(rm)), (d, Meta.contiguous((n, n))), O.ADD)
    assert _host(d)[:n * n].tobytes() == want.reshape(-1).tobytes()
    assert _host(d)[n * n:].tobytes() == buf[n * n:].tobytes()


# ----------------------------------------------------------------------------- two streams, one context
def test_reductions_issued_on_two_streams_through_one_context():
    """The workspace counters and partial slots are shared by every call of a context; a change of
    stream orders the new stream after the old one, so back-to-back reductions on alternating
    streams still give every result."""
    from rtensors_b200 import _lib as L
    be = _b()
    rng = np.random.default_rng(80)
    n = (1 << 22) + 77
    xs = [rng.normal(0, 1, n).astype(np.float32) for _ in range(2)]
    ds = [_dev(x) for x in xs]
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    outs = []
    for k in range(12):
        st = s1 if k % 2 == 0 else s2
        with torch.cuda.stream(st):
            be.sync_stream()
            o = torch.full((1,), -7.0, device="cuda", dtype=torch.float32)
            op = (L.SUM, L.MAX, L.MIN)[k % 3]
            be.apply_reduce_contiguous_flat(ds[k % 2], o, 0, n, op)
            col = torch.full((2048,), -7.0, device="cuda", dtype=torch.float32)
            be.apply_reduce((ds[k % 2], _m(O.Meta.contiguous((2048, 2048)))), col, 0, L.SUM)
            outs.append((k, op, o, col))
    torch.cuda.synchronize()
    be.sync_stream()
    for k, op, o, col in outs:
        x = xs[k % 2]
        got = float(_host(o)[0])
        if op == L.SUM:
            assert abs(got - float(x.sum(dtype=np.float64))) <= 1e-5 * math.log2(n) * float(np.abs(x).sum())
        else:
            assert got == float(x.max() if op == L.MAX else x.min())
        m = x[:2048 * 2048].reshape(2048, 2048)
        assert np.all(np.abs(_host(col).astype(np.float64) - m.sum(axis=0, dtype=np.float64))
                      <= 1e-5 * 11 * np.abs(m).sum(axis=0, dtype=np.float64))


# ----------------------------------------------------------------------------- graphs and the workspace
def test_a_captured_graph_stays_valid_when_the_workspace_grows_and_can_be_recorded_again():
    from rtensors_b200 import _lib as L
    from rtensors_b200._lib import lib
    from rtensors_b200.backend import CudaB200
    be = CudaB200(0)   # a fresh context: its workspace starts at the minimum size
    try:
        rng = np.random.default_rng(81)
        small = _dev(rng.normal(0, 1, 512 * 256).astype(np.float32))
        sm = _m(O.Meta.contiguous((512, 256)))
        col = be.alloc(256, torch.float32)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            be.sync_stream()
            be.apply_reduce((small, sm), col, 0, L.SUM)
            side.synchronize()
            gen0 = int(lib().rtb_ctx_workspace_generation(be._ctx))

            def record():
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    be.sync_stream()
                    be.apply_reduce((small, sm), col, 0, L.SUM)
                return g
            graph = record()
            eager = _host(col).copy()
            # a reduction that needs far more partial slots than the first one: the workspace moves
            big_rows, big_cols = 8, 1 << 21
            big = be.alloc(big_rows * big_cols, torch.float32)
            big.normal_()
            bigout = be.alloc(big_cols, torch.float32)
            be.apply_reduce((big, _m(O.Meta.contiguous((big_rows, big_cols)))), bigout, 0, L.SUM)
            for _ in range(3):
                bigv = be.reduce_ext_ori(big, 0, 1, big_rows, big_cols, L.VARIANCE)
            side.synchronize()
            gen1 = int(lib().rtb_ctx_workspace_generation(be._ctx))
            col.fill_(-1.0)
            graph.replay()                       # the old graph still owns a live (retired) workspace
            side.synchronize()
            assert _host(col).tobytes() == eager.tobytes()
            if gen1 != gen0:                     # the holder's rule: record again when the generation moved
                graph = record()
                col.fill_(-2.0)
                graph.replay()
                side.synchronize()
                assert _host(col).tobytes() == eager.tobytes()
            # growing during capture is refused instead of invalidating the capture
            huge = be.alloc(4 * (1 << 23), torch.float32)
            huge.zero_()
            hout = be.alloc(1 << 23, torch.float32)
            g2 = torch.cuda.CUDAGraph()
            refused = False
            with torch.cuda.graph(g2, stream=side):
                be.sync_stream()
                try:
                    be.reduce_ext_ori(huge, 0, 1, 4, 1 << 23, L.VARIANCE)
                    be.apply_reduce((huge, _m(O.Meta.contiguous((4, 1 << 23)))), hout, 0, L.SUM)
                except L.RtbError as e:
                    refused = "capture" in str(e)
            side.synchronize()
            assert refused or int(lib().rtb_ctx_workspace_generation(be._ctx)) == gen1
        torch.cuda.current_stream().wait_stream(side)
    finally:
        torch.cuda.synchronize()
        be.close()


# ----------------------------------------------------------------------------- config 2 at its own size
def test_scalar_chain_and_i32_add_at_2_pow_28_bit_exact():
    """f32 `a*=3; a+=2; a-=1` on 2^28 seeded uniform[-1,1) values and i32 `a+b` on two 2^28-element
    tensors in [-2^20, 2^20]: the buffers the benchmark's chain produces, compared in full with the
    CPU oracle (the reference's own large-chain check is src/ops/mod.rs:3215-3279)."""
    from rtensors_b200 import _lib as L
    from rtensors_b200.meta import Meta
    be = _b()
    n = 1 << 28
    rng = np.random.default_rng(0x5EED + 1)
    a = rng.random(n, dtype=np.float32)
    a *= 2
    a -= 1
    d = _dev(a)
    m = O.Meta.contiguous((n,))
    gm = Meta.contiguous((n,))
    for op, v in ((O.MUL, 3.0), (O.ADD, 2.0), (O.SUB, 1.0)):
        O.scalar_op(a, op, v, m, fast=True)
        be.scalar_apply(d, op, v, gm)
    got = _host(d)
    assert np.array_equal(got.view(np.uint32), a.view(np.uint32))
    del d, got, a
    ia = rng.integers(-(1 << 20), 1 << 20, n, endpoint=True, dtype=np.int32)
    ib = rng.integers(-(1 << 20), 1 << 20, n, endpoint=True, dtype=np.int32)
    want = np.empty_like(ia)
    O.broadcast(ia, m, ib, m, want, m, O.ADD, fast=True)
    da, db = _dev(ia), _dev(ib)
    out = be.alloc(n, torch.int32)
    be.broadcast((da, gm), (db, gm), (out, gm), L.ADD)
    assert np.array_equal(_host(out), want)
    assert int(want.astype(np.int64).sum()) == int(ia.astype(np.int64).sum()) + int(ib.astype(np.int64).sum())
