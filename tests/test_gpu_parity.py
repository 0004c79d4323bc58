"""Parity of the CUDA library (through the C ABI) with the CPU oracle on seeded inputs.

Bar: bit-exact for integer ops and for single-IEEE-op float elementwise work; float sums within
1e-5 * log2(n) relative to sum(|x|) (the reference CPU sum is one sequential accumulator, the GPU
sum is a tree); max / min exact.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

import oracle as O
from golden_runner import gather_view

pytestmark = pytest.mark.gpu

NP_DTYPES = [np.float32, np.float64, np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32,
             np.uint64, np.bool_]


def _b():
    from cuda_engine import backend
    return backend()


def _dev(a):
    return _b().alloc_from_slice(a)


def _host(t):
    return t.detach().cpu().numpy()


def _rand(rng, n, dt):
    dt = np.dtype(dt)
    if dt.kind == "f":
        return rng.uniform(-1, 1, n).astype(dt)
    if dt.kind == "b":
        return rng.integers(0, 2, n).astype(dt)
    info = np.iinfo(dt)
    lo, hi = max(info.min, -(1 << 20)), min(info.max, 1 << 20)
    return rng.integers(lo, hi, n, endpoint=True).astype(dt)


def _meta_pair(m):
    from rtensors_b200.meta import Meta
    return Meta(m.shape, m.strides, m.offset)


# ------------------------------------------------------------------------------------- scalar ops
@pytest.mark.parametrize("dt", NP_DTYPES, ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("n,off", [(1, 0), (3, 1), (1023, 0), (4099, 3), (1 << 16, 0), ((1 << 18) + 5, 7)])
def test_scalar_chain_contiguous(dt, n, off):
    rng = np.random.default_rng(n * 31 + off)
    buf = _rand(rng, n + off + 2, dt)
    meta = O.Meta((n,), (1,), off)
    ref = buf.copy()
    d = _dev(buf)
    chain = [(O.MUL, 3), (O.ADD, 2), (O.SUB, 1)] if np.dtype(dt).kind != "b" else [(O.MUL, 1), (O.ADD, 0), (O.SUB, 1)]
    if np.dtype(dt).kind in "fiu":
        chain.append((O.DIV, 7))
    for op, v in chain:
        O.scalar_op(ref, op, v, meta)
        _b().scalar_apply(d, op, v, _meta_pair(meta))
    assert _host(d).tobytes() == ref.tobytes()


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.int32, np.int64, np.int8])
@pytest.mark.parametrize("op", [O.NEG, O.RELU, O.ABS, O.SIGN])
def test_unary_layouts(dt, op):
    rng = np.random.default_rng(5)
    base = O.Meta.contiguous((6, 10, 12))
    views = [base, base.slice(2, None, None, 2), base.slice(0, None, None, -1).slice(2, None, None, -3),
             base.permute((2, 0, 1)), base.index(1, 3), base.slice(1, 8, 1, -2).index(2, 5),
             base.slice(0, None, None, -1).slice(1, None, None, -1).slice(2, None, None, -1)]
    for m in views:
        buf = _rand(rng, base.size, dt)
        if np.dtype(dt).kind == "f":
            buf[::7] = 0.0
            buf[3::11] = -0.0
        ref = buf.copy()
        if m.is_contiguous() and any(s < 0 for s in m.strides):
            # The reference dispatcher walks such a view forward from its offset (out of bounds);
            # the intended result is the op applied to every viewed element.
            idx = gather_index(m)
            tmp = ref[idx].copy()
            O.unary_op(tmp, op, O.Meta.contiguous((tmp.size,)))
            ref[idx] = tmp
        else:
            O.unary_op(ref, op, m)
        d = _dev(buf)
        _b().apply_unary(d, op, _meta_pair(m))
        assert _host(d).tobytes() == ref.tobytes(), m


def gather_index(m):
    idx = np.full(m.shape if m.shape else (), m.offset, dtype=np.int64)
    for k, (n, s) in enumerate(zip(m.shape, m.strides)):
        shp = [1] * len(m.shape)
        shp[k] = n
        idx = idx + (np.arange(n, dtype=np.int64) * s).reshape(shp)
    return idx.reshape(-1)


def test_relu_special_values_follow_cpu_backend():
    x = np.array([np.nan, -0.0, 0.0, -1.5, 2.5, np.inf, -np.inf], dtype=np.float32)
    ref = x.copy()
    O.unary_op(ref, O.RELU, O.Meta.contiguous((x.size,)))
    d = _dev(x)
    _b().apply_unary(d, O.RELU, _meta_pair(O.Meta.contiguous((x.size,))))
    assert _host(d).tobytes() == ref.tobytes()  # NaN -> 0 and -0 -> +0, as `x > 0 ? x : 0`
    s = x.copy()
    O.unary_op(s, O.SIGN, O.Meta.contiguous((x.size,)))
    d = _dev(x)
    _b().apply_unary(d, O.SIGN, _meta_pair(O.Meta.contiguous((x.size,))))
    assert _host(d).tobytes() == s.tobytes()


def test_fill_and_copy_view():
    rng = np.random.default_rng(9)
    base = O.Meta.contiguous((5, 8, 16))
    for m in [base, base.slice(2, 1, 15, 3), base.permute((1, 2, 0)).slice(0, None, None, -1), base.index(0, 2)]:
        buf = _rand(rng, base.size, np.float32)
        ref = buf.copy()
        O.fill(ref, 4.25, m)
        d = _dev(buf)
        _b().fill(d, 4.25, _meta_pair(m))
        assert _host(d).tobytes() == ref.tobytes()
        src = _rand(rng, base.size, np.int32)
        got = _host(_b().contiguous(_dev(src), _meta_pair(m)))[: m.size]
        assert np.array_equal(got, gather_view(src, m))


# ------------------------------------------------------------------------------------- broadcast
def _check_binary(a, am, b, bm, op):
    want, dm = O.binary(a, am, b, bm, op)
    out, gm = _b().binary(_dev(a), _meta_pair(am), _dev(b), _meta_pair(bm), op)
    assert tuple(gm.shape) == tuple(dm.shape)
    assert _host(out)[: dm.size].tobytes() == want.tobytes(), (am, bm, op)


def test_config_outer_product_add_then_axis_sum():
    rng = np.random.default_rng(0x5EED)
    a = rng.uniform(-1, 1, 4096).astype(np.float32)
    b = rng.uniform(-1, 1, 4096).astype(np.float32)
    am, bm = O.Meta.contiguous((4096, 1)), O.Meta.contiguous((1, 4096))
    want, dm = O.binary(a, am, b, bm, O.ADD)
    out, gm = _b().binary(_dev(a), _meta_pair(am), _dev(b), _meta_pair(bm), O.ADD)
    assert _host(out).tobytes() == want.tobytes()
    ref, om = O.reduce_axis(want, dm, 1, O.SUM)
    dst = _b().alloc(4096, torch.float32)
    _b().apply_reduce((out, gm), dst, 1, O.SUM)
    got = _host(dst)
    tol = 1e-5 * math.log2(4096)
    scale = np.abs(want.reshape(4096, 4096)).sum(axis=1, dtype=np.float64)
    assert np.all(np.abs(got.astype(np.float64) - ref.astype(np.float64)) <= tol * scale)


@pytest.mark.parametrize("scale", [16, 1])
def test_config_strided_negative_step_broadcast(scale):
    """A = permuted view of a (K,16,1,1) buffer, B = step -1 slice: the 4.3 GB configuration at
    full size (scale 1: checked on sampled rows) and 1/16 of it (checked everywhere)."""
    K, J, Lc = 1024 // scale, 64, 1024
    rng = np.random.default_rng(0x5EED + 3)
    bufa = rng.uniform(-1, 1, K * 16).astype(np.float32)
    bufb = rng.uniform(-1, 1, J * Lc).astype(np.float32)
    A = O.Meta.contiguous((K, 16, 1, 1)).view_as((1, K, 16, 1)).permute((2, 0, 1, 3))
    B = O.Meta.contiguous((1, J, 1, Lc)).slice(3, None, None, -1)
    out, gm = _b().binary(_dev(bufa), _meta_pair(A), _dev(bufb), _meta_pair(B), O.ADD)
    assert tuple(gm.shape) == (16, J, K, Lc)
    if scale > 1:
        want, _ = O.binary(bufa, A, bufb, B, O.ADD)
        assert _host(out).tobytes() == want.tobytes()
    else:
        o4 = out.view(16, J, K, Lc)
        ta = torch.from_numpy(bufa).cuda().view(K, 16).t().contiguous()  # [i, k] = bufa[16k + i]
        tb = torch.from_numpy(bufb).cuda().view(J, Lc).flip(1)           # [j, l] = bufb[1024 j + 1023 - l]
        # out[i,j,k,l] = bufa[16k+i] + bufb[1024j + 1023 - l]: one IEEE add, checked slab by slab
        for i in range(16):
            ref = ta[i].view(1, K, 1) + tb.view(J, 1, Lc)
            assert torch.equal(o4[i], ref)
        # and a sample of rows against the oracle's coordinate walk
        sub = O.Meta((1, 2, 3, Lc), (0, 0, 16, 0), 5)
        wa, _ = O.binary(bufa, O.Meta((2, 1, 3, 1), (1, 16384, 16, 1), 5), bufb, B.slice(1, 0, 2, 1), O.ADD)
        got = _host(o4[5:7, 0:2, 0:3, :].contiguous()).reshape(-1)
        assert got.tobytes() == wa.tobytes()


@pytest.mark.parametrize("dt", [np.float32, np.int32, np.float64, np.uint8, np.int64, np.bool_])
def test_random_broadcast_views(dt):
    rng = np.random.default_rng(77)
    for trial in range(40):
        rank = int(rng.integers(1, 5))
        full = [int(rng.choice([1, 2, 3, 5, 8, 33, 130])) for _ in range(rank)]
        sha = [d if rng.random() < 0.7 else 1 for d in full]
        shb = [d if rng.random() < 0.7 else 1 for d in full]
        shb = shb[int(rng.integers(0, rank)):] if rng.random() < 0.3 else shb

        def view_of(shape):
            # a buffer with padding, then random reversals / steps / permutes that keep the shape
            pad = [s * int(rng.choice([1, 2])) + int(rng.integers(0, 2)) for s in shape]
            m = O.Meta.contiguous(pad)
            for dim, s in enumerate(shape):
                step = int(rng.choice([1, 1, -1, 2, -2])) if pad[dim] >= 2 * s else int(rng.choice([1, -1]))
                if step > 0:
                    m = m.slice(dim, 0, min(pad[dim], (s - 1) * step + 1), step)
                else:
                    start = (s - 1) * (-step)
                    m = m.slice(dim, start, None, step)
                assert m.shape[dim] == s, (m, shape, dim, step)
            return int(np.prod(pad)), m
        na, am = view_of(sha)
        nb, bm = view_of(shb)
        a, b = _rand(rng, na, dt), _rand(rng, nb, dt)
        ops = [O.ADD, O.SUB, O.MUL] + ([O.DIV] if np.dtype(dt).kind == "f" else [])
        _check_binary(a, am, b, bm, int(rng.choice(ops)))


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.int32, np.uint8], ids=lambda d: np.dtype(d).name)
def test_long_rows_with_ragged_column_tiles(dt):
    """Rows of at least 128 vectors whose length is not a whole number of column tiles, with forward,
    reversed and broadcast operands, in and out of place."""
    rng = np.random.default_rng(4242)
    per = 16 // np.dtype(dt).itemsize
    for rows, inner in ((37, 250 * per), (5, 129 * per), (3, 1027 * per), (64, 513 * per)):
        a = _rand(rng, rows * inner, dt)
        b = _rand(rng, inner, dt)
        c = _rand(rng, rows, dt)
        am = O.Meta.contiguous((rows, inner))
        _check_binary(a, am, b, O.Meta.contiguous((inner,)), O.ADD)                                   # row-invariant right operand
        _check_binary(a, am, b, O.Meta.contiguous((inner,)).slice(0, None, None, -1), O.SUB)          # reversed
        _check_binary(c, O.Meta.contiguous((rows, 1)), b, O.Meta.contiguous((1, inner)), O.MUL)      # scalar per row x vector
        _check_binary(a, am.slice(1, None, None, -1), c, O.Meta.contiguous((rows, 1)), O.ADD)       # reversed left, scalar right
        # one-operand forms on a window of a wider buffer (pitch != row length)
        wide = _rand(rng, rows * (inner + 4 * per), dt)
        wm = O.Meta.contiguous((rows, inner + 4 * per)).slice(1, 0, inner, 1)
        ref = wide.copy()
        O.scalar_op(ref, O.ADD, 3, wm)
        d = _dev(wide)
        _b().scalar_apply(d, O.ADD, 3, _meta_pair(wm))
        assert _host(d).tobytes() == ref.tobytes(), (dt, rows, inner)
        ref2 = wide.copy()
        O.fill(ref2, 1, wm)
        d = _dev(wide)
        _b().fill(d, 1, _meta_pair(wm))
        assert _host(d).tobytes() == ref2.tobytes(), (dt, rows, inner)


def test_broadcast_in_place_forms():
    rng = np.random.default_rng(3)
    from rtensors_b200.meta import Meta
    for am, bshape in [(O.Meta.contiguous((64, 48)), (48,)), (O.Meta.contiguous((64, 48)).slice(1, None, None, -1), (1, 1)),
                       (O.Meta.contiguous((8, 64, 48)).permute((2, 0, 1)), (8, 1)),
                       (O.Meta.contiguous((64, 48)).slice(0, None, None, 2), (32, 48))]:
        a = _rand(rng, 8 * 64 * 48, np.float32)
        b = _rand(rng, int(np.prod(bshape)), np.float32)
        bm = O.Meta.contiguous(bshape)
        ref = a.copy()
        shape, sa, sb = O.broadcast_params(am, bm)
        ma = O.Meta(shape, sa, am.offset)
        O.broadcast(ref, ma, b, O.Meta(shape, sb, bm.offset), ref, ma, O.MUL)
        d = _dev(a)
        _b().binary_assign(d, _meta_pair(am), _dev(b), _meta_pair(bm), O.MUL)
        assert _host(d).tobytes() == ref.tobytes()


def test_i32_same_shape_add_bit_exact():
    rng = np.random.default_rng(0x5EED + 2)
    n = (1 << 22) + 3
    a = rng.integers(-(1 << 20), 1 << 20, n, endpoint=True).astype(np.int32)
    b = rng.integers(-(1 << 20), 1 << 20, n, endpoint=True).astype(np.int32)
    m = O.Meta.contiguous((n,))
    _check_binary(a, m, b, m, O.ADD)
    # wrap-around
    a[:4] = [2**31 - 1, -2**31, 2**31 - 1, 5]
    b[:4] = [1, -1, 2**31 - 1, -7]
    _check_binary(a, m, b, m, O.ADD)
    _check_binary(a, m, b, m, O.MUL)


def test_rank_above_plan_limit_is_peeled():
    rng = np.random.default_rng(4)
    shape = (2, 3) * 5  # rank 10; alternating strides below block merging
    pad = tuple(s + 1 for s in shape)
    m = O.Meta.contiguous(pad)
    for dim, s in enumerate(shape):
        m = m.slice(dim, 0, s, 1)
    a = _rand(rng, int(np.prod(pad)), np.float32)
    b = _rand(rng, 3, np.float32)
    _check_binary(a, m, b, O.Meta.contiguous((3,)), O.ADD)


def test_empty_and_scalar_shapes():
    a = np.array([2.5], dtype=np.float32)
    _check_binary(a, O.Meta.contiguous(()), a, O.Meta.contiguous(()), O.MUL)
    from rtensors_b200.meta import Meta
    z = _b().alloc(1, torch.float32)
    _b().scalar_apply(z, O.ADD, 1.0, Meta((0, 4), (4, 1), 0))  # empty view: no launch, no error
    out = _b().alloc(4, torch.float32)
    _b().apply_reduce((z, Meta((0, 4), (4, 1), 0)), out, 1, O.SUM)  # zero outputs: no launch


# ------------------------------------------------------------------------------------- reductions
def _sum_tol(n):
    return 1e-5 * max(math.log2(max(n, 2)), 1.0)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("n,start", [(1, 0), (2, 1), (31, 0), (1025, 3), (4096, 0), ((1 << 20) + 7, 1), (1 << 24, 0),
                                     # sizes that take one CTA per 32 KiB block: just above the one-wave limit with a
                                     # ragged last block, and a misaligned start with scalar head and tail elements
                                     ((5 << 20) + 1, 2), ((1 << 23) + 4099, 3)])
def test_flat_reductions(dt, n, start):
    rng = np.random.default_rng(n + start)
    x = rng.standard_normal(n + start + 1).astype(dt)
    d = _dev(x)
    absum = float(np.abs(x[start:start + n]).sum(dtype=np.float64))
    for op in (O.SUM, O.MEAN, O.MAX, O.MIN):
        want = O.reduce_flat(x, start, n, op)[0]
        out = _b().alloc(1, d.dtype)
        _b().apply_reduce_contiguous_flat(d, out, start, n, op)
        got = _host(out)[0]
        if op in (O.MAX, O.MIN):
            assert got.tobytes() == want.tobytes()
        else:
            scale = absum if op == O.SUM else absum / n
            assert abs(float(got) - float(want)) <= _sum_tol(n) * scale + 1e-30, (op, got, want)


@pytest.mark.parametrize("outer,r,inner", [(1, 8192, 1), (37, 1000, 1), (4096, 33, 1), (3, 70000, 1), (8, 5, 1),
                                           (1, 4096, 1024), (64, 128, 48), (5, 777, 130), (2, 3, 7), (300, 2, 4096),
                                           (1, 4096, 10), (7, 1, 9)])
def test_axis_reductions(outer, r, inner):
    rng = np.random.default_rng(outer * 7 + r + inner)
    x = rng.standard_normal(outer * r * inner).astype(np.float32)
    d = _dev(x)
    absum = np.abs(x.reshape(outer, r, inner)).sum(axis=1, dtype=np.float64).reshape(-1)
    for op in (O.SUM, O.MEAN, O.MAX, O.MIN):
        want = O.reduce_ori(x, outer, r, inner, op)
        got = _host(_b().reduce_axis_ori(d, 0, outer, r, inner, op))[: outer * inner]
        if op in (O.MAX, O.MIN):
            assert got.tobytes() == want.tobytes(), (op,)
        else:
            scale = absum if op == O.SUM else absum / r
            err = np.abs(got.astype(np.float64) - want.astype(np.float64))
            assert np.all(err <= _sum_tol(r) * scale + 1e-30), (op, err.max())


def test_axis_reduction_misaligned_offset_and_f64():
    rng = np.random.default_rng(21)
    x = rng.standard_normal(3 + 16 * 100 * 12).astype(np.float64)
    for off in (0, 1, 3):
        want = O.reduce_ori(x[off:off + 16 * 100 * 12].copy(), 16, 100, 12, O.SUM)
        got = _host(_b().reduce_axis_ori(_dev(x), off, 16, 100, 12, O.SUM))
        assert np.allclose(got, want, rtol=1e-12, atol=1e-12)
        want = O.reduce_ori(x[off:off + 16 * 100 * 12].copy(), 16 * 100, 12, 1, O.MAX)
        got = _host(_b().reduce_axis_ori(_dev(x), off, 16 * 100, 12, 1, O.MAX))
        assert got.tobytes() == want.tobytes()


def test_max_ignores_nan_and_starts_from_lowest_finite():
    x = np.array([np.nan, -np.inf, -np.inf, np.nan], dtype=np.float32)
    for op in (O.MAX, O.MIN):
        want = O.reduce_flat(x, 0, 4, op)
        out = _b().alloc(1, torch.float32)
        _b().apply_reduce_contiguous_flat(_dev(x), out, 0, 4, op)
        assert _host(out).tobytes() == want.tobytes()


def test_tensor_api_reductions_on_views():
    from rtensors_b200.tensor import Tensor
    rng = np.random.default_rng(8)
    x = rng.standard_normal((12, 20, 16)).astype(np.float32)
    t = Tensor.from_buf(x, x.shape, np.float32, _b())
    v = t.slice(2, None, None, -2).permute((1, 0, 2))  # non-contiguous: copied first, as the reference does
    xv = x[:, :, ::-2].transpose(1, 0, 2)
    got = v.sum_at(1).cpu()
    assert got.shape == (20, 1, 8)
    assert np.allclose(got[:, 0, :], xv.sum(axis=1), rtol=1e-5, atol=1e-5)
    assert v.max().item() == xv.max()
    assert abs(float(v.mean().item()) - float(xv.mean())) < 1e-5


# ------------------------------------------------------------------------------------- fused ops
@pytest.mark.parametrize("n", [1, 5, 4096, (1 << 20) + 3])
def test_l1_loss(n):
    rng = np.random.default_rng(n)
    a = rng.standard_normal(n).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    b[::5] = a[::5]  # exact zeros in the difference: sign(0) = 0
    for reduction in (0, 1):
        want, wg = O.l1_loss(a, b, reduction, True)
        loss, g = _b().l1_loss(_dev(a), _dev(b), reduction, True)
        scale = float(np.abs(a - b).sum(dtype=np.float64)) / (n if reduction == 0 else 1)
        assert abs(float(_host(loss)[0]) - float(want[0])) <= _sum_tol(n) * scale + 1e-30
        assert _host(g).tobytes() == wg.tobytes()
        loss2, _ = _b().l1_loss(_dev(a), _dev(b), reduction, False)
        assert _host(loss2).tobytes() == _host(loss).tobytes()


def test_reduce_to_shape():
    rng = np.random.default_rng(2)
    for shape, strides in [((4096, 1024), (0, 1)), ((4096, 10), (0, 1)), ((6, 5, 4, 3), (0, 12, 0, 1)),
                           ((6, 5, 4, 3), (0, 0, 3, 1)), ((8, 16), (16, 0)), ((7, 9), (0, 0)), ((3, 4), (4, 1))]:
        up = rng.standard_normal(int(np.prod(shape))).astype(np.float32)
        want, wshape = O.reduce_to_shape(up, shape, strides, intended=True)
        got, gshape = _b().reduce_to_shape(_dev(up), shape, strides)
        assert tuple(gshape) == tuple(wshape)
        g = _host(got)[: want.size]
        red = tuple(k for k, s in enumerate(strides) if s == 0)
        scale = np.abs(up.reshape(shape)).sum(axis=red, dtype=np.float64).reshape(-1) if red else np.abs(up)
        cnt = int(np.prod([shape[k] for k in red])) if red else 1
        assert np.all(np.abs(g.astype(np.float64) - want.astype(np.float64)) <= _sum_tol(cnt) * scale + 1e-30)


def test_relu_mask_sgd_and_u8_convert():
    rng = np.random.default_rng(6)
    x = rng.standard_normal(4096 * 33 + 4).astype(np.float32)
    x[::9] = 0.0
    ref = x.copy()
    wm = O.relu_mask(ref)
    d = _dev(x)
    m = _b().relu_mask(d)
    assert _host(d).tobytes() == ref.tobytes() and _host(m).tobytes() == wm.tobytes()
    p = rng.standard_normal(100003).astype(np.float32)
    g = rng.standard_normal(100003).astype(np.float32)
    rp = p.copy()
    O.sgd_update(rp, g, 0.01)
    dp = _dev(p)
    _b().sgd_update(dp, _dev(g), 0.01)
    assert _host(dp).tobytes() == rp.tobytes()
    u = rng.integers(0, 256, 28 * 28 * 17 + 1).astype(np.uint8)
    assert _host(_b().u8_to_f32_div(_dev(u), 255.0)).tobytes() == O.u8_to_f32_div(u, 255.0).tobytes()


# ------------------------------------------------------------------------------------- v1 launchers
def test_v1_reference_launchers():
    import rtensors_b200 as rt
    lib = rt.lib()
    rng = np.random.default_rng(10)
    torch.cuda.synchronize()
    x = rng.uniform(-1, 1, 5000).astype(np.float32)
    d = _dev(x)
    torch.cuda.synchronize()
    ref = x.copy()
    # contiguous scalar op: pointer already advanced by `start`
    lib.launch_mul_contiguous_f32(C.c_void_p(d.data_ptr() + 4 * 3), C.c_size_t(4000), C.c_float(3.0), C.c_uint(256))
    O.scalar_op(ref, O.MUL, 3.0, O.Meta((4000,), (1,), 3))
    lib.launch_add_strided_f32(C.c_void_p(d.data_ptr()), C.c_size_t(4999), C.c_ssize_t(-3), C.c_size_t(1000),
                               C.c_float(2.0), C.c_uint(256))
    O.scalar_op(ref, O.ADD, 2.0, O.Meta((1000,), (-3,), 4999))
    lib.launch_relu_contiguous_f32(C.c_void_p(d.data_ptr()), C.c_size_t(10), C.c_size_t(300), C.c_uint(256))
    O.unary_op(ref, O.RELU, O.Meta((300,), (1,), 10))
    # nd_affine takes shape / stride arrays in device memory
    shape = torch.tensor([10, 20], dtype=torch.int64, device="cuda")
    stride = torch.tensor([200, -2], dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    lib.launch_sub_nd_affine_f32(C.c_void_p(d.data_ptr()), C.c_size_t(100), C.c_void_p(stride.data_ptr()),
                                 C.c_void_p(shape.data_ptr()), C.c_size_t(2), C.c_size_t(200), C.c_float(1.0),
                                 C.c_uint(256))
    O.scalar_op(ref, O.SUB, 1.0, O.Meta((10, 20), (200, -2), 100))
    torch.cuda.synchronize()
    assert _host(d).tobytes() == ref.tobytes()
    # broadcast through the v1 symbol: (8,1) + (1,16)
    a, b = x[:8].copy(), x[8:24].copy()
    da, db, dd = _dev(a), _dev(b), _b().alloc(128, torch.float32)
    ls = torch.tensor([1, 0], dtype=torch.int64, device="cuda")
    rs = torch.tensor([0, 1], dtype=torch.int64, device="cuda")
    ds = torch.tensor([16, 1], dtype=torch.int64, device="cuda")
    sh = torch.tensor([8, 16], dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    lib.launch_binary_broadcast_elementwise_f32(C.c_void_p(da.data_ptr()), C.c_void_p(db.data_ptr()),
                                                C.c_void_p(dd.data_ptr()), C.c_size_t(0), C.c_size_t(0), C.c_size_t(0),
                                                C.c_size_t(2), C.c_size_t(128), C.c_void_p(ls.data_ptr()),
                                                C.c_void_p(rs.data_ptr()), C.c_void_p(ds.data_ptr()),
                                                C.c_void_p(sh.data_ptr()), C.c_uint8(0), C.c_uint(256))
    torch.cuda.synchronize()
    want, _ = O.binary(a, O.Meta.contiguous((8, 1)), b, O.Meta.contiguous((1, 16)), O.ADD)
    assert _host(dd).tobytes() == want.tobytes()
    # reductions
    out = _b().alloc(1, torch.float32)
    torch.cuda.synchronize()
    lib.launch_flat_contiguous_reduce_f32(C.c_void_p(d.data_ptr()), C.c_void_p(out.data_ptr()), C.c_size_t(5),
                                          C.c_size_t(4000), C.c_uint8(3), None, C.c_uint(256))
    torch.cuda.synchronize()
    assert _host(out).tobytes() == O.reduce_flat(ref, 5, 4000, O.MAX).tobytes()
    out2 = _b().alloc(50, torch.float32)
    lib.launch_nd_reduce_contiguous_f32(C.c_void_p(d.data_ptr()), C.c_void_p(out2.data_ptr()), C.c_size_t(0),
                                        C.c_size_t(5), C.c_size_t(100), C.c_size_t(10), C.c_uint8(4), None,
                                        C.c_uint(256))
    torch.cuda.synchronize()
    assert _host(out2).tobytes() == O.reduce_ori(ref[:5000], 5, 100, 10, O.MIN).tobytes()
    assert lib.rtensors_take_cuda_alloc_error() == 0


# ------------------------------------------------------------------------------------- MLP SGD step
@pytest.mark.parametrize("ref_quirks", [False, True], ids=["intended", "ref_quirks"])
def test_mlp_sgd_step_matches_oracle(ref_quirks):
    """GEMMs differ between cuBLAS and the oracle's GEMM, so the step is tolerance-checked
    (1e-4 of max|.| per tensor); the non-GEMM kernels are checked bit-exactly elsewhere."""
    from mlp_oracle import mlp_step
    from rtensors_b200.mlp import DenseMlp, synthetic_batch
    torch.backends.cuda.matmul.allow_tf32 = False
    sizes = (784, 256, 128, 10)
    batch = 192
    model = DenseMlp(_b(), sizes, lr=0.01, ref_quirks=ref_quirks)
    # non-zero biases so that the bias path matters
    params = model.host_params()
    rng = np.random.default_rng(1)
    for k in range(1, len(params), 2):
        params[k] = rng.uniform(-0.05, 0.05, params[k].shape).astype(np.float32)
    model.load_params(params)
    img, tgt, img_h, tgt_h = synthetic_batch(batch, "cuda:0")
    loss = model.step(img, tgt)
    want_loss, want_params, want_grads = mlp_step(params, sizes, img_h, tgt_h, 0.01, ref_quirks)
    assert abs(float(loss.item()) - want_loss) <= 1e-5 * abs(want_loss) + 1e-7
    got = model.host_params()
    for k, (g, w, p0) in enumerate(zip(got, want_params, params)):
        delta_w = w - p0
        scale = max(float(np.abs(delta_w).max()), 1e-12)
        assert np.abs((g - p0) - delta_w).max() <= 1e-3 * scale + 1e-9, (k, np.abs((g - p0) - delta_w).max(), scale)
    for k in range(len(params)):
        gg = model._view(model.grads, k).cpu().numpy()
        scale = max(float(np.abs(want_grads[k]).max()), 1e-12)
        assert np.abs(gg.reshape(-1) - want_grads[k].reshape(-1)).max() <= 1e-3 * scale, k


def test_mlp_loss_decreases_over_steps():
    from rtensors_b200.mlp import DenseMlp, synthetic_batch
    model = DenseMlp(_b(), (784, 128, 64, 10), lr=0.5)
    img, tgt, _, _ = synthetic_batch(256, "cuda:0")
    losses = [float(model.step(img, tgt).item()) for _ in range(30)]
    assert losses[-1] < losses[0]  # the reference's own autograd tests assert exactly this


def test_mlp_step_replayed_from_a_graph_equals_the_eager_step():
    """Two models with the same seed: one steps eagerly, the other through step_graphed (first call
    eager + capture, then replays) on a sequence of different batches; parameters stay bit-identical."""
    from rtensors_b200.mlp import DenseMlp, synthetic_batch
    eager = DenseMlp(_b(), (784, 128, 64, 10), lr=0.1)
    graphed = DenseMlp(_b(), (784, 128, 64, 10), lr=0.1)
    for k in range(5):
        img, tgt, _, _ = synthetic_batch(256, "cuda:0", seed=1000 + k)
        le = eager.step(img, tgt)
        lg = graphed.step_graphed(img, tgt)
        assert _host(le).tobytes() == _host(lg).tobytes(), k
        assert _host(eager.params).tobytes() == _host(graphed.params).tobytes(), k


# ------------------------------------------------------------------------------------- context / allocator
def test_context_allocator_and_copies():
    import rtensors_b200 as rt
    lib = rt.lib()
    ctx = C.c_void_p()
    assert lib.rtb_ctx_create(C.c_int(0), C.byref(ctx)) == 0
    try:
        assert lib.rtb_ctx_device(ctx) == 0 and lib.rtb_ctx_sm_count(ctx) > 0
        ptrs = []
        for nbytes in (1, 4096, 1 << 20, (3 << 20) + 5):
            p = C.c_void_p()
            assert lib.rtb_alloc(ctx, C.c_size_t(nbytes), C.byref(p)) == 0 and p.value
            assert p.value % 256 == 0
            ptrs.append(p)
        # round trip through the context's copy calls, with a kernel in between
        x = np.arange(1000, dtype=np.float32)
        p = ptrs[2]
        assert lib.rtb_h2d(ctx, p, x.ctypes.data_as(C.c_void_p), C.c_size_t(x.nbytes)) == 0
        v = np.array([2.0], dtype=np.float32)
        shape = (C.c_size_t * 1)(1000)
        strides = (C.c_ssize_t * 1)(1)
        assert lib.rtb_scalar_op(ctx, C.c_int(10), C.c_int(2), p, v.ctypes.data_as(C.c_void_p), C.c_size_t(1), shape,
                                 strides, C.c_size_t(0)) == 0
        assert lib.rtb_d2d(ctx, ptrs[3], p, C.c_size_t(x.nbytes)) == 0
        y = np.zeros_like(x)
        assert lib.rtb_d2h(ctx, y.ctypes.data_as(C.c_void_p), ptrs[3], C.c_size_t(x.nbytes)) == 0
        assert np.array_equal(y, x * 2)
        assert lib.rtb_ctx_launch_count(ctx) == 1
        # freed blocks are reused (caching) and foreign pointers are refused
        old = ptrs[1].value
        assert lib.rtb_free(ctx, ptrs[1]) == 0
        q = C.c_void_p()
        assert lib.rtb_alloc(ctx, C.c_size_t(4000), C.byref(q)) == 0 and q.value == old
        assert lib.rtb_free(ctx, C.c_void_p(12345)) == -1
        assert b"not allocated" in lib.rtb_last_error_string()
        for p in (ptrs[0], q, ptrs[2], ptrs[3]):
            assert lib.rtb_free(ctx, p) == 0
        assert lib.rtb_release_cached(ctx) == 0
        # a non-default stream
        s = torch.cuda.Stream()
        assert lib.rtb_ctx_set_stream(ctx, C.c_void_p(s.cuda_stream)) == 0
        assert lib.rtb_ctx_get_stream(ctx) == s.cuda_stream
        t = torch.ones(1 << 16, device="cuda")
        s.wait_stream(torch.cuda.current_stream())
        shape = (C.c_size_t * 1)(t.numel())
        assert lib.rtb_scalar_op(ctx, C.c_int(10), C.c_int(0), C.c_void_p(t.data_ptr()), v.ctypes.data_as(C.c_void_p),
                                 C.c_size_t(1), shape, strides, C.c_size_t(0)) == 0
        assert lib.rtb_ctx_sync(ctx) == 0
        assert float(t.sum().item()) == 3.0 * t.numel()
    finally:
        lib.rtb_ctx_destroy(ctx)


def test_error_codes_for_bad_arguments():
    import rtensors_b200 as rt
    from rtensors_b200.meta import Meta
    x = _b().alloc(16, torch.float32)
    with pytest.raises(rt.RtbError) as e:  # view runs past the buffer
        _b().scalar_apply(x, O.ADD, 1.0, Meta((4, 8), (8, 1), 0))
    assert e.value.code == -4
    flag = _b().alloc(4, torch.bool)
    with pytest.raises(rt.RtbError) as e:  # boolean division is not defined (todo!() in the reference)
        _b().scalar_apply(flag, O.DIV, True, Meta.contiguous((4,)))
    assert e.value.code == -2
    u = _b().alloc(4, torch.uint8)
    with pytest.raises(rt.RtbError):       # negation needs a signed type
        _b().apply_unary(u, O.NEG, Meta.contiguous((4,)))
    i = _b().alloc(4, torch.int32)
    with pytest.raises(rt.RtbError) as e:  # reductions are float-only, as in the reference
        _b().apply_reduce_contiguous_flat(i, i, 0, 4, O.SUM)
    assert e.value.code == -2
    with pytest.raises(rt.RtbError) as e:
        _b().apply_reduce((x, Meta.contiguous((4, 4)).permute((1, 0))), x, 0, O.SUM)
    assert e.value.code == -7


# ------------------------------------------------------------------------------------- 128-bit integers
def test_128_bit_integer_ops():
    """u128 / i128 have no numpy or torch dtype: drive them as raw 16-byte little-endian words."""
    import rtensors_b200 as rt
    from rtensors_b200.meta import Meta
    lib = rt.lib()
    rng = np.random.default_rng(128)
    n = 1000
    mask = (1 << 128) - 1

    def to_bytes(vals):
        return np.frombuffer(b"".join(int(v & mask).to_bytes(16, "little") for v in vals), dtype=np.uint8).copy()

    def from_bytes(buf):
        raw = buf.tobytes()
        return [int.from_bytes(raw[k:k + 16], "little") for k in range(0, len(raw), 16)]

    a = [int(rng.integers(0, 1 << 62)) << int(rng.integers(0, 66)) for _ in range(n)]
    b = [int(rng.integers(1, 1 << 62)) << int(rng.integers(0, 60)) for _ in range(n)]
    da, db = _dev(to_bytes(a)), _dev(to_bytes(b))
    out = _b().alloc(16 * n, torch.uint8)
    m = Meta.contiguous((n,))
    ctx = _b()._ctx
    for code, op, fn in ((5, 0, lambda x, y: (x + y) & mask), (5, 1, lambda x, y: (x - y) & mask),
                         (5, 2, lambda x, y: (x * y) & mask), (5, 3, lambda x, y: x // y)):
        rc = lib.rtb_broadcast(ctx, C.c_int(code), C.c_int(op), C.c_void_p(da.data_ptr()), (C.c_ssize_t * 1)(1),
                               C.c_size_t(0), C.c_void_p(db.data_ptr()), (C.c_ssize_t * 1)(1), C.c_size_t(0),
                               C.c_void_p(out.data_ptr()), (C.c_ssize_t * 1)(1), C.c_size_t(0), C.c_size_t(1),
                               (C.c_size_t * 1)(n))
        assert rc == 0
        assert from_bytes(_host(out)) == [fn(x, y) for x, y in zip(a, b)], op
    # signed: negate and relu through a reversed strided view
    sa = [int(rng.integers(-(1 << 62), 1 << 62)) * int(rng.integers(1, 1 << 40)) for _ in range(n)]
    ds = _dev(to_bytes(sa))
    view = Meta.contiguous((n,)).slice(0, None, None, -3)
    assert lib.rtb_unary_op(ctx, C.c_int(9), C.c_int(1), C.c_void_p(ds.data_ptr()), C.c_size_t(1),
                            (C.c_size_t * 1)(view.shape[0]), (C.c_ssize_t * 1)(view.strides[0]),
                            C.c_size_t(view.offset)) == 0
    want = list(sa)
    for k in range(view.shape[0]):
        idx = view.offset + k * view.strides[0]
        want[idx] = max(want[idx], 0)
    got = [v - (1 << 128) if v >> 127 else v for v in from_bytes(_host(ds))]
    assert got == want


def test_host_pipeline_matches_oracle():
    from rtensors_b200.host import HostPipeline
    from rtensors_b200.meta import Meta
    rng = np.random.default_rng(31)
    n = (1 << 20) + 777
    ha = torch.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)).pin_memory()
    hi = torch.from_numpy(rng.integers(-(1 << 20), 1 << 20, n).astype(np.int32)).pin_memory()
    hj = torch.from_numpy(rng.integers(-(1 << 20), 1 << 20, n).astype(np.int32)).pin_memory()
    ra, ri = torch.empty_like(ha).pin_memory(), torch.empty_like(hi).pin_memory()
    be = _b()

    def compute(v, length):
        mc = Meta.contiguous((length,))
        be.scalar_apply(v["a"], O.MUL, 3.0, mc)
        be.scalar_apply(v["a"], O.ADD, 2.0, mc)
        be.scalar_apply(v["a"], O.SUB, 1.0, mc)
        be.broadcast((v["ia"], mc), (v["ib"], mc), (v["iout"], mc), O.ADD)
    pipe = HostPipeline(be, chunk_elems=100_000)  # ragged last chunk, unaligned chunk starts
    for _ in range(2):
        pipe.run(n, {"a": ha, "ia": hi, "ib": hj}, {"a": (ra, torch.float32), "iout": (ri, torch.int32)}, compute)
    be.host_wait()
    ref = ha.numpy().copy()
    m = O.Meta.contiguous((n,))
    for op, v in ((O.MUL, 3.0), (O.ADD, 2.0), (O.SUB, 1.0)):
        O.scalar_op(ref, op, v, m)
    assert ra.numpy().tobytes() == ref.tobytes()
    assert np.array_equal(ri.numpy(), hi.numpy() + hj.numpy())


# ------------------------------------------------------------------------------------- remaining float families
_EXT_DOMAIN = {"SQRT": (0.01, 4), "RSQRT": (0.01, 4), "LN": (0.01, 4), "LN1P": (-0.9, 4), "ASIN": (-0.99, 0.99),
               "ACOS": (-0.99, 0.99), "ACOSH": (1.01, 5), "ATANH": (-0.99, 0.99), "RECIPROCAL": (0.05, 4)}


@pytest.mark.parametrize("dt,tol", [(np.float32, 2e-6), (np.float64, 1e-14)], ids=["f32", "f64"])
def test_remaining_unary_families_match_cpu_formulas(dt, tol):
    """The CUDA math library and glibc round transcendentals differently, so these are compared at
    a relative tolerance (the reference's own tests use |a-b| < 1e-5); the formulas are the CPU
    backend's (exp-based tanh, ln/sqrt-based asinh, ...), checked on all three layouts."""
    rng = np.random.default_rng(17)
    base = O.Meta.contiguous((37, 24))
    views = [base, base.slice(1, None, None, -2), base.permute((1, 0)).slice(0, 2, 20, 3)]
    names = ["SIGMOID", "TANH", "SQRT", "SIN", "COS", "TAN", "ASIN", "ACOS", "ATAN", "SINH", "COSH", "ASINH", "ACOSH",
             "ATANH", "RSQRT", "RECIPROCAL", "SQUARE", "CUBE", "EXP", "LN", "LN1P", "FLOOR", "CEIL", "ROUND", "TRUNC",
             "EXPM1", "SILU"]
    for name in names:
        lo, hi = _EXT_DOMAIN.get(name, (-3, 3))
        for m in views:
            buf = rng.uniform(lo, hi, base.size).astype(dt)
            if name in ("FLOOR", "CEIL", "ROUND", "TRUNC"):
                buf[:8] = [0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 0.0, -0.0]
            ref = buf.copy()
            O.unary_op(ref, getattr(O, name), m)
            d = _dev(buf)
            _b().apply_unary(d, getattr(O, name), _meta_pair(m))
            got = _host(d)
            if name in ("FLOOR", "CEIL", "ROUND", "TRUNC", "SQUARE", "CUBE", "RECIPROCAL", "SQRT"):
                assert got.tobytes() == ref.tobytes(), name  # single IEEE ops: exact
            else:
                assert np.allclose(got, ref, rtol=tol * 8, atol=tol), (name, np.abs(got - ref).max())


def test_remaining_scalar_families():
    rng = np.random.default_rng(18)
    m = O.Meta.contiguous((50, 100)).slice(1, None, None, -2).slice(0, 3, None, -1)
    for dt, tol in ((np.float32, 2e-6), (np.float64, 1e-14)):
        for op, v, lo in ((O.LOG, 2.0, 0.01), (O.LOG1P, 10.0, -0.9), (O.LEAKY_RELU, 0.1, -3), (O.ELU, 1.5, -3)):
            buf = rng.uniform(lo, 3, 5000).astype(dt)
            ref = buf.copy()
            O.scalar_op(ref, op, v, m)
            d = _dev(buf)
            _b().scalar_apply(d, op, v, _meta_pair(m))
            if op == O.LEAKY_RELU:
                assert _host(d).tobytes() == ref.tobytes()
            else:
                assert np.allclose(_host(d), ref, rtol=tol * 8, atol=tol), op
    # leaky_relu exists for integer types too (wrapping multiply on the negative side)
    for dt in (np.int32, np.int8, np.uint16):
        buf = _rand(rng, 5000, dt)
        ref = buf.copy()
        O.scalar_op(ref, O.LEAKY_RELU, 3, m)
        d = _dev(buf)
        _b().scalar_apply(d, O.LEAKY_RELU, 3, _meta_pair(m))
        assert _host(d).tobytes() == ref.tobytes()
    with pytest.raises(Exception):
        _b().scalar_apply(_dev(np.zeros(4, np.int32)), O.ELU, 1, _meta_pair(O.Meta.contiguous((4,))))
    with pytest.raises(Exception):
        _b().apply_unary(_dev(np.zeros(4, np.int32)), O.EXP, _meta_pair(O.Meta.contiguous((4,))))


def test_sign_dense_reversed_view_is_walked_from_its_lowest_address():
    """A fully reversed view counts as contiguous in the reference, whose dispatcher then walks
    forward from the view's offset and runs out of bounds (the Rust slice index panics; the oracle
    refuses).  The library applies the op to exactly the viewed elements."""
    x = np.arange(12, dtype=np.float32)
    m = O.Meta.contiguous((3, 4)).slice(0, None, None, -1).slice(1, None, None, -1)
    assert m.is_contiguous() and m.offset == 11
    with pytest.raises(O.OracleError):
        O.scalar_op(x.copy(), O.ADD, 1.0, m)
    d = _dev(x)
    _b().scalar_apply(d, O.ADD, 1.0, _meta_pair(m))
    assert np.array_equal(_host(d), x + 1)
    sub = O.Meta.contiguous((12,)).slice(0, 7, None, -1)  # elements 7..0 reversed
    d = _dev(x)
    _b().scalar_apply(d, O.MUL, 2.0, _meta_pair(sub))
    want = x.copy(); want[:8] *= 2
    assert np.array_equal(_host(d), want)


# ------------------------------------------------------------------------------------- beyond 2^31 elements
def test_more_than_2_31_elements_u8_and_f32():
    """64-bit indexing: the reference's flat reduce passes the count as `int`
    (cuda/kernels/reduction/reduce.cu:239-274); here sizes past 2^31 elements are first-class."""
    from rtensors_b200.meta import Meta
    free, _ = torch.cuda.mem_get_info()
    if free < 24 << 30:
        pytest.skip("needs 24 GiB of free device memory")
    n = (1 << 31) + 77
    x = torch.full((n,), 3, dtype=torch.uint8, device="cuda")
    x[-1] = 9
    x[1 << 31] = 5
    _b().scalar_apply(x, O.ADD, 250, Meta.contiguous((n,)))  # wraps: 3+250 = 253, 9+250 = 3, 5+250 = 255
    assert int(x[0]) == 253 and int(x[-1]) == 3 and int(x[1 << 31]) == 255 and int(x[(1 << 31) - 1]) == 253
    assert int((x == 253).sum()) == n - 2
    # strided view past 2^31: every other element of the upper half, reversed
    v = Meta.contiguous((n,)).slice(0, n - 1, 1 << 31, -2)
    _b().scalar_apply(x, O.SUB, 3, v)
    assert int(x[-1]) == 0 and int(x[-3]) == 250 and int(x[-2]) == 253
    del x
    torch.cuda.empty_cache()
    m = (1 << 31) + 1029
    y = torch.ones(m, dtype=torch.float32, device="cuda")
    y[-1] = 1025.0
    y[(1 << 31) + 3] = -7.0
    out = _b().alloc(1, torch.float32)
    _b().apply_reduce_contiguous_flat(y, out, 0, m, O.SUM)
    want = float(m - 2) + 1025.0 - 7.0
    assert abs(float(out.item()) - want) <= 1e-5 * 32 * want
    _b().apply_reduce_contiguous_flat(y, out, 5, m - 5, O.MAX)
    assert float(out.item()) == 1025.0
    _b().apply_reduce_contiguous_flat(y, out, 0, m, O.MIN)
    assert float(out.item()) == -7.0
    # axis reduction whose total size exceeds 2^31: [2, 2^30 + 515 (rounded), 1]... rows of ~2^30
    r = m // 2
    red = _b().reduce_axis_ori(y, 0, 2, r, 1, O.SUM)
    got = red.cpu().numpy()
    assert abs(got[0] - float(r)) <= 1e-5 * 31 * r
    assert abs(got[1] - (float(y[r:2 * r].sum(dtype=torch.float64)))) <= 1e-5 * 31 * r


# ------------------------------------------------------------------------------------- reductions over views
def test_reduce_view_matches_copy_then_reduce():
    """rtb_reduce_view against the reference's recipe (copy the view contiguous, then reduce), on
    views that reduce in place (contiguous inner run under strided / reversed / permuted outer dims,
    transposed matrices) and on views that take the copy fallback."""
    from rtensors_b200.meta import Meta
    rng = np.random.default_rng(99)
    base = O.Meta.contiguous((12, 40, 64))
    x = rng.standard_normal(base.size).astype(np.float32)
    d = _dev(x)
    views = [
        base,                                                     # dense
        base.slice(0, 2, 11, 3),                                  # strided outer, dense rest
        base.slice(0, None, None, -1),                            # reversed outer
        base.slice(1, 5, 35, 2),                                  # strided middle
        base.slice(1, None, None, -1).slice(0, 1, 9, 1),          # reversed middle
        base.slice(2, 8, 40, 1),                                  # inner window (row pitch > row length)
        base.slice(2, None, None, -1),                            # reversed inner -> copy fallback
        base.slice(2, None, None, 2),                             # strided inner -> copy fallback / strided rows
        base.permute((1, 0, 2)),                                  # permuted outer dims
        base.permute((2, 1, 0)),                                  # fully transposed
        base.permute((2, 0, 1)),                                  # contiguous dim moved to the front: rows with a pitch
        base.slice(1, 4, 36, 1).permute((2, 0, 1)),               # same over a window (outer dims do not collapse)
        base.index(0, 3).permute((1, 0)),                         # transposed matrix
        base.index(2, 7),                                         # (12, 40) with strides (2560, 64)
    ]
    for m in views:
        dense = gather_view(x, m)
        dm = O.Meta.contiguous(m.shape)
        for axis in [None] + list(range(len(m.shape))):
            for op in (O.SUM, O.MAX, O.MEAN, O.MIN):
                if axis is None:
                    want = O.reduce_flat(dense, 0, dense.size, op)
                    cnt = dense.size
                    scale = np.array([np.abs(dense).sum(dtype=np.float64)])
                else:
                    want, _ = O.reduce_axis(dense, dm, axis, op)
                    cnt = m.shape[axis]
                    scale = np.abs(dense.reshape(m.shape)).sum(axis=axis, dtype=np.float64).reshape(-1)
                got = _host(_b().reduce_view(d, _meta_pair(m), axis, op))[: want.size]
                if op in (O.MAX, O.MIN):
                    assert got.tobytes() == want.tobytes(), (m, axis, op)
                else:
                    s_ = scale if op == O.SUM else scale / cnt
                    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
                    assert np.all(err <= _sum_tol(cnt) * s_ + 1e-30), (m, axis, op, err.max())


def test_reduce_view_large_strided_outer_is_in_place():
    """A (4096, 4096) window of a (4096, 8192) matrix and its transpose: reduced without a copy
    (no allocation from the context allocator is needed for these layouts)."""
    from rtensors_b200.meta import Meta
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    big = torch.randn(4096 * 8192, device="cuda", generator=g)
    win = Meta.contiguous((4096, 8192)).slice(1, 1024, 5120, 1)
    ref = big.view(4096, 8192)[:, 1024:5120]
    got = _b().reduce_view(big, win, 1, O.SUM).view(4096)
    assert torch.allclose(got, ref.sum(dim=1), rtol=1e-4, atol=1e-3)
    got = _b().reduce_view(big, win, 0, O.MAX).view(4096)
    assert torch.equal(got, ref.max(dim=0).values)
    t = win.permute((1, 0))
    got = _b().reduce_view(big, t, 1, O.MIN).view(4096)  # reduce along the strided dim of the transpose
    assert torch.equal(got, ref.min(dim=0).values)
    got = _b().reduce_view(big, t, 0, O.SUM).view(4096)
    assert torch.allclose(got, ref.sum(dim=1), rtol=1e-4, atol=1e-3)


# ------------------------------------------------------------------------------------- fused broadcast + reduce
def test_broadcast_reduce_matches_materialise_then_reduce():
    rng = np.random.default_rng(5150)
    cases = [((4096, 1), (1, 4096), 1), ((4096, 1), (1, 4096), 0), ((33, 1, 17), (1, 300, 17), 1), ((33, 1, 17), (1, 300, 1), 2),
             ((8, 40, 64), (40, 64), 0), ((8, 40, 64), (8, 1, 64), 1), ((5, 6, 7, 8), (6, 1, 8), 2), ((1000,), (1000,), 0),
             ((16, 512), (512,), 1), ((2, 1000, 40), (1000, 1), 1)]
    for sha, shb, axis in cases:
        a = rng.uniform(-1, 1, int(np.prod(sha))).astype(np.float32)
        b = rng.uniform(0.5, 1.5, int(np.prod(shb))).astype(np.float32)
        am, bm = O.Meta.contiguous(sha), O.Meta.contiguous(shb)
        for binop in (O.ADD, O.MUL, O.SUB, O.DIV):
            full, fm = O.binary(a, am, b, bm, binop)
            for redop in (O.SUM, O.MAX, O.MEAN, O.MIN):
                if fm.rank == 1:
                    want = O.reduce_flat(full, 0, full.size, redop)
                else:
                    want, _ = O.reduce_axis(full, fm, axis, redop)
                got, om = _b().broadcast_reduce(_dev(a), _meta_pair(am), _dev(b), _meta_pair(bm), binop, axis, redop)
                g = _host(got)[: want.size]
                if redop in (O.MAX, O.MIN):
                    assert g.tobytes() == want.tobytes(), (sha, shb, axis, binop, redop)
                else:
                    cnt = fm.shape[axis]
                    scale = np.abs(full.reshape(fm.shape)).sum(axis=axis, dtype=np.float64).reshape(-1)
                    if redop == O.MEAN:
                        scale = scale / cnt
                    err = np.abs(g.astype(np.float64) - want.astype(np.float64))
                    assert np.all(err <= _sum_tol(cnt) * scale + 1e-30), (sha, shb, axis, binop, redop, err.max())
    # f64 through the same kernels (2-element vectors), k-contiguous and wide layouts
    for sha, shb, axis in (((64, 1), (1, 1024), 1), ((64, 1), (1, 1024), 0), ((3, 256, 40), (256, 1), 1)):
        a = rng.uniform(-1, 1, int(np.prod(sha)))
        b = rng.uniform(0.5, 1.5, int(np.prod(shb)))
        am, bm = O.Meta.contiguous(sha), O.Meta.contiguous(shb)
        full, fm = O.binary(a, am, b, bm, O.MUL)
        for redop in (O.SUM, O.MEAN, O.MAX):
            want, _ = O.reduce_axis(full, fm, axis, redop)
            got, _ = _b().broadcast_reduce(_dev(a), _meta_pair(am), _dev(b), _meta_pair(bm), O.MUL, axis, redop)
            assert np.allclose(_host(got)[: want.size], want, rtol=1e-12, atol=1e-12), (sha, shb, axis, redop)
    # strided / reversed operand views that collapse per group, and one that does not (fallback)
    a = rng.uniform(-1, 1, 64 * 48).astype(np.float32)
    b = rng.uniform(-1, 1, 48).astype(np.float32)
    for am in (O.Meta.contiguous((64, 48)).slice(0, None, None, -2), O.Meta.contiguous((64, 48)).slice(1, None, None, -1),
               O.Meta.contiguous((4, 16, 48)).slice(1, 0, 16, 3).slice(0, None, None, -1)):
        bm = O.Meta.contiguous((48,))
        full, fm = O.binary(a, am, b, bm, O.ADD)
        for axis in range(fm.rank):
            want, _ = O.reduce_axis(full, fm, axis, O.SUM)
            got, _ = _b().broadcast_reduce(_dev(a), _meta_pair(am), _dev(b), _meta_pair(bm), O.ADD, axis, O.SUM)
            assert np.allclose(_host(got)[: want.size], want, rtol=1e-5, atol=1e-5)


# ------------------------------------------------------------------------------------- variance / std / norm / logsumexp / argmax
_EXT_LAYOUTS = [(1, 1, 1), (2, 1, 50), (1, 1000003, 1), (7, 5000, 1), (300, 37, 1), (64, 9000, 1), (5, 333, 64), (3, 1000, 33),
                (1, 4096, 256), (40, 10, 1), (1, 70000, 8)]


def _ext_truth(x64, code, unbiased, is_std, norm_type):
    """f64 ground truth over axis 1 of a (outer, R, inner) array."""
    if code == O.VARIANCE:
        n = x64.shape[1]
        ddof = 1 if unbiased else 0
        v = x64.var(axis=1, ddof=ddof) if n - ddof > 0 else np.zeros((x64.shape[0], x64.shape[2]))
        return np.sqrt(v) if is_std else v
    if code == O.NORM:
        return np.abs(x64).sum(axis=1) if norm_type == 1 else np.sqrt((x64 * x64).sum(axis=1))
    m = x64.max(axis=1, keepdims=True)
    return (m + np.log(np.exp(x64 - m).sum(axis=1, keepdims=True)))[:, 0, :]


@pytest.mark.parametrize("dt", [np.float32, np.float64], ids=["f32", "f64"])
@pytest.mark.parametrize("outer,r,inner", _EXT_LAYOUTS)
def test_ext_reductions_match_oracle_and_f64_truth(dt, outer, r, inner):
    rng = np.random.default_rng(outer * 1315423911 % (1 << 31) + r * 7 + inner)
    off = 3  # an odd start: rows are not 16-byte aligned
    n = outer * r * inner
    buf = (rng.standard_normal(n + off) * 1.5 + 0.5).astype(dt)
    x = buf[off:]
    x64 = x.astype(np.float64).reshape(outer, r, inner)
    d = _dev(buf)
    from rtensors_b200.meta import Meta
    meta = Meta((outer, r, inner), (r * inner, inner, 1), off)
    eps = 1e-5 if dt == np.float32 else 1e-13
    tol = eps * max(math.log2(max(r, 2)), 1.0)
    for code, unbiased, is_std, norm_type in [(O.VARIANCE, True, False, 2), (O.VARIANCE, False, False, 2),
                                              (O.VARIANCE, True, True, 2), (O.VARIANCE, False, True, 2),
                                              (O.LOGSUMEXP, True, False, 2), (O.NORM, True, False, 1), (O.NORM, True, False, 2)]:
        out = _b().alloc(outer * inner, d.dtype)
        _b().apply_reduce_ex((d, meta), out, 1, code, unbiased, is_std, norm_type)
        got = _host(out).astype(np.float64).reshape(outer, inner)
        truth = _ext_truth(x64, code, unbiased, is_std, norm_type)
        scale = np.maximum(np.abs(truth), 1e-30)
        assert np.all(np.abs(got - truth) <= tol * scale + 1e-300), (code, unbiased, is_std, norm_type,
                                                                     float(np.max(np.abs(got - truth) / scale)))
        if r <= 70000:  # the sequential oracle itself drifts from the truth on longer runs
            want = O.reduce_ext_ori(x, outer, r, inner, code, unbiased, is_std, norm_type).astype(np.float64).reshape(outer, inner)
            otol = tol if dt == np.float64 or r <= 10000 else 20 * tol
            assert np.all(np.abs(got - want) <= otol * scale + 1e-300), (code, unbiased, is_std, norm_type)
    # positions: exact, also with many equal values (first position wins)
    for data in (buf, np.round(buf * 2).astype(dt)):
        dd = _dev(data)
        for code in (O.ARGMAX, O.ARGMIN):
            out = _b().alloc(outer * inner, torch.int64)
            _b().apply_reduce_ex((dd, meta), out, 1, code)
            want = O.argreduce_ori(data[off:], outer, r, inner, code)
            assert np.array_equal(_host(out).view(np.uint64), want), (code,)


@pytest.mark.parametrize("dt", [np.float32, np.float64], ids=["f32", "f64"])
@pytest.mark.parametrize("outer,r,inner,pitch", [(1, 4096, 1024, 1024), (2, 1000, 1156, 1156), (1, 257, 2048, 2048), (3, 300, 1024, 1024),
                                                 (1, 2048, 512, 1024), (1, 4099, 3072, 4096), (5, 67, 640, 640),
                                                 # rows of at least eight strips: the side-by-side form -- a ragged last strip, idle
                                                 # warps in the last group, chunk counts that fill the resident CTAs twice over,
                                                 # and enough (outer, group) items that nothing is chunked
                                                 (2, 513, 1924, 1924), (1, 130, 1792, 2048), (64, 515, 1024, 1024), (600, 128, 1024, 1024)])
def test_state_merging_column_reductions_on_aligned_rows(dt, outer, r, inner, pitch):
    """Few column tiles and 16-byte aligned rows -- the chunked one-wave regime of the vector column
    kernel (software-pipelined for variance and positions): ragged chunks, a ragged last tile, rows
    with a pitch.  Every op against the f64 truth, positions exact."""
    from rtensors_b200.meta import Meta
    be = _b()
    rng = np.random.default_rng(outer * 100003 + r * 17 + inner)
    buf = (rng.standard_normal(outer * r * pitch) * 1.5 + 0.5).astype(dt)
    x = buf.reshape(outer, r, pitch)[:, :, :inner]
    x64 = x.astype(np.float64)
    d = _dev(buf)
    meta = Meta((outer, r, inner), (r * pitch, pitch, 1), 0)
    eps = 1e-5 if dt == np.float32 else 1e-13
    tol = eps * math.log2(r)
    for code, unbiased, is_std, norm_type in [(O.VARIANCE, True, False, 2), (O.VARIANCE, False, True, 2), (O.LOGSUMEXP, True, False, 2),
                                              (O.NORM, True, False, 1), (O.NORM, True, False, 2)]:
        got = _host(be.reduce_view_ex(d, meta, 1, code, unbiased, is_std, norm_type)).astype(np.float64).reshape(outer, inner)
        truth = _ext_truth(x64, code, unbiased, is_std, norm_type)
        assert np.all(np.abs(got - truth) <= tol * np.maximum(np.abs(truth), 1e-30)), (code, unbiased, is_std, norm_type)
    dense = np.ascontiguousarray(x)
    for data in (dense, np.round(dense * 2).astype(dt)):
        wide = np.zeros((outer, r, pitch), dtype=dt)
        wide[:, :, :inner] = data
        dd = _dev(wide.reshape(-1))
        for code in (O.ARGMAX, O.ARGMIN):
            got = _host(be.reduce_view_ex(dd, meta, 1, code)).view(np.uint64)
            assert np.array_equal(got, O.argreduce_ori(data.reshape(-1), outer, r, inner, code)), code


def test_ext_reductions_flat_rank1_and_edge_values():
    from rtensors_b200.meta import Meta
    b = _b()
    x = np.array([3.0, -1.0, 3.0, 7.5, 7.5, -2.0], dtype=np.float32)
    d = _dev(x)
    m = Meta((6,), (1,), 0)
    for code, args, want in [(O.VARIANCE, (True, False, 2), np.var(x.astype(np.float64), ddof=1)),
                             (O.NORM, (True, False, 1), 24.0), (O.LOGSUMEXP, (True, False, 2), None)]:
        out = b.alloc(1, torch.float32)
        b.apply_reduce_ex((d, m), out, 0, code, *args)
        ref = O.reduce_ext_ori(x, 1, 6, 1, code, *args)[0]
        assert abs(float(_host(out)[0]) - float(ref)) <= 1e-6 * abs(float(ref))
        if want is not None:
            assert abs(float(_host(out)[0]) - want) <= 1e-6 * abs(want)
    for code, want in ((O.ARGMAX, 3), (O.ARGMIN, 5)):
        out = b.alloc(1, torch.int64)
        b.apply_reduce_ex((d, m), out, 0, code)
        assert int(_host(out)[0]) == want
    # one element: variance 0 (both denominators), std 0; logsumexp = the element; argmax 0
    one = _dev(np.array([4.25], dtype=np.float64))
    m1 = Meta((1,), (1,), 0)
    for args in ((True, False, 2), (False, False, 2), (True, True, 2)):
        out = b.alloc(1, torch.float64)
        b.apply_reduce_ex((one, m1), out, 0, O.VARIANCE, *args)
        assert float(_host(out)[0]) == 0.0
    out = b.alloc(1, torch.float64)
    b.apply_reduce_ex((one, m1), out, 0, O.LOGSUMEXP)
    assert float(_host(out)[0]) == 4.25
    # nothing compares above lowest(): position 0, as in the reference kernel
    ninf = _dev(np.full(70, -np.inf, dtype=np.float32))
    out = b.alloc(1, torch.int64)
    b.apply_reduce_ex((ninf, Meta((70,), (1,), 0)), out, 0, O.ARGMAX)
    assert int(_host(out)[0]) == 0
    # unknown norm type and unknown code are refused
    out = b.alloc(1, torch.float32)
    with pytest.raises(Exception):
        b.apply_reduce_ex((d, m), out, 0, O.NORM, True, False, 3)
    with pytest.raises(Exception):
        b.apply_reduce_ex((d, m), out, 0, 11)


def test_ext_reductions_over_views_and_tensor_api():
    import rtensors_b200 as rt
    from rtensors_b200.meta import Meta
    rng = np.random.default_rng(77)
    S = 96
    buf = rng.standard_normal(S * S).astype(np.float32)
    d = _dev(buf)
    full = O.Meta.contiguous((S, S))
    views = [full.slice(1, 8, 72, 1),                      # window: rows with a pitch
             full.permute((1, 0)),                         # transposed
             full.slice(0, None, None, -1),                # rows reversed
             full.slice(1, None, None, 2),                 # strided inner: copy fallback
             O.Meta.contiguous((S * S,)).slice(0, None, None, -1)]  # reversed flat run
    for vm in views:
        dense = gather_view(buf, vm).reshape(vm.shape)
        for axis in [None] + list(range(len(vm.shape))):
            for code, args in [(O.VARIANCE, (True, True, 2)), (O.LOGSUMEXP, (True, False, 2)), (O.NORM, (True, False, 2)),
                               (O.ARGMAX, (True, False, 2)), (O.ARGMIN, (True, False, 2))]:
                got = _host(_b().reduce_view_ex(d, _meta_pair(vm), axis, code, *args))
                if axis is None:
                    outer, r, inner = 1, dense.size, 1
                else:
                    outer = int(np.prod(dense.shape[:axis], dtype=np.int64))
                    r, inner = dense.shape[axis], int(np.prod(dense.shape[axis + 1:], dtype=np.int64))
                flat = np.ascontiguousarray(dense).reshape(-1)
                if code >= O.ARGMAX:
                    want = O.argreduce_ori(flat, outer, r, inner, code)
                    assert np.array_equal(got.view(np.uint64)[: want.size], want), (vm, axis, code)
                else:
                    want = O.reduce_ext_ori(flat, outer, r, inner, code, *args)
                    assert np.allclose(got[: want.size], want, rtol=2e-4, atol=1e-6), (vm, axis, code)
    # Tensor front end: names and result shapes of ReductionOp / TotalReductionOp
    t = rt.Tensor.from_buf([1., 2., 3., 4., 5., 6., 7., 8.], (4, 2), np.float64, _b())
    assert t.var_at(0).shape == (1, 2) and np.allclose(t.var_at(0).cpu().reshape(-1), [6.666666666666667] * 2)
    assert np.allclose(t.pop_var_at(0).cpu().reshape(-1), [5., 5.])
    assert np.allclose(t.std_at(0, False).cpu().reshape(-1), [2.23606797749979] * 2)
    assert np.allclose(t.logsumexp_at(0).cpu().reshape(-1), [7.145077938960783, 8.145077938960782])
    assert np.allclose(t.l1_norm_at(0).cpu().reshape(-1), [16., 20.])
    assert np.allclose(t.l2_norm_at(1).cpu().reshape(-1), np.sqrt([5., 25., 61., 113.]))
    assert float(t.var().cpu().reshape(-1)[0]) == 6.0 and abs(float(t.std(False).cpu().reshape(-1)[0]) - 2.29128784747792) < 1e-14
    assert int(t.argmax().cpu().reshape(-1)[0]) == 7 and int(t.argmin().cpu().reshape(-1)[0]) == 0
    assert t.argmax_at(1).shape == (4, 1) and t.argmax_at(1).cpu().reshape(-1).tolist() == [1, 1, 1, 1]


# ------------------------------------------------------------------------------------- CUDA graphs
def test_a_chain_of_library_calls_replays_from_a_cuda_graph():
    """After one eager pass (workspace and allocator blocks exist), a chain of calls -- broadcast add,
    in-place scalar op and relu, axis sum over a view, variance, fused broadcast+reduce -- is captured
    into a CUDA graph on a side stream and replayed on new input values; results equal the eager ones
    bit for bit (the kernels, their order and their partial-sum trees are the same)."""
    from rtensors_b200 import _lib as L
    from rtensors_b200._lib import check, lib
    from rtensors_b200.meta import Meta, broadcast_params
    be = _b()
    rng = np.random.default_rng(31337)
    rows, cols = 512, 1024
    am, bm = Meta.contiguous((rows, 1)), Meta.contiguous((1, cols))
    shape, sa, sb = broadcast_params(am, bm)
    dm = Meta.contiguous(shape)
    a = _dev(rng.uniform(-1, 1, rows).astype(np.float32))
    b = _dev(rng.uniform(-1, 1, cols).astype(np.float32))
    out = be.alloc(rows * cols, torch.float32)
    colsum = be.alloc(cols, torch.float32)
    rowvar = be.alloc(rows, torch.float32)
    fused = be.alloc(rows, torch.float32)
    win = dm.slice(1, 128, 896, 1)          # a strided window of the result
    winsum = be.alloc(rows, torch.float32)

    def chain():
        be.broadcast((a, Meta(shape, sa, 0)), (b, Meta(shape, sb, 0)), (out, dm), L.ADD)
        be.scalar_apply(out, L.MUL, 1.5, dm)
        be.apply_unary(out, L.RELU, dm)
        be.apply_reduce((out, dm), colsum, 0, L.SUM)
        be.apply_reduce_ex((out, dm), rowvar, 1, L.VARIANCE)
        check(lib().rtb_reduce_view(be._ctx, C.c_int(L.F32), C.c_int(L.SUM), be._p(out), C.c_size_t(win.rank), win.c_shape,
                                    win.c_strides, C.c_size_t(win.offset), C.c_ssize_t(1), be._p(winsum)))
        check(lib().rtb_broadcast_reduce(be._ctx, C.c_int(L.F32), C.c_int(L.ADD), C.c_int(L.SUM), be._p(a), L.diffs(sa), C.c_size_t(0),
                                         be._p(b), L.diffs(sb), C.c_size_t(0), C.c_size_t(2), L.sizes(shape), C.c_size_t(1),
                                         be._p(fused)))

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        be.sync_stream()
        chain()                               # eager pass: sizes the workspace, fills the allocator cache
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            be.sync_stream()
            chain()
        # new inputs, replay, then the same chain eagerly on the same inputs
        a.copy_(torch.from_numpy(rng.uniform(-1, 1, rows).astype(np.float32)))
        b.copy_(torch.from_numpy(rng.uniform(-1, 1, cols).astype(np.float32)))
        side.synchronize()
        launches_before = be.launches
        graph.replay()
        side.synchronize()
        assert be.launches == launches_before   # a replay goes through no library entry point
        replayed = [t.clone() for t in (out, colsum, rowvar, winsum, fused)]
        be.sync_stream()
        chain()
        side.synchronize()
        for r, e in zip(replayed, (out, colsum, rowvar, winsum, fused)):
            assert _host(r).tobytes() == _host(e).tobytes()
    torch.cuda.current_stream().wait_stream(side)
    be.sync_stream()
    # and the values are right
    want = np.maximum((_host(a)[:, None] + _host(b)[None, :]) * np.float32(1.5), 0).astype(np.float32)
    assert _host(out).tobytes() == want.reshape(-1).tobytes()
    assert np.allclose(_host(fused), (_host(a)[:, None] + _host(b)[None, :]).sum(axis=1), rtol=1e-5, atol=1e-4)


# ------------------------------------------------------------------------------------- config 4 at full size
def test_config4_reductions_at_full_size():
    """normal(0,1) data at the benchmark's own sizes: (8192,8192) x {sum, mean, max, min} x axis {0,1},
    (64,4096,1024) x 4 ops x axis 1, the flat sum of 2^30 and mean_l1_loss of two (4096,4096), each
    against the CPU oracle on the same values (the device draws them, the host gets a copy), plus the
    size-independent properties: max / min of the axis results equal the full max / min exactly, and
    the axis sums add up to the full sum."""
    b = _b()
    g = torch.Generator(device="cuda")
    g.manual_seed(0x5EED + 4)
    big = torch.randn(1 << 30, device="cuda", generator=g)
    host = big.cpu().numpy()

    def check_axis(outer, r, inner, axes_label):
        n = outer * r * inner
        x = host[:n]
        absum = np.abs(x.reshape(outer, r, inner)).sum(axis=1, dtype=np.float64).reshape(-1)
        res = {}
        for op in (O.SUM, O.MEAN, O.MAX, O.MIN):
            want = O.reduce_ori(x, outer, r, inner, op, fast=True)
            got = _host(b.reduce_axis_ori(big, 0, outer, r, inner, op))[: outer * inner]
            res[op] = got
            if op in (O.MAX, O.MIN):
                assert got.tobytes() == want.tobytes(), (axes_label, op)
            else:
                scale = absum if op == O.SUM else absum / r
                err = np.abs(got.astype(np.float64) - want.astype(np.float64))
                assert np.all(err <= _sum_tol(r) * scale + 1e-30), (axes_label, op, err.max())
        return res

    S = 8192
    r0 = check_axis(1, S, S, "8192^2 axis 0")
    r1 = check_axis(S, S, 1, "8192^2 axis 1")
    x2 = host[: S * S]
    assert r0[O.MAX].max() == r1[O.MAX].max() == x2.max() and r0[O.MIN].min() == r1[O.MIN].min() == x2.min()
    total64 = float(x2.sum(dtype=np.float64))
    tol = _sum_tol(S * S) * float(np.abs(x2).sum(dtype=np.float64))
    assert abs(float(r0[O.SUM].sum(dtype=np.float64)) - total64) <= tol and abs(float(r1[O.SUM].sum(dtype=np.float64)) - total64) <= tol
    check_axis(64, 4096, 1024, "(64,4096,1024) axis 1")

    # flat sum of 2^30: against the oracle's sequential f32 accumulator (backward-error bound) and the f64 truth
    out = b.alloc(1, torch.float32)
    b.apply_reduce_contiguous_flat(big, out, 0, 1 << 30, O.SUM)
    got = float(_host(out)[0])
    want = float(O.reduce_flat(host, 0, 1 << 30, O.SUM, fast=True)[0])
    abs_total = float(np.abs(host).sum(dtype=np.float64))
    truth = float(host.sum(dtype=np.float64))
    assert abs(got - want) <= _sum_tol(1 << 30) * abs_total
    assert abs(got - truth) <= abs(want - truth) + 1e-6 * abs_total  # the tree sum is at least as close to the truth
    for op in (O.MAX, O.MIN):
        b.apply_reduce_contiguous_flat(big, out, 0, 1 << 30, op)
        assert _host(out).tobytes() == O.reduce_flat(host, 0, 1 << 30, op, fast=True).tobytes()

    # mean_l1_loss of two (4096,4096)
    n = 4096 * 4096
    loss, gmap = b.l1_loss(big[:n], big[n: 2 * n], 0, True)
    wl, wg = O.l1_loss(host[:n], host[n: 2 * n], 0, True, fast=True)
    # 2^24 positive terms of about 1.1: the CPU backend's single f32 accumulator stalls once the sum
    # passes 2^24 (its result here is about 2 % low), so the bound is taken against the f64 truth and
    # the oracle value only has to be no closer to it than the device value
    truth = float(np.abs(host[:n].astype(np.float64) - host[n: 2 * n].astype(np.float64)).sum()) / n
    got = float(_host(loss)[0])
    assert abs(got - truth) <= _sum_tol(n) * truth
    assert abs(got - truth) <= abs(float(wl[0]) - truth) + 1e-7
    assert _host(gmap).tobytes() == wg.tobytes()


L_MUL, L_SUB = O.MUL, O.SUB  # the library's op codes are the oracle's


def test_long_chain_of_dependent_small_kernels_keeps_stream_order():
    """300 kernels back to back, each consuming what the previous one wrote (scalar ops on the whole
    buffer and on strided windows, a broadcast add of a reduced vector, reductions into a vector
    that is read again): with dependent launches every kernel starts before its predecessor has
    finished, so any access ahead of the wait would show up as a wrong value here."""
    from rtensors_b200.meta import Meta
    be = _b()
    rng = np.random.default_rng(2024)
    rows, cols = 96, 512
    x = rng.uniform(0.5, 1.5, rows * cols).astype(np.float32)
    ref = x.copy()
    d = _dev(x)
    full = Meta.contiguous((rows, cols))
    win = full.slice(0, None, None, 2).slice(1, 64, 448, 1)
    owin = O.Meta.contiguous((rows, cols)).slice(0, None, None, 2).slice(1, 64, 448, 1)
    ofull = O.Meta.contiguous((rows, cols))
    colmax = be.alloc(cols, torch.float32)
    for it in range(60):
        be.scalar_apply(d, L_MUL, 1.01, full)
        O.scalar_op(ref, O.MUL, 1.01, ofull)
        be.scalar_apply(d, L_SUB, 0.005, win)
        O.scalar_op(ref, O.SUB, 0.005, owin)
        be.apply_reduce((d, full), colmax, 0, O.MAX)
        cm, _ = O.reduce_axis(ref, ofull, 0, O.MAX)
        # x -= 0.01 * colmax, broadcast over the rows
        be.scalar_apply(colmax, L_MUL, 0.01, Meta.contiguous((cols,)))
        cm = cm.copy()
        O.scalar_op(cm, O.MUL, 0.01, O.Meta.contiguous((cols,)))
        be.binary_assign(d, full, colmax, Meta.contiguous((1, cols)), L_SUB)
        sh, sa, sb = O.broadcast_params(ofull, O.Meta.contiguous((1, cols)))
        O.broadcast(ref, O.Meta(sh, sa, 0), cm, O.Meta(sh, sb, 0), ref, O.Meta(sh, sa, 0), O.SUB)
    assert _host(d).tobytes() == ref.tobytes()



# ------------------------------------------------------------------------------------- dtype conversion
@pytest.mark.parametrize("src", list(range(13)), ids=lambda c: __import__("convert_cases").NAMES[c])
def test_convert_all_pairs_edge_values(src):
    """Every (src, dst) pair on edge values + seeded random ones, bit-exact with the oracle (any NaN
    matches any NaN).  Element counts are not a multiple of the per-thread pack, so the tail runs too."""
    from convert_cases import ALL_CODES, NAMES, decode, encode, same, samples
    rng = np.random.default_rng(2000 + src)
    raw = encode(src, samples(src, rng))
    d = _dev(np.frombuffer(raw, dtype=np.uint8).copy())
    for dst in ALL_CODES:
        got = _host(_b().convert_raw(d, src, dst)).tobytes()[: (len(raw) // O.DTYPE_SIZE[src]) * O.DTYPE_SIZE[dst]]
        want = O.convert(raw, src, dst)
        assert same(dst, decode(dst, got), decode(dst, want)), (NAMES[src], NAMES[dst])


@pytest.mark.parametrize("src,dst", [(np.float32, np.int32), (np.float32, np.float64), (np.uint8, np.float32),
                                     (np.float64, np.float32), (np.int64, np.float32), (np.float32, np.uint8),
                                     (np.int32, np.int8), (np.float32, np.bool_), (np.bool_, np.float64)])
@pytest.mark.parametrize("n", [1, 17, 4096, (1 << 20) + 13])
def test_convert_bulk_matches_oracle(src, dst, n):
    rng = np.random.default_rng(n + np.dtype(src).itemsize)
    if np.dtype(src).kind == "f":
        a = (rng.standard_normal(n) * 10.0 ** rng.integers(-2, 12, n)).astype(src)
    else:
        a = _rand(rng, n, src)
    got = _host(_b().convert(_dev(a), _b_torch(dst)))[:n]
    want = np.frombuffer(O.convert(a.tobytes(), O.NP_TO_CODE[np.dtype(src)], O.NP_TO_CODE[np.dtype(dst)]), dtype=dst)
    assert got.tobytes() == want.tobytes()


def _b_torch(npdt):
    from rtensors_b200.tensor import _NP_TO_TORCH
    return _NP_TO_TORCH[np.dtype(npdt)]


def test_convert_unaligned_views_and_errors():
    """Buffers that are element-aligned but not pack-aligned take the per-element path; a buffer
    that is not element-aligned, or an unknown dtype, is refused."""
    import rtensors_b200 as rt
    lib, ctx = rt.lib(), _b()._ctx
    rng = np.random.default_rng(77)
    a = (rng.standard_normal(1001) * 1000).astype(np.float32)
    d = _dev(np.concatenate([np.zeros(1, np.float32), a]))
    out = _b().alloc(1003, torch.int16)
    rc = lib.rtb_convert(ctx, C.c_int(O.F32), C.c_int(O.I16), C.c_void_p(d.data_ptr() + 4), C.c_void_p(out.data_ptr() + 2),
                         C.c_size_t(1001))
    assert rc == 0
    want = np.frombuffer(O.convert(a.tobytes(), O.F32, O.I16), dtype=np.int16)
    assert _host(out)[1:1002].tobytes() == want.tobytes()
    assert lib.rtb_convert(ctx, C.c_int(O.F32), C.c_int(O.I16), C.c_void_p(d.data_ptr() + 2), C.c_void_p(out.data_ptr()),
                           C.c_size_t(8)) != 0
    assert lib.rtb_convert(ctx, C.c_int(13), C.c_int(O.I16), C.c_void_p(d.data_ptr()), C.c_void_p(out.data_ptr()),
                           C.c_size_t(8)) != 0
    assert lib.rtb_convert(ctx, C.c_int(O.F32), C.c_int(O.I16), None, None, C.c_size_t(0)) == 0


def test_tensor_into_dtype_keeps_the_view():
    """into_dtype converts the whole buffer and clones the meta (core/primitives.rs:527-538), so a
    strided view stays the same view of the converted buffer."""
    from rtensors_b200.tensor import Tensor
    t = Tensor.from_buf([1.7, -2.2, 3.0, 2.5, -0.4, 300.2], (2, 3), np.float32, _b())
    assert t.into_dtype(np.int64).cpu().tolist() == [[2, -2, 3], [3, 0, 300]]
    assert t.into_dtype(np.bool_).cpu().tolist() == [[True, True, True], [True, True, True]]
    v = t.permute((1, 0)).slice(0, None, None, -1)
    assert v.into_dtype(np.uint8).cpu().tolist() == [[3, 255], [0, 0], [2, 3]]


def test_buffer_level_trait_methods():
    """copy / copy_from_slice / copy_range_within / read / write / len with the CPU backend's checks
    (backend/cpu.rs:151-207)."""
    import rtensors_b200._lib as L
    be = _b()
    a = _dev(np.arange(1, 7, dtype=np.int32))
    b = be.alloc(6, torch.int32)
    be.copy_from_slice(b, np.array([10, 20, 30, 40, 50, 60], dtype=np.int32))
    be.copy_range_within(b, a, 1, 3, 2)
    assert _host(b).tolist() == [10, 4, 5, 40, 50, 60]
    assert be.len(b) == 6 and be.read(b, 2) == 5
    be.write(b, 5, 7)
    assert be.read(b, 5) == 7
    c = be.copy(b)
    be.write(b, 0, -1)
    assert _host(c).tolist() == [10, 4, 5, 40, 50, 7]
    for bad, code in ((lambda: be.read(b, 6), L.ERR_BOUNDS), (lambda: be.write(b, 6, 1), L.ERR_BOUNDS),
                      (lambda: be.copy_range_within(b, a, 5, 0, 2), L.ERR_BOUNDS),
                      (lambda: be.copy_from_slice(b, np.zeros(1, np.int32)), L.ERR_SHAPE)):
        with pytest.raises(L.RtbError) as e:
            bad()
        assert e.value.code == code


def test_one_context_called_from_several_host_threads():
    """The reference's `Cuda` is Send + Sync and its launchers are called from any host thread
    (backend/cuda.rs:38-60).  Four threads share one context (one stream, one reduction workspace)
    and interleave elementwise ops, plain and extended reductions and the fused broadcast+reduce on
    buffers of their own; every result must equal what the same calls give alone."""
    import threading
    from rtensors_b200.meta import Meta
    be = _b()
    rng = np.random.default_rng(4242)
    rows, cols = 300, 1030
    data = [rng.standard_normal(rows * cols).astype(np.float32) for _ in range(4)]
    m = Meta.contiguous((rows, cols))

    def work(a, rounds):
        outs = []
        for _ in range(rounds):
            d = _dev(a)
            be.scalar_apply(d, L_MUL, 1.5, m)
            be.apply_unary(d, L_RELU, m)
            outs.append(_host(be.reduce_view(d, m, 0, L_SUM)).copy())
            outs.append(_host(be.reduce_view(d, m, 1, L_MAX)).copy())
            outs.append(_host(be.reduce_view(d, m, None, L_SUM)).copy())
            outs.append(_host(be.reduce_view_ex(d, m, 0, L_VAR)).copy())
            outs.append(_host(be.reduce_view_ex(d, m, 1, L_ARGMAX)).copy())
            col = _dev(a[:rows].copy())
            row = _dev(a[:cols].copy())
            outs.append(_host(be.broadcast_reduce(col, Meta.contiguous((rows, 1)), row, Meta.contiguous((1, cols)), 0, 0, L_SUM)[0]).copy())
        return outs

    alone = [work(a, 1) for a in data]
    got = [None] * 4
    errs = []

    def run(k):
        try:
            got[k] = work(data[k], 6)
        except Exception as e:  # pragma: no cover
            errs.append(e)

    ts = [threading.Thread(target=run, args=(k,)) for k in range(4)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errs, errs
    for k in range(4):
        n = len(alone[k])
        for j, o in enumerate(got[k]):
            assert o.tobytes() == alone[k][j % n].tobytes(), (k, j)


import rtensors_b200._lib as _L  # noqa: E402
L_MUL, L_RELU, L_SUM, L_MAX, L_VAR, L_ARGMAX = _L.MUL, _L.RELU, _L.SUM, _L.MAX, _L.VARIANCE, _L.ARGMAX


@pytest.mark.parametrize("dt", NP_DTYPES, ids=lambda d: np.dtype(d).name)
def test_relu_and_abs_gradient_maps_on_views(dt):
    """rtb_grad_mask (relu, abs, leaky_relu maps and the reciprocal) against the oracle on a contiguous
    tensor, a strided / reversed window and a permuted view, every dtype; abs needs a signed type and the
    reciprocal a non-boolean one, refused otherwise.  Integer buffers hold zeros: 1 / 0 gives 0."""
    import rtensors_b200._lib as L
    rng = np.random.default_rng(31 + np.dtype(dt).itemsize)
    buf = _rand(rng, 6 * 40 * 50 + 7, dt)
    if np.dtype(dt).kind == "f":
        buf[::11] = 0
        buf[5] = np.nan
    base = O.Meta.contiguous((6, 40, 50))
    views = [base, O.Meta((6, 40, 50), base.strides, 7), base.slice(1, 3, 37, 2).slice(2, None, None, -1),
             base.permute((2, 0, 1)), base.slice(0, 1, 2, 1).squeeze()]
    d = _dev(buf)
    signed = np.dtype(dt).kind in "fi"
    is_bool = np.dtype(dt).kind == "b"
    slope = True if is_bool else (0.125 if np.dtype(dt).kind == "f" else 3)
    for m in views:
        for kind in (L.MASK_RELU, L.MASK_ABS, L.MASK_LEAKY_RELU, L.MASK_RECIPROCAL):
            value = slope if kind == L.MASK_LEAKY_RELU else None
            if (kind == L.MASK_ABS and not signed) or (kind == L.MASK_RECIPROCAL and is_bool):
                with pytest.raises(L.RtbError):
                    _b().grad_mask(d, _meta_pair(m), kind, value)
                with pytest.raises(O.OracleError):
                    O.grad_mask(buf, kind, m, value)
                continue
            got = _host(_b().grad_mask(d, _meta_pair(m), kind, value))[: m.size]
            want = O.grad_mask(buf, kind, m, value)
            if kind == L.MASK_RECIPROCAL and np.dtype(dt).kind == "f":
                ok = (got.view(np.uint32 if got.itemsize == 4 else np.uint64) == want.view(np.uint32 if got.itemsize == 4 else np.uint64)) | (np.isnan(got) & np.isnan(want))
                assert ok.all(), (m, kind)
            else:
                assert got.tobytes() == want.tobytes(), (m, kind)


def test_tensor_gradient_maps():
    from rtensors_b200.tensor import Tensor
    t = Tensor.from_buf([-1.0, 0.0, 2.0, 3.0, -0.5, 0.25], (2, 3), np.float32, _b())
    assert t.relu_grad_map().cpu().tolist() == [[0, 0, 1], [1, 0, 1]]
    assert t.abs_grad_map().cpu().tolist() == [[-1, -1, 1], [1, -1, 1]]
    assert t.transpose().relu_grad_map().cpu().tolist() == [[0, 1], [0, 0], [1, 1]]
    assert t.leaky_relu_grad_map(0.125).cpu().tolist() == [[0.125, 0.125, 1], [1, 0.125, 1]]
    assert t.slice(1, 2, 3).reciprocal_map().cpu().tolist() == [[0.5], [4.0]]


@pytest.mark.parametrize("n", [1, 2, 4096 * 33 + 3, 100003])
def test_relu_mask_and_sgd_update_f64(n):
    rng = np.random.default_rng(600 + n)
    x = rng.standard_normal(n)
    x[::9] = 0.0
    ref = x.copy()
    wm = O.relu_mask(ref)
    d = _dev(x)
    m = _b().relu_mask(d)
    assert _host(d).tobytes() == ref.tobytes() and _host(m).tobytes() == wm.tobytes()
    p, g = rng.standard_normal(n), rng.standard_normal(n)
    rp = p.copy()
    O.sgd_update(rp, g, 0.0137)
    dp = _dev(p)
    _b().sgd_update(dp, _dev(g), 0.0137)
    assert _host(dp).tobytes() == rp.tobytes()


# ------------------------------------------------------------------------------------- transposing tiles
@pytest.mark.parametrize("dt", [np.float32, np.float64, np.int8, np.int16, np.uint8, np.bool_, np.int64],
                         ids=lambda d: np.dtype(d).name)
def test_transposed_and_permuted_operands(dt):
    """Views that are strided along the output's inner dim but dense along another one (transposes,
    permuted cubes) -- the transposing tile kernel: contiguous() copies, out-of-place and in-place
    binary ops with one or both operands transposed, ragged tile edges, a broadcast partner, and an
    operand that shares the output's buffer.  Bit-exact against the oracle."""
    rng = np.random.default_rng(515 + np.dtype(dt).itemsize)
    be = _b()
    for shape, perm in [((70, 45), (1, 0)), ((33, 64), (1, 0)), ((5, 40, 50), (2, 0, 1)), ((6, 37, 41), (0, 2, 1)),
                        ((3, 4, 20, 35), (0, 3, 1, 2)), ((17, 130), (1, 0)),
                        # vector-aligned extents and strides: the 16-byte tile kernel (full, ragged and many tiles)
                        ((72, 44), (1, 0)), ((260, 300), (1, 0)), ((8, 40, 132), (2, 0, 1)), ((6, 36, 40), (0, 2, 1)),
                        ((128, 256), (1, 0))]:
        base = O.Meta.contiguous(shape)
        n = base.size
        a, b = _rand(rng, n, dt), _rand(rng, n, dt)
        if np.dtype(dt).kind in "iu":
            a[a == 0] = 1
            b[b == 0] = 1
        va = base.permute(perm)
        da, db = _dev(a), _dev(b)
        # contiguous() of the permuted view
        assert _host(be.contiguous(da, _meta_pair(va)))[:n].tobytes() == gather_view(a, va).tobytes(), (shape, perm)
        dense = O.Meta.contiguous(va.shape)
        ops = (O.ADD, O.MUL) if np.dtype(dt).kind == "b" else (O.ADD, O.SUB, O.MUL, O.DIV)
        for op in ops:
            # a.T (op) b and b (op) a.T, fresh output
            for (x, mx, y, my) in ((a, va, b, dense), (b, dense, a, va), (a, va, b, va)):
                want, wm = O.binary(x, mx, y, my, op)
                got, gm = be.binary(_dev(x), _meta_pair(mx), _dev(y), _meta_pair(my), op)
                assert tuple(gm.shape) == tuple(wm.shape)
                assert _host(got)[: want.size].tobytes() == want.tobytes(), (shape, perm, op)
            # b (op)= a.T in place
            ref = b.copy()
            O.broadcast(ref, dense, a, va, ref, dense, op)
            dd = _dev(b)
            be.binary_assign(dd, _meta_pair(dense), da, _meta_pair(va), op)
            assert _host(dd).tobytes() == ref.tobytes(), (shape, perm, op, "in place")
        # a broadcast partner: a.T + row
        row_m = O.Meta.contiguous((va.shape[-1],))
        row = _rand(rng, va.shape[-1], dt)
        want, _ = O.binary(a, va, row, row_m, O.ADD)
        got, _ = be.binary(da, _meta_pair(va), _dev(row), _meta_pair(row_m), O.ADD)
        assert _host(got)[: want.size].tobytes() == want.tobytes(), (shape, perm, "row")
    # square matrix: a + a.T from the same buffer, fresh output
    m = O.Meta.contiguous((48, 48))
    a = _rand(rng, m.size, dt)
    want, _ = O.binary(a, m, a, m.permute((1, 0)), O.ADD)
    d = _dev(a)
    got, _ = be.binary(d, _meta_pair(m), d, _meta_pair(m.permute((1, 0))), O.ADD)
    assert _host(got)[: want.size].tobytes() == want.tobytes()
