"""This library against the reference's OWN CUDA kernels, recompiled unmodified for sm_100a
(baseline/_ref/libref_cuda.so): a second pin, besides the restated oracle, for the reductions that
only the reference's CUDA backend implements (variance / std, norms, logsumexp, argmax / argmin,
cuda/kernels/reduction/reduce.cu), plus the broadcast add and the plain reductions.  The reference
builds with --use_fast_math, so float results are compared within a tolerance; integer positions and
single IEEE adds are exact.  Contiguous inputs only."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref():
    from baseline import ref_cuda
    if not ref_cuda.available():
        pytest.skip("baseline/_ref/libref_cuda.so has not been built (needs the reference checkout)")
    return ref_cuda


def _b():
    from cuda_engine import backend
    return backend()


@pytest.mark.parametrize("tdt", [torch.float32, torch.float64], ids=["f32", "f64"])
@pytest.mark.parametrize("outer,r,inner", [(1, 600, 64), (5, 300, 1), (3, 1000, 33), (64, 257, 128)])
def test_axis_reductions_match_the_reference_kernels(tdt, outer, r, inner):
    R = _ref()
    from rtensors_b200 import _lib as L
    be = _b()
    g = torch.Generator(device="cuda")
    g.manual_seed(outer * 7 + r)
    x = torch.randn(outer * r * inner, device="cuda", dtype=tdt, generator=g) * 2 + 0.5
    tol = 2e-4 if tdt == torch.float32 else 1e-9
    cases = [(L.SUM, {}), (L.MEAN, {}), (L.MAX, {}), (L.MIN, {}), (L.VARIANCE, dict(unbiased=True)), (L.VARIANCE, dict(unbiased=False)),
             (L.VARIANCE, dict(unbiased=True, is_std=True)), (L.NORM, dict(norm_type=1)), (L.NORM, dict(norm_type=2)), (L.LOGSUMEXP, {})]
    for code, kw in cases:
        want = torch.full((outer * inner,), -7.0, device="cuda", dtype=tdt)
        R.reduce_nd(x, want, 0, outer, r, inner, code, **kw)
        got = be.reduce_ext_ori(x, 0, outer, r, inner, code, kw.get("unbiased", True), kw.get("is_std", False), kw.get("norm_type", 2)) \
            if code >= L.VARIANCE else be.reduce_axis_ori(x, 0, outer, r, inner, code)
        torch.cuda.synchronize()
        if code in (L.MAX, L.MIN):
            assert torch.equal(got, want), code
        else:
            scale = x.abs().view(outer, r, inner).sum(dim=1).reshape(-1).clamp_min(1.0) if code in (L.SUM, L.NORM) else 1.0
            assert torch.all((got - want).abs() <= tol * (want.abs() + scale)), (code, kw)
    # positions: distinct values, so the reference's thread-order tie rule cannot matter
    y = torch.randperm(outer * r * inner, device="cuda", generator=g).to(tdt)
    for code in (L.ARGMAX, L.ARGMIN):
        want = torch.zeros(outer * inner, device="cuda", dtype=torch.int64)
        R.reduce_nd(y, want, 0, outer, r, inner, code)
        got = be.reduce_ext_ori(y, 0, outer, r, inner, code)
        torch.cuda.synchronize()
        assert torch.equal(got, want), code


def test_flat_reductions_and_positions_match_the_reference_kernels():
    R = _ref()
    from rtensors_b200 import _lib as L
    from rtensors_b200.meta import Meta
    be = _b()
    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    n = (1 << 20) + 37
    x = torch.randn(n + 3, device="cuda", generator=g)
    for code in (L.SUM, L.MEAN, L.MAX, L.MIN):
        want = torch.zeros(1, device="cuda")
        got = torch.zeros(1, device="cuda")
        R.reduce_flat(x, want, 3, n, code)
        be.apply_reduce_contiguous_flat(x, got, 3, n, code)
        torch.cuda.synchronize()
        assert not R.alloc_failed()
        if code in (L.MAX, L.MIN):
            assert torch.equal(got, want)
        else:
            assert abs(float(got) - float(want)) <= 1e-5 * 20 * float(x[3:].abs().sum()) / (n if code == L.MEAN else 1)
    y = torch.randperm(n, device="cuda", generator=g).float()
    for code in (L.ARGMAX, L.ARGMIN):
        want = torch.zeros(1, device="cuda", dtype=torch.int64)
        got = torch.zeros(1, device="cuda", dtype=torch.int64)
        R.reduce_flat(y, want, 0, n, code)
        be.apply_reduce_ex((y, Meta.contiguous((n,))), got, 0, code)
        torch.cuda.synchronize()
        assert torch.equal(got, want)


def test_strided_negative_step_broadcast_add_matches_the_reference_kernel_bit_for_bit():
    """Config 3 at 1/64: the reference's generic broadcast kernel takes the same pre-broadcast
    strides (0 on broadcast dims, -1 on the reversed dim) and must give the same bits."""
    R = _ref()
    from rtensors_b200 import _lib as L
    from rtensors_b200.meta import Meta, broadcast_params
    be = _b()
    K = 16
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    bufa = torch.rand(K * 16, device="cuda", generator=g) * 2 - 1
    bufb = torch.rand(64 * 1024, device="cuda", generator=g) * 2 - 1
    Am = Meta.contiguous((K, 16, 1, 1)).view_as((1, K, 16, 1)).permute((2, 0, 1, 3))
    Bm = Meta.contiguous((1, 64, 1, 1024)).slice(3, None, None, -1)
    shape, sa, sb = broadcast_params(Am, Bm)
    dm = Meta.contiguous(shape)
    got = be.alloc(dm.size, torch.float32)
    want = torch.zeros(dm.size, device="cuda")
    lm, rm = Meta(shape, sa, Am.offset), Meta(shape, sb, Bm.offset)
    be.broadcast((bufa, lm), (bufb, rm), (got, dm), L.ADD)
    R.Broadcast(bufa, lm, bufb, rm, want, dm, R.ADD)()
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # scalar chain: the reference's fast-math build still does single IEEE mul / add / sub here
    a = torch.rand(1 << 20, device="cuda", generator=g) * 2 - 1
    b = a.clone()
    m = Meta.contiguous((a.numel(),))
    for name, code, v in (("mul", L.MUL, 3.0), ("add", L.ADD, 2.0), ("sub", L.SUB, 1.0)):
        be.scalar_apply(a, code, v, m)
        R.scalar_contiguous(b, name, v)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
