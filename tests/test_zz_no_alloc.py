"""The allocation-free full reduction (rtb_reduce_flat_noalloc) against the regular entry point.

Collected last on purpose: a run that stops at the first failure has then already exercised every
other test.  Callers of this entry point are hosts that may not call cudaMalloc (all device memory
already in their own pool, or a loop that cannot take the allocator's device-wide synchronisation);
the scratch it uses is a fixed array inside the library, shared by every call on the device and
still holding the previous call's values -- hence two calls in a row on different data here.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SUM, PROD, MAX, MIN, MEAN = 1, 2, 3, 4, 5
F32, F64 = 10, 11
MAX_LEN = 1 << 29


def _lib():
    import rtensors_b200 as rt
    return rt.lib()


def _noalloc(dtype, op, src, start, n, dst):
    stream = torch.cuda.current_stream().cuda_stream
    return _lib().rtb_reduce_flat_noalloc(C.c_int(dtype), C.c_int(op), C.c_void_p(src.data_ptr()), C.c_size_t(start),
                                          C.c_size_t(n), C.c_void_p(dst.data_ptr()), C.c_void_p(stream))


def _regular(ctx, dtype, op, src, start, n, dst):
    return _lib().rtb_reduce_flat(ctx, C.c_int(dtype), C.c_int(op), C.c_void_p(src.data_ptr()), C.c_size_t(start),
                                  C.c_size_t(n), C.c_void_p(dst.data_ptr()))


@pytest.fixture(scope="module")
def ctx():
    torch.cuda.set_device(0)
    c = C.c_void_p()
    assert _lib().rtb_ctx_create(C.c_int(0), C.byref(c)) == 0
    assert _lib().rtb_ctx_set_stream(c, C.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    yield c
    _lib().rtb_ctx_destroy(c)


@pytest.mark.parametrize("tdt,code", [(torch.float32, F32), (torch.float64, F64)], ids=["f32", "f64"])
def test_two_calls_in_a_row_match_the_regular_entry_point(ctx, tdt, code):
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    # first call: many CTAs (fills many scratch slots); second call: fewer CTAs, other data, an
    # unaligned start -- stale slots and a stale counter from the first call must not leak in
    cases = [((1 << 22) + 12345, 0), (200003, 3)]
    for n, start in cases:
        x = torch.randn(n + start + 5, device="cuda", dtype=tdt, generator=g)
        absum = float(x[start:start + n].abs().sum(dtype=torch.float64))
        for op in (SUM, MEAN, MAX, MIN):
            want = torch.zeros(1, device="cuda", dtype=tdt)
            got = torch.full((1,), 7.0, device="cuda", dtype=tdt)
            assert _regular(ctx, code, op, x, start, n, want) == 0
            assert _noalloc(code, op, x, start, n, got) == 0
            torch.cuda.synchronize()
            w, v = float(want.item()), float(got.item())
            if op in (MAX, MIN):
                assert v == w, (op, v, w)
                assert v == float(x[start:start + n].max() if op == MAX else x[start:start + n].min())
            else:
                # both are tree sums over different partitions: the float-sum tolerance of the suite
                eps_scale = 1e-5 if tdt == torch.float32 else 1e-12
                scale = absum if op == SUM else absum / n
                assert abs(v - w) <= eps_scale * math.log2(n) * scale, (op, v, w)


def test_rejects_lengths_beyond_the_builtin_scratch():
    x = torch.zeros(16, device="cuda")
    out = torch.zeros(1, device="cuda")
    rc = _noalloc(F32, SUM, x, 0, MAX_LEN + 1, out)
    assert rc == -10
    msg = _lib().rtb_last_error_string().decode()
    assert "RTB_NOALLOC_MAX_LEN" in msg and "exceeds" in msg
    assert _noalloc(9, SUM, x, 0, 4, out) == -2  # not a float dtype
    assert _noalloc(F32, 77, x, 0, 4, out) == -1  # unknown reduction code
    torch.cuda.synchronize()


def test_no_device_allocation_happens():
    x = torch.randn(1 << 20, device="cuda")
    out = torch.zeros(1, device="cuda")
    assert _noalloc(F32, SUM, x, 0, x.numel(), out) == 0  # set-up call for this device
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        assert _noalloc(F32, SUM, x, 0, x.numel(), out) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert abs(float(out.item()) - float(x.sum(dtype=torch.float64))) <= 1e-5 * 20 * float(x.abs().sum())


@pytest.mark.parametrize("tdt,code", [(torch.float32, F32), (torch.float64, F64)], ids=["f32", "f64"])
@pytest.mark.parametrize("start", [0, 1, 3])
def test_edges_of_the_head_vector_tail_split(ctx, tdt, code, start):
    """Lengths around the kernel's seams: nothing, less than one 16-byte vector behind a misaligned
    start, and one element either side of the 65 536-element boundary between one and two CTAs."""
    g = torch.Generator(device="cuda")
    g.manual_seed(99 + start)
    x = torch.rand(65537 + start + 4, device="cuda", dtype=tdt, generator=g) * 0.5 + 0.75   # products stay finite
    for n in (0, 1, 3, 5, 65535, 65536, 65537):
        for op in (SUM, PROD, MAX, MIN, MEAN):
            if op == PROD and n > 5:
                continue            # 65 536 factors in [0.75, 1.25) under- or overflow; the short runs cover PROD
            want = torch.full((1,), 3.0, device="cuda", dtype=tdt)
            got = torch.full((1,), 7.0, device="cuda", dtype=tdt)
            assert _regular(ctx, code, op, x, start, n, want) == 0
            assert _noalloc(code, op, x, start, n, got) == 0
            torch.cuda.synchronize()
            w, v = float(want.item()), float(got.item())
            if n == 0 and op == MEAN:
                assert math.isnan(v) and math.isnan(w)      # 0 / 0, as the CPU backend's mean of nothing
            elif op in (MAX, MIN) or n <= 1:
                assert v == w, (n, op, v, w)
            else:
                eps_scale = 1e-5 if tdt == torch.float32 else 1e-12
                assert abs(v - w) <= eps_scale * max(math.log2(n), 1.0) * max(abs(w), 1.0), (n, op, v, w)
