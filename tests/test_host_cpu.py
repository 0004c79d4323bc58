"""CPU-only checks: the library loads and exports every declared symbol, the host-side view
arithmetic agrees with the oracle's restatement of the reference, and the launch planner picks
the intended kernel class for the benchmark configurations.  No CUDA compute call is made."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle as O
import rtensors_b200 as rt
from rtensors_b200 import _lib as L
from rtensors_b200.meta import Meta, broadcast_params, plan_elementwise, shard_range

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    h = open(os.path.join(ROOT, "include", "rt_b200.h")).read()
    names.update(re.findall(r"\b(rtb_[a-z0-9_]+)\s*\(", h))
    # v1 header declares through macros: expand with the C preprocessor
    import subprocess
    pre = subprocess.run(["gcc", "-E", "-x", "c", os.path.join(ROOT, "include", "rt_b200_v1.h")],
                         capture_output=True, text=True, check=True).stdout
    names.update(re.findall(r"\b(launch_[a-z0-9_]+|rtensors_take_cuda_alloc_error)\s*\(", pre))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    lib = rt.lib()
    names = _declared_symbols()
    assert len(names) > 300
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing[:10]


def test_reference_launcher_names_are_covered():
    # the reference's own header set names these families for the hot path
    lib = rt.lib()
    for op in ("add", "sub", "mul", "div", "fill"):
        for layout in ("contiguous", "strided", "nd_affine"):
            for s in ("f32", "f64", "u8", "u16", "u32", "u64", "u128", "i8", "i16", "i32", "i64", "i128", "boolean"):
                assert hasattr(lib, f"launch_{op}_{layout}_{s}")
    for s in ("f32", "f64"):
        assert hasattr(lib, f"launch_flat_contiguous_reduce_{s}")
        assert hasattr(lib, f"launch_nd_reduce_contiguous_{s}")
        assert hasattr(lib, f"launch_binary_broadcast_elementwise_{s}")


def _rand_meta(rng, M):
    rank = int(rng.integers(0, 5))
    shape = tuple(int(rng.integers(1, 6)) for _ in range(rank))
    m = M.contiguous(shape)
    ops = []
    for _ in range(int(rng.integers(0, 4))):
        if m.rank == 0:
            break
        kind = rng.integers(0, 4)
        if kind == 0:
            dim = int(rng.integers(0, m.rank))
            step = int(rng.choice([-3, -2, -1, 1, 2, 3]))
            n = m.shape[dim]
            if step > 0:
                start = int(rng.integers(0, n)); end = int(rng.integers(start, n + 1))
            else:
                start = int(rng.integers(0, n)); end = int(rng.integers(-1, start + 1))
            ops.append(("slice", dim, start, None if end < 0 else end, step))
        elif kind == 1:
            ops.append(("permute", tuple(int(x) for x in rng.permutation(m.rank))))
        elif kind == 2:
            ops.append(("unsqueeze", int(rng.integers(0, m.rank + 1))))
        else:
            dim = int(rng.integers(0, m.rank))
            ops.append(("index", dim, int(rng.integers(0, m.shape[dim]))))
        op = ops[-1]
        m = getattr(m, op[0])(*op[1:])
    return shape, ops


def _apply(M, shape, ops):
    m = M.contiguous(shape)
    for op in ops:
        m = getattr(m, op[0])(*op[1:])
    return m


def test_view_arithmetic_matches_oracle():
    rng = np.random.default_rng(11)
    for _ in range(400):
        shape, ops = _rand_meta(rng, O.Meta)
        a = _apply(O.Meta, shape, ops)
        b = _apply(Meta, shape, ops)
        assert (a.shape, a.strides, a.offset) == (b.shape, b.strides, b.offset), (shape, ops)
        assert a.is_contiguous() == b.is_contiguous()
        assert a.squeeze().shape == b.squeeze().shape and a.squeeze().strides == b.squeeze().strides


def test_broadcast_params_match_oracle():
    rng = np.random.default_rng(12)
    hits = 0
    for _ in range(400):
        ra, rb = int(rng.integers(0, 5)), int(rng.integers(0, 5))
        base = [int(rng.integers(1, 5)) for _ in range(max(ra, rb))]
        sa = [d if rng.random() < 0.6 else 1 for d in base[len(base) - ra:]]
        sb = [d if rng.random() < 0.6 else 1 for d in base[len(base) - rb:]]
        if rng.random() < 0.1 and sa:
            sa[-1] += 7
        try:
            want = O.broadcast_params(O.Meta.contiguous(sa), O.Meta.contiguous(sb))
        except O.OracleError:
            with pytest.raises(rt.RtbError) as e:
                broadcast_params(Meta.contiguous(sa), Meta.contiguous(sb))
            assert e.value.code == -3
            continue
        assert broadcast_params(Meta.contiguous(sa), Meta.contiguous(sb)) == want
        hits += 1
    assert hits > 100


def test_slice_errors():
    m = Meta.contiguous((4, 3))
    with pytest.raises(rt.RtbError) as e:
        m.slice(2)
    assert e.value.code == -5
    with pytest.raises(rt.RtbError) as e:
        m.slice(0, 0, 4, 0)
    assert e.value.code == -6
    with pytest.raises(rt.RtbError) as e:
        m.slice(0, 5, None, 1)
    assert e.value.code == -4
    with pytest.raises(rt.RtbError):
        Meta.contiguous((2, 3)).permute((0, 0, 1))
    with pytest.raises(rt.RtbError):
        Meta((4,), (1,), 2).check_extent(5)
    Meta((4,), (-1,), 3).check_extent(4)
    with pytest.raises(rt.RtbError):
        Meta((4,), (-1,), 2).check_extent(4)


def _plan_list(p, name):
    return list(getattr(p, name))[: p.rank]


def test_plan_config_contiguous_chain_and_same_shape_add():
    n = 1 << 28
    m = Meta.contiguous((n,))
    p = plan_elementwise(L.F32, 1, (n,), m, m)
    assert p.kernel == 1 and p.rank == 1 and p.shape[0] == n
    m3 = Meta.contiguous((1 << 14, 1 << 14))
    p = plan_elementwise(L.I32, 2, m3.shape, m3, m3, m3)
    assert p.kernel == 1 and p.rank == 1 and p.shape[0] == n  # same-shape add collapses to one run


def test_plan_config_outer_product():
    shape, sa, sb = broadcast_params(Meta.contiguous((4096, 1)), Meta.contiguous((1, 4096)))
    d = Meta.contiguous(shape)
    p = plan_elementwise(L.F32, 2, shape, d, Meta(shape, sa, 0), Meta(shape, sb, 0))
    assert p.kernel == 3 and p.rank == 2
    assert (p.mode_d, p.mode_l, p.mode_r) == (0, 4, 0)  # vector store, broadcast scalar, vector load
    assert p.tile_x == 256 and p.ux == 4 and p.n_rows == 4096 and p.n_col_chunks == 1


def test_plan_config_strided_negative_step_broadcast():
    A = Meta.contiguous((1024, 16, 1, 1)).view_as((1, 1024, 16, 1)).permute((2, 0, 1, 3))
    B = Meta.contiguous((1, 64, 1, 1024)).slice(3, None, None, -1)
    assert A.shape == (16, 1, 1024, 1) and A.strides == (1, 16384, 16, 1)
    assert B.strides == (65536, 1024, 1024, -1) and B.offset == 1023
    shape, sa, sb = broadcast_params(A, B)
    assert shape == (16, 64, 1024, 1024) and sa == (1, 0, 16, 0) and sb == (0, 1024, 0, -1)
    d = Meta.contiguous(shape)
    p = plan_elementwise(L.F32, 2, shape, d, Meta(shape, sa, A.offset), Meta(shape, sb, B.offset))
    assert p.kernel == 3 and p.rank == 4
    assert (p.mode_d, p.mode_l, p.mode_r) == (0, 4, 2)  # vector store, broadcast, reversed vector load
    assert p.fast == 1 and p.ux == 4 and p.tile_x == 64 and p.tile_y == 4  # 4 rows x (64 x 4) vectors per CTA pass
    assert p.n_rows == 16 * 64 * 1024 and p.grid == p.n_rows // 4 and p.n_col_chunks == 1


def test_plan_flips_and_merges_reversed_inplace_view():
    # in place through a fully reversed view: one contiguous run walked from the lowest address
    m = Meta.contiguous((2, 3)).slice(1, None, None, -1).slice(0, None, None, -1)
    p = plan_elementwise(L.F32, 1, m.shape, m, m)
    assert p.kernel == 1 and p.rank == 1 and p.shape[0] == 6 and p.base_d == 0
    # permuted output: dims are reordered so the output is walked in address order
    t = Meta.contiguous((3, 4)).permute((1, 0))
    p = plan_elementwise(L.F32, 1, t.shape, t, t)
    assert p.kernel == 1 and p.shape[0] == 12


def test_plan_misaligned_operands_use_row_kernel_modes():
    n = 1000
    m = Meta.contiguous((n,))
    p = plan_elementwise(L.F32, 2, (n,), m, Meta((n,), (1,), 1), m, ptr_d=0, ptr_l=0, ptr_r=0)
    assert p.kernel == 3 and p.mode_d == 0 and p.mode_l == 1 and p.mode_r == 0


def test_plan_rejects_zero_stride_output():
    with pytest.raises(rt.RtbError):
        plan_elementwise(L.F32, 1, (4, 4), Meta((4, 4), (0, 1), 0), Meta.contiguous((4, 4)))


def test_plan_high_rank_collapses():
    shape = (2,) * 20
    m = Meta.contiguous(shape)
    p = plan_elementwise(L.F32, 2, shape, m, m, m)
    assert p.kernel == 1 and p.shape[0] == 1 << 20


def test_shard_range_partitions_exactly():
    for extent in (0, 1, 7, 16, 4096, 1000003):
        for parts in (1, 2, 3, 4, 8):
            spans = [shard_range(extent, parts, k) for k in range(parts)]
            assert spans[0][0] == 0 and spans[-1][1] == extent
            for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
                assert e0 == b1
            sizes_ = [e - b for b, e in spans]
            assert max(sizes_) - min(sizes_) <= 1


def test_no_device_compute_fails_loudly_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    ctx = C.c_void_p()
    rc = rt.lib().rtb_ctx_create(C.c_int(0), C.byref(ctx))
    assert rc != 0
    with pytest.raises(RuntimeError):
        rt.CudaB200(0)


def test_host_buffer_entry_points_check_their_arguments_before_any_cuda_call():
    """Null contexts and null buffers are refused with RTB_ERR_INVALID (-1) on a box without a GPU too."""
    lib = rt.lib()
    null = C.c_void_p(0)
    out = C.c_void_p()
    one = (C.c_size_t * 1)(4)
    st = (C.c_ssize_t * 1)(1)
    assert lib.rtb_host_stage_in(null, null, C.c_size_t(16), C.byref(out)) == -1
    assert lib.rtb_host_scratch(null, C.c_size_t(16), C.byref(out)) == -1
    assert lib.rtb_host_ready(null, null) == -1
    assert lib.rtb_host_stage_out(null, null, null, C.c_size_t(16)) == -1
    assert lib.rtb_host_release(null, null) == -1
    assert lib.rtb_host_join(null) == -1 and lib.rtb_host_wait(null) == -1 and lib.rtb_host_trim(null) == -1
    assert lib.rtb_host_set_stage_bytes(null, C.c_size_t(1 << 20)) == -1
    assert lib.rtb_host_pin(null, C.c_size_t(16)) == -1
    assert lib.rtb_host_alloc(C.c_size_t(16), None) == -1
    assert lib.rtb_host_reduce_view(null, C.c_int(10), C.c_int(1), None, null, C.c_size_t(4), C.c_size_t(1), one, st, C.c_size_t(0),
                                    C.c_ssize_t(0), null) == -1
    assert lib.rtb_host_broadcast(null, C.c_int(10), C.c_int(0), null, C.c_size_t(4), st, C.c_size_t(0), null, C.c_size_t(4), st,
                                  C.c_size_t(0), null, C.c_size_t(1), one, C.c_size_t(0), C.c_size_t(4)) == -1
    assert b"null" in lib.rtb_last_error_string()


# ---- the reference's view-arithmetic tests, replayed on the library's host-side planner (no GPU)
_HOST_KINDS = ("view_check", "view_set", "view_values", "slice_error", "permute_error", "view_as_error", "strides_of", "meta_check", "broadcast_error", "assign_shape_error")


class _HostEngine:
    """The part of the engine interface that needs no device: view metadata from the library."""
    Meta = Meta

    @staticmethod
    def broadcast_params(a, b):
        return broadcast_params(a, b)

    @staticmethod
    def error_kind(e):
        return {-4: "bounds", -6: "shape", -5: "dim"}.get(getattr(e, "code", None))


def _host_cases():
    from golden.reference_cases import CASES
    return [c for c in CASES if c["kind"] in _HOST_KINDS]


@pytest.mark.parametrize("case", _host_cases(), ids=[c["name"] for c in _host_cases()])
def test_reference_view_case_on_host_planner(case):
    from golden_runner import run_case
    run_case(case, _HostEngine())
