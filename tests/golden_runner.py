"""Replays the transcribed reference known-answer cases against an engine.

An engine is any object with the small interface used below (the CPU oracle adapter lives in
this file; the CUDA adapter in tests/cuda_engine.py).  Buffers are 1-D numpy arrays holding the
whole underlying storage; metas describe the view (shape, strides, offset in elements).
"""
from __future__ import annotations

import numpy as np

NP = {"f32": np.float32, "f64": np.float64, "i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64,
      "u8": np.uint8, "u16": np.uint16, "u32": np.uint32, "u64": np.uint64, "bool": np.bool_}
BIN = {"add": 0, "sub": 1, "mul": 2, "div": 3, "log": 4, "log1p": 5, "leaky_relu": 6, "elu": 7}
# truth closures of ops/scalar/mod.rs, evaluated in the tensor's own dtype (x, operand) -> value
SCALAR_TRUTH = {
    "log_base": lambda x, v: (np.log(x) / np.log(x.dtype.type(v))).astype(x.dtype),
    "log1p_base": lambda x, v: (np.log1p(x) / np.log(x.dtype.type(v))).astype(x.dtype),
    "leaky": lambda x, v: np.where(x > 0, x, x * x.dtype.type(v)).astype(x.dtype),
    "elu": lambda x, v: np.where(x >= 0, x, np.expm1(np.minimum(x, 0)) * x.dtype.type(v)).astype(x.dtype),
}
UN = {n: i for i, n in enumerate(
    ["neg", "relu", "abs", "sign", "sigmoid", "tanh", "sqrt", "sin", "cos", "tan", "asin", "acos", "atan", "sinh", "cosh",
     "asinh", "acosh", "atanh", "rsqrt", "reciprocal", "square", "cube", "exp", "ln", "ln1p", "floor", "ceil", "round",
     "trunc", "expm1", "silu"])}
TRUTH = {
    "neg": lambda x: -x, "max0": lambda x: np.maximum(x, 0.0), "signum": np.sign,
    "sigmoid": lambda x: 1.0 / (1.0 + np.exp(-x)), "silu": lambda x: x / (1.0 + np.exp(-x)), "tanh": np.tanh,
    "sqrt": np.sqrt, "ln": np.log, "sin": np.sin, "cos": np.cos, "tan": np.tan, "asin": np.arcsin, "acos": np.arccos,
    "atan": np.arctan, "sinh": np.sinh, "cosh": np.cosh, "asinh": np.arcsinh, "acosh": np.arccosh, "atanh": np.arctanh,
    "rsqrt": lambda x: 1.0 / np.sqrt(x), "reciprocal": lambda x: 1.0 / x, "square": lambda x: x * x,
    "cube": lambda x: x * x * x, "exp": np.exp, "expm1": np.expm1, "ln1p": np.log1p, "floor": np.floor, "ceil": np.ceil,
    "trunc": np.trunc, "round": lambda x: np.trunc(x + np.copysign(0.5, x)),  # Rust f.round(): halves away from zero
}
RED = {"sum": 1, "prod": 2, "max": 3, "min": 4, "mean": 5}
# name -> (code, unbiased, is_std, norm_type): the ReductionSettings the reference front end sends
# (ops/reduction/mod.rs:413-510)
RED_EXT = {"var": (6, True, False, 2), "pop_var": (6, False, False, 2), "std": (6, True, True, 2),
           "pop_std": (6, False, True, 2), "logsumexp": (7, True, False, 2), "l1": (8, True, False, 1),
           "l2": (8, True, False, 2), "argmax": (9, True, False, 2), "argmin": (10, True, False, 2)}


def build_tensor(spec, dtype, engine):
    """-> (buffer, meta) for a tensor spec of tests/golden/reference_cases.py."""
    dt = NP[dtype]
    if "buf" in spec:
        shape = tuple(spec["shape"])
        buf = np.array(spec["buf"], dtype=dt)
    elif "ones" in spec:
        shape = tuple(spec["ones"])
        buf = np.ones(int(np.prod(shape, dtype=np.int64)) if shape else 1, dtype=dt)
    else:
        shape = tuple(spec["zeros"])
        buf = np.zeros(int(np.prod(shape, dtype=np.int64)) if shape else 1, dtype=dt)
    meta = engine.Meta.contiguous(shape)
    for coord, value in spec.get("set", []):
        buf[sum(c * s for c, s in zip(coord, meta.strides))] = value
    return buf, apply_view(meta, spec.get("view", []))


def apply_view(meta, ops):
    for v in ops:
        if v[0] == "slice":
            meta = meta.slice(v[1], v[2], v[3], v[4])
        elif v[0] == "index":
            meta = meta.index(v[1], v[2])
        elif v[0] == "permute":
            meta = meta.permute(v[1])
        elif v[0] == "unsqueeze":
            meta = meta.unsqueeze(v[1])
        elif v[0] == "squeeze":
            meta = meta.squeeze(v[1])
        elif v[0] == "view_as":
            meta = meta.view_as(v[1])
        else:
            raise ValueError(v)
    return meta


def check_values(case, out, shape):
    assert list(shape) == list(case["shape"]), (case["name"], shape)
    n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
    out = np.asarray(out)[:n]
    if "values" in case:
        exp = np.array(case["values"], dtype=out.dtype)
        assert np.array_equal(out, exp), (case["name"], out, exp)
    if "all" in case:
        assert np.all(out == np.array(case["all"], dtype=out.dtype)), (case["name"], out)
    if "spots" in case:
        strides = [1] * len(shape)
        for k in range(len(shape) - 2, -1, -1):
            strides[k] = strides[k + 1] * shape[k + 1]
        for coord, v in case["spots"]:
            got = out[sum(c * s for c, s in zip(coord, strides))]
            assert got == np.array(v, dtype=out.dtype), (case["name"], coord, got, v)


def run_case(case, engine):
    kind = case["kind"]
    if kind == "scalar_assign":
        buf, meta = build_tensor(case["a"], case["dtype"], engine)
        em = case.get("expect_meta")
        if em:
            assert list(meta.shape) == em["shape"] and list(meta.strides) == em["strides"]
            assert meta.offset == em["offset"] and meta.is_contiguous() == em["contiguous"]
        for op, value in case["ops"]:
            buf = engine.scalar_assign(buf, meta, BIN[op], value)
        if "buf" in case:
            assert np.array_equal(buf, np.array(case["buf"], dtype=buf.dtype)), (case["name"], buf)
        if "buf_close" in case:
            exp, eps = case["buf_close"]
            assert np.all(np.abs(buf.astype(np.float64) - np.array(exp, dtype=buf.dtype).astype(np.float64)) < eps), (case["name"], buf)
        for idx, v in case.get("buf_at", []):
            assert buf[idx] == v, (case["name"], idx, buf[idx])
    elif kind == "program":
        buf, meta = build_tensor(case["a"], case["dtype"], engine)
        for step in case["steps"]:
            m = apply_view(meta, step[1])
            if step[0] == "assign":
                buf = engine.scalar_assign(buf, m, BIN[step[2]], step[3])
            else:
                before = buf.copy()
                out, _ = engine.scalar_out(buf, m, BIN[step[2]], step[3])
                assert np.asarray(out)[: len(step[4])].tolist() == step[4], (case["name"], step, out)
                assert np.array_equal(buf, before), case["name"]
        assert np.array_equal(buf, np.array(case["buf"], dtype=buf.dtype)), (case["name"], buf)
    elif kind == "fill":
        buf, meta = build_tensor(case["a"], case["dtype"], engine)
        base = engine.Meta.contiguous(case["a"]["shape"])
        buf = engine.fill(buf, meta, case["value"])
        if "buf" in case:
            assert np.array_equal(buf, np.array(case["buf"], dtype=buf.dtype)), (case["name"], buf)
        for coord, v in case.get("base_spots", []):
            assert buf[sum(c * s for c, s in zip(coord, base.strides))] == v, (case["name"], coord)
    elif kind == "owned":
        buf, meta = build_tensor(case["a"], case["dtype"], engine)
        if "view_contiguous" in case:
            assert meta.is_contiguous() == case["view_contiguous"], case["name"]
        out = engine.owned(buf, meta)
        assert list(meta.shape) == list(case["shape"]), (case["name"], meta.shape)
        if "values" in case:
            assert np.asarray(out)[: len(case["values"])].tolist() == case["values"], (case["name"], out)
        if "ends" in case:
            n = int(np.prod(case["shape"], dtype=np.int64))
            assert (np.asarray(out)[0], np.asarray(out)[n - 1]) == case["ends"], case["name"]
    elif kind == "view_check":
        buf, meta = build_tensor(case["a"], case["dtype"], engine)
        assert list(meta.shape) == list(case["shape"]), (case["name"], meta.shape)
        if "strides" in case:
            assert list(meta.strides) == list(case["strides"]), (case["name"], meta.strides)
        for coord, v in case["spots"]:
            got = buf[meta.offset + sum(c * s for c, s in zip(coord, meta.strides))]
            assert got == v, (case["name"], coord, got, v)
    elif kind == "view_set":
        buf, base = build_tensor(case["a"], case["dtype"], engine)
        meta = apply_view(base, case["view"])
        assert list(meta.shape) == list(case["shape"]), (case["name"], meta.shape)
        for coord, v in case["sets"]:
            buf[meta.offset + sum(c * s for c, s in zip(coord, meta.strides))] = v
        for coord, v in case["base_spots"]:
            assert buf[base.offset + sum(c * s for c, s in zip(coord, base.strides))] == v, (case["name"], coord)
    elif kind == "slice_error":
        m = engine.Meta.contiguous(case["a_shape"])
        dim, start, end, step = case["slice"]
        try:
            m.slice(dim, start, end, step)
        except Exception as e:
            assert engine.error_kind(e) == case["error"], (case["name"], e)
            return
        raise AssertionError(f"{case['name']}: slice should be refused")
    elif kind == "meta_check":
        if "a_meta" in case:
            shape, strides, offset = case["a_meta"]
            meta = engine.Meta(tuple(shape), tuple(strides), offset)
        else:
            _, meta = build_tensor(case["a"], "i32", engine)
        if "size" in case:
            assert meta.size == case["size"], case["name"]
        if "offset" in case:
            assert meta.offset == case["offset"], case["name"]
        if "contiguous" in case:
            assert meta.is_contiguous() == case["contiguous"], case["name"]
    elif kind == "view_as_error":
        m = engine.Meta.contiguous(case["a_shape"])
        try:
            m.view_as(case["new_shape"])
        except Exception:
            return
        raise AssertionError(f"{case['name']}: view_as should be refused")
    elif kind == "strides_of":
        assert list(engine.Meta.contiguous(case["shape"]).strides) == list(case["strides"]), case["name"]
    elif kind == "permute_error":
        m = engine.Meta.contiguous(case["a_shape"])
        try:
            m.permute(case["dims"])
        except Exception as e:
            assert engine.error_kind(e) == "dim", (case["name"], e)
            return
        raise AssertionError(f"{case['name']}: permute should be refused")
    elif kind == "view_values":
        buf, meta = build_tensor(case["a"], case["dtype"], engine)
        assert list(meta.shape) == list(case["shape"]), (case["name"], meta.shape)
        got = gather_view(buf, meta)
        assert np.asarray(got).reshape(-1).tolist() == case["values"], (case["name"], got)
    elif kind == "scalar":
        buf, meta = build_tensor(case["a"], case["dtype"], engine)
        before = buf.copy()
        out, shape = engine.scalar_out(buf, meta, BIN[case["op"]], case["value"])
        check_values(case, out, shape)
        assert np.array_equal(buf, before), case["name"]
    elif kind == "binary":
        a, am = build_tensor(case["a"], case["dtype"], engine)
        b, bm = build_tensor(case["b"], case["dtype"], engine)
        out, shape = engine.binary(a, am, b, bm, BIN[case["op"]])
        check_values(case, out, shape)
    elif kind == "binary_assign":
        a, am = build_tensor(case["a"], case["dtype"], engine)
        b, bm = build_tensor(case["b"], case["dtype"], engine)
        a = engine.binary_assign(a, am, b, bm, BIN[case["op"]])
        assert np.array_equal(a, np.array(case["buf"], dtype=a.dtype)), (case["name"], a)
    elif kind == "broadcast_error":
        ma = engine.Meta.contiguous(case["a_shape"])
        mb = engine.Meta.contiguous(case["b_shape"])
        try:
            engine.broadcast_params(ma, mb)
        except Exception:
            return
        raise AssertionError(f"{case['name']}: shapes should not broadcast")
    elif kind == "assign_shape_error":
        # `a op= b` requires the broadcast shape to equal a's shape (ops/broadcast/add.rs:26-31)
        ma = engine.Meta.contiguous(case["a_shape"])
        mb = engine.Meta.contiguous(case["b_shape"])
        shape, _, _ = engine.broadcast_params(ma, mb)
        assert tuple(shape) != tuple(ma.shape)
    elif kind == "reduce_total":
        a, am = build_tensor(case["a"], case["dtype"], engine)
        got = engine.reduce_total(a, am, RED[case["op"]])
        want = case["cuda_value"] if getattr(engine, "tree_sums", False) and "cuda_value" in case else case["value"]
        assert got == np.array(want, dtype=a.dtype), (case["name"], repr(got))
    elif kind == "reduce_axis":
        a, am = build_tensor(case["a"], case["dtype"], engine)
        out, shape = engine.reduce_axis(a, am, case["axis"], RED[case["op"]])
        check_values(case, out, shape)
    elif kind == "reduce_ext":
        a, am = build_tensor(case["a"], case["dtype"], engine)
        code, unbiased, is_std, norm_type = RED_EXT[case["op"]]
        out, shape = engine.reduce_ext(a, am, case["axis"], code, unbiased, is_std, norm_type)
        assert list(shape) == list(case["shape"]), (case["name"], shape)
        out = np.asarray(out)[: len(case["values"])]
        if code >= 9:
            assert out.dtype == np.uint64 and out.tolist() == case["values"], (case["name"], out)
        else:
            exp = np.array(case["values"], dtype=a.dtype)
            # a device engine merges partial states in tree order: a few ulps from the listed values
            ulps = 8 if getattr(engine, "tree_sums", False) else 0
            assert np.all(np.abs(out - exp) <= ulps * np.spacing(np.abs(exp))), (case["name"], out, exp)
    elif kind == "scalar_fixture":
        dt = NP[case["dtype"]]
        d = np.array(case["definition"], dtype=dt)
        if case["layout"] == "contiguous":
            meta = engine.Meta.contiguous((2, 1))
        elif case["layout"] == "1d":
            meta = engine.Meta.contiguous((3, 1)).slice(0, None, None, 2)
        else:
            meta = engine.Meta.contiguous((4, 4, 1)).slice(0, None, None, 2).slice(1, None, None, 2)
        by = [s * d.itemsize for s in meta.strides]
        view = np.lib.stride_tricks.as_strided(d[meta.offset:], shape=meta.shape, strides=by)
        exp = d.copy()
        expv = np.lib.stride_tricks.as_strided(exp[meta.offset:], shape=meta.shape, strides=by)
        expv[...] = SCALAR_TRUTH[case["truth"]](view, case["value"])
        got = engine.scalar_assign(d.copy(), meta, BIN[case["op"]], case["value"])
        if np.dtype(dt).kind == "f":  # eps_eq of the reference: |a - b| < tolerance
            assert np.all(np.abs(got - exp) < case["tol"]), (case["name"], got, exp)
        else:
            assert np.array_equal(got, exp), (case["name"], got, exp)
    elif kind == "unary_fixture":
        dt = NP[case["dtype"]]
        d = np.array(case["definition"], dtype=dt)
        if case["layout"] == "contiguous":
            meta = engine.Meta.contiguous((2, 1))
        elif case["layout"] == "1d":
            meta = engine.Meta.contiguous((3, 1)).slice(0, None, None, 2)
        else:
            meta = engine.Meta.contiguous((4, 4, 1)).slice(0, None, None, 2).slice(1, None, None, 2)
        truth = TRUTH[case["truth"]]
        view = np.lib.stride_tricks.as_strided(d[meta.offset:], shape=meta.shape,
                                               strides=[s * d.itemsize for s in meta.strides])
        exp = d.copy()
        expv = np.lib.stride_tricks.as_strided(exp[meta.offset:], shape=meta.shape,
                                               strides=[s * d.itemsize for s in meta.strides])
        expv[...] = truth(view)
        got = engine.unary_assign(d.copy(), meta, UN[case["op"]])
        if "tol" in case:  # eps_eq of the reference: |a - b| < tolerance
            assert np.all(np.abs(got - exp) < case["tol"]), (case["name"], got, exp)
        else:
            assert np.array_equal(got, exp), (case["name"], got, exp)
    else:
        raise ValueError(kind)


def gather_view(buf, meta):
    """Row-major copy of the viewed elements (what `contiguous()` / `owned()` produce)."""
    if meta.size == 0:
        return np.zeros(0, dtype=buf.dtype)
    idx = np.full(meta.shape if meta.shape else (), meta.offset, dtype=np.int64)
    for k, (n, s) in enumerate(zip(meta.shape, meta.strides)):
        shp = [1] * len(meta.shape)
        shp[k] = n
        idx = idx + (np.arange(n, dtype=np.int64) * s).reshape(shp)
    return buf[idx.reshape(-1)].copy()


class OracleEngine:
    """Adapter: the CPU oracle behind the engine interface."""

    def __init__(self, fast=False):
        import oracle
        self.o = oracle
        self.Meta = oracle.Meta
        self.fast = fast

    def broadcast_params(self, a, b):
        return self.o.broadcast_params(a, b)

    def scalar_assign(self, buf, meta, op, value):
        self.o.scalar_op(buf, op, value, meta, self.fast)
        return buf

    def unary_assign(self, buf, meta, op):
        self.o.unary_op(buf, op, meta, self.fast)
        return buf

    def fill(self, buf, meta, value):
        self.o.fill(buf, value, meta, self.fast)
        return buf

    def owned(self, buf, meta):
        # view_to_contiguous, core/tensor.rs:299-325: element by element in row-major order
        return gather_view(buf, meta).reshape(-1)

    def scalar_out(self, buf, meta, op, value):
        # out-of-place scalar op = owned() copy, then in place (ops/scalar/add.rs:93-97)
        out = gather_view(buf, meta)
        m = self.Meta.contiguous(meta.shape)
        self.o.scalar_op(out, op, value, m, self.fast)
        return out, meta.shape

    def binary(self, a, am, b, bm, op):
        out, dm = self.o.binary(a, am, b, bm, op, self.fast)
        return out, dm.shape

    def binary_assign(self, a, am, b, bm, op):
        shape, sa, sb = self.o.broadcast_params(am, bm)
        assert tuple(shape) == tuple(am.shape)
        ma = self.Meta(shape, sa, am.offset)
        self.o.broadcast(a, ma, b, self.Meta(shape, sb, bm.offset), a, ma, op, self.fast)
        return a

    def reduce_total(self, a, am, op):
        return self.o.reduce_flat(a, am.offset, am.size, op, self.fast)[0]

    def reduce_axis(self, a, am, axis, op):
        out, om = self.o.reduce_axis(a, am, axis, op, self.fast)
        return out, om.shape

    @staticmethod
    def error_kind(e):
        return {-2: "bounds", -3: "shape", -1: "dim"}.get(getattr(e, "code", None))

    def reduce_ext(self, a, am, axis, code, unbiased, is_std, norm_type):
        assert am.is_contiguous()
        if axis is None:
            outer, r, inner, shape = 1, am.size, 1, ()
        else:
            outer = int(np.prod(am.shape[:axis], dtype=np.int64))
            r, inner = am.shape[axis], int(np.prod(am.shape[axis + 1:], dtype=np.int64))
            shape = tuple(1 if k == axis else s for k, s in enumerate(am.shape))
        src = a[am.offset:]
        if code >= 9:
            return self.o.argreduce_ori(src, outer, r, inner, code, self.fast), shape
        return self.o.reduce_ext_ori(src, outer, r, inner, code, unbiased, is_std, norm_type, self.fast), shape
