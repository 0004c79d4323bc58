"""rtensors_b200 -- the rtensors tensor hot path (scalar elementwise ops, N-d broadcast binary ops
over strided / permuted / negative-step views, axis and full reductions, mean_l1_loss,
reduce-to-shape) as hand-written CUDA for sm_100a behind a C ABI.

The compute library is `librt_b200.so` (C ABI in include/rt_b200.h, built by
`python -m rtensors_b200.build`).  This package is the thin host side: a ctypes binding, the
view-metadata mirror and a `TensorBase`-like front end used by the tests and the bench.  There
is no CPU or eager fallback: without the built library or without a GPU the ops raise.
"""
from . import _lib
from ._lib import (ABS, ADD, BOOL, DIV, F32, F64, I8, I16, I32, I64, I128, MAX, MEAN, MIN, MUL, NEG, PROD, RELU,
                   SIGN, SUB, SUM, U8, U16, U32, U64, U128, RtbError, lib)
from .meta import Meta, broadcast_params, plan_elementwise, shard_range

__all__ = ["Meta", "broadcast_params", "plan_elementwise", "shard_range", "lib", "RtbError"]


def __getattr__(name):
    # torch-dependent parts are imported on first use so that `import rtensors_b200` stays light
    import importlib
    if name in ("CudaB200", "backend"):
        mod = importlib.import_module(".backend", __name__)
        return mod if name == "backend" else mod.CudaB200
    if name in ("Tensor", "tensor", "mean_l1_loss"):
        mod = importlib.import_module(".tensor", __name__)
        return mod if name == "tensor" else getattr(mod, name)
    raise AttributeError(name)
