"""ctypes binding of librt_b200.so (the C ABI declared in include/rt_b200.h)."""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "librt_b200.so")

# dtype codes (rtb_dtype) = DType discriminants of the reference, src/core/value.rs:567-581
U8, I8, U16, I16, U32, U128, I32, U64, I64, I128, F32, F64, BOOL = range(13)
DTYPE_SIZE = {U8: 1, I8: 1, BOOL: 1, U16: 2, I16: 2, U32: 4, I32: 4, F32: 4, U64: 8, I64: 8, F64: 8, U128: 16, I128: 16}
ADD, SUB, MUL, DIV, LOG, LOG1P, LEAKY_RELU, ELU = range(8)
(NEG, RELU, ABS, SIGN, SIGMOID, TANH, SQRT, SIN, COS, TAN, ASIN, ACOS, ATAN, SINH, COSH, ASINH, ACOSH, ATANH, RSQRT,
 RECIPROCAL, SQUARE, CUBE, EXP, LN, LN1P, FLOOR, CEIL, ROUND, TRUNC, EXPM1, SILU) = range(31)
SUM, PROD, MAX, MIN, MEAN = 1, 2, 3, 4, 5
VARIANCE, LOGSUMEXP, NORM, ARGMAX, ARGMIN = 6, 7, 8, 9, 10
OK = 0


MASK_RELU, MASK_ABS, MASK_LEAKY_RELU, MASK_RECIPROCAL = 1, 2, 3, 4   # rtb_grad_mask kinds
# rtb_status codes used by host-side checks (include/rt_b200.h)
ERR_INVALID, ERR_DTYPE, ERR_BROADCAST, ERR_BOUNDS, ERR_DIM, ERR_SHAPE, ERR_NONCONTIG = -1, -2, -3, -4, -5, -6, -7


class RtbError(RuntimeError):
    """A non-zero rtb_status; `.code` is the status, the text comes from rtb_last_error_string()."""

    def __init__(self, code: int, text: str):
        super().__init__(f"rtb status {code}: {text}")
        self.code = code


class ReduceSettings(C.Structure):
    """rtb_reduce_settings = the reference's ReductionSettings (cuda/include/common.h:13-17)."""
    _fields_ = [("unbiased", C.c_bool), ("is_std", C.c_bool), ("norm_type", C.c_int)]


class Plan(C.Structure):
    _fields_ = [("kernel", C.c_int), ("rank", C.c_int), ("shape", C.c_uint64 * 8), ("stride_d", C.c_int64 * 8),
                ("stride_l", C.c_int64 * 8), ("stride_r", C.c_int64 * 8), ("base_d", C.c_int64),
                ("base_l", C.c_int64), ("base_r", C.c_int64), ("vec", C.c_int), ("mode_d", C.c_int),
                ("mode_l", C.c_int), ("mode_r", C.c_int), ("tile_x", C.c_int), ("tile_y", C.c_int),
                ("n_rows", C.c_uint64), ("n_col_chunks", C.c_uint64), ("grid", C.c_uint64),
                ("fast", C.c_int), ("ux", C.c_int)]


_lib = None


def lib() -> C.CDLL:
    """Loads the library; there is no fallback -- a missing build is an error."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m rtensors_b200.build` "
                               "(this package has no CPU or eager fallback)")
        l = C.CDLL(LIB_PATH)
        l.rtb_last_error_string.restype = C.c_char_p
        l.rtb_ctx_get_stream.restype = C.c_void_p
        l.rtb_ctx_launch_count.restype = C.c_uint64
        l.rtb_ctx_workspace_generation.restype = C.c_uint64
        l.rtb_meta_contiguous_strides.restype = None
        l.rtb_shard_range.restype = None
        l.rtb_ctx_destroy.restype = None
        _lib = l
    return _lib


def check(rc: int) -> None:
    if rc != OK:
        raise RtbError(rc, (lib().rtb_last_error_string() or b"").decode())


def sizes(xs):
    return (C.c_size_t * max(len(xs), 1))(*[int(x) for x in xs])


def diffs(xs):
    return (C.c_ssize_t * max(len(xs), 1))(*[int(x) for x in xs])
