"""Harness over the reference's own CUDA kernels recompiled for sm_100a (baseline/_ref/libref_cuda.so,
built by baseline/ref_cuda/Makefile) -- TEST AND BENCH INFRASTRUCTURE, never imported by the product
package.  Calls go through the reference's `extern "C" launch_*` symbols with the launch parameters
its Rust host uses: block size 256 (src/backend/cuda.rs:36), shape / stride arrays uploaded to device
memory as u64 / i64 before a broadcast call (src/backend/cuda.rs:1044-1084), settings passed as a host
pointer, everything on the legacy default stream.

Only contiguous or plainly strided inputs are handed to it: a view whose strides are dense up to sign
would be walked out of bounds by the reference's dispatcher, so no such call is made here.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libref_cuda.so")
BLOCK = 256
SUM, PROD, MAX, MIN, MEAN, VARIANCE, LOGSUMEXP, NORM, ARGMAX, ARGMIN = range(1, 11)
ADD, SUB, MUL, DIV = range(4)


class Settings(C.Structure):
    _fields_ = [("unbiased", C.c_bool), ("is_std", C.c_bool), ("norm_type", C.c_int)]


def build(reference: str = "/root/reference") -> bool:
    """Compiles the shared object if the reference checkout is present; True if it exists afterwards."""
    if os.path.isdir(os.path.join(reference, "libs", "rtensors", "cuda", "kernels")):
        subprocess.run(["make", "-C", os.path.join(_HERE, "ref_cuda"), f"REF={reference}"], check=True, capture_output=True)
    return os.path.exists(LIB_PATH)


def available() -> bool:
    return os.path.exists(LIB_PATH)


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(LIB_PATH, mode=os.RTLD_LOCAL)
    return _lib


def _p(t: torch.Tensor):
    return C.c_void_p(t.data_ptr())


_SUFFIX = {torch.float32: "f32", torch.float64: "f64", torch.int32: "i32", torch.uint8: "u8", torch.int64: "i64"}


class Broadcast:
    """One prepared call of launch_binary_broadcast_elementwise_<S>: the four index arrays live in
    device memory, as the Rust host uploads them before the launch."""

    def __init__(self, left, lmeta, right, rmeta, dst, dmeta, op: int):
        dev = dst.device
        self.args = (left, right, dst)
        self.shape = torch.tensor(list(dmeta.shape), dtype=torch.int64, device=dev)
        self.ls = torch.tensor(list(lmeta.strides), dtype=torch.int64, device=dev)
        self.rs = torch.tensor(list(rmeta.strides), dtype=torch.int64, device=dev)
        self.ds = torch.tensor(list(dmeta.strides), dtype=torch.int64, device=dev)
        size = 1
        for n in dmeta.shape:
            size *= n
        self.fn = getattr(lib(), "launch_binary_broadcast_elementwise_" + _SUFFIX[dst.dtype])
        self.fn.restype = None
        self.call = (_p(left), _p(right), _p(dst), C.c_size_t(lmeta.offset), C.c_size_t(rmeta.offset), C.c_size_t(dmeta.offset),
                     C.c_size_t(len(dmeta.shape)), C.c_size_t(size), _p(self.ls), _p(self.rs), _p(self.ds), _p(self.shape),
                     C.c_uint8(op), C.c_uint(BLOCK))

    def __call__(self):
        self.fn(*self.call)


def scalar_contiguous(buf: torch.Tensor, op: str, value):
    """launch_<add|sub|mul|div>_contiguous_<S>(data, n, value, block)"""
    fn = getattr(lib(), f"launch_{op}_contiguous_{_SUFFIX[buf.dtype]}")
    fn.restype = None
    v = {torch.float32: C.c_float, torch.float64: C.c_double, torch.int32: C.c_int32}[buf.dtype](value)
    fn(_p(buf), C.c_size_t(buf.numel()), v, C.c_uint(BLOCK))


def reduce_flat(src: torch.Tensor, out: torch.Tensor, start: int, n: int, code: int, unbiased=True, is_std=False, norm_type=2):
    st = Settings(unbiased, is_std, norm_type)
    name = "argmax" if code in (ARGMAX, ARGMIN) else "reduce"
    fn = getattr(lib(), f"launch_flat_contiguous_{name}_{_SUFFIX[src.dtype]}")
    fn.restype = None
    fn(_p(src), _p(out), C.c_size_t(start), C.c_size_t(n), C.c_uint8(code), C.byref(st), C.c_uint(BLOCK))


def reduce_nd(src: torch.Tensor, out: torch.Tensor, offset: int, outer: int, r: int, inner: int, code: int, unbiased=True,
              is_std=False, norm_type=2):
    st = Settings(unbiased, is_std, norm_type)
    name = "nd_argmax_contiguous" if code in (ARGMAX, ARGMIN) else "nd_reduce_contiguous"
    fn = getattr(lib(), f"launch_{name}_{_SUFFIX[src.dtype]}")
    fn.restype = None
    fn(_p(src), _p(out), C.c_size_t(offset), C.c_size_t(outer), C.c_size_t(r), C.c_size_t(inner), C.c_uint8(code), C.byref(st),
       C.c_uint(BLOCK))


def alloc_failed() -> bool:
    return bool(lib().rtensors_take_cuda_alloc_error())
