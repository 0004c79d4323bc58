"""Inputs and an exact-arithmetic model for dtype conversion tests.

`model_convert` restates the Rust `as` rules that DTypeConversion applies (core/value.rs:270-290,
333-460, 770-822) with Python integers and fractions (only f64 -> f32 leans on numpy's IEEE cast) so that it checks
the C oracle independently; the CUDA kernels are then checked against the oracle.
"""
import math
import struct
from fractions import Fraction

import numpy as np

import oracle as O

INT_BITS = {O.U8: (8, False), O.I8: (8, True), O.U16: (16, False), O.I16: (16, True), O.U32: (32, False),
            O.I32: (32, True), O.U64: (64, False), O.I64: (64, True), O.U128: (128, False), O.I128: (128, True)}
ALL_CODES = list(range(13))
NAMES = {O.U8: "u8", O.I8: "i8", O.U16: "u16", O.I16: "i16", O.U32: "u32", O.U128: "u128", O.I32: "i32",
         O.U64: "u64", O.I64: "i64", O.I128: "i128", O.F32: "f32", O.F64: "f64", O.BOOL: "boolean"}


def encode(code, values) -> bytes:
    """Python values -> little-endian element bytes of dtype `code`."""
    if code == O.F32:
        return np.array(values, dtype=np.float32).tobytes()
    if code == O.F64:
        return np.array(values, dtype=np.float64).tobytes()
    if code == O.BOOL:
        return bytes(1 if v else 0 for v in values)
    bits, signed = INT_BITS[code]
    return b"".join(int(v).to_bytes(bits // 8, "little", signed=signed) for v in values)


def decode(code, raw: bytes):
    if code == O.F32:
        return list(np.frombuffer(raw, dtype=np.float32))
    if code == O.F64:
        return list(np.frombuffer(raw, dtype=np.float64))
    if code == O.BOOL:
        return [b != 0 for b in raw]
    bits, signed = INT_BITS[code]
    w = bits // 8
    return [int.from_bytes(raw[k:k + w], "little", signed=signed) for k in range(0, len(raw), w)]


def _round_half_away(x: float) -> int:
    f = Fraction(x)
    q = abs(f)
    n = q.numerator // q.denominator
    if q - n >= Fraction(1, 2):
        n += 1
    return -n if f < 0 else n


def _int_to_float_rne(v: int, mant: int, emax: int) -> float:
    """Nearest-even float with `mant` significand bits of the exact integer v; overflow -> inf."""
    if v == 0:
        return 0.0
    s, a = (-1.0 if v < 0 else 1.0), abs(v)
    drop = max(a.bit_length() - mant, 0)
    if drop:
        q, rem = a >> drop, a & ((1 << drop) - 1)
        half = 1 << (drop - 1)
        if rem > half or (rem == half and (q & 1)):
            q += 1
        a = q << drop
    if a.bit_length() > emax:
        return s * math.inf
    return s * float(a)  # exact: at most `mant` <= 53 significant bits


def model_convert(src_code, dst_code, values):
    """values: decoded source elements -> list of destination elements (ints, floats or bools)."""
    out = []
    for v in values:
        src_float = src_code in (O.F32, O.F64)
        if src_code == O.BOOL:
            v, src_float = (1 if v else 0), False
        if dst_code == O.BOOL:
            out.append(bool(v != 0))  # NaN != 0 is true
        elif dst_code in (O.F32, O.F64):
            if src_float:
                with np.errstate(over="ignore"):
                    out.append(np.float32(v) if dst_code == O.F32 else np.float64(v))
            else:
                f = _int_to_float_rne(int(v), 24 if dst_code == O.F32 else 53, 128 if dst_code == O.F32 else 1024)
                out.append(np.float32(f) if dst_code == O.F32 else np.float64(f))
        else:
            bits, signed = INT_BITS[dst_code]
            lo, hi = (-(1 << (bits - 1)), (1 << (bits - 1)) - 1) if signed else (0, (1 << bits) - 1)
            if src_float:
                x = float(v)
                if math.isnan(x):
                    out.append(0)
                elif math.isinf(x):
                    out.append(hi if x > 0 else lo)
                else:
                    out.append(min(max(_round_half_away(x), lo), hi))
            else:
                w = int(v) & ((1 << bits) - 1)
                out.append(w - (1 << bits) if signed and w >> (bits - 1) else w)
    return out


def same(dst_code, got, want) -> bool:
    """Element lists equal; floats by bit pattern except that any NaN matches any NaN."""
    if len(got) != len(want):
        return False
    if dst_code in (O.F32, O.F64):
        fmt = "<f" if dst_code == O.F32 else "<d"
        for g, w in zip(got, want):
            if math.isnan(float(g)) and math.isnan(float(w)):
                continue
            if struct.pack(fmt, float(g)) != struct.pack(fmt, float(w)):
                return False
        return True
    return list(got) == list(want)


def samples(code, rng, n_random=256):
    """Edge values plus seeded random ones for source dtype `code`."""
    if code == O.BOOL:
        return [False, True] + [bool(b) for b in rng.integers(0, 2, n_random)]
    if code in (O.F32, O.F64):
        dt = np.float32 if code == O.F32 else np.float64
        edge = [0.0, -0.0, 0.5, -0.5, 1.5, -1.5, 2.5, -2.5, 0.49999997, 1.7, -2.2, 3.0, 127.5, -128.5, 255.5, 32767.5,
                65535.5, 2147483648.0, -2147483648.0, 2147483520.0, 4294967296.0, 9.223372036854775807e18,
                -9.223372036854775808e18, 1.8446744073709552e19, 1.7014118346046923e38, -1.7014118346046923e38,
                3.0e38, -3.0e38, 1e-45, 16777217.0, math.inf, -math.inf, math.nan]
        if code == O.F64:
            edge += [3.4028234663852886e38, 3.4028235677973366e38, 1e39, -1e39, 3.402823669209385e38, 1e300, -1e300,
                     4503599627370497.5, 9007199254740993.0, 1e-320, 0.1, 16777217.0, 33554435.0]
        vals = list(np.array(edge, dtype=dt))
        mags = rng.uniform(-1, 1, n_random) * np.exp2(rng.integers(-4, 130 if code == O.F32 else 140, n_random))
        with np.errstate(over="ignore"):
            vals += list(mags.astype(dt))
        vals += list((rng.integers(-300, 300, 64) + 0.5).astype(dt))
        return vals
    bits, signed = INT_BITS[code]
    lo, hi = (-(1 << (bits - 1)), (1 << (bits - 1)) - 1) if signed else (0, (1 << bits) - 1)
    edge = [0, 1, hi, lo, hi - 1, lo + 1, 127, 128, 255, 256, (1 << 24) + 1, (1 << 24) + 3, (1 << 53) + 1, (1 << 53) + 3,
            (1 << 63) - 1, 1 << 63, (1 << 64) + 1, (1 << 100) + (1 << 76) + 1, (1 << 100) + (1 << 76), (1 << 127) + 1,
            ((1 << 24) - 1) << 104, (((1 << 24) - 1) << 104) + (1 << 103), (((1 << 25) - 1) << 103)]
    if signed:
        edge += [-e for e in edge]
    vals = [e for e in edge if lo <= e <= hi]
    for _ in range(n_random):
        width = int(rng.integers(1, bits + 1))
        v = int.from_bytes(rng.bytes(16), "little") >> (128 - width)
        if signed:
            v = v - (1 << (width - 1)) if width > 1 else -v
        vals.append(min(max(v, lo), hi))
    return vals
