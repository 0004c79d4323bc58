// Element type conversion between any two of the 13 dtypes: the device form of Backend::convert
// (backend/mod.rs:234), which the reference's CUDA backend performs as one host read and one host
// write per element (backend/cuda.rs:682-703).  Here it is one streaming kernel per (src, dst) pair.
//
// Per-element rule = DTypeConversion::convert (core/value.rs:270-290) = Rust `as` casts:
//   float -> int   : round() (half away from zero), then saturate; NaN -> 0   (core/value.rs:333-372)
//   float -> float : nearest-even                                              (core/value.rs:373-380)
//   int   -> int   : two's-complement truncation / sign extension              (core/value.rs:402-444)
//   int   -> float : nearest-even of the exact value                           (core/value.rs:445-452)
//   any   -> bool  : value != 0 (NaN is true); bool -> any : 0 or 1            (core/value.rs:381-388, 770-822)
//
// Layout: both buffers are flat and dense.  A thread converts U packs of E consecutive elements, a
// pack being 16 bytes of the wider type.  HBM-bound: sizeof(S) + sizeof(D) bytes per element.
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

#include "rtb_internal.h"

namespace rtb {
namespace {

using u128 = unsigned __int128;
using i128 = __int128;

struct BoolByte { uint8_t v; };  // the reference's `boolean`: one byte, 0 or 1

template <int CODE> struct TypeOf;
template <> struct TypeOf<RTB_U8> { using type = uint8_t; };
template <> struct TypeOf<RTB_I8> { using type = int8_t; };
template <> struct TypeOf<RTB_U16> { using type = uint16_t; };
template <> struct TypeOf<RTB_I16> { using type = int16_t; };
template <> struct TypeOf<RTB_U32> { using type = uint32_t; };
template <> struct TypeOf<RTB_U128> { using type = u128; };
template <> struct TypeOf<RTB_I32> { using type = int32_t; };
template <> struct TypeOf<RTB_U64> { using type = uint64_t; };
template <> struct TypeOf<RTB_I64> { using type = int64_t; };
template <> struct TypeOf<RTB_I128> { using type = i128; };
template <> struct TypeOf<RTB_F32> { using type = float; };
template <> struct TypeOf<RTB_F64> { using type = double; };
template <> struct TypeOf<RTB_BOOL> { using type = BoolByte; };

template <typename T> constexpr bool kIsFloat = std::is_same<T, float>::value || std::is_same<T, double>::value;
template <typename T> constexpr bool kIsBool = std::is_same<T, BoolByte>::value;
template <typename T> constexpr bool kIs128 = std::is_same<T, u128>::value || std::is_same<T, i128>::value;
template <typename T> constexpr bool kIsSigned =
    std::is_same<T, int8_t>::value || std::is_same<T, int16_t>::value || std::is_same<T, int32_t>::value ||
    std::is_same<T, int64_t>::value || std::is_same<T, i128>::value;

// 2^k as F; one past the top of the exponent range (k = 128 for f32) gives +inf
template <typename F> __device__ __forceinline__ F pow2(int k) {
    if constexpr (std::is_same<F, float>::value) return __int_as_float((127 + k) << 23);
    else return __longlong_as_double((long long)(1023 + k) << 52);
}

// Nearest-even F of an unsigned 128-bit value: keep the top 64 significant bits, fold everything
// below them into a sticky last bit (it sits at least 10 places under F's rounding position), let
// the hardware round that once, then scale by a power of two (exact, or +inf for u128 -> f32 at
// the very top, as `as` gives).
template <typename F> __device__ __forceinline__ F u128_to_float(u128 x) {
    uint64_t hi = (uint64_t)(x >> 64), lo = (uint64_t)x;
    if (hi == 0) return (F)lo;
    int sh = 64 - __clzll((long long)hi);  // 1..64 low bits to drop
    uint64_t top = sh == 64 ? hi : ((hi << (64 - sh)) | (lo >> sh));
    uint64_t dropped = sh == 64 ? lo : (lo << (64 - sh));
    top |= (dropped != 0) ? 1u : 0u;
    return (F)top * pow2<F>(sh);
}

// integral, finite, 0 <= a < 2^128
__device__ __forceinline__ u128 float_to_u128(double a) {
    if (a < pow2<double>(64)) return (u128)(uint64_t)a;
    double h = floor(a * pow2<double>(-64));  // exact
    double l = a - h * pow2<double>(64);      // exact: h * 2^64 shares a's leading bits
    return ((u128)(uint64_t)h << 64) | (u128)(uint64_t)l;
}

template <typename S, typename D> __device__ __forceinline__ D cast_one(S v) {
    if constexpr (kIsBool<S>) {
        const unsigned b = v.v ? 1u : 0u;
        if constexpr (kIsBool<D>) return v;
        else return (D)b;
    } else if constexpr (kIsBool<D>) {
        return BoolByte{(uint8_t)(v != (S)0 ? 1 : 0)};
    } else if constexpr (kIsFloat<S> && kIsFloat<D>) {
        return (D)v;
    } else if constexpr (kIsFloat<S>) {
        // float -> integer
        constexpr int bits = (int)sizeof(D) * 8;
        S r;
        if constexpr (std::is_same<S, float>::value) r = roundf(v); else r = round(v);
        if (r != r) return (D)0;
        if constexpr (kIsSigned<D>) {
            const D hi = (D)(((u128)1 << (bits - 1)) - 1), lo = (D)(-hi - 1);
            // 2^(bits-1) is representable in S for every width here (f32 reaches 2^127)
            if (r >= pow2<S>(bits - 1)) return hi;
            if (r <= -pow2<S>(bits - 1)) return lo;
            if constexpr (kIs128<D>) {
                u128 m = float_to_u128(fabs((double)r));
                return r < (S)0 ? (D)(~m + 1) : (D)m;
            } else {
                return (D)(long long)r;
            }
        } else {
            if (!(r > (S)0)) return (D)0;
            const D hi = (D)~(D)0;
            if (r >= pow2<S>(bits)) return hi;  // u128 from f32: only +inf
            if constexpr (kIs128<D>) return (D)float_to_u128((double)r);
            else return (D)(unsigned long long)r;
        }
    } else if constexpr (kIsFloat<D>) {
        // integer -> float
        if constexpr (std::is_same<S, u128>::value) {
            return u128_to_float<D>(v);
        } else if constexpr (std::is_same<S, i128>::value) {
            const bool neg = v < 0;
            u128 m = neg ? (~(u128)v + 1) : (u128)v;
            D f = u128_to_float<D>(m);
            return neg ? -f : f;
        } else {
            return (D)v;
        }
    } else {
        return (D)v;  // integer -> integer: modular
    }
}

template <typename T, int E> struct alignas((sizeof(T) * E) < 16 ? (sizeof(T) * E) : 16) Pack { T e[E]; };

// Per-thread shape, from a sweep on 2^28 elements: a pack is 16 bytes on the WIDER side, so that both
// sides of a warp's access are dense (a 64-byte-per-thread store pattern ran at 0.7 of this); a
// thread owns U packs one block-width apart, loaded before any is stored.  U = 2 is best up to a
// size ratio of 4 when widening (u8 -> f32: 6.7 TB/s against 6.6 at U = 4 and 5.5 at U = 1), 4
// beyond that and when narrowing by 4 or more.
template <typename S, typename D> constexpr int pack_elems() {
    constexpr int mx = (int)(sizeof(S) < sizeof(D) ? sizeof(D) : sizeof(S));
    return 16 / mx < 1 ? 1 : 16 / mx;
}
template <typename S, typename D> constexpr int packs_per_thread() {
    constexpr int s = (int)sizeof(S), d = (int)sizeof(D);
    if (d > s) return d / s >= 8 ? 4 : 2;
    if (s > d) return s / d >= 4 ? 4 : 2;
    return 2;
}

constexpr int kConvBlock = 256;

template <typename S, typename D, int E, int U>
__global__ void __launch_bounds__(kConvBlock) convert_kernel(const S *__restrict__ src, D *__restrict__ dst, size_t n, int packed) {
    grid_dep_sync();
    const size_t base = (size_t)blockIdx.x * (kConvBlock * E * U) + (size_t)threadIdx.x * E;
    if (packed && (size_t)(blockIdx.x + 1) * (kConvBlock * E * U) <= n) {
        Pack<S, E> in[U];
#pragma unroll
        for (int u = 0; u < U; ++u) in[u] = *reinterpret_cast<const Pack<S, E> *>(src + base + (size_t)u * kConvBlock * E);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            Pack<D, E> out;
#pragma unroll
            for (int k = 0; k < E; ++k) out.e[k] = cast_one<S, D>(in[u].e[k]);
            *reinterpret_cast<Pack<D, E> *>(dst + base + (size_t)u * kConvBlock * E) = out;
        }
    } else {
        // last tile, or buffers that are not pack-aligned: element by element, same ownership
        for (int u = 0; u < U; ++u) {
            const size_t i = base + (size_t)u * kConvBlock * E;
            for (size_t k = i; k < i + E && k < n; ++k) dst[k] = cast_one<S, D>(src[k]);
        }
    }
}

template <int SC, int DC> int convert_typed(Ctx *ctx, const void *src, void *dst, size_t n) {
    using S = typename TypeOf<SC>::type;
    using D = typename TypeOf<DC>::type;
    constexpr int E = pack_elems<S, D>(), U = packs_per_thread<S, D>();
    if (((uintptr_t)src % alignof(S)) != 0 || ((uintptr_t)dst % alignof(D)) != 0)
        return fail(RTB_ERR_INVALID, "convert: buffers must be aligned to their element type");
    const int packed = (((uintptr_t)src % alignof(Pack<S, E>)) == 0 && ((uintptr_t)dst % alignof(Pack<D, E>)) == 0) ? 1 : 0;
    const size_t tile = (size_t)kConvBlock * E * U, blocks = (n + tile - 1) / tile;
    if (blocks > 0x7fffffffull) return fail(RTB_ERR_INVALID, "convert: too many elements for one launch");
    launch_dep(ctx, (unsigned)blocks, (unsigned)kConvBlock, convert_kernel<S, D, E, U>, (const S *)src, (D *)dst, n, packed);
    return check_launch(ctx, "convert_kernel");
}

template <int SC> int convert_from(Ctx *ctx, int dst_dtype, const void *src, void *dst, size_t n) {
    switch (dst_dtype) {
        case RTB_U8: return convert_typed<SC, RTB_U8>(ctx, src, dst, n);
        case RTB_I8: return convert_typed<SC, RTB_I8>(ctx, src, dst, n);
        case RTB_U16: return convert_typed<SC, RTB_U16>(ctx, src, dst, n);
        case RTB_I16: return convert_typed<SC, RTB_I16>(ctx, src, dst, n);
        case RTB_U32: return convert_typed<SC, RTB_U32>(ctx, src, dst, n);
        case RTB_U128: return convert_typed<SC, RTB_U128>(ctx, src, dst, n);
        case RTB_I32: return convert_typed<SC, RTB_I32>(ctx, src, dst, n);
        case RTB_U64: return convert_typed<SC, RTB_U64>(ctx, src, dst, n);
        case RTB_I64: return convert_typed<SC, RTB_I64>(ctx, src, dst, n);
        case RTB_I128: return convert_typed<SC, RTB_I128>(ctx, src, dst, n);
        case RTB_F32: return convert_typed<SC, RTB_F32>(ctx, src, dst, n);
        case RTB_F64: return convert_typed<SC, RTB_F64>(ctx, src, dst, n);
        case RTB_BOOL: return convert_typed<SC, RTB_BOOL>(ctx, src, dst, n);
    }
    return fail(RTB_ERR_DTYPE, "convert: unknown destination dtype");
}

}  // namespace

int launch_convert(Ctx *ctx, int src_dtype, int dst_dtype, const void *src, void *dst, size_t n) {
    if (n == 0) return RTB_OK;
    switch (src_dtype) {
        case RTB_U8: return convert_from<RTB_U8>(ctx, dst_dtype, src, dst, n);
        case RTB_I8: return convert_from<RTB_I8>(ctx, dst_dtype, src, dst, n);
        case RTB_U16: return convert_from<RTB_U16>(ctx, dst_dtype, src, dst, n);
        case RTB_I16: return convert_from<RTB_I16>(ctx, dst_dtype, src, dst, n);
        case RTB_U32: return convert_from<RTB_U32>(ctx, dst_dtype, src, dst, n);
        case RTB_U128: return convert_from<RTB_U128>(ctx, dst_dtype, src, dst, n);
        case RTB_I32: return convert_from<RTB_I32>(ctx, dst_dtype, src, dst, n);
        case RTB_U64: return convert_from<RTB_U64>(ctx, dst_dtype, src, dst, n);
        case RTB_I64: return convert_from<RTB_I64>(ctx, dst_dtype, src, dst, n);
        case RTB_I128: return convert_from<RTB_I128>(ctx, dst_dtype, src, dst, n);
        case RTB_F32: return convert_from<RTB_F32>(ctx, dst_dtype, src, dst, n);
        case RTB_F64: return convert_from<RTB_F64>(ctx, dst_dtype, src, dst, n);
        case RTB_BOOL: return convert_from<RTB_BOOL>(ctx, dst_dtype, src, dst, n);
    }
    return fail(RTB_ERR_DTYPE, "convert: unknown source dtype");
}

}  // namespace rtb
