// Reductions for f32 / f64: flat (whole range -> one value), inner-axis (rows), outer-axis
// (columns, threads along the contiguous inner dim), fused L1 loss, and the small fused kernels
// of the autograd MLP step.  All HBM-bound: each input element is read exactly once.
//
// Accumulator semantics follow the reference CPU backend (src/ops/reduction/mod.rs:9-137):
// sum / mean start at 0, prod at 1, max at the lowest finite value with `v > acc`, min at the
// highest finite value with `v < acc` (so NaNs are skipped); mean divides by (T)(float)count
// (src/core/value.rs:54-56).  Float sums are tree-ordered here (sequential on the CPU), which is
// why sums carry a tolerance while max / min are exact.  Every kernel combines in a fixed order,
// so results are run-to-run deterministic.
#include <cfloat>
#include <type_traits>

#include "rtb_internal.h"
#include "rtb_mg.cuh"

namespace rtb {
namespace {

constexpr int kBlock = 256;
constexpr int kWarps = kBlock / 32;
// Workspace header (see workspace()): 64 completion counters for the flat kernel, then
// kMaxTileCounters per-tile counters for the axis kernels; scratch data starts after the header.
// Kernels leave every counter at zero.
constexpr size_t kTileCounterOffset = 64;      // in counters
constexpr size_t kMaxTileCounters = 16384 - 64;
constexpr size_t kWorkspaceHeader = 65536;     // bytes
// Resident CTAs per SM for the streaming reductions.  Measured on B200 with a read-only probe:
// 7.29 TB/s at 4 CTAs of 256 threads per SM, 7.14 at 8, 6.97 at 16 -- fewer concurrent streams keep
// DRAM pages open longer -- so the flat reduction runs a persistent grid of 4 CTAs per SM.
constexpr unsigned kStreamCtasPerSm = 4;
// The axis kernels end every item with a block-wide barrier; they run one CTA per item (measured
// faster than a persistent grid), bounded only by the 2^31 grid limit: 2^31 / 256 SMs.
constexpr unsigned kAxisGridCap = 1u << 22;

template <typename T> struct Limits;
template <> struct Limits<float> {
    static __host__ __device__ float lowest() { return -FLT_MAX; }
    static __host__ __device__ float highest() { return FLT_MAX; }
};
template <> struct Limits<double> {
    static __host__ __device__ double lowest() { return -DBL_MAX; }
    static __host__ __device__ double highest() { return DBL_MAX; }
};

// OP: rtb_redop without MEAN (mean = SUM + divide at the end)
template <typename T, int OP> struct Comb {
    static __device__ __forceinline__ T identity() {
        if (OP == RTB_PROD) return (T)1;
        if (OP == RTB_MAX) return Limits<T>::lowest();
        if (OP == RTB_MIN) return Limits<T>::highest();
        return (T)0;
    }
    // `a` is the running value, `b` the incoming one
    static __device__ __forceinline__ T apply(T a, T b) {
        if (OP == RTB_PROD) return a * b;
        if (OP == RTB_MAX) return b > a ? b : a;
        if (OP == RTB_MIN) return b < a ? b : a;
        return a + b;
    }
};

template <typename T> struct VecOf {
    static constexpr int N = 16 / (int)sizeof(T);
    union U {
        uint4 q;
        T e[N];
    };
};

template <typename T> __device__ __forceinline__ T shfl_down(T v, int delta) { return __shfl_down_sync(0xffffffffu, v, delta); }

template <typename T, int OP> __device__ __forceinline__ T warp_reduce(T v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = Comb<T, OP>::apply(v, shfl_down(v, d));
    return v;
}

// result valid in thread 0
template <typename T, int OP> __device__ __forceinline__ T block_reduce(T v, T *smem /* kWarps */) {
    v = warp_reduce<T, OP>(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    T out = Comb<T, OP>::identity();
    if (warp == 0) {
        out = lane < kWarps ? smem[lane] : Comb<T, OP>::identity();
#pragma unroll
        for (int d = kWarps / 2; d > 0; d >>= 1) out = Comb<T, OP>::apply(out, shfl_down(out, d));
    }
    __syncthreads();
    return out;
}

template <typename T> __device__ __forceinline__ T finish(T acc, int mean, size_t count) {
    return mean ? acc / (T)(float)count : acc;
}

// Element sources for the flat kernel.
template <typename T> struct SrcPlain {
    const T *p;
    __device__ __forceinline__ T scalar(size_t i) const { return p[i]; }
    __device__ __forceinline__ void vec(size_t iv, T out[VecOf<T>::N]) const {
        typename VecOf<T>::U u;
        u.q = reinterpret_cast<const uint4 *>(p)[iv];
#pragma unroll
        for (int j = 0; j < VecOf<T>::N; ++j) out[j] = u.e[j];
    }
    __device__ __forceinline__ uintptr_t phase() const { return (uintptr_t)p & 15u; }
    __device__ __forceinline__ SrcPlain advanced(size_t n) const { return SrcPlain{p + n}; }
    __device__ __forceinline__ bool vector_ok() const { return true; }
};

// |a - b| with an optional gradient map sign(a - b) [/ count] written on the way (L1 loss).
template <typename T> struct SrcL1 {
    const T *a;
    const T *b;
    T *g;       // may be null
    T scale;    // divisor for the gradient map (1 for the sum form)
    int same_phase;
    __device__ __forceinline__ T one(T x, T y, T *gout) const {
        T d = x - y;
        T s = d < (T)0 ? (T)-1 : (d > (T)0 ? (T)1 : (T)0);
        if (gout) *gout = s / scale;
        return sizeof(T) == 4 ? (T)fabsf((float)d) : (T)fabs((double)d);
    }
    __device__ __forceinline__ T scalar(size_t i) const { return one(a[i], b[i], g ? g + i : nullptr); }
    __device__ __forceinline__ void vec(size_t iv, T out[VecOf<T>::N]) const {
        typename VecOf<T>::U x, y, s;
        x.q = reinterpret_cast<const uint4 *>(a)[iv];
        y.q = reinterpret_cast<const uint4 *>(b)[iv];
#pragma unroll
        for (int j = 0; j < VecOf<T>::N; ++j) out[j] = one(x.e[j], y.e[j], g ? &s.e[j] : nullptr);
        if (g) reinterpret_cast<uint4 *>(g)[iv] = s.q;
    }
    __device__ __forceinline__ uintptr_t phase() const { return (uintptr_t)a & 15u; }
    __device__ __forceinline__ SrcL1 advanced(size_t n) const { return SrcL1{a + n, b + n, g ? g + n : nullptr, scale, same_phase}; }
    __device__ __forceinline__ bool vector_ok() const { return same_phase != 0; }
};

// ---- flat: grid-wide partials, the last CTA to finish folds them ---------------------------------
// ws layout: counter [0] of the header (left at zero), partials start after the header.
// Peers = MgPeers: the last CTA also exchanges this GPU's total with the other ranks over peer memory
// (rtb_mg.cuh) and `count` is the global element count; Peers = NoPeers: single GPU, count = n.
template <typename T, int OP, typename Src, typename Peers>
__global__ void __launch_bounds__(kBlock) flat_reduce_kernel(Src src, size_t n, T *partials, unsigned int *counter,
                                                             T *out, int mean, size_t count, Peers peers, size_t block_vecs) {
    grid_dep_wait();
    __shared__ T smem[kWarps];
    __shared__ bool is_last;
    constexpr int N = VecOf<T>::N;
    T acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = Comb<T, OP>::identity();

    size_t head = 0, nvec = 0;
    if (src.vector_ok()) {
        head = ((16u - (unsigned)src.phase()) & 15u) / sizeof(T);
        if (head > n) head = n;
        nvec = (n - head) / N;
    }
    const size_t tail0 = head + nvec * N;
    const Src body = src.advanced(head);
    const size_t gstride = (size_t)gridDim.x * kBlock;
    // block_vecs == 0: the grid sweeps the array together (CTA b takes vectors b*256 + t, + grid*256, ...);
    // otherwise CTA b owns the contiguous vectors [b*block_vecs, (b+1)*block_vecs)
    const size_t stride = block_vecs ? (size_t)kBlock : gstride;
    size_t i = block_vecs ? (size_t)blockIdx.x * block_vecs + threadIdx.x : (size_t)blockIdx.x * kBlock + threadIdx.x;
    if (block_vecs) {
        const size_t hi = ((size_t)blockIdx.x + 1) * block_vecs;
        if (hi < nvec) nvec = hi;
    }
    // four independent 16-byte loads in flight per thread
    for (; i + 3 * stride < nvec; i += 4 * stride) {
        T v[4][N];
#pragma unroll
        for (int u = 0; u < 4; ++u) body.vec(i + u * stride, v[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < N; ++j) acc[u] = Comb<T, OP>::apply(acc[u], v[u][j]);
    }
    for (; i < nvec; i += stride) {
        T v[N];
        body.vec(i, v);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[0] = Comb<T, OP>::apply(acc[0], v[j]);
    }
    // scalar head and tail (at most 2*(N-1) elements when vectorised; everything otherwise)
    for (size_t k = (size_t)blockIdx.x * kBlock + threadIdx.x; k < head; k += gstride)
        acc[1] = Comb<T, OP>::apply(acc[1], src.scalar(k));
    for (size_t k = tail0 + (size_t)blockIdx.x * kBlock + threadIdx.x; k < n; k += gstride)
        acc[2] = Comb<T, OP>::apply(acc[2], src.scalar(k));

    grid_dep_launch();  // streaming done: the next kernel of the stream may start to move in
    T v = Comb<T, OP>::apply(Comb<T, OP>::apply(acc[0], acc[1]), Comb<T, OP>::apply(acc[2], acc[3]));
    v = block_reduce<T, OP>(v, smem);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = v;
        __threadfence();
        unsigned int done = atomicAdd(counter, 1u);
        is_last = (done == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    T t = Comb<T, OP>::identity();
    for (unsigned int k = threadIdx.x; k < gridDim.x; k += kBlock) t = Comb<T, OP>::apply(t, __ldcg(partials + k));
    t = block_reduce<T, OP>(t, smem);
    if constexpr (std::is_same<Peers, MgPeers>::value)
        t = mg_exchange_scalar<T>(t, peers, [](T a, T b) { return Comb<T, OP>::apply(a, b); });
    if (threadIdx.x == 0) {
        out[0] = finish(t, mean, count);
        *counter = 0;  // ready for the next launch on this stream
    }
}

// ---- inner axis (inner == 1): src is [rows, R], one value per row --------------------------------
// GROUP threads cooperate on a row (32 = a warp, 256 = the CTA); split > 1 cuts R into `split`
// chunks whose partial results go to dst[row * split + chunk] for a second pass.
template <typename T, int OP, int GROUP>
__global__ void __launch_bounds__(kBlock) row_reduce_kernel(const T *src, size_t rows, size_t R, ptrdiff_t pitch,
                                                            size_t split, T *dst, int mean, size_t count) {
    grid_dep_sync();
    __shared__ T smem[kWarps];
    constexpr int N = VecOf<T>::N;
    constexpr int rows_per_block = kBlock / GROUP;
    const int g = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
    const size_t items = rows * split;
    const size_t per = (R + split - 1) / split;
    // persistent: a CTA walks items b, b + grid, ... (the grid is capped at a few CTAs per SM)
    for (size_t first = (size_t)blockIdx.x * rows_per_block; first < items; first += (size_t)gridDim.x * rows_per_block) {
        const size_t item = first + g;  // (row, chunk)
        const bool live = item < items;
        T acc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u] = Comb<T, OP>::identity();
        if (live) {
            const size_t row = item / split, chunk = item % split;
            const size_t k0 = chunk * per, k1 = k0 + per < R ? k0 + per : R;
            const T *p = src + (ptrdiff_t)row * pitch;  // pitch = elements between rows (R when dense)
            // vector body over the 16-byte aligned part of [k0, k1)
            size_t a0 = k0 + (((16u - (unsigned)((uintptr_t)(p + k0) & 15u)) & 15u) / sizeof(T));
            if (a0 > k1) a0 = k1;
            const size_t nvec = (k1 - a0) / N;
            const uint4 *pv = reinterpret_cast<const uint4 *>(p + a0);
            size_t i = t;
            for (; i + 7 * GROUP < nvec; i += 8 * GROUP) {  // eight 16-byte loads in flight per thread
                typename VecOf<T>::U v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u].q = pv[i + u * GROUP];
#pragma unroll
                for (int u = 0; u < 8; ++u)
#pragma unroll
                    for (int j = 0; j < N; ++j) acc[u & 3] = Comb<T, OP>::apply(acc[u & 3], v[u].e[j]);
            }
            for (; i + 3 * GROUP < nvec; i += 4 * GROUP) {
                typename VecOf<T>::U v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u].q = pv[i + u * GROUP];
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int j = 0; j < N; ++j) acc[u] = Comb<T, OP>::apply(acc[u], v[u].e[j]);
            }
            for (; i < nvec; i += GROUP) {
                typename VecOf<T>::U v;
                v.q = pv[i];
#pragma unroll
                for (int j = 0; j < N; ++j) acc[0] = Comb<T, OP>::apply(acc[0], v.e[j]);
            }
            for (size_t k = k0 + t; k < a0; k += GROUP) acc[1] = Comb<T, OP>::apply(acc[1], p[k]);
            for (size_t k = a0 + nvec * N + t; k < k1; k += GROUP) acc[2] = Comb<T, OP>::apply(acc[2], p[k]);
        }
        T v = Comb<T, OP>::apply(Comb<T, OP>::apply(acc[0], acc[1]), Comb<T, OP>::apply(acc[2], acc[3]));
        if (GROUP == 32) {
            v = warp_reduce<T, OP>(v);
        } else {
            v = block_reduce<T, OP>(v, smem);
        }
        if (t == 0 && live) dst[item] = split == 1 ? finish(v, mean, count) : v;
    }
}

// ---- outer axis (inner > 1): src is [outer, R, inner]; threads run along inner ---------------------
// CTA = TX lanes along inner (VW columns each) x TY = 256/TX lanes along R (TX = 32 in use).
// `split` cuts R into chunks, one CTA each.  With split > 1 every CTA stores its partial row, and the last CTA of a column tile to
// finish (per-tile completion counter) folds the `split` partial rows in chunk order -- one launch,
// and the fold order does not depend on which CTA came last.
template <bool CG, typename T> __device__ __forceinline__ uint4 ld128(const T *p) {
    return CG ? __ldcg(reinterpret_cast<const uint4 *>(p)) : *reinterpret_cast<const uint4 *>(p);
}
template <bool CG, typename T> __device__ __forceinline__ T ld1(const T *p) { return CG ? __ldcg(p) : *p; }

// CG: read through L2 only (__ldcg) -- used when the rows are chunk partials that other CTAs of
// this launch have just written, which an L1 line fetched earlier on this SM could hide
template <typename T, int OP, int VW, int TY, bool CG = false>
__device__ __forceinline__ void col_accumulate(const T *p, ptrdiff_t row_stride, size_t k0, size_t k1, int ly, T acc[VW]) {
    constexpr int B = 8;  // rows in flight per thread
    size_t k = k0 + ly;
    if (VW > 1) {
        for (; k + (B - 1) * TY < k1; k += B * TY) {
            typename VecOf<T>::U v[B];
#pragma unroll
            for (int u = 0; u < B; ++u) v[u].q = ld128<CG>(p + (ptrdiff_t)(k + TY * u) * row_stride);
#pragma unroll
            for (int u = 0; u < B; ++u)
#pragma unroll
                for (int j = 0; j < VW; ++j) acc[j] = Comb<T, OP>::apply(acc[j], v[u].e[j]);
        }
        for (; k < k1; k += TY) {
            typename VecOf<T>::U v;
            v.q = ld128<CG>(p + (ptrdiff_t)k * row_stride);
#pragma unroll
            for (int j = 0; j < VW; ++j) acc[j] = Comb<T, OP>::apply(acc[j], v.e[j]);
        }
    } else {
        for (; k + (B - 1) * TY < k1; k += B * TY) {
            T v[B];
#pragma unroll
            for (int u = 0; u < B; ++u) v[u] = ld1<CG>(p + (ptrdiff_t)(k + TY * u) * row_stride);
#pragma unroll
            for (int u = 0; u < B; ++u) acc[0] = Comb<T, OP>::apply(acc[0], v[u]);
        }
        for (; k < k1; k += TY) acc[0] = Comb<T, OP>::apply(acc[0], ld1<CG>(p + (ptrdiff_t)k * row_stride));
    }
}

// TY partial rows of the tile (in shared memory) -> 1; thread c owns column c
template <typename T, int OP, int TW, int TY>
__device__ __forceinline__ T col_combine(const T (*smem)[TW + 1], int c) {
    T v = smem[0][c];
#pragma unroll
    for (int y = 1; y < TY; ++y) v = Comb<T, OP>::apply(v, smem[y][c]);
    return v;
}

template <typename T, int OP, int VW, int TX>
__global__ void __launch_bounds__(kBlock) col_reduce_kernel(const T *src, size_t outer, size_t R, size_t inner,
                                                            ptrdiff_t outer_stride, ptrdiff_t row_stride,
                                                            size_t split, size_t col_tiles, T *partial,
                                                            unsigned int *counters, T *dst, int mean, size_t count) {
    grid_dep_wait();
    constexpr int TY = kBlock / TX;
    constexpr int TW = TX * VW;  // columns per tile
    __shared__ T smem[TY][TW + 1];
    __shared__ bool is_last;
    const int lx = threadIdx.x % TX, ly = threadIdx.x / TX;
    const size_t items = outer * split * col_tiles;
    const size_t per = (R + split - 1) / split;
    // a CTA walks items b, b + grid, ... (normally one); neighbouring CTAs read neighbouring column
    // tiles of the same rows
    for (size_t b = blockIdx.x; b < items; b += gridDim.x) {
        size_t q = b;
        const size_t tile = q % col_tiles; q /= col_tiles;
        const size_t chunk = q % split;
        const size_t o = q / split;
        const size_t col = (tile * TX + lx) * VW;
        const size_t k0 = chunk * per, k1 = k0 + per < R ? k0 + per : R;
        T acc[VW];
#pragma unroll
        for (int j = 0; j < VW; ++j) acc[j] = Comb<T, OP>::identity();
        // element (o, k, i) of the source sits at o*outer_stride + k*row_stride + i (dense: R*inner, inner)
        if (col < inner && k0 < k1)
            col_accumulate<T, OP, VW, TY>(src + (ptrdiff_t)o * outer_stride + (ptrdiff_t)col, row_stride, k0, k1, ly, acc);
        grid_dep_launch();
#pragma unroll
        for (int j = 0; j < VW; ++j) smem[ly][lx * VW + j] = acc[j];
        __syncthreads();
        for (int c = threadIdx.x; c < TW; c += kBlock) {
            T v = col_combine<T, OP, TW, TY>(smem, c);
            const size_t gc = tile * TW + c;
            if (gc < inner) {
                if (split == 1) dst[o * inner + gc] = finish(v, mean, count);
                else partial[(o * split + chunk) * inner + gc] = v;
            }
        }
        if (split == 1) {
            __syncthreads();  // smem is reused by the next item
            continue;
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned int done = atomicAdd(counters + o * col_tiles + tile, 1u);
            is_last = done == (unsigned int)split - 1u;
        }
        __syncthreads();
        if (!is_last) continue;  // uniform per CTA
        __threadfence();
#pragma unroll
        for (int j = 0; j < VW; ++j) acc[j] = Comb<T, OP>::identity();
        if (col < inner) col_accumulate<T, OP, VW, TY, true>(partial + (o * split) * inner + col, (ptrdiff_t)inner, 0, split, ly, acc);
#pragma unroll
        for (int j = 0; j < VW; ++j) smem[ly][lx * VW + j] = acc[j];
        __syncthreads();
        for (int c = threadIdx.x; c < TW; c += kBlock) {
            T v = col_combine<T, OP, TW, TY>(smem, c);
            const size_t gc = tile * TW + c;
            if (gc < inner) dst[o * inner + gc] = finish(v, mean, count);
        }
        if (threadIdx.x == 0) counters[o * col_tiles + tile] = 0;  // ready for the next launch
        __syncthreads();
    }
}

// ---- fused broadcast + axis reduce: dst[a, b] = reduce_k f(l[a, k, b], r[a, k, b]) ------------------
// The binary op is applied on the fly and never written out (config 1: (4096,1) + (1,4096) followed
// by sum over axis 1 touches 48 KiB instead of a 64 MiB intermediate).  Each operand is addressed
// as a*sa + k*sk + b*sb with its own strides (0 on broadcast dims).  Two layouts: lanes along b
// when the output row is wide (coalesced in b), a warp per output with lanes along k otherwise.
struct Strides3 {
    ptrdiff_t a, k, b;
};

template <typename T> __device__ __forceinline__ T apply_binop(int op, T x, T y) {
    switch (op) {
        case RTB_ADD: return x + y;
        case RTB_SUB: return x - y;
        case RTB_MUL: return x * y;
        default: return x / y;
    }
}

template <typename T, int OP, bool WIDE>
__global__ void __launch_bounds__(kBlock) bcast_reduce_kernel(const T *l, Strides3 sl, const T *r, Strides3 sr, int binop,
                                                              size_t A, size_t R, size_t B, size_t split, T *dst, int mean) {
    grid_dep_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (WIDE) {
        // CTA = 32 outputs along b x 8 lanes along k, one CTA per (a, chunk of k, b tile); with
        // split > 1, dst holds [A, split, B] partial results for a second pass
        __shared__ T smem[kWarps][33];
        const size_t b_tiles = (B + 31) / 32;
        const size_t per = (R + split - 1) / split;
        for (size_t item = blockIdx.x; item < A * split * b_tiles; item += gridDim.x) {
            size_t q = item;
            const size_t b = (q % b_tiles) * 32 + lane; q /= b_tiles;
            const size_t chunk = q % split;
            const size_t a = q / split;
            const size_t k0 = chunk * per, k1 = k0 + per < R ? k0 + per : R;
            T acc = Comb<T, OP>::identity();
            if (b < B) {
                const T *pl = l + (ptrdiff_t)a * sl.a + (ptrdiff_t)b * sl.b;
                const T *pr = r + (ptrdiff_t)a * sr.a + (ptrdiff_t)b * sr.b;
                size_t k = k0 + warp;
                for (; k + 3 * kWarps < k1; k += 4 * kWarps) {
                    T x[4], y[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        x[u] = pl[(ptrdiff_t)(k + u * kWarps) * sl.k];
                        y[u] = pr[(ptrdiff_t)(k + u * kWarps) * sr.k];
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc = Comb<T, OP>::apply(acc, apply_binop(binop, x[u], y[u]));
                }
                for (; k < k1; k += kWarps) acc = Comb<T, OP>::apply(acc, apply_binop(binop, pl[(ptrdiff_t)k * sl.k], pr[(ptrdiff_t)k * sr.k]));
            }
            smem[warp][lane] = acc;
            __syncthreads();
            if (warp == 0) {
                T v = smem[0][lane];
#pragma unroll
                for (int y = 1; y < kWarps; ++y) v = Comb<T, OP>::apply(v, smem[y][lane]);
                if (b < B) dst[(a * split + chunk) * B + b] = split == 1 ? finish(v, mean, R) : v;
            }
            __syncthreads();
        }
    } else {
        // a warp per output element, lanes along k
        const size_t outputs = A * B;
        for (size_t o = (size_t)blockIdx.x * kWarps + warp; o < outputs; o += (size_t)gridDim.x * kWarps) {
            const size_t a = o / B, b = o % B;
            const T *pl = l + (ptrdiff_t)a * sl.a + (ptrdiff_t)b * sl.b;
            const T *pr = r + (ptrdiff_t)a * sr.a + (ptrdiff_t)b * sr.b;
            T acc[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[u] = Comb<T, OP>::identity();
            // cursors advance by a precomputed step, so the loop body has no 64-bit multiplies
            const ptrdiff_t dl = sl.k * 32, dr = sr.k * 32;
            const T *ql = pl + (ptrdiff_t)lane * sl.k, *qr = pr + (ptrdiff_t)lane * sr.k;
            size_t k = lane;
            for (; k + 96 < R; k += 128, ql += 4 * dl, qr += 4 * dr) {
                T x[4], y[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    x[u] = ql[u * dl];
                    y[u] = qr[u * dr];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[u] = Comb<T, OP>::apply(acc[u], apply_binop(binop, x[u], y[u]));
            }
            for (; k < R; k += 32, ql += dl, qr += dr) acc[0] = Comb<T, OP>::apply(acc[0], apply_binop(binop, *ql, *qr));
            T v = Comb<T, OP>::apply(Comb<T, OP>::apply(acc[0], acc[1]), Comb<T, OP>::apply(acc[2], acc[3]));
            v = warp_reduce<T, OP>(v);
            if (lane == 0) dst[o] = finish(v, mean, R);
        }
    }
}

// Both operands either contiguous or invariant along k: a warp per output element, every lane
// reading 128-bit vectors of consecutive k; an invariant operand is read once per output.
template <typename T, int OP, int BINOP>
__global__ void __launch_bounds__(kBlock) bcast_reduce_kvec_kernel(const T *l, Strides3 sl, const T *r, Strides3 sr, size_t A,
                                                                   size_t R, size_t B, T *dst, int mean) {
    grid_dep_sync();
    constexpr int N = VecOf<T>::N;
    using U = typename VecOf<T>::U;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t outputs = A * B, nvec = R / N;
    for (size_t o = (size_t)blockIdx.x * kWarps + warp; o < outputs; o += (size_t)gridDim.x * kWarps) {
        const size_t a = o / B, b = o % B;
        const T *pl = l + (ptrdiff_t)a * sl.a + (ptrdiff_t)b * sl.b;
        const T *pr = r + (ptrdiff_t)a * sr.a + (ptrdiff_t)b * sr.b;
        U x[2], y[2];
        if (sl.k == 0) {
#pragma unroll
            for (int e = 0; e < N; ++e) x[0].e[e] = x[1].e[e] = pl[0];
        }
        if (sr.k == 0) {
#pragma unroll
            for (int e = 0; e < N; ++e) y[0].e[e] = y[1].e[e] = pr[0];
        }
        T acc[2][N];
#pragma unroll
        for (int e = 0; e < N; ++e) acc[0][e] = acc[1][e] = Comb<T, OP>::identity();
        size_t kv = lane;
        for (; kv + 32 < nvec; kv += 64) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (sl.k) x[u].q = reinterpret_cast<const uint4 *>(pl)[kv + 32 * u];
                if (sr.k) y[u].q = reinterpret_cast<const uint4 *>(pr)[kv + 32 * u];
            }
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int e = 0; e < N; ++e) acc[u][e] = Comb<T, OP>::apply(acc[u][e], apply_binop(BINOP, x[u].e[e], y[u].e[e]));
        }
        if (kv < nvec) {
            if (sl.k) x[0].q = reinterpret_cast<const uint4 *>(pl)[kv];
            if (sr.k) y[0].q = reinterpret_cast<const uint4 *>(pr)[kv];
#pragma unroll
            for (int e = 0; e < N; ++e) acc[0][e] = Comb<T, OP>::apply(acc[0][e], apply_binop(BINOP, x[0].e[e], y[0].e[e]));
        }
        T v = Comb<T, OP>::apply(acc[0][0], acc[1][0]);
#pragma unroll
        for (int e = 1; e < N; ++e) v = Comb<T, OP>::apply(v, Comb<T, OP>::apply(acc[0][e], acc[1][e]));
        v = warp_reduce<T, OP>(v);
        if (lane == 0) dst[o] = finish(v, mean, R);
    }
}

// Both operands either contiguous or invariant along b: a CTA covers 32 x N consecutive outputs
// (every lane one 128-bit vector of them) with its 8 warps along k; an operand that is also
// invariant along k is read once.  With split > 1, dst holds [A, split, B] partial rows.
template <typename T, int OP, int BINOP>
__global__ void __launch_bounds__(kBlock) bcast_reduce_bvec_kernel(const T *l, Strides3 sl, const T *r, Strides3 sr, size_t A,
                                                                   size_t R, size_t B, size_t split, T *dst, int mean) {
    grid_dep_sync();
    constexpr int N = VecOf<T>::N;
    using U = typename VecOf<T>::U;
    __shared__ uint4 smem[kWarps][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t bvecs = B / N, b_tiles = (bvecs + 31) / 32;
    const size_t per = (R + split - 1) / split;
    auto fetch = [&](U &v, const T *p, ptrdiff_t sb) {
        if (sb) {
            v.q = *reinterpret_cast<const uint4 *>(p);
        } else {
            const T s = *p;
#pragma unroll
            for (int e = 0; e < N; ++e) v.e[e] = s;
        }
    };
    for (size_t item = blockIdx.x; item < A * split * b_tiles; item += gridDim.x) {
        size_t q = item;
        const size_t bv = (q % b_tiles) * 32 + lane; q /= b_tiles;
        const size_t chunk = q % split;
        const size_t a = q / split;
        const size_t k0 = chunk * per, k1 = k0 + per < R ? k0 + per : R;
        U acc;
#pragma unroll
        for (int e = 0; e < N; ++e) acc.e[e] = Comb<T, OP>::identity();
        if (bv < bvecs) {
            const T *pl = l + (ptrdiff_t)a * sl.a + (ptrdiff_t)(bv * N) * sl.b;
            const T *pr = r + (ptrdiff_t)a * sr.a + (ptrdiff_t)(bv * N) * sr.b;
            U x[2], y[2];
            if (sl.k == 0) { fetch(x[0], pl, sl.b); x[1] = x[0]; }
            if (sr.k == 0) { fetch(y[0], pr, sr.b); y[1] = y[0]; }
            size_t k = k0 + warp;
            for (; k + kWarps < k1; k += 2 * kWarps) {
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (sl.k) fetch(x[u], pl + (ptrdiff_t)(k + u * kWarps) * sl.k, sl.b);
                    if (sr.k) fetch(y[u], pr + (ptrdiff_t)(k + u * kWarps) * sr.k, sr.b);
                }
#pragma unroll
                for (int u = 0; u < 2; ++u)
#pragma unroll
                    for (int e = 0; e < N; ++e) acc.e[e] = Comb<T, OP>::apply(acc.e[e], apply_binop(BINOP, x[u].e[e], y[u].e[e]));
            }
            if (k < k1) {
                if (sl.k) fetch(x[0], pl + (ptrdiff_t)k * sl.k, sl.b);
                if (sr.k) fetch(y[0], pr + (ptrdiff_t)k * sr.k, sr.b);
#pragma unroll
                for (int e = 0; e < N; ++e) acc.e[e] = Comb<T, OP>::apply(acc.e[e], apply_binop(BINOP, x[0].e[e], y[0].e[e]));
            }
        }
        smem[warp][lane] = acc.q;
        __syncthreads();
        if (warp == 0) {
            U v;
            v.q = smem[0][lane];
#pragma unroll
            for (int w = 1; w < kWarps; ++w) {
                U o;
                o.q = smem[w][lane];
#pragma unroll
                for (int e = 0; e < N; ++e) v.e[e] = Comb<T, OP>::apply(v.e[e], o.e[e]);
            }
            if (bv < bvecs) {
                if (split == 1) {
#pragma unroll
                    for (int e = 0; e < N; ++e) v.e[e] = finish(v.e[e], mean, R);
                }
                *reinterpret_cast<uint4 *>(dst + (a * split + chunk) * B + bv * N) = v.q;
            }
        }
        __syncthreads();
    }
}

// ---- fused MLP pieces ----------------------------------------------------------------------------
__global__ void __launch_bounds__(kBlock) relu_mask_kernel(float *x, float *mask, size_t n) {
    grid_dep_sync();
    const size_t nvec = n / 4;
    const size_t stride = (size_t)gridDim.x * kBlock;
    for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < nvec; i += stride) {
        float4 v = reinterpret_cast<float4 *>(x)[i];
        float4 m, o;
        m.x = v.x > 0.f ? 1.f : 0.f; o.x = v.x > 0.f ? v.x : 0.f;
        m.y = v.y > 0.f ? 1.f : 0.f; o.y = v.y > 0.f ? v.y : 0.f;
        m.z = v.z > 0.f ? 1.f : 0.f; o.z = v.z > 0.f ? v.z : 0.f;
        m.w = v.w > 0.f ? 1.f : 0.f; o.w = v.w > 0.f ? v.w : 0.f;
        reinterpret_cast<float4 *>(x)[i] = o;
        reinterpret_cast<float4 *>(mask)[i] = m;
    }
    for (size_t k = nvec * 4 + (size_t)blockIdx.x * kBlock + threadIdx.x; k < n; k += stride) {
        float v = x[k];
        mask[k] = v > 0.f ? 1.f : 0.f;
        x[k] = v > 0.f ? v : 0.f;
    }
}

// z[r, c] = relu(z[r, c] + bias[c]) in place, mask[r, c] = (z[r, c] + bias[c]) > 0 ? 1 : 0: the bias
// broadcast add, relu_inplace and its gradient map (three launches and 5 passes over the
// activations when run one by one) as ONE pass that reads z once and writes z and mask.  A thread keeps
// its VW bias values in registers and walks kRowsPerCta rows, all loads issued before the first store.
// The sum is the same single IEEE add and the comparisons the same `x > 0` as in the separate calls.
constexpr int kBiasRows = 8;
template <typename T, int VW>
__global__ void __launch_bounds__(kBlock) bias_relu_mask_kernel(T *z, const T *bias, T *mask, size_t rows, size_t cols,
                                                                size_t col_blocks) {
    grid_dep_sync();
    using U = typename VecOf<T>::U;
    const size_t cb = blockIdx.x % col_blocks, rb = blockIdx.x / col_blocks;
    const size_t c = (cb * kBlock + threadIdx.x) * VW;
    if (c >= cols) return;
    const size_t r0 = rb * kBiasRows;
    T b[VW], v[kBiasRows][VW];
    if (VW > 1) {
        U u;
        u.q = __ldg(reinterpret_cast<const uint4 *>(bias + c));
#pragma unroll
        for (int j = 0; j < VW; ++j) b[j] = u.e[j];
    } else {
        b[0] = __ldg(bias + c);
    }
#pragma unroll
    for (int k = 0; k < kBiasRows; ++k) {
        if (r0 + k < rows) {
            if (VW > 1) {
                U u;
                u.q = *reinterpret_cast<const uint4 *>(z + (r0 + k) * cols + c);
#pragma unroll
                for (int j = 0; j < VW; ++j) v[k][j] = u.e[j];
            } else {
                v[k][0] = z[(r0 + k) * cols + c];
            }
        }
    }
#pragma unroll
    for (int k = 0; k < kBiasRows; ++k) {
        if (r0 + k < rows) {
            U o, m;
#pragma unroll
            for (int j = 0; j < VW; ++j) {
                const T t = v[k][j] + b[j];
                o.e[j] = t > (T)0 ? t : (T)0;
                m.e[j] = t > (T)0 ? (T)1 : (T)0;
            }
            if (VW > 1) {
                *reinterpret_cast<uint4 *>(z + (r0 + k) * cols + c) = o.q;
                *reinterpret_cast<uint4 *>(mask + (r0 + k) * cols + c) = m.q;
            } else {
                z[(r0 + k) * cols + c] = o.e[0];
                mask[(r0 + k) * cols + c] = m.e[0];
            }
        }
    }
}

__global__ void __launch_bounds__(kBlock) sgd_kernel(float *p, const float *g, float lr, size_t n) {
    grid_dep_sync();
    const size_t nvec = n / 4;
    const size_t stride = (size_t)gridDim.x * kBlock;
    for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < nvec; i += stride) {
        float4 w = reinterpret_cast<float4 *>(p)[i];
        float4 q = reinterpret_cast<const float4 *>(g)[i];
        // two roundings, as `update = grad * lr; param -= update` on the CPU (no FMA)
        w.x = w.x - __fmul_rn(q.x, lr); w.y = w.y - __fmul_rn(q.y, lr);
        w.z = w.z - __fmul_rn(q.z, lr); w.w = w.w - __fmul_rn(q.w, lr);
        reinterpret_cast<float4 *>(p)[i] = w;
    }
    for (size_t k = nvec * 4 + (size_t)blockIdx.x * kBlock + threadIdx.x; k < n; k += stride)
        p[k] = p[k] - __fmul_rn(g[k], lr);
}

// f64 forms of the two kernels above (the reference's relu map and SGD::step are generic over the
// float type); 2 elements per 128-bit access
__global__ void __launch_bounds__(kBlock) relu_mask_f64_kernel(double *x, double *mask, size_t n) {
    grid_dep_sync();
    const size_t nvec = n / 2;
    const size_t stride = (size_t)gridDim.x * kBlock;
    for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < nvec; i += stride) {
        double2 v = reinterpret_cast<const double2 *>(x)[i];
        double2 m, o;
        m.x = v.x > 0.0 ? 1.0 : 0.0; o.x = v.x > 0.0 ? v.x : 0.0;
        m.y = v.y > 0.0 ? 1.0 : 0.0; o.y = v.y > 0.0 ? v.y : 0.0;
        reinterpret_cast<double2 *>(x)[i] = o;
        reinterpret_cast<double2 *>(mask)[i] = m;
    }
    if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0) {
        double v = x[n - 1];
        mask[n - 1] = v > 0.0 ? 1.0 : 0.0;
        x[n - 1] = v > 0.0 ? v : 0.0;
    }
}

__global__ void __launch_bounds__(kBlock) sgd_f64_kernel(double *p, const double *g, double lr, size_t n) {
    grid_dep_sync();
    const size_t nvec = n / 2;
    const size_t stride = (size_t)gridDim.x * kBlock;
    for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < nvec; i += stride) {
        double2 w = reinterpret_cast<double2 *>(p)[i];
        double2 q = reinterpret_cast<const double2 *>(g)[i];
        w.x = w.x - __dmul_rn(q.x, lr);  // two roundings, no FMA
        w.y = w.y - __dmul_rn(q.y, lr);
        reinterpret_cast<double2 *>(p)[i] = w;
    }
    if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0) p[n - 1] = p[n - 1] - __dmul_rn(g[n - 1], lr);
}

__global__ void __launch_bounds__(kBlock) u8_f32_kernel(const uint8_t *src, float *dst, float divisor, size_t n) {
    grid_dep_sync();
    const size_t nvec = n / 4;
    const size_t stride = (size_t)gridDim.x * kBlock;
    for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < nvec; i += stride) {
        uchar4 v = reinterpret_cast<const uchar4 *>(src)[i];
        float4 o;
        o.x = __fdiv_rn((float)v.x, divisor); o.y = __fdiv_rn((float)v.y, divisor);
        o.z = __fdiv_rn((float)v.z, divisor); o.w = __fdiv_rn((float)v.w, divisor);
        reinterpret_cast<float4 *>(dst)[i] = o;
    }
    for (size_t k = nvec * 4 + (size_t)blockIdx.x * kBlock + threadIdx.x; k < n; k += stride)
        dst[k] = __fdiv_rn((float)src[k], divisor);
}

// ---- host side -----------------------------------------------------------------------------------
unsigned grid_for(Ctx *ctx, size_t work_items, unsigned per_sm) {
    size_t cap = (size_t)ctx->sm_count * per_sm;
    size_t g = work_items < cap ? work_items : cap;
    return (unsigned)(g ? g : 1);
}

template <typename T, int OP, typename Src, typename Peers = NoPeers>
int flat_launch(Ctx *ctx, Src src, size_t n, T *out, int mean, size_t count = 0, Peers peers = Peers{}) {
    if (!std::is_same<Peers, MgPeers>::value) count = n;
    constexpr int N = VecOf<T>::N;
    // one CTA per 4 KiB-vector-iterations, capped at 4 CTAs per SM: a read-bandwidth probe on B200 gives
    // 7.29 TB/s at 4 CTAs/SM, 7.14 at 8 and 6.97 at 16 (fewer concurrent streams, better DRAM locality)
    size_t items = (n / N + (size_t)kBlock * 4 - 1) / ((size_t)kBlock * 4);
    unsigned grid = grid_for(ctx, items, kStreamCtasPerSm);
    // Plain inputs of more than one wave of 32 KiB blocks: one CTA per contiguous block, many waves, the block
    // size doubled until at most 16384 blocks remain (their partials are folded by one CTA).  The hardware's
    // CTA scheduler then evens out the SMs, which the one-wave sweep cannot: measured 2^25 f32 26.2 -> 23.8 us,
    // 2^26 46.4 -> 42.6, 2^27 84.7 -> 79.5, 2^28 158.8 -> 152.8, 2^30 595.4 -> 590.4.  The two-stream L1
    // source gains nothing and keeps the sweep.
    size_t block_vecs = 0;
    if (std::is_same<Src, SrcPlain<T>>::value) {
        size_t bv = 2048;
        size_t blocks = (n / N + bv - 1) / bv;
        if (blocks > grid) {
            while (blocks > 16384) {
                bv *= 2;
                blocks = (n / N + bv - 1) / bv;
            }
            block_vecs = bv;
            grid = (unsigned)blocks;
        }
    }
    void *ws = nullptr;
    int rc = workspace(ctx, (size_t)grid * sizeof(T), &ws);
    if (rc != RTB_OK) return rc;
    unsigned int *counter = reinterpret_cast<unsigned int *>(ws);
    T *partials = reinterpret_cast<T *>(reinterpret_cast<char *>(ws) + kWorkspaceHeader);
    launch_dep(ctx, grid, kBlock, flat_reduce_kernel<T, OP, Src, Peers>, src, n, partials, counter, out, mean, count, peers, block_vecs);
    return check_launch(ctx, "flat_reduce_kernel");
}

template <typename T, typename Src, typename Peers = NoPeers>
int flat_by_op(Ctx *ctx, int redop, Src src, size_t n, T *out, size_t count = 0, Peers peers = Peers{}) {
    switch (redop) {
        case RTB_SUM: return flat_launch<T, RTB_SUM, Src, Peers>(ctx, src, n, out, 0, count, peers);
        case RTB_MEAN: return flat_launch<T, RTB_SUM, Src, Peers>(ctx, src, n, out, 1, count, peers);
        case RTB_PROD: return flat_launch<T, RTB_PROD, Src, Peers>(ctx, src, n, out, 0, count, peers);
        case RTB_MAX: return flat_launch<T, RTB_MAX, Src, Peers>(ctx, src, n, out, 0, count, peers);
        case RTB_MIN: return flat_launch<T, RTB_MIN, Src, Peers>(ctx, src, n, out, 0, count, peers);
    }
    return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
}

template <typename T, int OP>
int rows_launch(Ctx *ctx, const T *src, size_t rows, size_t R, ptrdiff_t pitch, T *dst, int mean) {
    // few long rows: cut each row into chunks so every SM has work, then fold the chunks
    size_t split = 1;
    const size_t min_items = (size_t)ctx->sm_count * 4;
    if (rows < min_items && R >= 8192) {
        split = (min_items + rows - 1) / rows;
        size_t max_split = R / 4096;
        if (split > max_split) split = max_split;
        if (split < 1) split = 1;
    }
    T *target = dst;
    if (split > 1) {
        void *ws = nullptr;
        int rc = workspace(ctx, rows * split * sizeof(T), &ws);
        if (rc != RTB_OK) return rc;
        target = reinterpret_cast<T *>(reinterpret_cast<char *>(ws) + kWorkspaceHeader);
    }
    const size_t items = rows * split;
    const size_t chunk_len = (R + split - 1) / split;
    // One CTA (or warp) per row.  A persistent grid of 4 CTAs/SM was measured and is slower here
    // (8192x8192 axis 1: 5.9 vs 6.3 TB/s): every row ends in a block-wide tree reduction, and with few
    // resident CTAs nothing hides that barrier.  The kernel still loops, so any grid size is legal.
    if (chunk_len >= 1024) {
        unsigned grid = grid_for(ctx, items, kAxisGridCap);
        launch_dep(ctx, grid, kBlock, row_reduce_kernel<T, OP, kBlock>, src, rows, R, pitch, split, target, mean, R);
    } else {
        unsigned grid = grid_for(ctx, (items + kWarps - 1) / kWarps, kAxisGridCap);
        launch_dep(ctx, grid, kBlock, row_reduce_kernel<T, OP, 32>, src, rows, R, pitch, split, target, mean, R);
    }
    int rc = check_launch(ctx, "row_reduce_kernel");
    if (rc != RTB_OK || split == 1) return rc;
    unsigned fold_grid = grid_for(ctx, (rows + kWarps - 1) / kWarps, kAxisGridCap);
    launch_dep(ctx, fold_grid, kBlock, row_reduce_kernel<T, OP, 32>, target, rows, split, (ptrdiff_t)split, 1, dst, mean, R);
    return check_launch(ctx, "row_reduce_kernel(fold)");
}

// Number of R-chunks per column tile.  CTAs do equal work, so a launch that needs slightly more
// than one wave of resident CTAs takes two rounds.  Measured on B200 (sweep over the split factor,
// (8192,8192) axis 0 = 64 tiles): the kernel is fastest when all CTAs are resident at once and the
// wave is nearly full -- 10 chunks (640 CTAs, 740 resident) 5.5 TB/s, 8 chunks 5.2, 12 chunks
// (768 CTAs, two rounds) 4.0.  So: as many chunks as fit in ONE wave, each at least 64 rows.
size_t pick_split(size_t base_ctas, size_t resident, size_t max_split) {
    if (max_split < 1) max_split = 1;
    size_t split = resident / (base_ctas ? base_ctas : 1);
    if (split < 1) split = 1;
    if (split > max_split) split = max_split;
    return split;
}

template <typename K>
size_t resident_ctas(Ctx *ctx, K kernel) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kBlock, 0) != cudaSuccess || per_sm < 1) per_sm = 4;
    return (size_t)ctx->sm_count * (size_t)per_sm;
}

template <typename T, int OP, int VW, int TX>
int cols_launch_t(Ctx *ctx, const T *src, size_t outer, size_t R, size_t inner, ptrdiff_t outer_stride,
                  ptrdiff_t row_stride, T *dst, int mean, size_t count) {
    const size_t tile_cols = (size_t)TX * VW;
    const size_t col_tiles = (inner + tile_cols - 1) / tile_cols;
    const size_t base_ctas = outer * col_tiles;
    size_t split = 1;
    if (base_ctas <= kMaxTileCounters) split = pick_split(base_ctas, resident_ctas(ctx, col_reduce_kernel<T, OP, VW, TX>), R / 64);
    T *partial = nullptr;
    unsigned int *counters = nullptr;
    if (split > 1) {
        void *ws = nullptr;
        int rc = workspace(ctx, outer * split * inner * sizeof(T), &ws);
        if (rc != RTB_OK) return rc;
        counters = reinterpret_cast<unsigned int *>(ws) + kTileCounterOffset;
        partial = reinterpret_cast<T *>(reinterpret_cast<char *>(ws) + kWorkspaceHeader);
    }
    const unsigned grid = grid_for(ctx, base_ctas * split, kAxisGridCap);  // one CTA per (tile, chunk)
    launch_dep(ctx, grid, kBlock, col_reduce_kernel<T, OP, VW, TX>, src, outer, R, inner, outer_stride, row_stride, split,
                                                                       col_tiles, partial, counters, dst, mean, count);
    return check_launch(ctx, "col_reduce_kernel");
}

template <typename T, int OP>
int cols_launch(Ctx *ctx, const T *src, size_t outer, size_t R, size_t inner, ptrdiff_t outer_stride,
                ptrdiff_t row_stride, T *dst, int mean, size_t count = 0) {
    if (count == 0) count = R;  // the divisor of a mean; differs from R only when folding partial sums
    constexpr int N = VecOf<T>::N;
    // 128-bit loads need every (o, k) row start on a 16-byte boundary
    const bool vec = (inner % N == 0) && (((uintptr_t)src & 15u) == 0) && (outer_stride % N == 0) && (row_stride % N == 0);
    // TX = 32 (tile = 32 x 128-bit columns, 8 rows in flight per CTA).  A 256-lane tile (whole 4 KiB
    // row segments per CTA) was measured and is not faster: (64,4096,1024) axis 1 6.50 vs 6.5-6.7 TB/s,
    // (8192,8192) axis 0 4.72 vs 5.3-5.5 TB/s -- the fold of many chunk partials by one CTA per wide
    // tile costs more than the longer DRAM bursts gain.
    if (vec) return cols_launch_t<T, OP, N, 32>(ctx, src, outer, R, inner, outer_stride, row_stride, dst, mean, count);
    return cols_launch_t<T, OP, 1, 32>(ctx, src, outer, R, inner, outer_stride, row_stride, dst, mean, count);
}

// src element (o, k, i) at o*outer_stride + k*row_stride + i; dst[o*inner + i]
template <typename T, int OP>
int axis_launch(Ctx *ctx, const T *src, size_t outer, size_t R, size_t inner, ptrdiff_t outer_stride,
                ptrdiff_t row_stride, T *dst, int mean) {
    if (inner == 1 && row_stride == 1) return rows_launch<T, OP>(ctx, src, outer, R, outer_stride, dst, mean);
    return cols_launch<T, OP>(ctx, src, outer, R, inner, outer_stride, row_stride, dst, mean);
}

template <typename T>
int axis_by_op(Ctx *ctx, int redop, const T *src, size_t outer, size_t R, size_t inner, ptrdiff_t so, ptrdiff_t sr, T *dst) {
    switch (redop) {
        case RTB_SUM: return axis_launch<T, RTB_SUM>(ctx, src, outer, R, inner, so, sr, dst, 0);
        case RTB_MEAN: return axis_launch<T, RTB_SUM>(ctx, src, outer, R, inner, so, sr, dst, 1);
        case RTB_PROD: return axis_launch<T, RTB_PROD>(ctx, src, outer, R, inner, so, sr, dst, 0);
        case RTB_MAX: return axis_launch<T, RTB_MAX>(ctx, src, outer, R, inner, so, sr, dst, 0);
        case RTB_MIN: return axis_launch<T, RTB_MIN>(ctx, src, outer, R, inner, so, sr, dst, 0);
    }
    return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
}

template <typename T, int OP>
int bcast_reduce_launch(Ctx *ctx, const T *l, Strides3 sl, const T *r, Strides3 sr, int binop, size_t A, size_t R, size_t B,
                        T *dst, int mean) {
    if (B >= 32) {
        constexpr size_t NB = VecOf<T>::N;
        auto bvec_ok = [&](const T *p, const Strides3 &s) {
            const bool al = reinterpret_cast<uintptr_t>(p) % 16 == 0 && (A == 1 || s.a % (ptrdiff_t)NB == 0) && s.k % (ptrdiff_t)NB == 0;
            return s.b == 0 || (s.b == 1 && al);
        };
        const bool bvec = B % NB == 0 && B >= 32 * NB && bvec_ok(l, sl) && bvec_ok(r, sr) && binop >= RTB_ADD && binop <= RTB_DIV &&
                          reinterpret_cast<uintptr_t>(dst) % 16 == 0;
        const size_t base = bvec ? A * ((B / NB + 31) / 32) : A * ((B + 31) / 32);
        // few output tiles: cut k into chunks so that every SM has work, then fold the partial rows
        size_t split = 1;
        const size_t want = (size_t)ctx->sm_count * 2;
        if (base < want && R >= 128) {
            split = (want + base - 1) / base;
            if (split > R / 64) split = R / 64;
            if (split < 1) split = 1;
        }
        T *target = dst;
        if (split > 1) {
            void *tmp = nullptr;  // not the reduction workspace: the fold below uses that
            int rc = rtb_alloc(reinterpret_cast<rtb_ctx *>(ctx), A * split * B * sizeof(T), &tmp);
            if (rc != RTB_OK) return rc;
            target = static_cast<T *>(tmp);
        }
        const unsigned wgrid = grid_for(ctx, base * split, kAxisGridCap);
        if (bvec) {
#define RTB_BVEC(BOP)                                                                                                          \
    case BOP:                                                                                                                   \
        launch_dep(ctx, wgrid, kBlock, bcast_reduce_bvec_kernel<T, OP, BOP>, l, sl, r, sr, A, R, B, split, target, mean);    \
        break;
            switch (binop) {
                RTB_BVEC(RTB_ADD) RTB_BVEC(RTB_SUB) RTB_BVEC(RTB_MUL) RTB_BVEC(RTB_DIV)
            }
#undef RTB_BVEC
        } else {
            launch_dep(ctx, wgrid, kBlock, bcast_reduce_kernel<T, OP, true>, l, sl, r, sr, binop, A, R, B, split, target, mean);
        }
        int rc = check_launch(ctx, "bcast_reduce_kernel");
        if (split > 1) {
            if (rc == RTB_OK) rc = cols_launch<T, OP>(ctx, target, A, split, B, (ptrdiff_t)(split * B), (ptrdiff_t)B, dst, mean, R);
            rtb_free(reinterpret_cast<rtb_ctx *>(ctx), target);  // reuse is ordered by the stream
        }
        return rc;
    }
    size_t blocks = (A * B + kWarps - 1) / kWarps;
    constexpr size_t N = VecOf<T>::N;
    auto vec_ok = [&](const T *p, const Strides3 &s) {
        if (s.k == 0) return true;
        return s.k == 1 && reinterpret_cast<uintptr_t>(p) % 16 == 0 && (A == 1 || s.a % (ptrdiff_t)N == 0) &&
               (B == 1 || s.b % (ptrdiff_t)N == 0);
    };
    if (R % N == 0 && R >= 32 * N && vec_ok(l, sl) && vec_ok(r, sr) && binop >= RTB_ADD && binop <= RTB_DIV) {
        const unsigned grid = grid_for(ctx, blocks, kAxisGridCap);
#define RTB_KVEC(BOP)                                                                                                 \
    case BOP:                                                                                                          \
        launch_dep(ctx, grid, kBlock, bcast_reduce_kvec_kernel<T, OP, BOP>, l, sl, r, sr, A, R, B, dst, mean);      \
        break;
        switch (binop) {
            RTB_KVEC(RTB_ADD) RTB_KVEC(RTB_SUB) RTB_KVEC(RTB_MUL) RTB_KVEC(RTB_DIV)
        }
#undef RTB_KVEC
        return check_launch(ctx, "bcast_reduce_kvec_kernel");
    }
    launch_dep(ctx, grid_for(ctx, blocks, kAxisGridCap), kBlock, bcast_reduce_kernel<T, OP, false>, l, sl, r, sr, binop, A, R, B, 1,
                                                                                                dst, mean);
    return check_launch(ctx, "bcast_reduce_kernel");
}

template <typename T>
int bcast_reduce_by_op(Ctx *ctx, int redop, const T *l, Strides3 sl, const T *r, Strides3 sr, int binop, size_t A, size_t R,
                       size_t B, T *dst) {
    switch (redop) {
        case RTB_SUM: return bcast_reduce_launch<T, RTB_SUM>(ctx, l, sl, r, sr, binop, A, R, B, dst, 0);
        case RTB_MEAN: return bcast_reduce_launch<T, RTB_SUM>(ctx, l, sl, r, sr, binop, A, R, B, dst, 1);
        case RTB_PROD: return bcast_reduce_launch<T, RTB_PROD>(ctx, l, sl, r, sr, binop, A, R, B, dst, 0);
        case RTB_MAX: return bcast_reduce_launch<T, RTB_MAX>(ctx, l, sl, r, sr, binop, A, R, B, dst, 0);
        case RTB_MIN: return bcast_reduce_launch<T, RTB_MIN>(ctx, l, sl, r, sr, binop, A, R, B, dst, 0);
    }
    return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
}

}  // namespace

int launch_reduce_flat(Ctx *ctx, int dtype, int redop, const void *src, size_t len, void *dst) {
    std::lock_guard<std::mutex> lock(ctx->ws_mu);
    if (dtype == RTB_F32) return flat_by_op<float>(ctx, redop, SrcPlain<float>{(const float *)src}, len, (float *)dst);
    if (dtype == RTB_F64) return flat_by_op<double>(ctx, redop, SrcPlain<double>{(const double *)src}, len, (double *)dst);
    return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
}

int launch_reduce_axis(Ctx *ctx, int dtype, int redop, const void *src, size_t outer, size_t r, size_t inner,
                       void *dst) {
    return launch_reduce_axis_strided(ctx, dtype, redop, src, outer, r, inner, (ptrdiff_t)(r * inner), (ptrdiff_t)inner, dst);
}

int launch_reduce_axis_strided(Ctx *ctx, int dtype, int redop, const void *src, size_t outer, size_t r, size_t inner,
                               ptrdiff_t outer_stride, ptrdiff_t row_stride, void *dst) {
    std::lock_guard<std::mutex> lock(ctx->ws_mu);
    if (dtype == RTB_F32)
        return axis_by_op<float>(ctx, redop, (const float *)src, outer, r, inner, outer_stride, row_stride, (float *)dst);
    if (dtype == RTB_F64)
        return axis_by_op<double>(ctx, redop, (const double *)src, outer, r, inner, outer_stride, row_stride, (double *)dst);
    return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
}

template <typename T>
static int l1_typed(Ctx *ctx, const T *a, const T *b, size_t n, int reduction, T *loss, T *g) {
    uintptr_t pa = (uintptr_t)a & 15u, pb = (uintptr_t)b & 15u, pg = g ? ((uintptr_t)g & 15u) : pa;
    SrcL1<T> src{a, b, g, reduction == 0 ? (T)(float)n : (T)1, (pa == pb && pa == pg) ? 1 : 0};
    return flat_launch<T, RTB_SUM, SrcL1<T>>(ctx, src, n, loss, reduction == 0 ? 1 : 0);
}

// the same over a tensor split across ranks: the gradient map is scaled by the GLOBAL count and
// the per-GPU sums of |a - b| are exchanged by the last CTA
template <typename T>
static int l1_typed_mg(Ctx *ctx, const T *a, const T *b, size_t n, int reduction, T *loss, T *g, const MgPeers &peers,
                       size_t global_count) {
    uintptr_t pa = (uintptr_t)a & 15u, pb = (uintptr_t)b & 15u, pg = g ? ((uintptr_t)g & 15u) : pa;
    SrcL1<T> src{a, b, g, reduction == 0 ? (T)(float)global_count : (T)1, (pa == pb && pa == pg) ? 1 : 0};
    return flat_launch<T, RTB_SUM, SrcL1<T>, MgPeers>(ctx, src, n, loss, reduction == 0 ? 1 : 0, global_count, peers);
}

int launch_l1_mg(Ctx *ctx, int dtype, const void *a, const void *b, size_t n, int reduction, void *loss, void *gmap,
                 const MgPeers &peers, size_t global_count) {
    std::lock_guard<std::mutex> lock(ctx->ws_mu);
    if (dtype == RTB_F32)
        return l1_typed_mg<float>(ctx, (const float *)a, (const float *)b, n, reduction, (float *)loss, (float *)gmap, peers, global_count);
    if (dtype == RTB_F64)
        return l1_typed_mg<double>(ctx, (const double *)a, (const double *)b, n, reduction, (double *)loss, (double *)gmap, peers, global_count);
    return fail(RTB_ERR_DTYPE, "l1 loss is defined for f32 and f64 only");
}

int launch_reduce_flat_mg(Ctx *ctx, int dtype, int redop, const void *src, size_t len, void *dst, const MgPeers &peers,
                          size_t global_count) {
    std::lock_guard<std::mutex> lock(ctx->ws_mu);
    if (dtype == RTB_F32)
        return flat_by_op<float, SrcPlain<float>, MgPeers>(ctx, redop, SrcPlain<float>{(const float *)src}, len, (float *)dst, global_count, peers);
    if (dtype == RTB_F64)
        return flat_by_op<double, SrcPlain<double>, MgPeers>(ctx, redop, SrcPlain<double>{(const double *)src}, len, (double *)dst, global_count, peers);
    return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
}

int launch_l1(Ctx *ctx, int dtype, const void *a, const void *b, size_t n, int reduction, void *loss, void *gmap) {
    std::lock_guard<std::mutex> lock(ctx->ws_mu);
    if (dtype == RTB_F32) return l1_typed<float>(ctx, (const float *)a, (const float *)b, n, reduction, (float *)loss, (float *)gmap);
    if (dtype == RTB_F64) return l1_typed<double>(ctx, (const double *)a, (const double *)b, n, reduction, (double *)loss, (double *)gmap);
    return fail(RTB_ERR_DTYPE, "l1 loss is defined for f32 and f64 only");
}

int launch_relu_mask(Ctx *ctx, float *x, float *mask, size_t n) {
    if ((((uintptr_t)x | (uintptr_t)mask) & 15u) != 0) return fail(RTB_ERR_INVALID, "relu_mask needs 16-byte aligned buffers");
    unsigned grid = grid_for(ctx, (n / 4 + kBlock - 1) / kBlock, 16);
    launch_dep(ctx, grid, kBlock, relu_mask_kernel, x, mask, n);
    return check_launch(ctx, "relu_mask_kernel");
}

template <typename T>
static int bias_relu_mask_typed(Ctx *ctx, T *z, const T *bias, T *mask, size_t rows, size_t cols) {
    constexpr int N = VecOf<T>::N;
    const bool vec = cols % N == 0 && (((uintptr_t)z | (uintptr_t)bias | (uintptr_t)mask) & 15u) == 0;
    const size_t per = vec ? (size_t)N : 1;
    const size_t col_blocks = (cols / per + kBlock - 1) / kBlock;
    const size_t grid = col_blocks * ((rows + kBiasRows - 1) / kBiasRows);
    if (grid > 0x7fffffffu) return fail(RTB_ERR_TOO_LARGE, "bias_relu_mask: %zu x %zu is beyond one launch", rows, cols);
    if (vec) launch_dep(ctx, (unsigned)grid, kBlock, bias_relu_mask_kernel<T, N>, z, bias, mask, rows, cols, col_blocks);
    else launch_dep(ctx, (unsigned)grid, kBlock, bias_relu_mask_kernel<T, 1>, z, bias, mask, rows, cols, col_blocks);
    return check_launch(ctx, "bias_relu_mask_kernel");
}

int launch_bias_relu_mask(Ctx *ctx, int dtype, void *z, const void *bias, void *mask, size_t rows, size_t cols) {
    if (rows == 0 || cols == 0) return RTB_OK;
    if (dtype == RTB_F32) return bias_relu_mask_typed<float>(ctx, (float *)z, (const float *)bias, (float *)mask, rows, cols);
    if (dtype == RTB_F64) return bias_relu_mask_typed<double>(ctx, (double *)z, (const double *)bias, (double *)mask, rows, cols);
    return fail(RTB_ERR_DTYPE, "bias_relu_mask is defined for f32 and f64 only");
}

int launch_sgd(Ctx *ctx, float *p, const float *g, float lr, size_t n) {
    if ((((uintptr_t)p | (uintptr_t)g) & 15u) != 0) return fail(RTB_ERR_INVALID, "sgd_update needs 16-byte aligned buffers");
    unsigned grid = grid_for(ctx, (n / 4 + kBlock - 1) / kBlock, 16);
    launch_dep(ctx, grid, kBlock, sgd_kernel, p, g, lr, n);
    return check_launch(ctx, "sgd_kernel");
}

int launch_relu_mask_f64(Ctx *ctx, double *x, double *mask, size_t n) {
    if ((((uintptr_t)x | (uintptr_t)mask) & 15u) != 0) return fail(RTB_ERR_INVALID, "relu_mask needs 16-byte aligned buffers");
    unsigned grid = grid_for(ctx, (n / 2 + kBlock - 1) / kBlock, 16);
    launch_dep(ctx, grid, kBlock, relu_mask_f64_kernel, x, mask, n);
    return check_launch(ctx, "relu_mask_f64_kernel");
}

int launch_sgd_f64(Ctx *ctx, double *p, const double *g, double lr, size_t n) {
    if ((((uintptr_t)p | (uintptr_t)g) & 15u) != 0) return fail(RTB_ERR_INVALID, "sgd_update needs 16-byte aligned buffers");
    unsigned grid = grid_for(ctx, (n / 2 + kBlock - 1) / kBlock, 16);
    launch_dep(ctx, grid, kBlock, sgd_f64_kernel, p, g, lr, n);
    return check_launch(ctx, "sgd_f64_kernel");
}

int launch_u8_f32(Ctx *ctx, const uint8_t *src, float *dst, float divisor, size_t n) {
    if (((uintptr_t)src & 3u) != 0 || ((uintptr_t)dst & 15u) != 0) return fail(RTB_ERR_INVALID, "u8_to_f32 needs aligned buffers");
    unsigned grid = grid_for(ctx, (n / 4 + kBlock - 1) / kBlock, 16);
    launch_dep(ctx, grid, kBlock, u8_f32_kernel, src, dst, divisor, n);
    return check_launch(ctx, "u8_f32_kernel");
}

}  // namespace rtb

namespace rtb {
int launch_bcast_reduce(Ctx *ctx, int dtype, int binop, int redop, const void *l, const ptrdiff_t sl[3], const void *r,
                        const ptrdiff_t sr[3], size_t A, size_t R, size_t B, void *dst) {
    Strides3 a{sl[0], sl[1], sl[2]}, b{sr[0], sr[1], sr[2]};
    if (dtype == RTB_F32)
        return bcast_reduce_by_op<float>(ctx, redop, (const float *)l, a, (const float *)r, b, binop, A, R, B, (float *)dst);
    if (dtype == RTB_F64)
        return bcast_reduce_by_op<double>(ctx, redop, (const double *)l, a, (const double *)r, b, binop, A, R, B, (double *)dst);
    return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
}
}  // namespace rtb
