// Reductions whose running value is a small state rather than one number: variance / standard
// deviation (Welford states merged with Chan's formula), logsumexp (running max + rescaled sum),
// L1 / L2 norm, argmax / argmin (value + position).  The reference implements them only in its CUDA
// backend (cuda/kernels/reduction/reduce.cu:166-240, 324-420, 560-716, 845-990); semantics kept:
// variance of n <= 1 elements is 0, denominators n-1 / n, argmax / argmin return the first
// position of the extreme value (0 when nothing compares above lowest() / below max()).
//
// Layout handled: source element (o, k, i) at o*outer_stride + k*row_stride + i, reduced over k,
// output row-major over (o, i).  inner == 1 with row_stride == 1 runs one CTA (or warp) per row
// reading 128-bit vectors; everything else runs tiles of 32 x VW columns with the 8 warps of a
// CTA along k.  When there are too few outputs to fill the GPU, k is cut into chunks whose partial
// states go to the context workspace; the CTA that finishes a row / column tile last (a completion
// counter in the workspace header, left at zero again) merges them -- one launch.
#include "rtb_internal.h"

#include <cfloat>
#include <cmath>

namespace rtb {
namespace {

constexpr int kBlock = 256;
constexpr int kWarps = kBlock / 32;
constexpr size_t kWorkspaceHeader = 65536;  // bytes of completion counters in front of the scratch
constexpr unsigned kGridCap = 1u << 22;
// completion counters in the workspace header: [0, 64) belong to the flat sum kernel, the rest to
// per-row / per-tile counters of the chunked axis kernels (shared with the plain reductions; every
// kernel leaves them at zero and launches on one context are ordered)
constexpr size_t kTileCounterOffset = 64;
constexpr size_t kMaxTileCounters = 16384 - 64;

struct ExtSettings {
    int unbiased;
    int is_std;
};

// f32 logsumexp terms use the hardware exponential (2 ulp), as the reference's fast-math build does
__device__ __forceinline__ float t_exp(float x) { return __expf(x); }
__device__ __forceinline__ double t_exp(double x) { return exp(x); }
__device__ __forceinline__ float t_log(float x) { return logf(x); }
__device__ __forceinline__ double t_log(double x) { return log(x); }
__device__ __forceinline__ float t_sqrt(float x) { return sqrtf(x); }
__device__ __forceinline__ double t_sqrt(double x) { return sqrt(x); }
__device__ __forceinline__ float t_abs(float x) { return fabsf(x); }
__device__ __forceinline__ double t_abs(double x) { return fabs(x); }
// The library is built without FMA contraction so that single operations round as on the CPU; these
// reductions are tolerance-checked (the reference's own build contracts them), so they fuse by hand.
__device__ __forceinline__ float t_fma(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double t_fma(double a, double b, double c) { return fma(a, b, c); }
// weight nb / (na + nb) of a state merge: a 2-ulp quotient is ample for f32 weights
__device__ __forceinline__ float t_ratio(float a, float b) { return __fdividef(a, b); }
__device__ __forceinline__ double t_ratio(double a, double b) { return a / b; }
template <typename T> __device__ __forceinline__ T t_lowest();
template <> __device__ __forceinline__ float t_lowest<float>() { return -FLT_MAX; }
template <> __device__ __forceinline__ double t_lowest<double>() { return -DBL_MAX; }
template <typename T> __device__ __forceinline__ T t_ninf();
template <> __device__ __forceinline__ float t_ninf<float>() { return -INFINITY; }
template <> __device__ __forceinline__ double t_ninf<double>() { return -(double)INFINITY; }

template <typename V> __device__ __forceinline__ V shfl_down_any(V v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }

// ---- reducers ----------------------------------------------------------------------------------
// State identity(); add_one(state, x, k); add_batch<NB>(state, x[NB], k0, kstep) for NB values at
// positions k0 + e*kstep; merge(a, b); shfl(state, delta); Out finish(state, settings).

template <typename T> struct RedVar {
    using Out = T;
    static constexpr bool kPositional = false;
    static constexpr bool kHeavyMerge = true;  // merging two states costs tens of instructions
    static constexpr bool kPipelineCols = true;  // column kernel: prefetch the next batch while merging
    // The count is kept in the element type: merges then need no 64-bit integer arithmetic and no
    // integer -> float conversions (both multi-instruction), and the state is 12 bytes instead of 16
    // for f32.  Counts are exact up to 2^24 (f32) / 2^53 (f64); beyond that a merged count may round by
    // 6e-8 relative, far inside the tolerance of a float variance.
    struct State {
        T mean, m2, n;
    };
    __device__ static State identity() { return State{(T)0, (T)0, (T)0}; }
    __device__ static State merge(const State &a, const State &b) {
        if (b.n == (T)0) return a;
        if (a.n == (T)0) return b;
        const T w = t_ratio(b.n, a.n + b.n);
        const T delta = b.mean - a.mean;
        State r;
        r.mean = t_fma(delta, w, a.mean);
        r.m2 = t_fma(delta * delta, a.n * w, a.m2 + b.m2);
        r.n = a.n + b.n;
        return r;
    }
    // a batch becomes one state (its own mean and squared deviations), merged with one division
    template <int NB> __device__ static void add_batch(State &s, const T (&x)[NB], unsigned long long, unsigned long long) {
        T sum = x[0];
#pragma unroll
        for (int e = 1; e < NB; ++e) sum += x[e];
        const T bm = sum * ((T)1 / (T)NB);
        T m2 = (T)0;
#pragma unroll
        for (int e = 0; e < NB; ++e) {
            const T d = x[e] - bm;
            m2 = t_fma(d, d, m2);
        }
        s = merge(s, State{bm, m2, (T)NB});
    }
    __device__ static void add_one(State &s, T x, unsigned long long) { s = merge(s, State{x, (T)0, (T)1}); }
    __device__ static State shfl(const State &s, int d) {
        return State{shfl_down_any(s.mean, d), shfl_down_any(s.m2, d), shfl_down_any(s.n, d)};
    }
    __device__ static Out finish(const State &s, ExtSettings st) {
        const T den = st.unbiased ? (s.n > (T)1 ? s.n - (T)1 : (T)1) : (s.n > (T)0 ? s.n : (T)1);
        const T v = s.m2 / den;
        return st.is_std ? t_sqrt(v) : v;
    }
};

template <typename T> struct RedLse {
    using Out = T;
    static constexpr bool kPositional = false;
    static constexpr bool kHeavyMerge = true;
    static constexpr bool kPipelineCols = false;  // column kernel: prefetch the next batch while merging
    struct State {
        T m, s;  // running max, sum of exp(x - m); s == 0 marks "empty"
    };
    __device__ static State identity() { return State{t_ninf<T>(), (T)0}; }
    __device__ static State merge(const State &a, const State &b) {
        if (b.s == (T)0) return a;
        if (a.s == (T)0) return b;
        const T m = a.m > b.m ? a.m : b.m;
        return State{m, a.s * t_exp(a.m - m) + b.s * t_exp(b.m - m)};
    }
    template <int NB> __device__ static void add_batch(State &s, const T (&x)[NB], unsigned long long, unsigned long long) {
        T vm = x[0];
#pragma unroll
        for (int e = 1; e < NB; ++e) vm = x[e] > vm ? x[e] : vm;
        T vs = (T)0;
#pragma unroll
        for (int e = 0; e < NB; ++e) vs += t_exp(x[e] - vm);
        // one more exponential rescales whichever side has the smaller max
        if (s.s == (T)0) {
            s = State{vm, vs};
        } else if (vm <= s.m) {
            s.s += vs * t_exp(vm - s.m);
        } else {
            s.s = s.s * t_exp(s.m - vm) + vs;
            s.m = vm;
        }
    }
    __device__ static void add_one(State &s, T x, unsigned long long) { s = merge(s, State{x, (T)1}); }
    __device__ static State shfl(const State &s, int d) { return State{shfl_down_any(s.m, d), shfl_down_any(s.s, d)}; }
    __device__ static Out finish(const State &s, ExtSettings) { return s.m + t_log(s.s); }
};

template <typename T, int P> struct RedNorm {
    using Out = T;
    static constexpr bool kPositional = false;
    static constexpr bool kHeavyMerge = false;
    static constexpr bool kPipelineCols = false;  // column kernel: prefetch the next batch while merging
    struct State {
        T v;
    };
    __device__ static State identity() { return State{(T)0}; }
    __device__ static State merge(const State &a, const State &b) { return State{a.v + b.v}; }
    __device__ static T accum(T acc, T x) { return P == 1 ? acc + t_abs(x) : t_fma(x, x, acc); }
    template <int NB> __device__ static void add_batch(State &s, const T (&x)[NB], unsigned long long, unsigned long long) {
        T acc = accum((T)0, x[0]);
#pragma unroll
        for (int e = 1; e < NB; ++e) acc = accum(acc, x[e]);
        s.v += acc;
    }
    __device__ static void add_one(State &s, T x, unsigned long long) { s.v = accum(s.v, x); }
    __device__ static State shfl(const State &s, int d) { return State{shfl_down_any(s.v, d)}; }
    __device__ static Out finish(const State &s, ExtSettings) { return P == 2 ? t_sqrt(s.v) : s.v; }
};

template <typename T, bool MAXI> struct RedArg {
    using Out = unsigned long long;
    static constexpr bool kPositional = true;
    static constexpr bool kHeavyMerge = true;
    static constexpr bool kPipelineCols = true;  // column kernel: prefetch the next batch while merging
    static constexpr unsigned long long kNone = ~0ull;
    struct State {
        T v;
        unsigned long long k;
    };
    __device__ static State identity() { return State{MAXI ? t_lowest<T>() : -t_lowest<T>(), kNone}; }
    __device__ static bool better(T x, T best) { return MAXI ? x > best : x < best; }
    __device__ static State merge(const State &a, const State &b) {
        return (better(b.v, a.v) || (b.v == a.v && b.k < a.k)) ? b : a;
    }
    __device__ static void add_one(State &s, T x, unsigned long long k) {
        if (better(x, s.v)) { s.v = x; s.k = k; }  // positions arrive in increasing order: strict keeps the first
    }
    template <int NB> __device__ static void add_batch(State &s, const T (&x)[NB], unsigned long long k0, unsigned long long kstep) {
#pragma unroll
        for (int e = 0; e < NB; ++e) add_one(s, x[e], k0 + (unsigned long long)e * kstep);
    }
    __device__ static State shfl(const State &s, int d) { return State{shfl_down_any(s.v, d), shfl_down_any(s.k, d)}; }
    __device__ static Out finish(const State &s, ExtSettings) { return s.k == kNone ? 0ull : s.k; }
};

template <typename T> struct Vec128 {
    static constexpr int N = 16 / (int)sizeof(T);
    union U {
        uint4 q;
        T e[N];
    };
};

// A chunk state written by another CTA of this launch: read word by word through L2 (__ldcg), so
// that an L1 line fetched earlier on this SM cannot hide it.
template <typename S> __device__ __forceinline__ S load_state_cg(const S *p) {
    static_assert(sizeof(S) % 4 == 0, "states are made of 4-byte words");
    union {
        S s;
        unsigned int w[sizeof(S) / 4];
    } u;
#pragma unroll
    for (int i = 0; i < (int)(sizeof(S) / 4); ++i) u.w[i] = __ldcg(reinterpret_cast<const unsigned int *>(p) + i);
    return u.s;
}

template <typename R> __device__ __forceinline__ typename R::State warp_merge(typename R::State s) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s = R::merge(s, R::shfl(s, d));
    return s;
}

// all threads call; the merged state is valid in thread 0
template <typename R> __device__ __forceinline__ typename R::State block_merge(typename R::State s, typename R::State *smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    s = warp_merge<R>(s);
    if (lane == 0) smem[warp] = s;
    __syncthreads();
    if (warp == 0) {
        s = lane < kWarps ? smem[lane] : R::identity();
#pragma unroll
        for (int d = kWarps / 2; d > 0; d >>= 1) s = R::merge(s, R::shfl(s, d));
    }
    __syncthreads();
    return s;
}

// ---- inner == 1: one CTA (GROUP == kBlock) or one warp (GROUP == 32) per (row, chunk) -----------
template <typename T, typename R, int GROUP>
__global__ void __launch_bounds__(kBlock) ext_rows_kernel(const T *__restrict__ src, size_t rows, size_t len, ptrdiff_t pitch,
                                                          size_t split, typename R::State *partial, unsigned int *counters,
                                                          typename R::Out *dst, ExtSettings st) {
    grid_dep_wait();
    using State = typename R::State;
    using V = Vec128<T>;
    constexpr int N = V::N;
    constexpr int U = 4;  // vectors in flight per thread
    __shared__ State smem[kWarps];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tid = GROUP == kBlock ? (int)threadIdx.x : lane;
    const size_t items = rows * split;
    const size_t per = (len + split - 1) / split;
    const size_t first = GROUP == kBlock ? blockIdx.x : (size_t)blockIdx.x * kWarps + warp;
    const size_t step = GROUP == kBlock ? gridDim.x : (size_t)gridDim.x * kWarps;
    // every thread of a CTA runs the same number of iterations when GROUP == kBlock (block barriers)
    for (size_t item = first; item < items; item += step) {
        const size_t row = item / split, chunk = item % split;
        const size_t k0 = chunk * per < len ? chunk * per : len;
        const size_t k1 = k0 + per < len ? k0 + per : len;
        const T *p = src + (ptrdiff_t)row * pitch;
        State s = R::identity();
        if (k0 < k1) {
            const size_t mis = (reinterpret_cast<uintptr_t>(p + k0) / sizeof(T)) % N;
            size_t head = mis ? N - mis : 0;
            if (head > k1 - k0) head = k1 - k0;
            if ((size_t)tid < head) R::add_one(s, p[k0 + tid], k0 + tid);
            const size_t kb = k0 + head;
            const size_t nvec = (k1 - kb) / N;
            const uint4 *pv = reinterpret_cast<const uint4 *>(p + kb);
            size_t v = tid;
            for (; v + (U - 1) * GROUP < nvec; v += U * GROUP) {
                typename V::U x[U];
#pragma unroll
                for (int u = 0; u < U; ++u) x[u].q = pv[v + u * GROUP];
                if (!R::kPositional) {
                    T flat[U * N];
#pragma unroll
                    for (int u = 0; u < U; ++u)
#pragma unroll
                        for (int e = 0; e < N; ++e) flat[u * N + e] = x[u].e[e];
                    R::template add_batch<U * N>(s, flat, 0ull, 0ull);
                } else {
#pragma unroll
                    for (int u = 0; u < U; ++u) R::template add_batch<N>(s, x[u].e, kb + (v + u * GROUP) * N, 1ull);
                }
            }
            for (; v < nvec; v += GROUP) {
                typename V::U x;
                x.q = pv[v];
                R::template add_batch<N>(s, x.e, kb + v * N, 1ull);
            }
            const size_t kt = kb + nvec * N;
            if (kt + tid < k1) R::add_one(s, p[kt + tid], kt + tid);
        }
        grid_dep_launch();
        if (GROUP != kBlock) {  // warp per row; rows this short are never chunked
            s = warp_merge<R>(s);
            if (lane == 0) dst[row] = R::finish(s, st);
            continue;
        }
        s = block_merge<R>(s, smem);
        if (split == 1) {
            if (threadIdx.x == 0) dst[row] = R::finish(s, st);
            continue;
        }
        if (threadIdx.x == 0) {
            partial[row * split + chunk] = s;
            __threadfence();
            is_last = atomicAdd(counters + row, 1u) == (unsigned int)split - 1u;
        }
        __syncthreads();
        if (!is_last) continue;  // uniform per CTA
        __threadfence();
        s = R::identity();
        for (size_t c = threadIdx.x; c < split; c += kBlock) s = R::merge(s, load_state_cg(partial + row * split + c));
        s = block_merge<R>(s, smem);
        if (threadIdx.x == 0) {
            dst[row] = R::finish(s, st);
            counters[row] = 0;  // ready for the next launch
        }
    }
}

// ---- inner > 1 (or strided rows): tiles of 32 x VW columns, the 8 warps of a CTA along k --------
template <typename T, typename R, int VW, bool PIPE = false>
__global__ void __launch_bounds__(kBlock) ext_cols_kernel(const T *__restrict__ src, size_t outer, size_t len, size_t inner,
                                                          ptrdiff_t outer_stride, ptrdiff_t row_stride, size_t split,
                                                          typename R::State *partial, unsigned int *counters,
                                                          typename R::Out *dst, ExtSettings st) {
    grid_dep_wait();
    using State = typename R::State;
    constexpr int U = 8;  // rows in flight per thread (4 measured slower, also for the heavy states)
    constexpr bool kPipelined = PIPE;
    __shared__ State smem[kWarps][32][VW];
    __shared__ bool is_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t col_tiles = (inner + 32 * VW - 1) / (32 * VW);
    const size_t per = (len + split - 1) / split;
    const size_t items = outer * split * col_tiles;
    for (size_t item = blockIdx.x; item < items; item += gridDim.x) {
        size_t q = item;
        const size_t col = ((q % col_tiles) * 32 + lane) * VW; q /= col_tiles;
        const size_t chunk = q % split;
        const size_t o = q / split;
        const size_t k0 = chunk * per < len ? chunk * per : len;
        const size_t k1 = k0 + per < len ? k0 + per : len;
        State s[VW];
#pragma unroll
        for (int c = 0; c < VW; ++c) s[c] = R::identity();
        if (col < inner) {
            const T *p = src + (ptrdiff_t)o * outer_stride + (ptrdiff_t)col;
            size_t k = k0 + warp;
            auto fetch = [&](T (&x)[U][VW], size_t kk) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const T *pr = p + (ptrdiff_t)(kk + u * kWarps) * row_stride;
                    if (VW > 1) {
                        typename Vec128<T>::U t;
                        t.q = *reinterpret_cast<const uint4 *>(pr);
#pragma unroll
                        for (int c = 0; c < VW; ++c) x[u][c] = t.e[c];
                    } else {
                        x[u][0] = *pr;
                    }
                }
            };
            auto absorb = [&](const T (&x)[U][VW], size_t kk) {
#pragma unroll
                for (int c = 0; c < VW; ++c) {
                    T colv[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) colv[u] = x[u][c];
                    R::template add_batch<U>(s[c], colv, kk, (unsigned long long)kWarps);
                }
            };
            if (kPipelined) {
                // the next batch's loads are issued before this batch is absorbed, so the merge
                // arithmetic (a division per column for Welford) runs under the load latency
                T x[U][VW];
                bool have = k + (U - 1) * kWarps < k1;
                if (have) fetch(x, k);
                while (have) {
                    const size_t kn = k + U * kWarps;
                    const bool next = kn + (U - 1) * kWarps < k1;
                    T y[U][VW];
                    if (next) fetch(y, kn);
                    absorb(x, k);
                    if (next) {
#pragma unroll
                        for (int u = 0; u < U; ++u)
#pragma unroll
                            for (int c = 0; c < VW; ++c) x[u][c] = y[u][c];
                    }
                    k = kn;
                    have = next;
                }
            } else {
                for (; k + (U - 1) * kWarps < k1; k += U * kWarps) {
                    T x[U][VW];
                    fetch(x, k);
                    absorb(x, k);
                }
            }
            for (; k < k1; k += kWarps) {
                const T *pr = p + (ptrdiff_t)k * row_stride;
                if (VW > 1) {
                    typename Vec128<T>::U t;
                    t.q = *reinterpret_cast<const uint4 *>(pr);
#pragma unroll
                    for (int c = 0; c < VW; ++c) R::add_one(s[c], t.e[c], k);
                } else {
                    R::add_one(s[0], *pr, k);
                }
            }
        }
        grid_dep_launch();
        // merge the 8 warps of the CTA: warp 0 ends with the state of (o, chunk, col + c)
        auto across_warps = [&](bool last_pass) {
#pragma unroll
            for (int c = 0; c < VW; ++c) smem[warp][lane][c] = s[c];
            __syncthreads();
            if (warp == 0 && col < inner) {
#pragma unroll
                for (int c = 0; c < VW; ++c) {
                    State t = smem[0][lane][c];
#pragma unroll
                    for (int w = 1; w < kWarps; ++w) t = R::merge(t, smem[w][lane][c]);
                    if (last_pass) dst[o * inner + col + c] = R::finish(t, st);
                    else partial[(o * split + chunk) * inner + col + c] = t;
                }
                if (!last_pass) __threadfence();  // chunk states visible device-wide before the counter moves
            }
            __syncthreads();
        };
        across_warps(split == 1);
        if (split == 1) continue;
        if (threadIdx.x == 0) {
            __threadfence();
            is_last = atomicAdd(counters + o * col_tiles + (item % col_tiles), 1u) == (unsigned int)split - 1u;
        }
        __syncthreads();
        if (!is_last) continue;  // uniform per CTA
        __threadfence();
#pragma unroll
        for (int c = 0; c < VW; ++c) s[c] = R::identity();
        if (col < inner)
            for (size_t ch = warp; ch < split; ch += kWarps)
#pragma unroll
                for (int c = 0; c < VW; ++c) s[c] = R::merge(s[c], load_state_cg(partial + (o * split + ch) * inner + col + c));
        across_warps(true);
        if (threadIdx.x == 0) counters[o * col_tiles + (item % col_tiles)] = 0;  // ready for the next launch
    }
}

// CTAs of `kernel` that are resident at once on the whole GPU
template <typename K> size_t resident_ctas(Ctx *ctx, K kernel) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kBlock, 0) != cudaSuccess || per_sm < 1) per_sm = 4;
    return (size_t)ctx->sm_count * (size_t)per_sm;
}

unsigned grid_of(size_t items) { return (unsigned)(items < kGridCap ? (items ? items : 1) : kGridCap); }

template <typename T, typename R>
int ext_launch(Ctx *ctx, const T *src, size_t outer, size_t len, size_t inner, ptrdiff_t outer_stride, ptrdiff_t row_stride,
               void *dst_raw, ExtSettings st) {
    using State = typename R::State;
    using Out = typename R::Out;
    constexpr size_t N = Vec128<T>::N;
    Out *dst = static_cast<Out *>(dst_raw);
    if (outer == 0 || inner == 0) return RTB_OK;
    std::lock_guard<std::mutex> lock(ctx->ws_mu);
    const size_t want = (size_t)ctx->sm_count * 4;  // work items that fill the GPU
    State *partial = nullptr;
    unsigned int *counters = nullptr;
    size_t split = 1;
    auto get_partial = [&](size_t states) {
        void *ws = nullptr;
        int rc = workspace(ctx, states * sizeof(State), &ws);
        if (rc != RTB_OK) return rc;
        partial = reinterpret_cast<State *>(reinterpret_cast<char *>(ws) + kWorkspaceHeader);
        counters = reinterpret_cast<unsigned int *>(ws) + kTileCounterOffset;
        return rc;
    };
    int rc = RTB_OK;
    if (inner == 1 && row_stride == 1) {
        if (outer < want && outer <= kMaxTileCounters && len >= 8192) {
            split = (want + outer - 1) / outer;
            if (split > len / 4096) split = len / 4096;  // chunks stay >= 4096 elements: always the CTA form
        }
        if (split > 1 && (rc = get_partial(outer * split)) != RTB_OK) return rc;
        const size_t items = outer * split;
        // A block-wide merge of heavy states costs more than reducing a few thousand elements, so such
        // rows up to 16384 elements go to one warp each when there are enough rows to fill the GPU.
        const bool warp_rows = len < 1024 || (R::kHeavyMerge && split == 1 && len <= 16384 && outer >= (size_t)ctx->sm_count * 32);
        if (!warp_rows)
            launch_dep(ctx, grid_of(items), kBlock, ext_rows_kernel<T, R, kBlock>, src, outer, len, outer_stride, split, partial, counters,
                                                                                     dst, st);
        else
            launch_dep(ctx, grid_of((items + kWarps - 1) / kWarps), kBlock, ext_rows_kernel<T, R, 32>, src, outer, len, outer_stride, 1,
                                                                                                 nullptr, nullptr, dst, st);
        return check_launch(ctx, "ext_rows_kernel");
    }
    const bool vec = inner % N == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 && outer_stride % (ptrdiff_t)N == 0 &&
                     row_stride % (ptrdiff_t)N == 0;
    const size_t cols_per_tile = 32 * (vec ? N : 1);
    const size_t base = outer * ((inner + cols_per_tile - 1) / cols_per_tile);
    // CTAs do equal work, so the launch is fastest as ONE wave of resident CTAs: as many chunks of k
    // per tile as fit, each at least 64 rows
    // Few column tiles (the chunked one-wave regime) and a reducer whose merge is long: the
    // software-pipelined instantiation (next batch loaded before this one is absorbed; twice the
    // registers, half the resident CTAs).  Measured on (8192,8192) axis 0: variance 59 -> 53 us,
    // argmax 56 -> 52 us; with many tiles and long loops it is 3-5 % slower, and logsumexp (121
    // registers) loses a third, so those stay on the plain loop.
    const bool pipe = vec && R::kPipelineCols && base < (size_t)ctx->sm_count * 2;
    const size_t resident = !vec ? resident_ctas(ctx, ext_cols_kernel<T, R, 1>)
                                 : (pipe ? resident_ctas(ctx, ext_cols_kernel<T, R, (int)N, R::kPipelineCols>)
                                         : resident_ctas(ctx, ext_cols_kernel<T, R, (int)N>));
    split = base <= kMaxTileCounters ? resident / base : 1;  // one completion counter per tile
    if (split > len / 64) split = len / 64;
    if (split < 1) split = 1;
    if (split > 1 && (rc = get_partial(outer * split * inner)) != RTB_OK) return rc;
    const unsigned grid = grid_of(base * split);
    if (pipe)
        launch_dep(ctx, grid, kBlock, ext_cols_kernel<T, R, (int)N, R::kPipelineCols>, src, outer, len, inner, outer_stride,
                   row_stride, split, partial, counters, dst, st);
    else if (vec)
        launch_dep(ctx, grid, kBlock, ext_cols_kernel<T, R, (int)N>, src, outer, len, inner, outer_stride, row_stride, split, partial,
                                                                        counters, dst, st);
    else
        launch_dep(ctx, grid, kBlock, ext_cols_kernel<T, R, 1>, src, outer, len, inner, outer_stride, row_stride, split, partial,
                                                                   counters, dst, st);
    return check_launch(ctx, "ext_cols_kernel");
}

template <typename T>
int ext_by_op(Ctx *ctx, int redop, const rtb_reduce_settings *set, const T *src, size_t outer, size_t len, size_t inner,
              ptrdiff_t outer_stride, ptrdiff_t row_stride, void *dst) {
    ExtSettings st{set ? (int)set->unbiased : 1, set ? (int)set->is_std : 0};
    switch (redop) {
        case RTB_VARIANCE: return ext_launch<T, RedVar<T>>(ctx, src, outer, len, inner, outer_stride, row_stride, dst, st);
        case RTB_LOGSUMEXP: return ext_launch<T, RedLse<T>>(ctx, src, outer, len, inner, outer_stride, row_stride, dst, st);
        case RTB_NORM: {
            const int p = set ? set->norm_type : 2;
            if (p == 1) return ext_launch<T, RedNorm<T, 1>>(ctx, src, outer, len, inner, outer_stride, row_stride, dst, st);
            if (p == 2) return ext_launch<T, RedNorm<T, 2>>(ctx, src, outer, len, inner, outer_stride, row_stride, dst, st);
            return fail(RTB_ERR_INVALID, "norm type %d is not 1 or 2", p);
        }
        case RTB_ARGMAX: return ext_launch<T, RedArg<T, true>>(ctx, src, outer, len, inner, outer_stride, row_stride, dst, st);
        case RTB_ARGMIN: return ext_launch<T, RedArg<T, false>>(ctx, src, outer, len, inner, outer_stride, row_stride, dst, st);
    }
    return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
}

}  // namespace

int launch_reduce_ext(Ctx *ctx, int dtype, int redop, const rtb_reduce_settings *settings, const void *src, size_t outer, size_t r,
                      size_t inner, ptrdiff_t outer_stride, ptrdiff_t row_stride, void *dst) {
    if (dtype == RTB_F32)
        return ext_by_op<float>(ctx, redop, settings, (const float *)src, outer, r, inner, outer_stride, row_stride, dst);
    if (dtype == RTB_F64)
        return ext_by_op<double>(ctx, redop, settings, (const double *)src, outer, r, inner, outer_stride, row_stride, dst);
    return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
}

}  // namespace rtb
