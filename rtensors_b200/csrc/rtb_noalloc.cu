// rtb_reduce_flat_noalloc: a full reduction (sum / prod / max / min / mean of a contiguous range)
// that never asks the CUDA allocator for anything.
//
// Why it exists.  The regular flat reduction keeps its per-CTA partial results and a completion
// counter in a workspace that the library grows with cudaMalloc on first use.  Some hosts cannot
// tolerate that: a process that has already handed every byte of device memory to its own pool
// (so a further cudaMalloc simply fails), a latency-critical loop in which cudaMalloc's implicit
// device-wide synchronisation is forbidden, or an embedding runtime whose rule is that foreign
// libraries do not allocate.  For them the scratch lives in a fixed array inside the library
// image; the caller still supplies the input and the one-element output.
//
// What that costs.  Every GPU that loads the library carries the array (64.25 KiB) until the
// process exits.  The array bounds the problem: one partial slot per CTA, one CTA per 65,536
// elements, 8,192 slots -> at most RTB_NOALLOC_MAX_LEN = 2^29 elements per call; longer ranges
// are rejected, not split.  All calls on a device share the one array, and it still holds
// whatever the previous call left there: the counter word is cleared on the stream before every
// launch (the partial slots need no clearing, each is written before it is read).  Two calls
// whose kernels could run at the same time on one device -- different streams, different host
// threads -- would race on the array; callers must order them (same stream, or an event).
//
// Set-up.  Host code cannot use the array's name as a device address (on the host the symbol is
// only a stand-in).  The first call on each device therefore resolves the address once with
// cudaGetSymbolAddress while that device is current, and caches it.  Make that first call
// outside any stream capture.
//
// Accumulator semantics are those of the regular reduction (reference CPU backend,
// src/ops/reduction/mod.rs:9-137): max / min start from the lowest / highest finite value and use
// `v > acc` / `v < acc`; mean divides by (T)(float)len; float sums are tree-ordered.
#include <cfloat>
#include <mutex>

#include "rtb_internal.h"

namespace {

constexpr int kThreads = 256;
constexpr size_t kTileElems = 65536;                 // elements reduced by one CTA
constexpr size_t kSlots = 8192;                      // partial results the scratch can hold
constexpr size_t kHeaderBytes = 256;                 // counter word lives here
constexpr size_t kScratchBytes = kHeaderBytes + kSlots * sizeof(double);
static_assert(kTileElems * kSlots == RTB_NOALLOC_MAX_LEN, "header constant out of date");

static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

template <typename T> struct Lim;
template <> struct Lim<float> {
    static __device__ float lo() { return -FLT_MAX; }
    static __device__ float hi() { return FLT_MAX; }
};
template <> struct Lim<double> {
    static __device__ double lo() { return -DBL_MAX; }
    static __device__ double hi() { return DBL_MAX; }
};

template <typename T, int OP> struct Acc {
    static __device__ __forceinline__ T identity() {
        return OP == RTB_PROD ? (T)1 : OP == RTB_MAX ? Lim<T>::lo() : OP == RTB_MIN ? Lim<T>::hi() : (T)0;
    }
    static __device__ __forceinline__ T apply(T a, T b) {
        if (OP == RTB_PROD) return a * b;
        if (OP == RTB_MAX) return b > a ? b : a;
        if (OP == RTB_MIN) return b < a ? b : a;
        return a + b;
    }
};

template <typename T, int OP>
__device__ __forceinline__ T cta_reduce(T v, T *smem) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = Acc<T, OP>::apply(v, __shfl_down_sync(0xffffffffu, v, d));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    T out = Acc<T, OP>::identity();
    if (warp == 0) {
        out = lane < kThreads / 32 ? smem[lane] : Acc<T, OP>::identity();
#pragma unroll
        for (int d = kThreads / 64; d > 0; d >>= 1) out = Acc<T, OP>::apply(out, __shfl_down_sync(0xffffffffu, out, d));
    }
    __syncthreads();
    return out;
}

// CTA b reduces src[b*kTileElems, ...) into scratch slot b; the last CTA to finish folds the slots
// in index order and writes dst[0].  `scratch` is the device address of g_noalloc_scratch.
template <typename T, int OP>
__global__ void __launch_bounds__(kThreads) noalloc_reduce_kernel(const T *src, size_t n, unsigned char *scratch,
                                                                  T *dst, int mean) {
    __shared__ T smem[kThreads / 32];
    __shared__ bool is_last;
    constexpr int N = 16 / (int)sizeof(T);
    unsigned int *counter = reinterpret_cast<unsigned int *>(scratch);
    T *slots = reinterpret_cast<T *>(scratch + kHeaderBytes);

    const size_t begin = (size_t)blockIdx.x * kTileElems;
    const size_t end = begin + kTileElems < n ? begin + kTileElems : n;
    const T *p = src + begin;
    const size_t len = end - begin;
    size_t head = ((16u - (unsigned)((uintptr_t)p & 15u)) & 15u) / sizeof(T);
    if (head > len) head = len;
    const size_t nvec = (len - head) / N;
    const uint4 *pv = reinterpret_cast<const uint4 *>(p + head);
    union V { uint4 q; T e[N]; };

    T acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = Acc<T, OP>::identity();
    size_t i = threadIdx.x;
    for (; i + 3 * kThreads < nvec; i += 4 * kThreads) {
        V v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u].q = pv[i + u * kThreads];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < N; ++j) acc[u] = Acc<T, OP>::apply(acc[u], v[u].e[j]);
    }
    for (; i < nvec; i += kThreads) {
        V v;
        v.q = pv[i];
#pragma unroll
        for (int j = 0; j < N; ++j) acc[0] = Acc<T, OP>::apply(acc[0], v.e[j]);
    }
    for (size_t k = threadIdx.x; k < head; k += kThreads) acc[1] = Acc<T, OP>::apply(acc[1], p[k]);
    for (size_t k = head + nvec * N + threadIdx.x; k < len; k += kThreads) acc[2] = Acc<T, OP>::apply(acc[2], p[k]);

    T v = Acc<T, OP>::apply(Acc<T, OP>::apply(acc[0], acc[1]), Acc<T, OP>::apply(acc[2], acc[3]));
    v = cta_reduce<T, OP>(v, smem);
    if (threadIdx.x == 0) {
        slots[blockIdx.x] = v;
        __threadfence();
        is_last = atomicAdd(counter, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    T t = Acc<T, OP>::identity();
    for (unsigned int k = threadIdx.x; k < gridDim.x; k += kThreads) t = Acc<T, OP>::apply(t, __ldcg(slots + k));
    t = cta_reduce<T, OP>(t, smem);
    if (threadIdx.x == 0) dst[0] = mean ? t / (T)(float)n : t;
}

// Device address of the scratch array, resolved once per device (index = device ordinal).
std::mutex g_mu;
unsigned char *g_scratch_addr[64] = {};

int scratch_address(unsigned char **out) {
    int dev = -1;
    RTB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return rtb::fail(RTB_ERR_INVALID, "device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_addr[dev]) {
        void *p = nullptr;
        RTB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_scratch_addr[dev] = static_cast<unsigned char *>(p);
    }
    *out = g_scratch_addr[dev];
    return RTB_OK;
}

template <typename T, int OP>
int run(const T *src, size_t n, unsigned char *scratch, T *dst, int mean, cudaStream_t stream) {
    const unsigned grid = (unsigned)((n + kTileElems - 1) / kTileElems);
    // the counter word must be zero when the kernel starts, whatever an earlier call left behind
    RTB_CUDA(cudaMemsetAsync(scratch, 0, kHeaderBytes, stream));
    noalloc_reduce_kernel<T, OP><<<grid ? grid : 1, kThreads, 0, stream>>>(src, n, scratch, dst, mean);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return rtb::cuda_fail(e, "noalloc_reduce_kernel");
    return RTB_OK;
}

template <typename T>
int by_op(int redop, const T *src, size_t n, unsigned char *scratch, T *dst, cudaStream_t stream) {
    switch (redop) {
        case RTB_SUM: return run<T, RTB_SUM>(src, n, scratch, dst, 0, stream);
        case RTB_MEAN: return run<T, RTB_SUM>(src, n, scratch, dst, 1, stream);
        case RTB_PROD: return run<T, RTB_PROD>(src, n, scratch, dst, 0, stream);
        case RTB_MAX: return run<T, RTB_MAX>(src, n, scratch, dst, 0, stream);
        case RTB_MIN: return run<T, RTB_MIN>(src, n, scratch, dst, 0, stream);
    }
    return rtb::fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
}

}  // namespace

RTB_API int rtb_reduce_flat_noalloc(int dtype, int redop, const void *src, size_t start, size_t len, void *dst,
                                    void *stream) {
    if (!src || !dst) return rtb::fail(RTB_ERR_INVALID, "null argument");
    if (dtype != RTB_F32 && dtype != RTB_F64) return rtb::fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
    if (len > RTB_NOALLOC_MAX_LEN)
        return rtb::fail(RTB_ERR_TOO_LARGE,
                         "rtb_reduce_flat_noalloc: len %zu exceeds RTB_NOALLOC_MAX_LEN (%zu elements); the built-in "
                         "scratch has one slot per 65536 elements and 8192 slots -- use rtb_reduce_flat, or reduce in pieces",
                         len, (size_t)RTB_NOALLOC_MAX_LEN);
    unsigned char *scratch = nullptr;
    int rc = scratch_address(&scratch);
    if (rc != RTB_OK) return rc;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (dtype == RTB_F32) return by_op<float>(redop, (const float *)src + start, len, scratch, (float *)dst, s);
    return by_op<double>(redop, (const double *)src + start, len, scratch, (double *)dst, s);
}
