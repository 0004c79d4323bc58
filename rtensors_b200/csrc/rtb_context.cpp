// Device context: one per device, created once and reused -- stream, reduction workspace and a
// caching device allocator.  Replaces the per-call context / handle creation and the raw
// cuMemAlloc / cuMemFree per tensor of the reference CUDA backend (src/backend/cuda.rs:38-51,
// 155-185, 668-836).
#include "rtb_internal.h"

namespace rtb {

static constexpr size_t kCounterBytes = 65536;  // header of completion counters, kept at zero by the kernels

int workspace(Ctx *ctx, size_t bytes, void **out) {
    size_t need = kCounterBytes + ((bytes + 255) & ~size_t(255));
    if (need > ctx->ws_bytes) {
        size_t grow = need < (size_t(1) << 20) ? (size_t(1) << 20) : need;
        void *p = nullptr;
        // earlier kernels may still be using the old workspace
        RTB_CUDA(cudaStreamSynchronize(ctx->stream));
        RTB_CUDA(cudaMalloc(&p, grow));
        cudaError_t e = cudaMemsetAsync(p, 0, kCounterBytes, ctx->stream);
        if (e != cudaSuccess) {
            cudaFree(p);
            return cuda_fail(e, "cudaMemsetAsync(workspace)");
        }
        if (ctx->ws) cudaFree(ctx->ws);
        ctx->ws = p;
        ctx->ws_bytes = grow;
    }
    *out = ctx->ws;
    return RTB_OK;
}

int check_launch(Ctx *ctx, const char *what) {
    count_launch(ctx);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, what);
    return RTB_OK;
}

static std::mutex g_default_mu;
static std::map<int, Ctx *> g_default;

Ctx *default_ctx() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lock(g_default_mu);
    auto it = g_default.find(dev);
    if (it != g_default.end()) return it->second;
    rtb_ctx *c = nullptr;
    if (rtb_ctx_create(dev, &c) != RTB_OK) return nullptr;
    g_default[dev] = reinterpret_cast<Ctx *>(c);
    return g_default[dev];
}

static size_t round_block(size_t bytes) {
    if (bytes < 512) return 512;
    if (bytes < (size_t(1) << 20)) return (bytes + 511) & ~size_t(511);
    return (bytes + (size_t(2) << 20) - 1) & ~((size_t(2) << 20) - 1);
}

}  // namespace rtb

using rtb::Ctx;

static inline Ctx *C(rtb_ctx *c) { return reinterpret_cast<Ctx *>(c); }

RTB_API int rtb_ctx_create(int device, rtb_ctx **out) {
    if (!out) return rtb::fail(RTB_ERR_INVALID, "null out pointer");
    int count = 0;
    RTB_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return rtb::fail(RTB_ERR_INVALID, "device %d not in [0,%d)", device, count);
    RTB_CUDA(cudaSetDevice(device));
    Ctx *ctx = new Ctx();
    ctx->device = device;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) {
        delete ctx;
        return rtb::cuda_fail(e, "cudaGetDeviceProperties");
    }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->l2_bytes = (size_t)prop.l2CacheSize;
    *out = reinterpret_cast<rtb_ctx *>(ctx);
    return RTB_OK;
}

RTB_API void rtb_ctx_destroy(rtb_ctx *c) {
    if (!c) return;
    Ctx *ctx = C(c);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    rtb_release_cached(c);
    for (auto &kv : ctx->live_blocks) cudaFree(kv.first);
    if (ctx->ws) cudaFree(ctx->ws);
    delete ctx;
}

RTB_API int rtb_ctx_set_stream(rtb_ctx *c, void *stream) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    C(c)->stream = reinterpret_cast<cudaStream_t>(stream);
    return RTB_OK;
}
RTB_API void *rtb_ctx_get_stream(rtb_ctx *c) { return c ? (void *)C(c)->stream : nullptr; }
RTB_API int rtb_ctx_device(rtb_ctx *c) { return c ? C(c)->device : -1; }
RTB_API int rtb_ctx_sm_count(rtb_ctx *c) { return c ? C(c)->sm_count : 0; }
RTB_API uint64_t rtb_ctx_launch_count(rtb_ctx *c) { return c ? C(c)->launches.load() : 0; }

RTB_API int rtb_ctx_sync(rtb_ctx *c) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    RTB_CUDA(cudaStreamSynchronize(C(c)->stream));
    return RTB_OK;
}

RTB_API int rtb_alloc(rtb_ctx *c, size_t bytes, void **out) {
    if (!c || !out) return rtb::fail(RTB_ERR_INVALID, "null argument");
    Ctx *ctx = C(c);
    size_t want = rtb::round_block(bytes);
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = ctx->free_blocks.lower_bound(want);
    // reuse a cached block unless it would waste more than a quarter of itself
    if (it != ctx->free_blocks.end() && it->first - want <= it->first / 4) {
        *out = it->second;
        ctx->live_blocks[it->second] = it->first;
        ctx->free_blocks.erase(it);
        return RTB_OK;
    }
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e == cudaErrorMemoryAllocation) {  // give cached blocks back and retry once
        cudaGetLastError();
        for (auto &kv : ctx->free_blocks) cudaFree(kv.second);
        ctx->free_blocks.clear();
        e = cudaMalloc(&p, want);
    }
    if (e != cudaSuccess) return rtb::cuda_fail(e, "cudaMalloc");
    ctx->live_blocks[p] = want;
    *out = p;
    return RTB_OK;
}

RTB_API int rtb_free(rtb_ctx *c, void *ptr) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    if (!ptr) return RTB_OK;
    Ctx *ctx = C(c);
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = ctx->live_blocks.find(ptr);
    if (it == ctx->live_blocks.end()) return rtb::fail(RTB_ERR_INVALID, "pointer was not allocated by this ctx");
    // Stream order makes reuse safe: the next owner's kernels are enqueued after the last user's.
    ctx->free_blocks.emplace(it->second, ptr);
    ctx->live_blocks.erase(it);
    return RTB_OK;
}

RTB_API int rtb_release_cached(rtb_ctx *c) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    Ctx *ctx = C(c);
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaStreamSynchronize(ctx->stream);
    for (auto &kv : ctx->free_blocks) cudaFree(kv.second);
    ctx->free_blocks.clear();
    return RTB_OK;
}

RTB_API int rtb_h2d(rtb_ctx *c, void *dst, const void *src, size_t bytes) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    RTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, C(c)->stream));
    return RTB_OK;
}
RTB_API int rtb_d2h(rtb_ctx *c, void *dst, const void *src, size_t bytes) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    RTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, C(c)->stream));
    RTB_CUDA(cudaStreamSynchronize(C(c)->stream));
    return RTB_OK;
}
RTB_API int rtb_d2d(rtb_ctx *c, void *dst, const void *src, size_t bytes) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    RTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, C(c)->stream));
    return RTB_OK;
}
