// Device context: one per device, created once and reused -- stream, reduction workspace and a
// caching device allocator.  Replaces the per-call context / handle creation and the raw
// cuMemAlloc / cuMemFree per tensor of the reference CUDA backend (src/backend/cuda.rs:38-51,
// 155-185, 668-836).
#include "rtb_internal.h"

namespace rtb {

static constexpr size_t kCounterBytes = 65536;  // header of completion counters, kept at zero by the kernels

int use_device(Ctx *ctx) {
    int cur = -1;
    RTB_CUDA(cudaGetDevice(&cur));
    if (cur != ctx->device) RTB_CUDA(cudaSetDevice(ctx->device));
    return RTB_OK;
}

static bool stream_capturing(cudaStream_t stream) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return st != cudaStreamCaptureStatusNone;
}
static bool capturing(Ctx *ctx) { return stream_capturing(ctx->stream); }

// A superseded workspace is never freed before rtb_ctx_destroy: kernels already enqueued, and CUDA
// graphs captured earlier, still hold its address.  It moves to ctx->retired instead, and
// ws_generation tells a holder of a captured graph that the graph should be recorded again.
int workspace(Ctx *ctx, size_t bytes, void **out) {
    size_t need = kCounterBytes + ((bytes + 255) & ~size_t(255));
    if (need > ctx->ws_bytes) {
        if (capturing(ctx))
            return fail(RTB_ERR_INVALID,
                        "the reduction workspace (%zu bytes) would have to grow to %zu bytes during stream capture: "
                        "run the sequence once eagerly or call rtb_ctx_reserve_workspace first",
                        ctx->ws_bytes, need);
        size_t grow = need < (size_t(1) << 20) ? (size_t(1) << 20) : need;
        void *p = nullptr;
        RTB_CUDA(cudaMalloc(&p, grow));
        // cudaMemset on the stream: ordered before every later kernel of this context
        cudaError_t e = cudaMemsetAsync(p, 0, kCounterBytes, ctx->stream);
        if (e != cudaSuccess) {
            cudaFree(p);
            return cuda_fail(e, "cudaMemsetAsync(workspace)");
        }
        if (ctx->ws) ctx->retired.push_back(ctx->ws);
        ctx->ws = p;
        ctx->ws_bytes = grow;
        ctx->ws_generation.fetch_add(1, std::memory_order_relaxed);
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
    rtb::host_release(ctx);
    rtb::mg_release(ctx);
    rtb_release_cached(c);
    for (auto &kv : ctx->live_blocks) cudaFree(kv.first);
    if (ctx->ws) cudaFree(ctx->ws);
    for (void *p : ctx->retired) cudaFree(p);
    if (ctx->order_event) cudaEventDestroy(ctx->order_event);
    delete ctx;
}

// The context's state (workspace counters and partial slots, the allocator's free list) is only
// ordered by the stream.  When the stream changes, the new stream is made to wait for everything
// enqueued so far on the old one, so that work issued through this context keeps one total order.
RTB_API int rtb_ctx_set_stream(rtb_ctx *c, void *stream) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    Ctx *ctx = C(c);
    cudaStream_t next = reinterpret_cast<cudaStream_t>(stream);
    if (next == ctx->stream) return RTB_OK;
    int rc = rtb::use_device(ctx);
    if (rc) return rc;
    if (!ctx->order_event) RTB_CUDA(cudaEventCreateWithFlags(&ctx->order_event, cudaEventDisableTiming));
    if (!rtb::capturing(ctx) && !rtb::stream_capturing(next)) {
        // (a stream that is being captured cannot be joined with work outside its graph: whoever set
        // up the capture has ordered the capturing stream after the earlier work)
        RTB_CUDA(cudaEventRecord(ctx->order_event, ctx->stream));
        RTB_CUDA(cudaStreamWaitEvent(next, ctx->order_event, 0));
    }
    ctx->stream = next;
    return RTB_OK;
}
RTB_API void *rtb_ctx_get_stream(rtb_ctx *c) { return c ? (void *)C(c)->stream : nullptr; }
RTB_API int rtb_ctx_device(rtb_ctx *c) { return c ? C(c)->device : -1; }
RTB_API int rtb_ctx_sm_count(rtb_ctx *c) { return c ? C(c)->sm_count : 0; }
RTB_API uint64_t rtb_ctx_launch_count(rtb_ctx *c) { return c ? C(c)->launches.load() : 0; }
RTB_API uint64_t rtb_ctx_workspace_generation(rtb_ctx *c) { return c ? C(c)->ws_generation.load() : 0; }

RTB_API int rtb_ctx_reserve_workspace(rtb_ctx *c, size_t bytes) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    Ctx *ctx = C(c);
    int rc = rtb::use_device(ctx);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(ctx->ws_mu);
    void *p = nullptr;
    return rtb::workspace(ctx, bytes, &p);
}

RTB_API int rtb_ctx_sync(rtb_ctx *c) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    int rc = rtb::use_device(C(c));
    if (rc) return rc;
    RTB_CUDA(cudaStreamSynchronize(C(c)->stream));
    return rtb::host_sync(C(c));  // copy-outs of host-buffer operations follow the compute stream
}

RTB_API int rtb_alloc(rtb_ctx *c, size_t bytes, void **out) {
    if (!c || !out) return rtb::fail(RTB_ERR_INVALID, "null argument");
    Ctx *ctx = C(c);
    int rc = rtb::use_device(ctx);
    if (rc) return rc;
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
    // Nothing is allocated or freed while the stream is being captured: a graph must only hold
    // addresses that stay valid for its replays.
    if (rtb::capturing(ctx))
        return rtb::fail(RTB_ERR_ALLOC, "rtb_alloc: no cached block of %zu bytes during stream capture "
                         "(run the sequence once eagerly so the allocator holds the blocks)", want);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e == cudaErrorMemoryAllocation) {  // give cached blocks back and retry once
        cudaGetLastError();
        cudaStreamSynchronize(ctx->stream);  // kernels enqueued earlier may still use freed blocks
        for (auto &kv : ctx->free_blocks) cudaFree(kv.second);
        ctx->free_blocks.clear();
        ctx->ws_generation.fetch_add(1, std::memory_order_relaxed);  // addresses a graph may hold are gone
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
    int rc = rtb::use_device(ctx);
    if (rc) return rc;
    if (rtb::capturing(ctx)) return rtb::fail(RTB_ERR_INVALID, "rtb_release_cached during stream capture");
    std::lock_guard<std::mutex> lock(ctx->mu);
    cudaStreamSynchronize(ctx->stream);
    for (auto &kv : ctx->free_blocks) cudaFree(kv.second);
    if (!ctx->free_blocks.empty()) ctx->ws_generation.fetch_add(1, std::memory_order_relaxed);
    ctx->free_blocks.clear();
    return RTB_OK;
}

RTB_API int rtb_h2d(rtb_ctx *c, void *dst, const void *src, size_t bytes) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    if (int rc = rtb::use_device(C(c))) return rc;
    RTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, C(c)->stream));
    return RTB_OK;
}
RTB_API int rtb_d2h(rtb_ctx *c, void *dst, const void *src, size_t bytes) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    if (int rc = rtb::use_device(C(c))) return rc;
    RTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, C(c)->stream));
    RTB_CUDA(cudaStreamSynchronize(C(c)->stream));
    return RTB_OK;
}
RTB_API int rtb_d2d(rtb_ctx *c, void *dst, const void *src, size_t bytes) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    if (int rc = rtb::use_device(C(c))) return rc;
    RTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, C(c)->stream));
    return RTB_OK;
}
