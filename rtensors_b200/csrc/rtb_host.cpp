// Host-buffer operations: work whose inputs and results live in HOST memory.  The reference moves whole
// tensors synchronously (alloc_from_slice / dump, src/backend/cuda.rs:668-680, 770-788: one blocking
// cuMemcpy each way per tensor); here a context owns an upload lane and a download lane (two more
// streams) and a pool of device slots, so that a tensor's upload, the kernels and the copy-out of the
// results run concurrently (PCIe is full duplex) and the compute stream never waits for a transfer it
// does not need.
//
// Ordering is by events only; no call in this file blocks the host except rtb_host_wait.
//   slot      a device block of the pool with three events: `ready` (the end of its upload) and two
//             `idle` events (its last reader is done: one for kernels on the compute stream, one for
//             copies on the download lane).  Whoever takes a slot from the pool makes the stream that
//             writes it first wait for both.
//   stage_in  takes a slot, copies host -> slot on the upload lane, records `ready`.  The compute
//             stream waits for it only when the caller says it needs the data (rtb_host_ready).
//   stage_out makes the download lane wait for the compute stream's work so far, copies device -> host
//             there and, when the source is a slot, records its `idle`.
#include <algorithm>

#include "rtb_internal.h"

namespace rtb {

struct HostSlot {
    void *ptr = nullptr;
    size_t bytes = 0;
    bool taken = false;
    bool output = false;  // written first by the compute stream (results, staging); else by the upload lane
    cudaEvent_t ready = nullptr;
    cudaEvent_t idle_compute = nullptr, idle_down = nullptr;  // the last kernel that read it / its last copy-out
    bool compute_set = false, down_set = false;               // the event has been recorded at least once
};

struct HostLanes {
    cudaStream_t up = nullptr, down = nullptr;
    cudaEvent_t mark = nullptr;  // scratch event: "the compute stream's work so far"
    cudaEvent_t join_up = nullptr, join_down = nullptr;
    std::mutex mu;
    std::vector<HostSlot> slots;
    size_t stage_bytes = size_t(64) << 20;  // one stage of rtb_host_broadcast
};

static bool host_capturing(Ctx *ctx) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->stream, &st) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return st != cudaStreamCaptureStatusNone;
}

static int lanes(Ctx *ctx, HostLanes **out) {
    if (int rc = use_device(ctx)) return rc;
    if (host_capturing(ctx)) return fail(RTB_ERR_INVALID, "host-buffer operations cannot be captured into a CUDA graph");
    std::lock_guard<std::mutex> create_lock(ctx->mu);
    if (!ctx->host) {
        HostLanes *h = new HostLanes();
        cudaError_t e = cudaStreamCreateWithFlags(&h->up, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->down, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->mark, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->join_up, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->join_down, cudaEventDisableTiming);
        if (e != cudaSuccess) {
            if (h->up) cudaStreamDestroy(h->up);
            if (h->down) cudaStreamDestroy(h->down);
            if (h->mark) cudaEventDestroy(h->mark);
            if (h->join_up) cudaEventDestroy(h->join_up);
            if (h->join_down) cudaEventDestroy(h->join_down);
            delete h;
            return cuda_fail(e, "creating the transfer lanes");
        }
        ctx->host = h;
    }
    *out = ctx->host;
    return RTB_OK;
}

static bool slot_is_idle(const HostSlot &s) {
    if (s.compute_set && cudaEventQuery(s.idle_compute) != cudaSuccess) return false;
    if (s.down_set && cudaEventQuery(s.idle_down) != cudaSuccess) return false;
    return true;
}

// A free slot of the same kind that holds `bytes` and is not more than twice as large.  One whose last
// readers are already done is preferred (the smallest of those).  If all candidates are still in use and
// the pool holds fewer than kPoolDepth blocks of this kind and size class, a new block is allocated instead
// of waiting (triple buffering: a chunk's upload, kernels and copy-out each need a block of their own);
// otherwise -- or when the device has no room for another -- the smallest busy candidate is taken and its
// first writer waits.  Inputs and outputs never trade blocks: an input's last reader is a kernel, an
// output's is a copy on the download lane, so an upload never has to wait for a copy-out (a 256 MiB input
// that took over a 256 MiB staging block was measured to serialise the two directions: 179 ms instead of
// 110 ms for 5.6 GB up and 4.3 GB down).
static constexpr size_t kPoolDepth = 3;

// frees a block's memory and events; the entry stays in the table as an empty one (ptr == nullptr)
static void drop_block(HostSlot &s) {
    cudaFree(s.ptr);
    cudaEventDestroy(s.ready);
    cudaEventDestroy(s.idle_compute);
    cudaEventDestroy(s.idle_down);
    s = HostSlot();
}

static int new_slot(HostLanes *h, size_t bytes, bool output, size_t *index) {
    HostSlot s;
    s.output = output;
    s.bytes = (bytes + 511) & ~size_t(511);
    cudaError_t e = cudaMalloc(&s.ptr, s.bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return RTB_ERR_CUDA;
    }
    e = cudaEventCreateWithFlags(&s.ready, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s.idle_compute, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&s.idle_down, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        cudaFree(s.ptr);
        if (s.ready) cudaEventDestroy(s.ready);
        if (s.idle_compute) cudaEventDestroy(s.idle_compute);
        cudaGetLastError();
        return RTB_ERR_CUDA;
    }
    for (size_t i = 0; i < h->slots.size(); ++i)
        if (!h->slots[i].ptr) {  // an empty entry left by drop_block
            h->slots[i] = s;
            *index = i;
            return RTB_OK;
        }
    h->slots.push_back(s);
    *index = h->slots.size() - 1;
    return RTB_OK;
}

static int take_slot(HostLanes *h, size_t bytes, bool output, size_t *index) {
    if (bytes == 0) bytes = 1;
    size_t best = SIZE_MAX, in_class = 0;
    bool best_idle = false;
    for (size_t i = 0; i < h->slots.size(); ++i) {
        const HostSlot &s = h->slots[i];
        if (!s.ptr || s.output != output || s.bytes < bytes || s.bytes / 2 > bytes) continue;
        ++in_class;
        if (s.taken) continue;
        const bool idle = slot_is_idle(s);
        if (best == SIZE_MAX || (idle && !best_idle) || (idle == best_idle && s.bytes < h->slots[best].bytes)) {
            best = i;
            best_idle = idle;
        }
    }
    cudaGetLastError();  // cudaEventQuery reports cudaErrorNotReady through the last-error state
    if (best == SIZE_MAX || (!best_idle && in_class < kPoolDepth)) {
        size_t fresh = 0;
        if (new_slot(h, bytes, output, &fresh) == RTB_OK) {
            best = fresh;
        } else if (best == SIZE_MAX) {
            // the device is full and nothing in the pool fits: give the pool's unused blocks whose readers
            // are done back to the device (blocks of other sizes pile up when a host moves tensors of many
            // different sizes) and ask once more.  Entries keep their positions: callers hold indices.
            for (HostSlot &s : h->slots)
                if (!s.taken && s.ptr && slot_is_idle(s)) drop_block(s);
            cudaGetLastError();
            if (new_slot(h, bytes, output, &fresh) != RTB_OK)
                return fail(RTB_ERR_CUDA, "no device memory for a host-buffer block of %zu bytes", bytes);
            best = fresh;
        }
    }
    h->slots[best].taken = true;
    *index = best;
    return RTB_OK;
}

static HostSlot *find_slot(HostLanes *h, const void *ptr) {
    for (HostSlot &s : h->slots)
        if (s.taken && s.ptr == ptr) return &s;
    return nullptr;
}

void host_release(Ctx *ctx) {
    HostLanes *h = ctx->host;
    if (!h) return;
    cudaStreamSynchronize(h->up);
    cudaStreamSynchronize(h->down);
    for (HostSlot &s : h->slots)
        if (s.ptr) drop_block(s);
    cudaStreamDestroy(h->up);
    cudaStreamDestroy(h->down);
    cudaEventDestroy(h->mark);
    cudaEventDestroy(h->join_up);
    cudaEventDestroy(h->join_down);
    delete h;
    ctx->host = nullptr;
}

int host_sync(Ctx *ctx) {
    HostLanes *h = ctx->host;
    if (!h) return RTB_OK;
    RTB_CUDA(cudaStreamSynchronize(h->up));
    RTB_CUDA(cudaStreamSynchronize(h->down));
    return RTB_OK;
}

// ---- the primitives, on a locked HostLanes ---------------------------------------------------------
static int wait_idle(cudaStream_t writer, const HostSlot &s) {
    if (s.compute_set) RTB_CUDA(cudaStreamWaitEvent(writer, s.idle_compute, 0));
    if (s.down_set) RTB_CUDA(cudaStreamWaitEvent(writer, s.idle_down, 0));
    return RTB_OK;
}

static int stage_in(Ctx *ctx, HostLanes *h, const void *src_host, size_t bytes, size_t *index) {
    if (int rc = take_slot(h, bytes, false, index)) return rc;
    HostSlot &s = h->slots[*index];
    int rc = wait_idle(h->up, s);
    if (rc == RTB_OK && bytes) {
        cudaError_t e = cudaMemcpyAsync(s.ptr, src_host, bytes, cudaMemcpyHostToDevice, h->up);
        if (e != cudaSuccess) rc = cuda_fail(e, "cudaMemcpyAsync(host to block)");
    }
    if (rc == RTB_OK) {
        cudaError_t e = cudaEventRecord(s.ready, h->up);
        if (e != cudaSuccess) rc = cuda_fail(e, "cudaEventRecord(ready)");
    }
    if (rc != RTB_OK) s.taken = false;  // nothing was enqueued on it that a later user would not wait for
    return rc;
}

// a slot the compute stream writes first (a result or a staging block)
static int take_output(Ctx *ctx, HostLanes *h, size_t bytes, size_t *index) {
    if (int rc = take_slot(h, bytes, true, index)) return rc;
    int rc = wait_idle(ctx->stream, h->slots[*index]);
    if (rc != RTB_OK) h->slots[*index].taken = false;
    return rc;
}

static int stage_out(Ctx *ctx, HostLanes *h, const void *src_dev, void *dst_host, size_t bytes, HostSlot *slot) {
    RTB_CUDA(cudaEventRecord(h->mark, ctx->stream));
    RTB_CUDA(cudaStreamWaitEvent(h->down, h->mark, 0));
    if (bytes) RTB_CUDA(cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, h->down));
    if (slot) {
        RTB_CUDA(cudaEventRecord(slot->idle_down, h->down));
        slot->down_set = true;
    }
    return RTB_OK;
}

// returns a slot whose last reader is the compute stream (an input) to the pool
static int give_back_after_compute(Ctx *ctx, HostSlot &s) {
    RTB_CUDA(cudaEventRecord(s.idle_compute, ctx->stream));
    s.compute_set = true;
    s.taken = false;
    return RTB_OK;
}

// Blocks a composite call holds: whatever is still listed when the call leaves (an error path) goes back
// to the pool.
struct Held {
    HostLanes *h;
    std::vector<size_t> idx;
    explicit Held(HostLanes *lanes) : h(lanes) {}
    ~Held() {
        for (size_t i : idx) h->slots[i].taken = false;
    }
    void done() { idx.clear(); }
};

static size_t product(const size_t *shape, size_t from, size_t rank) {
    size_t n = 1;
    for (size_t d = from; d < rank; ++d) n *= shape[d];
    return n;
}

}  // namespace rtb

using rtb::Ctx;
using rtb::HostLanes;
using rtb::HostSlot;
static inline Ctx *C(rtb_ctx *c) { return reinterpret_cast<Ctx *>(c); }

// ---- pinned host memory ------------------------------------------------------------------------------
RTB_API int rtb_host_alloc(size_t bytes, void **out) {
    if (!out) return rtb::fail(RTB_ERR_INVALID, "null argument");
    RTB_CUDA(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocPortable));
    return RTB_OK;
}
RTB_API int rtb_host_free(void *ptr) {
    if (ptr) RTB_CUDA(cudaFreeHost(ptr));
    return RTB_OK;
}
RTB_API int rtb_host_pin(void *ptr, size_t bytes) {
    if (!ptr || !bytes) return rtb::fail(RTB_ERR_INVALID, "rtb_host_pin needs a buffer");
    RTB_CUDA(cudaHostRegister(ptr, bytes, cudaHostRegisterPortable));
    return RTB_OK;
}
RTB_API int rtb_host_unpin(void *ptr) {
    if (ptr) RTB_CUDA(cudaHostUnregister(ptr));
    return RTB_OK;
}

// ---- primitives ----------------------------------------------------------------------------------------
RTB_API int rtb_host_stage_in(rtb_ctx *c, const void *src_host, size_t bytes, void **dev_out) {
    if (!c || !dev_out || (!src_host && bytes)) return rtb::fail(RTB_ERR_INVALID, "null argument");
    HostLanes *h = nullptr;
    if (int rc = rtb::lanes(C(c), &h)) return rc;
    std::lock_guard<std::mutex> lock(h->mu);
    size_t i = 0;
    if (int rc = rtb::stage_in(C(c), h, src_host, bytes, &i)) return rc;
    *dev_out = h->slots[i].ptr;
    return RTB_OK;
}

RTB_API int rtb_host_scratch(rtb_ctx *c, size_t bytes, void **dev_out) {
    if (!c || !dev_out) return rtb::fail(RTB_ERR_INVALID, "null argument");
    HostLanes *h = nullptr;
    if (int rc = rtb::lanes(C(c), &h)) return rc;
    std::lock_guard<std::mutex> lock(h->mu);
    size_t i = 0;
    if (int rc = rtb::take_output(C(c), h, bytes, &i)) return rc;
    *dev_out = h->slots[i].ptr;
    return RTB_OK;
}

RTB_API int rtb_host_ready(rtb_ctx *c, const void *dev) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    HostLanes *h = nullptr;
    if (int rc = rtb::lanes(C(c), &h)) return rc;
    std::lock_guard<std::mutex> lock(h->mu);
    HostSlot *s = rtb::find_slot(h, dev);
    if (!s) return rtb::fail(RTB_ERR_INVALID, "rtb_host_ready: not a block handed out by rtb_host_stage_in");
    RTB_CUDA(cudaStreamWaitEvent(C(c)->stream, s->ready, 0));
    return RTB_OK;
}

RTB_API int rtb_host_stage_out(rtb_ctx *c, const void *src_dev, void *dst_host, size_t bytes) {
    if (!c || ((!src_dev || !dst_host) && bytes)) return rtb::fail(RTB_ERR_INVALID, "null argument");
    HostLanes *h = nullptr;
    if (int rc = rtb::lanes(C(c), &h)) return rc;
    std::lock_guard<std::mutex> lock(h->mu);
    // the source may lie inside a slot (a staging block cut into pieces)
    HostSlot *slot = nullptr;
    for (HostSlot &s : h->slots)
        if (s.taken && (const char *)src_dev >= (const char *)s.ptr && (const char *)src_dev < (const char *)s.ptr + s.bytes) slot = &s;
    if (slot && (const char *)src_dev + bytes > (const char *)slot->ptr + slot->bytes)
        return rtb::fail(RTB_ERR_BOUNDS, "rtb_host_stage_out: %zu bytes from this address run past the end of its pool block", bytes);
    return rtb::stage_out(C(c), h, src_dev, dst_host, bytes, slot);
}

RTB_API int rtb_host_release(rtb_ctx *c, void *dev) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    if (!dev) return RTB_OK;
    HostLanes *h = nullptr;
    if (int rc = rtb::lanes(C(c), &h)) return rc;
    std::lock_guard<std::mutex> lock(h->mu);
    HostSlot *s = rtb::find_slot(h, dev);
    if (!s) return rtb::fail(RTB_ERR_INVALID, "rtb_host_release: not a block of the host-buffer pool");
    // its readers so far: copies on the download lane (their event is already recorded) and kernels on
    // the compute stream (recorded now)
    return rtb::give_back_after_compute(C(c), *s);
}

RTB_API int rtb_host_join(rtb_ctx *c) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    HostLanes *h = nullptr;
    if (int rc = rtb::lanes(C(c), &h)) return rc;
    std::lock_guard<std::mutex> lock(h->mu);
    RTB_CUDA(cudaEventRecord(h->join_up, h->up));
    RTB_CUDA(cudaEventRecord(h->join_down, h->down));
    RTB_CUDA(cudaStreamWaitEvent(C(c)->stream, h->join_up, 0));
    RTB_CUDA(cudaStreamWaitEvent(C(c)->stream, h->join_down, 0));
    return RTB_OK;
}

RTB_API int rtb_host_wait(rtb_ctx *c) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    if (int rc = rtb::use_device(C(c))) return rc;
    RTB_CUDA(cudaStreamSynchronize(C(c)->stream));
    return rtb::host_sync(C(c));
}

RTB_API int rtb_host_trim(rtb_ctx *c) {
    if (!c) return rtb::fail(RTB_ERR_INVALID, "null ctx");
    if (int rc = rtb_host_wait(c)) return rc;
    HostLanes *h = C(c)->host;
    if (!h) return RTB_OK;
    std::lock_guard<std::mutex> lock(h->mu);
    for (HostSlot &s : h->slots)
        if (!s.taken && s.ptr) rtb::drop_block(s);
    return RTB_OK;
}

RTB_API int rtb_host_set_stage_bytes(rtb_ctx *c, size_t bytes) {
    if (!c || !bytes) return rtb::fail(RTB_ERR_INVALID, "rtb_host_set_stage_bytes needs a context and a size");
    HostLanes *h = nullptr;
    if (int rc = rtb::lanes(C(c), &h)) return rc;
    std::lock_guard<std::mutex> lock(h->mu);
    h->stage_bytes = bytes;
    return RTB_OK;
}

// ---- composites ----------------------------------------------------------------------------------------
RTB_API int rtb_host_reduce_view(rtb_ctx *c, int dtype, int redop, const rtb_reduce_settings *settings, const void *src_host,
                                 size_t src_len, size_t rank, const size_t *shape, const ptrdiff_t *strides, size_t offset,
                                 ptrdiff_t axis, void *dst_host) {
    if (!c || !src_host || !dst_host || (rank && (!shape || !strides))) return rtb::fail(RTB_ERR_INVALID, "null argument");
    const size_t es = rtb::dtype_size(dtype);
    if (!es) return rtb::fail(RTB_ERR_DTYPE, "unknown dtype %d", dtype);
    if (axis >= (ptrdiff_t)rank) return rtb::fail(RTB_ERR_INVALID, "axis %td out of range for rank %zu", axis, rank);
    if (int rc = rtb_meta_check_extent(rank, shape, strides, offset, src_len)) return rc;
    size_t out_elems = 1;
    if (axis >= 0)
        for (size_t d = 0; d < rank; ++d)
            if ((ptrdiff_t)d != axis) out_elems *= shape[d];
    const size_t out_es = (redop == RTB_ARGMAX || redop == RTB_ARGMIN) ? sizeof(uint64_t) : es;
    HostLanes *h = nullptr;
    if (int rc = rtb::lanes(C(c), &h)) return rc;
    std::lock_guard<std::mutex> lock(h->mu);
    size_t in = 0, out = 0;
    rtb::Held held(h);
    if (int rc = rtb::stage_in(C(c), h, src_host, src_len * es, &in)) return rc;
    held.idx.push_back(in);
    if (int rc = rtb::take_output(C(c), h, out_elems * out_es, &out)) return rc;
    held.idx.push_back(out);
    RTB_CUDA(cudaStreamWaitEvent(C(c)->stream, h->slots[in].ready, 0));
    held.done();  // from here on both blocks are returned below, with the events that protect them
    int rc = rtb_reduce_view_ex(c, dtype, redop, settings, h->slots[in].ptr, rank, shape, strides, offset, axis, h->slots[out].ptr);
    if (rc == RTB_OK) rc = rtb::stage_out(C(c), h, h->slots[out].ptr, dst_host, out_elems * out_es, &h->slots[out]);
    h->slots[out].taken = false;  // idle once the copy-out just enqueued is done
    int rc2 = rtb::give_back_after_compute(C(c), h->slots[in]);
    return rc ? rc : rc2;
}

RTB_API int rtb_host_broadcast(rtb_ctx *c, int dtype, int binop, const void *left_host, size_t left_len, const ptrdiff_t *stride_l,
                               size_t off_l, const void *right_host, size_t right_len, const ptrdiff_t *stride_r, size_t off_r,
                               void *dst_host, size_t rank, const size_t *shape, size_t begin, size_t end) {
    if (!c || !left_host || !right_host || !dst_host || (rank && (!shape || !stride_l || !stride_r)))
        return rtb::fail(RTB_ERR_INVALID, "null argument");
    const size_t es = rtb::dtype_size(dtype);
    if (!es) return rtb::fail(RTB_ERR_DTYPE, "unknown dtype %d", dtype);
    if (int rc = rtb_meta_check_extent(rank, shape, stride_l, off_l, left_len)) return rc;
    if (int rc = rtb_meta_check_extent(rank, shape, stride_r, off_r, right_len)) return rc;
    const size_t extent0 = rank ? shape[0] : 1;
    if (begin > end || end > extent0) return rtb::fail(RTB_ERR_INVALID, "range [%zu, %zu) of an outermost dim of %zu", begin, end, extent0);
    const size_t per = rtb::product(shape, 1, rank);  // elements per index of the outermost dim
    if (begin == end || per == 0) return RTB_OK;
    // indices of the outermost dim per stage: about 64 MiB by default, so that a stage's copy-out is long
    // against its launch and the ring of three stays small
    HostLanes *h = nullptr;
    if (int rc = rtb::lanes(C(c), &h)) return rc;
    std::lock_guard<std::mutex> lock(h->mu);
    const size_t target = h->stage_bytes;
    size_t group = std::max<size_t>(1, target / std::max<size_t>(per * es, 1));
    group = std::min(group, end - begin);
    const size_t stage_bytes = group * per * es;
    const size_t n_stages = (end - begin + group - 1) / group;
    const size_t ring = std::min<size_t>(3, n_stages);
    size_t l = 0, r = 0, st[3] = {0, 0, 0};
    rtb::Held held(h);
    if (int rc = rtb::stage_in(C(c), h, left_host, left_len * es, &l)) return rc;
    held.idx.push_back(l);
    if (int rc = rtb::stage_in(C(c), h, right_host, right_len * es, &r)) return rc;
    held.idx.push_back(r);
    for (size_t k = 0; k < ring; ++k) {
        if (int rc = rtb::take_output(C(c), h, stage_bytes, &st[k])) return rc;
        held.idx.push_back(st[k]);
    }
    RTB_CUDA(cudaStreamWaitEvent(C(c)->stream, h->slots[l].ready, 0));
    RTB_CUDA(cudaStreamWaitEvent(C(c)->stream, h->slots[r].ready, 0));
    held.done();  // from here on every block is returned below, with the events that protect it

    std::vector<size_t> sshape(shape, shape + rank);
    std::vector<ptrdiff_t> sd(rank);
    int rc = RTB_OK;
    for (size_t k = 0, i = begin; i < end && rc == RTB_OK; ++k, i += group) {
        const size_t n = std::min(group, end - i);
        HostSlot &stage = h->slots[st[k % ring]];
        if (k >= ring) {  // the block's previous copy-out is done
            cudaError_t e = cudaStreamWaitEvent(C(c)->stream, stage.idle_down, 0);
            if (e != cudaSuccess) {
                rc = rtb::cuda_fail(e, "cudaStreamWaitEvent(stage)");
                break;
            }
        }
        if (rank) sshape[0] = n;
        rtb_meta_contiguous_strides(rank, sshape.data(), sd.data());
        rc = rtb_broadcast(c, dtype, binop, h->slots[l].ptr, stride_l, off_l + (rank ? i * stride_l[0] : 0), h->slots[r].ptr, stride_r,
                           off_r + (rank ? i * stride_r[0] : 0), stage.ptr, sd.data(), 0, rank, sshape.data());
        if (rc == RTB_OK)
            rc = rtb::stage_out(C(c), h, stage.ptr, (char *)dst_host + (i - begin) * per * es, n * per * es, &stage);
    }
    for (size_t k = 0; k < ring; ++k) h->slots[st[k]].taken = false;  // idle once their last copy-out is done
    int rc2 = rtb::give_back_after_compute(C(c), h->slots[l]);
    int rc3 = rtb::give_back_after_compute(C(c), h->slots[r]);
    return rc ? rc : (rc2 ? rc2 : rc3);
}
