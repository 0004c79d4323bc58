// Multi-GPU layer behind the C ABI (`rtb_mg_*`): one rank per GPU, one communicator per context.
//
// The reference is single-device (`Cuda::new()` -> device 0 with `// TODO multiple devices`,
// src/backend/cuda.rs:155-162, 815-818).  The path shards by slabs with no data-path collective for
// elementwise / broadcast work; a collective appears only where a reduction runs across the
// sharded dim.  Two transports:
//   * small results (one value, a partial vector of up to 64 KiB): the peer-memory exchange of
//     rtb_mg.cuh, fused into the reduction's last CTA for full reductions and L1 loss, a small
//     kernel of its own for partial vectors -- a few microseconds instead of a collective launch;
//   * everything else (the gradient bucket): ncclAllReduce on the context's stream, or on the
//     communicator's side stream between rtb_mg_allreduce_begin / _join so that it overlaps compute.
// NCCL is bound at run time (dlopen of libnccl.so.2, reusing the copy the host process already
// loaded), so the library itself has no link dependency on it and single-GPU hosts need no NCCL.
#include <dlfcn.h>
#include <nccl.h>
#include <unistd.h>

#include <cstdlib>

#include "rtb_mg.cuh"

namespace rtb {

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
};

std::mutex g_nccl_mu;
NcclApi g_nccl;

int load_nccl() {
    std::lock_guard<std::mutex> lock(g_nccl_mu);
    if (g_nccl.handle) return RTB_OK;
    // the copy the process already holds (a framework's bundled NCCL) wins over the system one
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(RTB_ERR_INVALID, "NCCL is not available: %s", dlerror());
    NcclApi a;
    a.handle = h;
#define RTB_SYM(field, name)                                                      \
    a.field = reinterpret_cast<decltype(a.field)>(dlsym(h, name));               \
    if (!a.field) return fail(RTB_ERR_INVALID, "NCCL symbol %s is missing", name);
    RTB_SYM(GetUniqueId, "ncclGetUniqueId")
    RTB_SYM(CommInitRank, "ncclCommInitRank")
    RTB_SYM(CommDestroy, "ncclCommDestroy")
    RTB_SYM(AllReduce, "ncclAllReduce")
    RTB_SYM(AllGather, "ncclAllGather")
    RTB_SYM(GetErrorString, "ncclGetErrorString")
    RTB_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
#undef RTB_SYM
    g_nccl = a;
    return RTB_OK;
}

int nccl_fail(ncclResult_t r, const char *what) {
    return fail(RTB_ERR_CUDA, "%s: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "NCCL error");
}
#define RTB_NCCL(call)                                              \
    do {                                                            \
        ncclResult_t r__ = (call);                                  \
        if (r__ != ncclSuccess) return nccl_fail(r__, #call);       \
    } while (0)

}  // namespace

struct Mg {
    ncclComm_t comm = nullptr;
    int nranks = 1, rank = 0;
    uint2 *local = nullptr;                 // this rank's exchange buffer
    uint2 *slots[kMgMaxRanks] = {};         // every rank's buffer as seen from this process
    bool mapped = false;                    // peers' buffers are mapped (CUDA IPC, or peer access inside one process)
    bool same_process[kMgMaxRanks] = {};    // slots[p] is a raw pointer of this process: nothing to close
    unsigned int *state = nullptr;          // device: epoch, status, counter, pad
    unsigned long long wait_ns = 2000000000ull;
    cudaStream_t side = nullptr;
    cudaEvent_t fork_ev = nullptr, join_ev = nullptr;
    bool side_busy = false;
};

bool mg_peers(Ctx *ctx, MgPeers *out) {
    Mg *mg = ctx->mg;
    if (!mg || !mg->mapped) return false;
    out->nranks = mg->nranks;
    out->rank = mg->rank;
    out->wait_ns = mg->wait_ns;
    for (int p = 0; p < kMgMaxRanks; ++p) out->slots[p] = mg->slots[p];
    out->state = mg->state;
    return true;
}

namespace {

constexpr int kBlock = 256;

template <typename T, int OP> struct Fold {
    static __device__ __forceinline__ T apply(T a, T b) {
        if (OP == RTB_PROD) return a * b;
        if (OP == RTB_MAX) return b > a ? b : a;
        if (OP == RTB_MIN) return b < a ? b : a;
        return a + b;
    }
};

// Partial vectors: out[i] = fold over ranks of partial_r[i], i < n, n * sizeof(T) <= 64 KiB.
// Every thread sends its elements to all ranks first, then collects; `partial` may be `out`.
template <typename T, int OP>
__global__ void __launch_bounds__(kBlock) mg_combine_kernel(MgPeers m, const T *partial, T *out, size_t n, int mean, size_t count) {
    grid_dep_wait();
    constexpr int W = sizeof(T) / 4;
    union Word {
        T v;
        uint32_t w[W];
    };
    const uint32_t epoch = mg_next_epoch(m.state);
    const size_t base = (size_t)(epoch & 1u) * kMgMaxRanks * kMgSlotWords;
    const size_t stride = (size_t)gridDim.x * kBlock;
    const size_t first = (size_t)blockIdx.x * kBlock + threadIdx.x;
    for (size_t i = first; i < n; i += stride) {
        Word u;
        u.v = partial[i];
        for (int p = 0; p < m.nranks; ++p) {
            uint2 *dst = m.slots[p] + base + (size_t)m.rank * kMgSlotWords + i * W;
#pragma unroll
            for (int w = 0; w < W; ++w) mg_store(dst + w, u.w[w], epoch);
        }
    }
    bool dead = false;
    for (size_t i = first; i < n; i += stride) {
        T acc = (T)0;
        for (int p = 0; p < m.nranks; ++p) {
            const uint2 *src = m.slots[m.rank] + base + (size_t)p * kMgSlotWords + i * W;
            Word u;
#pragma unroll
            for (int w = 0; w < W; ++w) {
                // after one wait ran out (here or in any other thread) nothing waits again
                if (!dead && (*reinterpret_cast<volatile unsigned int *>(m.state + 1) & 1u)) dead = true;
                uint32_t got = 0;
                if (dead) {
                    got = mg_load(src + w).x;
                } else if (!mg_wait(src + w, epoch, m.wait_ns, &got)) {
                    dead = true;
                    atomicOr(m.state + 1, 1u);
                }
                u.w[w] = got;
            }
            acc = p == 0 ? u.v : Fold<T, OP>::apply(acc, u.v);
        }
        if (dead) acc = mg_nan<T>();
        out[i] = mean ? acc / (T)(float)count : acc;
    }
    // the last CTA to finish publishes the epoch
    __shared__ bool is_last;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        is_last = atomicAdd(m.state + 2, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (is_last && threadIdx.x == 0) {
        m.state[2] = 0;
        *reinterpret_cast<volatile unsigned int *>(m.state) = epoch;
    }
}

template <typename T> __global__ void __launch_bounds__(kBlock) mg_scale_kernel(T *x, size_t n, size_t count) {
    grid_dep_wait();
    const T d = (T)(float)count;
    for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (size_t)gridDim.x * kBlock) x[i] = x[i] / d;
}

template <typename T>
int combine_typed(Ctx *ctx, const MgPeers &peers, int redop, const T *partial, T *out, size_t n, size_t count) {
    const int mean = redop == RTB_MEAN;
    size_t blocks = (n + kBlock - 1) / kBlock;
    if (blocks > (size_t)ctx->sm_count) blocks = (size_t)ctx->sm_count;
    const unsigned grid = (unsigned)(blocks ? blocks : 1);
    switch (redop) {
        case RTB_SUM:
        case RTB_MEAN: launch_dep(ctx, grid, kBlock, mg_combine_kernel<T, RTB_SUM>, peers, partial, out, n, mean, count); break;
        case RTB_PROD: launch_dep(ctx, grid, kBlock, mg_combine_kernel<T, RTB_PROD>, peers, partial, out, n, 0, count); break;
        case RTB_MAX: launch_dep(ctx, grid, kBlock, mg_combine_kernel<T, RTB_MAX>, peers, partial, out, n, 0, count); break;
        case RTB_MIN: launch_dep(ctx, grid, kBlock, mg_combine_kernel<T, RTB_MIN>, peers, partial, out, n, 0, count); break;
        default: return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
    }
    return check_launch(ctx, "mg_combine_kernel");
}

bool nccl_type(int dtype, ncclDataType_t *t) {
    switch (dtype) {
        case RTB_I8: *t = ncclInt8; return true;
        case RTB_U8: *t = ncclUint8; return true;
        case RTB_I32: *t = ncclInt32; return true;
        case RTB_U32: *t = ncclUint32; return true;
        case RTB_I64: *t = ncclInt64; return true;
        case RTB_U64: *t = ncclUint64; return true;
        case RTB_F32: *t = ncclFloat32; return true;
        case RTB_F64: *t = ncclFloat64; return true;
    }
    return false;
}

bool nccl_op(int redop, ncclRedOp_t *o) {
    switch (redop) {
        case RTB_SUM:
        case RTB_MEAN: *o = ncclSum; return true;
        case RTB_PROD: *o = ncclProd; return true;
        case RTB_MAX: *o = ncclMax; return true;
        case RTB_MIN: *o = ncclMin; return true;
    }
    return false;
}

int nccl_allreduce(Ctx *ctx, cudaStream_t stream, int dtype, int redop, void *buf, size_t n, size_t mean_count) {
    Mg *mg = ctx->mg;
    ncclDataType_t t;
    ncclRedOp_t o;
    if (!nccl_type(dtype, &t)) return fail(RTB_ERR_DTYPE, "dtype %d has no all-reduce", dtype);
    if (!nccl_op(redop, &o)) return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
    if (n == 0) return RTB_OK;
    RTB_NCCL(g_nccl.AllReduce(buf, buf, n, t, o, mg->comm, stream));
    if (redop == RTB_MEAN) {
        if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "mean is defined for f32 and f64 only");
        size_t blocks = (n + kBlock - 1) / kBlock;
        if (blocks > (size_t)ctx->sm_count * 8) blocks = (size_t)ctx->sm_count * 8;
        cudaStream_t keep = ctx->stream;
        ctx->stream = stream;
        if (dtype == RTB_F32) launch_dep(ctx, (unsigned)blocks, kBlock, mg_scale_kernel<float>, (float *)buf, n, mean_count);
        else launch_dep(ctx, (unsigned)blocks, kBlock, mg_scale_kernel<double>, (double *)buf, n, mean_count);
        ctx->stream = keep;
        return check_launch(ctx, "mg_scale_kernel");
    }
    return RTB_OK;
}

int need_mg(rtb_ctx *c, Mg **mg) {
    if (!c) return fail(RTB_ERR_INVALID, "null ctx");
    Ctx *ctx = reinterpret_cast<Ctx *>(c);
    if (!ctx->mg) return fail(RTB_ERR_INVALID, "this context has no communicator: call rtb_mg_init first");
    *mg = ctx->mg;
    return use_device(ctx);
}

void destroy_mg(Mg *mg) {
    if (!mg) return;
    if (mg->mapped)
        for (int p = 0; p < mg->nranks; ++p)
            if (p != mg->rank && mg->slots[p] && !mg->same_process[p]) cudaIpcCloseMemHandle(mg->slots[p]);
    if (mg->comm) g_nccl.CommDestroy(mg->comm);
    if (mg->local) cudaFree(mg->local);
    if (mg->state) cudaFree(mg->state);
    if (mg->side) cudaStreamDestroy(mg->side);
    if (mg->fork_ev) cudaEventDestroy(mg->fork_ev);
    if (mg->join_ev) cudaEventDestroy(mg->join_ev);
    delete mg;
}

// every rank has passed this point (a 1-element all-reduce + host wait)
int barrier(Ctx *ctx) {
    Mg *mg = ctx->mg;
    RTB_NCCL(g_nccl.AllReduce(mg->state + 3, mg->state + 3, 1, ncclUint32, ncclMax, mg->comm, ctx->stream));
    RTB_CUDA(cudaStreamSynchronize(ctx->stream));
    return RTB_OK;
}

}  // namespace

void mg_release(Ctx *ctx) {
    if (!ctx->mg) return;
    cudaStreamSynchronize(ctx->stream);
    destroy_mg(ctx->mg);
    ctx->mg = nullptr;
}

}  // namespace rtb

using namespace rtb;
static inline Ctx *C(rtb_ctx *c) { return reinterpret_cast<Ctx *>(c); }

RTB_API int rtb_mg_unique_id(void *id_out) {
    if (!id_out) return fail(RTB_ERR_INVALID, "null id");
    int rc = load_nccl();
    if (rc) return rc;
    static_assert(sizeof(ncclUniqueId) == RTB_MG_ID_BYTES, "ncclUniqueId size");
    ncclUniqueId id;
    RTB_NCCL(g_nccl.GetUniqueId(&id));
    std::memcpy(id_out, &id, sizeof(id));
    return RTB_OK;
}

RTB_API int rtb_mg_init(rtb_ctx *c, int nranks, int rank, const void *id_bytes) {
    if (!c || !id_bytes) return fail(RTB_ERR_INVALID, "null argument");
    if (nranks < 1 || nranks > kMgMaxRanks || rank < 0 || rank >= nranks)
        return fail(RTB_ERR_INVALID, "rank %d of %d ranks (at most %d)", rank, nranks, kMgMaxRanks);
    Ctx *ctx = C(c);
    if (ctx->mg) return fail(RTB_ERR_INVALID, "this context already has a communicator");
    int rc = load_nccl();
    if (rc) return rc;
    if ((rc = use_device(ctx))) return rc;
    Mg *mg = new Mg();
    mg->nranks = nranks;
    mg->rank = rank;
    ncclUniqueId id;
    std::memcpy(&id, id_bytes, sizeof(id));
    ncclResult_t nr = g_nccl.CommInitRank(&mg->comm, nranks, id, rank);
    if (nr != ncclSuccess) {
        mg->comm = nullptr;
        destroy_mg(mg);
        return nccl_fail(nr, "ncclCommInitRank");
    }
    ctx->mg = mg;
    auto bail = [&](int code) {
        destroy_mg(mg);
        ctx->mg = nullptr;
        return code;
    };
    cudaError_t e;
    if ((e = cudaMalloc(&mg->local, kMgBufferPackets * sizeof(uint2))) != cudaSuccess) return bail(cuda_fail(e, "cudaMalloc(exchange buffer)"));
    if ((e = cudaMalloc(&mg->state, 64)) != cudaSuccess) return bail(cuda_fail(e, "cudaMalloc(exchange state)"));
    if ((e = cudaMemsetAsync(mg->local, 0, kMgBufferPackets * sizeof(uint2), ctx->stream)) != cudaSuccess) return bail(cuda_fail(e, "cudaMemsetAsync"));
    if ((e = cudaMemsetAsync(mg->state, 0, 64, ctx->stream)) != cudaSuccess) return bail(cuda_fail(e, "cudaMemsetAsync"));
    if ((e = cudaStreamCreateWithFlags(&mg->side, cudaStreamNonBlocking)) != cudaSuccess) return bail(cuda_fail(e, "cudaStreamCreate"));
    if ((e = cudaEventCreateWithFlags(&mg->fork_ev, cudaEventDisableTiming)) != cudaSuccess) return bail(cuda_fail(e, "cudaEventCreate"));
    if ((e = cudaEventCreateWithFlags(&mg->join_ev, cudaEventDisableTiming)) != cudaSuccess) return bail(cuda_fail(e, "cudaEventCreate"));
    mg->slots[rank] = mg->local;
    if (nranks == 1) {
        mg->mapped = true;
        return RTB_OK;
    }
    // Exchange the IPC handles of the buffers with one all-gather, then map every peer's buffer.  Each
    // record carries a flag saying whether the handle could be made; mapping is all or nothing.
    // A rank in the SAME process (one host thread per device) cannot open an IPC handle of its own
    // process; there the raw pointer is used directly after enabling peer access to its device.
    struct Record {
        cudaIpcMemHandle_t handle;
        int ok;
        int device;
        long long pid;
        unsigned long long ptr;
        int pad[10];
    };
    static_assert(sizeof(Record) == 128, "record size");
    Record mine{};
    mine.ok = cudaIpcGetMemHandle(&mine.handle, mg->local) == cudaSuccess ? 1 : 0;
    if (!mine.ok) cudaGetLastError();
    // RTB_MG_NO_PEER=1 on any rank keeps every rank off the peer-memory path (everything then goes
    // through NCCL): for hosts that forbid IPC mappings, and for testing that path
    if (const char *no_peer = std::getenv("RTB_MG_NO_PEER"))
        if (no_peer[0] == '1') mine.ok = 0;
    mine.device = ctx->device;
    mine.pid = (long long)getpid();
    mine.ptr = (unsigned long long)(uintptr_t)mg->local;
    Record *dev = nullptr;
    if ((e = cudaMalloc(&dev, sizeof(Record) * (size_t)nranks)) != cudaSuccess) return bail(cuda_fail(e, "cudaMalloc(handles)"));
    std::vector<Record> all((size_t)nranks);
    e = cudaMemcpyAsync(dev + rank, &mine, sizeof(Record), cudaMemcpyHostToDevice, ctx->stream);
    nr = e == cudaSuccess ? g_nccl.AllGather(dev + rank, dev, sizeof(Record), ncclUint8, mg->comm, ctx->stream) : ncclSuccess;
    if (e == cudaSuccess && nr == ncclSuccess) e = cudaMemcpyAsync(all.data(), dev, sizeof(Record) * (size_t)nranks, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess && nr == ncclSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(dev);
    if (nr != ncclSuccess) return bail(nccl_fail(nr, "ncclAllGather(handles)"));
    if (e != cudaSuccess) return bail(cuda_fail(e, "handle exchange"));
    bool every = true;
    for (int p = 0; p < nranks; ++p) every = every && all[(size_t)p].ok;
    int opened = 0;
    if (every) {
        for (int p = 0; p < nranks && every; ++p) {
            if (p == rank) continue;
            const Record &r = all[(size_t)p];
            if (r.pid == mine.pid) {
                int can = 0;
                if (r.device != ctx->device && cudaDeviceCanAccessPeer(&can, ctx->device, r.device) == cudaSuccess && can) {
                    cudaError_t pe = cudaDeviceEnablePeerAccess(r.device, 0);
                    if (pe == cudaSuccess || pe == cudaErrorPeerAccessAlreadyEnabled) {
                        cudaGetLastError();
                        mg->slots[p] = reinterpret_cast<uint2 *>((uintptr_t)r.ptr);
                        mg->same_process[p] = true;
                        continue;
                    }
                }
                cudaGetLastError();
                every = false;
                continue;
            }
            void *ptr = nullptr;
            if (cudaIpcOpenMemHandle(&ptr, r.handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                cudaGetLastError();
                every = false;
            } else {
                mg->slots[p] = static_cast<uint2 *>(ptr);
                ++opened;
            }
        }
    }
    // all ranks agree on whether the peer path is usable (min over ranks of "I mapped everyone")
    unsigned int flag = every ? 1u : 0u;
    e = cudaMemcpyAsync(mg->state + 3, &flag, sizeof(flag), cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) nr = g_nccl.AllReduce(mg->state + 3, mg->state + 3, 1, ncclUint32, ncclMin, mg->comm, ctx->stream);
    if (e == cudaSuccess && nr == ncclSuccess) e = cudaMemcpyAsync(&flag, mg->state + 3, sizeof(flag), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess && nr == ncclSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (nr != ncclSuccess) return bail(nccl_fail(nr, "ncclAllReduce(peer agreement)"));
    if (e != cudaSuccess) return bail(cuda_fail(e, "peer agreement"));
    mg->mapped = flag == 1u;
    if (!mg->mapped) {
        for (int p = 0; p < nranks; ++p)
            if (p != rank && mg->slots[p]) {
                if (!mg->same_process[p]) cudaIpcCloseMemHandle(mg->slots[p]);
                mg->slots[p] = nullptr;
            }
    }
    (void)opened;
    return RTB_OK;
}

RTB_API int rtb_mg_finalize(rtb_ctx *c) {
    if (!c) return fail(RTB_ERR_INVALID, "null ctx");
    Ctx *ctx = C(c);
    if (!ctx->mg) return RTB_OK;
    int rc = use_device(ctx);
    if (rc) return rc;
    Mg *mg = ctx->mg;
    if (mg->nranks > 1) {
        // nobody may still be storing into a buffer that is about to be unmapped or freed
        if ((rc = barrier(ctx))) return rc;
        if (mg->mapped) {
            for (int p = 0; p < mg->nranks; ++p)
                if (p != mg->rank && mg->slots[p]) {
                    if (!mg->same_process[p]) cudaIpcCloseMemHandle(mg->slots[p]);
                    mg->slots[p] = nullptr;
                }
            mg->mapped = false;
            if ((rc = barrier(ctx))) return rc;
        }
    }
    mg_release(ctx);
    return RTB_OK;
}

RTB_API int rtb_mg_info(rtb_ctx *c, int *nranks, int *rank, int *peer_mapped) {
    if (!c) return fail(RTB_ERR_INVALID, "null ctx");
    Mg *mg = C(c)->mg;
    if (nranks) *nranks = mg ? mg->nranks : 1;
    if (rank) *rank = mg ? mg->rank : 0;
    if (peer_mapped) *peer_mapped = mg && mg->mapped && mg->nranks > 1 ? 1 : 0;
    return RTB_OK;
}

RTB_API int rtb_mg_set_wait_ns(rtb_ctx *c, uint64_t ns) {
    Mg *mg = nullptr;
    int rc = need_mg(c, &mg);
    if (rc) return rc;
    if (ns < 1000 || ns > 60000000000ull) return fail(RTB_ERR_INVALID, "wait limit must be between 1 us and 60 s");
    mg->wait_ns = ns;
    return RTB_OK;
}

RTB_API int rtb_mg_status(rtb_ctx *c, unsigned int *bits) {
    Mg *mg = nullptr;
    int rc = need_mg(c, &mg);
    if (rc) return rc;
    if (!bits) return fail(RTB_ERR_INVALID, "null bits");
    Ctx *ctx = C(c);
    RTB_CUDA(cudaMemcpyAsync(bits, mg->state + 1, sizeof(unsigned int), cudaMemcpyDeviceToHost, ctx->stream));
    RTB_CUDA(cudaStreamSynchronize(ctx->stream));
    ncclResult_t async = ncclSuccess;
    if (g_nccl.CommGetAsyncError(mg->comm, &async) == ncclSuccess && async != ncclSuccess && async != ncclInProgress) *bits |= 2u;
    return RTB_OK;
}

RTB_API int rtb_mg_realign(rtb_ctx *c) {
    Mg *mg = nullptr;
    int rc = need_mg(c, &mg);
    if (rc) return rc;
    Ctx *ctx = C(c);
    // everyone adopts the highest epoch any rank has reached, and the status word is cleared
    RTB_NCCL(g_nccl.AllReduce(mg->state, mg->state, 1, ncclUint32, ncclMax, mg->comm, ctx->stream));
    RTB_CUDA(cudaMemsetAsync(mg->state + 1, 0, 2 * sizeof(unsigned int), ctx->stream));
    return barrier(ctx);
}

RTB_API int rtb_mg_allreduce(rtb_ctx *c, int dtype, int redop, void *buf, size_t n, size_t mean_count) {
    Mg *mg = nullptr;
    int rc = need_mg(c, &mg);
    if (rc) return rc;
    if (!buf && n) return fail(RTB_ERR_INVALID, "null buffer");
    if (mg->nranks == 1 && redop != RTB_MEAN) return RTB_OK;
    return nccl_allreduce(C(c), C(c)->stream, dtype, redop, buf, n, mean_count);
}

RTB_API int rtb_mg_allreduce_begin(rtb_ctx *c, int dtype, int redop, void *buf, size_t n, size_t mean_count) {
    Mg *mg = nullptr;
    int rc = need_mg(c, &mg);
    if (rc) return rc;
    if (!buf && n) return fail(RTB_ERR_INVALID, "null buffer");
    Ctx *ctx = C(c);
    RTB_CUDA(cudaEventRecord(mg->fork_ev, ctx->stream));
    RTB_CUDA(cudaStreamWaitEvent(mg->side, mg->fork_ev, 0));
    if (!(mg->nranks == 1 && redop != RTB_MEAN)) {
        rc = nccl_allreduce(ctx, mg->side, dtype, redop, buf, n, mean_count);
        if (rc) return rc;
    }
    RTB_CUDA(cudaEventRecord(mg->join_ev, mg->side));
    mg->side_busy = true;
    return RTB_OK;
}

RTB_API int rtb_mg_allreduce_join(rtb_ctx *c) {
    Mg *mg = nullptr;
    int rc = need_mg(c, &mg);
    if (rc) return rc;
    if (!mg->side_busy) return RTB_OK;
    RTB_CUDA(cudaStreamWaitEvent(C(c)->stream, mg->join_ev, 0));
    mg->side_busy = false;
    return RTB_OK;
}

RTB_API int rtb_mg_combine(rtb_ctx *c, int dtype, int redop, void *buf, size_t n, size_t mean_count) {
    Mg *mg = nullptr;
    int rc = need_mg(c, &mg);
    if (rc) return rc;
    if (!buf && n) return fail(RTB_ERR_INVALID, "null buffer");
    if (redop < RTB_SUM || redop > RTB_MEAN) return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
    if (n == 0) return RTB_OK;
    Ctx *ctx = C(c);
    MgPeers peers;
    const size_t es = dtype_size(dtype);
    const bool small = (dtype == RTB_F32 || dtype == RTB_F64) && n * es <= (size_t)kMgSlotWords * 4;
    if (small && mg_peers(ctx, &peers)) {
        if (dtype == RTB_F32) return combine_typed<float>(ctx, peers, redop, (const float *)buf, (float *)buf, n, mean_count);
        return combine_typed<double>(ctx, peers, redop, (const double *)buf, (double *)buf, n, mean_count);
    }
    return nccl_allreduce(ctx, ctx->stream, dtype, redop, buf, n, mean_count);
}

RTB_API int rtb_mg_reduce_flat(rtb_ctx *c, int dtype, int redop, const void *src, size_t start, size_t local_len,
                               size_t global_len, void *dst) {
    Mg *mg = nullptr;
    int rc = need_mg(c, &mg);
    if (rc) return rc;
    if (!src || !dst) return fail(RTB_ERR_INVALID, "null argument");
    if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
    if (redop < RTB_SUM || redop > RTB_MEAN) return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
    Ctx *ctx = C(c);
    const char *p = (const char *)src + start * dtype_size(dtype);
    MgPeers peers;
    if (mg_peers(ctx, &peers)) return launch_reduce_flat_mg(ctx, dtype, redop, p, local_len, dst, peers, global_len);
    // no peer mapping: local partial (sum for a mean), then NCCL
    rc = launch_reduce_flat(ctx, dtype, redop == RTB_MEAN ? RTB_SUM : redop, p, local_len, dst);
    if (rc) return rc;
    return nccl_allreduce(ctx, ctx->stream, dtype, redop, dst, 1, global_len);
}

RTB_API int rtb_mg_reduce_axis(rtb_ctx *c, int dtype, int redop, const void *src, size_t offset, size_t outer,
                               size_t r_local, size_t inner, ptrdiff_t outer_stride, ptrdiff_t row_stride, size_t global_r,
                               void *dst) {
    Mg *mg = nullptr;
    int rc = need_mg(c, &mg);
    if (rc) return rc;
    if (!src || !dst) return fail(RTB_ERR_INVALID, "null argument");
    if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "reductions are defined for f32 and f64 only");
    if (redop < RTB_SUM || redop > RTB_MEAN) return fail(RTB_ERR_INVALID, "unsupported reduction code %d", redop);
    if (outer == 0 || inner == 0) return RTB_OK;
    Ctx *ctx = C(c);
    const char *p = (const char *)src + (ptrdiff_t)offset * (ptrdiff_t)dtype_size(dtype);
    rc = launch_reduce_axis_strided(ctx, dtype, redop == RTB_MEAN ? RTB_SUM : redop, p, outer, r_local, inner, outer_stride,
                                    row_stride, dst);
    if (rc) return rc;
    return rtb_mg_combine(c, dtype, redop, dst, outer * inner, global_r);
}

RTB_API int rtb_mg_l1_loss(rtb_ctx *c, int dtype, const void *a, const void *b, size_t local_n, size_t global_n,
                           int reduction, void *loss, void *grad_map) {
    Mg *mg = nullptr;
    int rc = need_mg(c, &mg);
    if (rc) return rc;
    if (!a || !b || !loss) return fail(RTB_ERR_INVALID, "null argument");
    if (reduction != 0 && reduction != 1) return fail(RTB_ERR_INVALID, "reduction must be 0 (mean) or 1 (sum)");
    if (dtype != RTB_F32 && dtype != RTB_F64) return fail(RTB_ERR_DTYPE, "l1 loss is defined for f32 and f64 only");
    Ctx *ctx = C(c);
    MgPeers peers;
    if (mg_peers(ctx, &peers)) return launch_l1_mg(ctx, dtype, a, b, local_n, reduction, loss, grad_map, peers, global_n);
    // no peer mapping: the same kernel exchanging with itself only (loss = this rank's share, the
    // map already scaled by the global count), then NCCL sums the shares
    MgPeers solo{};
    solo.nranks = 1;
    solo.rank = 0;
    solo.wait_ns = mg->wait_ns;
    solo.slots[0] = mg->local;
    solo.state = mg->state;
    rc = launch_l1_mg(ctx, dtype, a, b, local_n, reduction, loss, grad_map, solo, global_n);
    if (rc) return rc;
    return nccl_allreduce(ctx, ctx->stream, dtype, RTB_SUM, loss, 1, 0);
}
