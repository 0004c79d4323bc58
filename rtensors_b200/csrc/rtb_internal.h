// Internal declarations shared by the translation units of librt_b200.so.
#pragma once
#include <cstddef>
#include <cstdint>
#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include <cuda_runtime.h>

#include "rt_b200.h"

#define RTB_API extern "C" __attribute__((visibility("default")))

namespace rtb {

// ---- per-thread error text -------------------------------------------------------------------
int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

#define RTB_CUDA(call)                                                       \
    do {                                                                     \
        cudaError_t e__ = (call);                                            \
        if (e__ != cudaSuccess) return ::rtb::cuda_fail(e__, #call);         \
    } while (0)

// ---- dtype properties ------------------------------------------------------------------------
size_t dtype_size(int dtype);  // 0 for an unknown code

// ---- context -----------------------------------------------------------------------------------
struct Mg;         // multi-GPU communicator state (rtb_mg.cu)
struct HostLanes;  // transfer lanes and device slots of the host-buffer operations (rtb_host.cpp)
struct Ctx {
    int device = 0;
    int sm_count = 0;
    size_t l2_bytes = 0;
    cudaStream_t stream = nullptr;
    std::atomic<uint64_t> launches{0};
    // reduction workspace (partials + completion counters), grown on demand.  ws_mu serialises the
    // host threads that enqueue workspace-using kernels on this context: the kernels share the
    // counters and partial slots and rely on stream order, so their enqueue order must be total.
    std::mutex ws_mu;
    void *ws = nullptr;
    size_t ws_bytes = 0;
    std::vector<void *> retired;              // superseded workspaces, freed only with the context
    std::atomic<uint64_t> ws_generation{0};   // bumped whenever device memory a captured graph may hold goes away
    cudaEvent_t order_event = nullptr;        // joins the old stream into the new one in rtb_ctx_set_stream
    Mg *mg = nullptr;                         // set by rtb_mg_init
    HostLanes *host = nullptr;                // created by the first host-buffer operation
    // caching allocator: free blocks by rounded size; live blocks by pointer
    std::mutex mu;
    std::multimap<size_t, void *> free_blocks;
    std::map<void *, size_t> live_blocks;
};

// Returns a workspace with a 64 KiB header followed by at least `bytes` bytes of scratch.  The
// header holds completion counters that kernels leave at zero; it is zeroed when the workspace is
// created.
int workspace(Ctx *ctx, size_t bytes, void **out);
void mg_release(Ctx *ctx);  // frees ctx->mg without any collective (context teardown)
void host_release(Ctx *ctx);  // waits for the transfer lanes and frees them with their device slots
int host_sync(Ctx *ctx);      // waits for the transfer lanes (no-op if there are none)
int use_device(Ctx *ctx);  // makes ctx->device current for the calling thread
Ctx *default_ctx();  // ctx on the current device bound to the legacy default stream (ABI v1)

inline void count_launch(Ctx *ctx) { ctx->launches.fetch_add(1, std::memory_order_relaxed); }
int check_launch(Ctx *ctx, const char *what);

// ---- programmatic dependent launch ---------------------------------------------------------------
// Every kernel of the library is launched with the "programmatic stream serialization" attribute and
// begins with grid_dep_sync().  A kernel that follows another kernel of the library on the same
// stream is then scheduled while its predecessor's last wave is still running -- its CTAs become
// resident as SMs free up -- and only blocks (griddepcontrol.wait) until the predecessor has
// completed and its writes are visible.  Nothing before that wait touches global memory, so stream
// order is kept exactly; what is saved is the launch gap and the drain of the tail, measured at
// 2.0 - 2.7 us per kernel boundary on B200 (a 64 MiB read-modify-write: 14.4 -> 11.7 us each when
// run back to back).  After a kernel that does not cooperate (a copy, another library's kernel)
// the launch behaves like a plain one.
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Kernels of many short CTAs release their dependents at once: that only takes effect when the
// LAST CTA has started.  Kernels whose CTAs are all resident from the start and run long (the
// one-wave reductions) release them after their main loop instead -- CTAs of the next kernel
// that sit waiting next to a 600 us streaming loop were measured to slow it by up to 10 %.
__device__ __forceinline__ void grid_dep_sync() {
    grid_dep_launch();
    grid_dep_wait();
}

template <typename... KArgs, typename... Args>
inline void launch_dep_smem(Ctx *ctx, unsigned grid, unsigned block, size_t smem_bytes, void (*kernel)(KArgs...), Args &&...args);

template <typename... KArgs, typename... Args>
inline void launch_dep(Ctx *ctx, unsigned grid, unsigned block, void (*kernel)(KArgs...), Args &&...args) {
    launch_dep_smem(ctx, grid, block, 0, kernel, std::forward<Args>(args)...);
}

// the same with dynamic shared memory (the caller has raised the kernel's limit if it exceeds 48 KB)
template <typename... KArgs, typename... Args>
inline void launch_dep_smem(Ctx *ctx, unsigned grid, unsigned block, size_t smem_bytes, void (*kernel)(KArgs...), Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    (void)cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);  // the caller reads the error with check_launch()
}
#endif

// ---- planner (host) ----------------------------------------------------------------------------
constexpr int kMaxPlanRank = 8;
enum AccessMode { kContigVec = 0, kContigScalar = 1, kRevVec = 2, kRevScalar = 3, kBroadcast = 4, kStrided = 5 };
enum PlanKernel { kNothing = 0, kFlatVec = 1, kFlatScalar = 2, kRows = 3 };

struct ViewArg {
    const ptrdiff_t *strides;  // rank entries (elements)
    size_t offset;             // elements
    uintptr_t ptr;             // buffer base address (only its alignment matters to the planner)
};

// Builds the plan; returns RTB_OK, or RTB_ERR_TOO_LARGE when more than kMaxPlanRank dims remain
// after collapsing (the caller then peels outer dims).
int make_plan(size_t elem_size, int n_inputs, size_t rank, const size_t *shape, const ViewArg &d, const ViewArg &l,
              const ViewArg &r, rtb_plan *out);

// ---- launchers implemented in the .cu files ----------------------------------------------------
// op families for the elementwise engine
enum EwFamily { kFamBinary = 0, kFamScalar = 1, kFamUnary = 2, kFamFill = 3, kFamCopy = 4 };

struct EwCall {
    int dtype;
    int family;  // EwFamily
    int op;      // rtb_binop or rtb_unop
    unsigned char value[16];  // scalar operand / fill value
    void *d;
    const void *l;
    const void *r;
};
// Runs one planned elementwise call (any family) on ctx->stream.
int launch_elementwise(Ctx *ctx, const EwCall &call, const rtb_plan &plan);
// Plans and runs, peeling outer dims on the host if the collapsed rank exceeds kMaxPlanRank.
int run_elementwise(Ctx *ctx, const EwCall &call, size_t rank, const size_t *shape, const ptrdiff_t *sd, size_t od,
                    const ptrdiff_t *sl, size_t ol, const ptrdiff_t *sr, size_t orr);

int launch_reduce_flat(Ctx *ctx, int dtype, int redop, const void *src, size_t len, void *dst);
int launch_reduce_axis(Ctx *ctx, int dtype, int redop, const void *src, size_t outer, size_t r, size_t inner,
                       void *dst);
// same with explicit element strides: source element (o, k, i) at o*outer_stride + k*row_stride + i
int launch_reduce_axis_strided(Ctx *ctx, int dtype, int redop, const void *src, size_t outer, size_t r, size_t inner,
                               ptrdiff_t outer_stride, ptrdiff_t row_stride, void *dst);
// codes RTB_VARIANCE .. RTB_ARGMIN over the same addressing; dst holds uint64_t for the arg codes
int launch_reduce_ext(Ctx *ctx, int dtype, int redop, const rtb_reduce_settings *settings, const void *src, size_t outer,
                      size_t r, size_t inner, ptrdiff_t outer_stride, ptrdiff_t row_stride, void *dst);
// fused broadcast binary op + axis reduce: operands addressed as a*s[0] + k*s[1] + b*s[2]
int launch_bcast_reduce(Ctx *ctx, int dtype, int binop, int redop, const void *l, const ptrdiff_t sl[3], const void *r,
                        const ptrdiff_t sr[3], size_t A, size_t R, size_t B, void *dst);
int launch_l1(Ctx *ctx, int dtype, const void *a, const void *b, size_t n, int reduction, void *loss, void *gmap);
int launch_relu_mask(Ctx *ctx, float *x, float *mask, size_t n);
int launch_bias_relu_mask(Ctx *ctx, int dtype, void *z, const void *bias, void *mask, size_t rows, size_t cols);
int launch_sgd(Ctx *ctx, float *p, const float *g, float lr, size_t n);
int launch_relu_mask_f64(Ctx *ctx, double *x, double *mask, size_t n);
int launch_sgd_f64(Ctx *ctx, double *p, const double *g, double lr, size_t n);
int launch_convert(Ctx *ctx, int src_dtype, int dst_dtype, const void *src, void *dst, size_t n);
int launch_u8_f32(Ctx *ctx, const uint8_t *src, float *dst, float divisor, size_t n);

}  // namespace rtb
