// Multi-GPU exchange of small partial results over NVLink peer memory (device side).
//
// Every rank owns one exchange buffer; every rank maps all the others' (CUDA IPC).  A value travels
// as 8-byte packets {32-bit payload word, 32-bit epoch}: one naturally aligned 8-byte store, so a
// reader that sees the expected epoch also sees the payload -- no fence, no separate flag.  A rank
// stores its packets into slot [epoch parity][its rank] of EVERY rank's buffer (its own included)
// with plain st.global over NVLink, then polls the nranks slots of its own buffer and folds them in
// rank order, so all ranks compute the same bits.  No bulk-copy engine, no switch-side replication,
// and no library kernel ever sees a peer pointer.
//
// Two buffers by epoch parity are enough: a rank can only enter exchange e+2 after it has read every
// rank's packets of e+1, and a rank sends those only after it has finished reading exchange e.
//
// Every wait is bounded (a time limit on %globaltimer plus an iteration cap).  A wait that runs out
// sets bit 0 of the status word, the result becomes NaN, and the kernel returns normally; the host
// reads the word with rtb_mg_status().  Nothing traps and nothing spins forever.
#pragma once
#include <cmath>

#include "rtb_internal.h"

namespace rtb {

constexpr int kMgMaxRanks = 16;
constexpr int kMgSlotWords = 16384;  // 32-bit payload words one rank can send per exchange (64 KiB)
constexpr size_t kMgBufferPackets = (size_t)2 * kMgMaxRanks * kMgSlotWords;  // [parity][sender][word]

// Kernel parameter.  state: [0] epoch of the last finished exchange (device resident, so a captured
// graph replays correctly), [1] status bits, [2] CTA completion counter (left at zero).
struct MgPeers {
    int nranks, rank;
    unsigned long long wait_ns;
    uint2 *slots[kMgMaxRanks];  // slots[rank] is this GPU's own buffer, the others are peer mappings
    unsigned int *state;
};
struct NoPeers {};

#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long mg_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mg_store(uint2 *p, uint32_t word, uint32_t epoch) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(word), "r"(epoch) : "memory");
}
__device__ __forceinline__ uint2 mg_load(const uint2 *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// Polls one packet of this GPU's own buffer until it carries `epoch`.  false = the limit ran out.
__device__ __forceinline__ bool mg_wait(const uint2 *p, uint32_t epoch, unsigned long long wait_ns, uint32_t *word) {
    uint2 v = mg_load(p);
    if (v.y != epoch) {
        const unsigned long long t0 = mg_now();
        unsigned long long spins = (wait_ns >> 5) + 4096;  // second bound, should the timer stand still
        while (spins-- > 0) {
            v = mg_load(p);
            if (v.y == epoch || mg_now() - t0 >= wait_ns) break;
            __nanosleep(40);
        }
    }
    *word = v.x;
    return v.y == epoch;
}
__device__ __forceinline__ uint32_t mg_next_epoch(const unsigned int *state) {
    uint32_t e = *reinterpret_cast<const volatile unsigned int *>(state) + 1u;
    return e ? e : 1u;  // 0 is what an untouched buffer holds
}
template <typename T> __device__ __forceinline__ T mg_nan() { return (T)NAN; }

// One value per rank, exchanged by the calling CTA (all its threads must call; blockDim >= 2 * nranks).
// `mine` is read from thread 0; the combined value is returned in thread 0.  COMB(a, b) folds.
template <typename T, typename COMB>
__device__ __forceinline__ T mg_exchange_scalar(T mine, const MgPeers &m, COMB comb) {
    constexpr int W = sizeof(T) / 4;
    __shared__ uint32_t s_mine[2];
    __shared__ uint32_t s_all[kMgMaxRanks * 2];
    __shared__ uint32_t s_epoch;
    __shared__ int s_failed;
    union {
        T v;
        uint32_t w[W];
    } u;
    if (threadIdx.x == 0) {
        u.v = mine;
#pragma unroll
        for (int w = 0; w < W; ++w) s_mine[w] = u.w[w];
        s_epoch = mg_next_epoch(m.state);
        s_failed = 0;
    }
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const int tid = threadIdx.x;
    const size_t base = (size_t)(epoch & 1u) * kMgMaxRanks * kMgSlotWords;
    if (tid < m.nranks * W) {
        const int p = tid / W, w = tid % W;
        mg_store(m.slots[p] + base + (size_t)m.rank * kMgSlotWords + w, s_mine[w], epoch);
        uint32_t got = 0;
        if (!mg_wait(m.slots[m.rank] + base + (size_t)p * kMgSlotWords + w, epoch, m.wait_ns, &got)) s_failed = 1;
        s_all[tid] = got;
    }
    __syncthreads();
    T total = mine;
    if (tid == 0) {
        for (int p = 0; p < m.nranks; ++p) {
#pragma unroll
            for (int w = 0; w < W; ++w) u.w[w] = s_all[p * W + w];
            total = p == 0 ? u.v : comb(total, u.v);
        }
        if (s_failed) {
            atomicOr(m.state + 1, 1u);
            total = mg_nan<T>();
        }
        *reinterpret_cast<volatile unsigned int *>(m.state) = epoch;
    }
    return total;
}
#endif

// ---- host side (rtb_mg.cu) -----------------------------------------------------------------------
struct Mg;
// the peers of ctx's communicator as a kernel parameter; false when ctx has no communicator or the
// exchange buffers could not be mapped (then callers fall back to NCCL)
bool mg_peers(Ctx *ctx, MgPeers *out);
int launch_reduce_flat_mg(Ctx *ctx, int dtype, int redop, const void *src, size_t len, void *dst, const MgPeers &peers,
                          size_t global_count);
int launch_l1_mg(Ctx *ctx, int dtype, const void *a, const void *b, size_t n, int reduction, void *loss, void *gmap,
                 const MgPeers &peers, size_t global_count);

}  // namespace rtb
