// The multi-GPU entry points driven from compiled code: one host thread per device in ONE process
// (the form in which a Rust host would own its devices), through the plain C ABI only.
// Each thread owns a context, joins the communicator, reduces its half of a tensor and ends with the
// global result; an axis sum whose reduced dim is split combines partial vectors the same way.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

#include "rt_b200.h"
#include "rtensors_b200.hpp"

static int g_fail = 0;
#define CHECK(cond)                                                              \
    do {                                                                         \
        if (!(cond)) {                                                           \
            std::printf("FAILED %s:%d: %s  [%s]\n", __FILE__, __LINE__, #cond, rtb_last_error_string()); \
            ++g_fail;                                                            \
            return;                                                              \
        }                                                                        \
    } while (0)

static void worker(int rank, int nranks, const unsigned char *id, const std::vector<float> *x, double *out_sum, float *out_max,
                   std::vector<float> *col_sums, int *peer_mapped) {
    rtb_ctx *ctx = nullptr;
    CHECK(rtb_ctx_create(rank, &ctx) == RTB_OK);
    CHECK(rtb_mg_init(ctx, nranks, rank, id) == RTB_OK);
    int n = 0, r = 0;
    CHECK(rtb_mg_info(ctx, &n, &r, peer_mapped) == RTB_OK && n == nranks && r == rank);
    // flat range of this rank
    size_t b = 0, e = 0;
    rtb_shard_range(x->size(), (size_t)nranks, (size_t)rank, &b, &e);
    void *dev = nullptr, *res = nullptr;
    CHECK(rtb_alloc(ctx, (e - b) * sizeof(float), &dev) == RTB_OK);
    CHECK(rtb_alloc(ctx, 4096 * sizeof(float), &res) == RTB_OK);
    CHECK(rtb_h2d(ctx, dev, x->data() + b, (e - b) * sizeof(float)) == RTB_OK);
    float v = 0;
    CHECK(rtb_mg_reduce_flat(ctx, RTB_F32, RTB_SUM, dev, 0, e - b, x->size(), res) == RTB_OK);
    CHECK(rtb_d2h(ctx, &v, res, sizeof(float)) == RTB_OK);
    out_sum[rank] = v;
    CHECK(rtb_mg_reduce_flat(ctx, RTB_F32, RTB_MAX, dev, 0, e - b, x->size(), res) == RTB_OK);
    CHECK(rtb_d2h(ctx, &out_max[rank], res, sizeof(float)) == RTB_OK);
    // the same buffer as rows of a (rows, 256) matrix whose ROWS are split: column sums need a combine
    const size_t cols = 256, rows_local = (e - b) / cols, rows_global = x->size() / cols;
    CHECK(rtb_mg_reduce_axis(ctx, RTB_F32, RTB_SUM, dev, 0, 1, rows_local, cols, (ptrdiff_t)(rows_local * cols), (ptrdiff_t)cols,
                             rows_global, res) == RTB_OK);
    col_sums[rank].resize(cols);
    CHECK(rtb_d2h(ctx, col_sums[rank].data(), res, cols * sizeof(float)) == RTB_OK);
    unsigned bits = 99;
    CHECK(rtb_mg_status(ctx, &bits) == RTB_OK && bits == 0);
    CHECK(rtb_free(ctx, dev) == RTB_OK && rtb_free(ctx, res) == RTB_OK);
    CHECK(rtb_mg_finalize(ctx) == RTB_OK);
    rtb_ctx_destroy(ctx);
}

// The same through the C++ mirror's `Cuda` class (one object per device): mean over the split tensor, a
// partial-vector combine, and an all-reduce begun on the side stream and joined.
static void mirror_worker(int rank, int nranks, const std::vector<unsigned char> *id, const std::vector<float> *x, float *out_mean,
                          float *out_vec) {
    using namespace rtb200;
    try {
        Cuda cuda(rank);
        cuda.mg_init(nranks, rank, *id);
        size_t b = 0, e = 0;
        rtb_shard_range(x->size(), (size_t)nranks, (size_t)rank, &b, &e);
        auto local = cuda.alloc_from_slice(std::vector<float>(x->begin() + b, x->begin() + e));
        auto res = cuda.alloc<float>(1);
        cuda.mg_reduce_flat(*local, 0, e - b, x->size(), ReductionOpTypes::Mean, *res);
        out_mean[rank] = cuda.dump(*res)[0];
        auto vec = cuda.alloc_from_slice(std::vector<float>(64, (float)(rank + 1)));
        cuda.mg_combine(*vec, 64, ReductionOpTypes::Sum);
        auto big = cuda.alloc_from_slice(std::vector<float>(100000, (float)(rank + 1)));
        cuda.mg_allreduce(*big, 100000, ReductionOpTypes::Sum, /*overlap=*/true);
        cuda.mg_allreduce_join();
        out_vec[rank] = cuda.dump(*vec)[63] + cuda.dump(*big)[99999];
        if (cuda.mg_status() != 0 || cuda.mg_world() != nranks || cuda.mg_rank() != rank) ++g_fail;
        cuda.mg_finalize();
    } catch (const std::exception &ex) {
        std::printf("FAILED (mirror, rank %d): %s\n", rank, ex.what());
        ++g_fail;
    }
}

int main() {
    rtb_ctx *probe = nullptr;
    if (rtb_ctx_create(1, &probe) != RTB_OK) {
        std::printf("skipped: needs 2 GPUs\n");
        return 0;
    }
    rtb_ctx_destroy(probe);
    // host-only partition arithmetic first
    {
        const size_t shape[2] = {8192, 8192};
        if (rtb_mg_pick_reduce_dim(2, shape, 0, 8) != 1 || rtb_mg_pick_reduce_dim(2, shape, 1, 8) != 0) {
            std::printf("FAILED: partitioner\n");
            return 1;
        }
        const ptrdiff_t sl[2] = {1, 0}, sr[2] = {0, 1};
        size_t slab[2], b, e, ol, orr;
        int dim = rtb_mg_slab(2, shape, sl, 0, sr, 0, 8, 3, slab, &b, &e, &ol, &orr);
        if (dim != 0 || b != 3072 || e != 4096 || slab[0] != 1024 || ol != 3072 || orr != 0) {
            std::printf("FAILED: slab\n");
            return 1;
        }
    }
    const int nranks = 2;
    unsigned char id[RTB_MG_ID_BYTES];
    if (rtb_mg_unique_id(id) != RTB_OK) {
        std::printf("FAILED: unique id: %s\n", rtb_last_error_string());
        return 1;
    }
    std::vector<float> x((size_t)1 << 20);
    double truth = 0;
    float mx = -1e30f;
    for (size_t i = 0; i < x.size(); ++i) {
        x[i] = (float)((double)((i * 2654435761u) % 2001) / 1000.0 - 1.0);
        truth += x[i];
        mx = x[i] > mx ? x[i] : mx;
    }
    double sums[2] = {0, 0};
    float maxs[2] = {0, 0};
    std::vector<float> cols[2];
    int mapped[2] = {0, 0};
    std::thread t0(worker, 0, nranks, id, &x, sums, maxs, cols, &mapped[0]);
    std::thread t1(worker, 1, nranks, id, &x, sums, maxs, cols, &mapped[1]);
    t0.join();
    t1.join();
    if (g_fail) return 1;
    if (sums[0] != sums[1] || maxs[0] != maxs[1] || maxs[0] != mx || std::fabs(sums[0] - truth) > 1e-5 * 20 * (double)x.size()) {
        std::printf("FAILED: sum %.6f / %.6f vs %.6f, max %.6f / %.6f vs %.6f\n", sums[0], sums[1], truth, maxs[0], maxs[1], mx);
        return 1;
    }
    for (size_t c = 0; c < 256; ++c) {
        double want = 0;
        for (size_t r = 0; r < x.size() / 256; ++r) want += x[r * 256 + c];
        if (cols[0][c] != cols[1][c] || std::fabs(cols[0][c] - want) > 1e-5 * 12 * 4096) {
            std::printf("FAILED: column %zu: %.6f / %.6f vs %.6f\n", c, cols[0][c], cols[1][c], want);
            return 1;
        }
    }
    {
        std::vector<unsigned char> id2 = rtb200::Cuda::mg_unique_id();
        float means[2] = {0, 0}, vecs[2] = {0, 0};
        std::thread m0(mirror_worker, 0, nranks, &id2, &x, means, vecs);
        std::thread m1(mirror_worker, 1, nranks, &id2, &x, means, vecs);
        m0.join();
        m1.join();
        if (g_fail) return 1;
        const double want_mean = truth / (double)x.size();
        if (means[0] != means[1] || std::fabs(means[0] - want_mean) > 1e-5 || vecs[0] != 6.0f || vecs[1] != 6.0f) {
            std::printf("FAILED: mirror mean %.7f / %.7f vs %.7f, sums %.1f %.1f\n", means[0], means[1], want_mean, vecs[0], vecs[1]);
            return 1;
        }
    }
    std::printf("ok: two ranks in one process, peer exchange mapped = %d %d\n", mapped[0], mapped[1]);
    return 0;
}
