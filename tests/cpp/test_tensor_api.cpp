// The reference's own tensor tests, restated against the C++ host mirror (include/rtensors_b200.hpp).
// Each block cites the test it mirrors (paths relative to libs/rtensors/src/ of the reference).
// Exit code 0 = all passed; prints the first failure otherwise.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "rtensors_b200.hpp"

using namespace rtb200;
template <typename T> using Tensor = TensorBase<T>;

static int g_checks = 0;
#define ASSERT_EQ(a, b)                                                                          \
    do {                                                                                         \
        ++g_checks;                                                                              \
        if (!((a) == (b))) { std::printf("FAIL %s:%d: %s != %s\n", __FILE__, __LINE__, #a, #b); std::exit(1); } \
    } while (0)
#define ASSERT_TRUE(x) ASSERT_EQ(static_cast<bool>(x), true)

template <typename T> static std::vector<T> iota(int lo, int hi) {
    std::vector<T> v;
    for (int i = lo; i <= hi; ++i) v.push_back((T)i);
    return v;
}

int main() {
    Cuda cuda(0);

    {  // ops/mod.rs:127-142 test_add_after_slice
        auto tensor = Tensor<int32_t>::from_buf(cuda, {1, 2, 3, 4, 5, 6}, {2, 3});
        auto slice = tensor.slice(0, Slice::range(1, 1));  // second row
        ASSERT_EQ(slice.get({0}), 4);
        slice += 100;
        ASSERT_EQ(cuda.dump(*tensor.buf), (std::vector<int32_t>{1, 2, 3, 104, 105, 106}));
    }
    {  // ops/mod.rs:200-215 test_mul_after_column_slice
        auto tensor = Tensor<int32_t>::from_buf(cuda, {1, 2, 3, 4, 5, 6}, {2, 3});
        auto col = tensor.slice(1, Slice::range(1, 1));
        ASSERT_TRUE(!col.is_contiguous());
        col *= 3;
        ASSERT_EQ(cuda.dump(*tensor.buf), (std::vector<int32_t>{1, 6, 3, 4, 15, 6}));
    }
    {  // ops/mod.rs:922-951 test_3d_noncontiguous_slice
        auto tensor = Tensor<int32_t>::from_buf(cuda, iota<int32_t>(1, 24), {2, 3, 4});
        auto slice = tensor.slice(1, Slice::range(1, 1));
        ASSERT_EQ(slice.shape(), (std::vector<size_t>{2, 4}));
        ASSERT_EQ(slice.strides(), (std::vector<ptrdiff_t>{12, 1}));
        ASSERT_EQ(slice.offset(), (size_t)4);
        slice += 100;
        auto expect = iota<int32_t>(1, 24);
        for (int i : {5, 6, 7, 8, 17, 18, 19, 20}) expect[i - 1] += 100;
        ASSERT_EQ(cuda.dump(*tensor.buf), expect);
    }
    {  // ops/mod.rs:340-357 test_mul_not_inplace_with_noncontiguous_slice
        auto tensor = Tensor<int32_t>::from_buf(cuda, {1, 2, 3, 4, 5, 6}, {2, 3});
        auto result = tensor.slice(1, Slice::range(1, 1)) * 3;
        ASSERT_EQ(result.cpu(), (std::vector<int32_t>{6, 15}));
        ASSERT_TRUE(result.is_contiguous());
        ASSERT_EQ(cuda.dump(*tensor.buf), (std::vector<int32_t>{1, 2, 3, 4, 5, 6}));
    }
    {  // ops/mod.rs:1154-1171 test_broadcast_flipped
        auto veca = Tensor<float>::ones(cuda, {1, 3});
        auto vecb = Tensor<float>::ones(cuda, {3, 1});
        veca.set({0, 0}, 22.0f);
        auto vecc = veca + vecb;
        ASSERT_EQ(vecc.shape(), (std::vector<size_t>{3, 3}));
        for (size_t i = 0; i < 3; ++i)
            for (size_t j = 0; j < 3; ++j) ASSERT_EQ(vecc.get({i, j}), j == 0 ? 23.0f : 2.0f);
    }
    {  // ops/mod.rs:1474-1487 test_broadcast_div_2d_matrices
        auto veca = Tensor<float>::from_buf(cuda, {100, 200, 300, 400}, {2, 2});
        auto vecb = Tensor<float>::from_buf(cuda, {10, 20}, {1, 2});
        ASSERT_EQ((veca / vecb).cpu(), (std::vector<float>{10, 10, 30, 20}));
    }
    {  // ops/mod.rs:1491-1498 test_broadcast_incompatible_dimensions_3d (should_panic)
        auto veca = Tensor<float>::ones(cuda, {3, 4});
        auto vecb = Tensor<float>::ones(cuda, {2, 5, 6});
        bool threw = false;
        try { auto c = veca + vecb; } catch (const TensorError &e) { threw = e.code == RTB_ERR_BROADCAST; }
        ASSERT_TRUE(threw);
    }
    {  // ops/mod.rs:2455-2479 test_broadcast_with_negative_step_slice
        auto a = Tensor<float>::from_buf(cuda, iota<float>(1, 12), {4, 3});
        auto sliced = a.slice(0, Slice::full().step(-1));
        auto b = Tensor<float>::from_buf(cuda, {10, 20, 30}, {3});
        ASSERT_EQ((sliced + b).cpu(), (std::vector<float>{20, 31, 42, 17, 28, 39, 14, 25, 36, 11, 22, 33}));
    }
    {  // ops/mod.rs:2580-2601 test_broadcast_inplace_with_negative_step
        auto a = Tensor<float>::from_buf(cuda, {1, 2, 3, 4, 5, 6}, {2, 3});
        auto sliced = a.slice(1, Slice::full().step(-1));
        sliced += Tensor<float>::from_buf(cuda, {10}, {1, 1});
        ASSERT_EQ(cuda.dump(*a.buf), (std::vector<float>{11, 12, 13, 14, 15, 16}));
    }
    {  // ops/mod.rs:2604-2635 test_broadcast_chained_slices_with_negative_steps
        auto a = Tensor<float>::from_buf(cuda, iota<float>(1, 16), {4, 4});
        auto s2 = a.slice(0, Slice::full().step(-1)).slice(1, Slice::full().step(2));
        ASSERT_EQ(s2.shape(), (std::vector<size_t>{4, 2}));
        auto b = Tensor<float>::from_buf(cuda, {100, 200}, {1, 2});
        ASSERT_EQ((s2 + b).cpu(), (std::vector<float>{113, 215, 109, 211, 105, 207, 101, 203}));
    }
    {  // ops/mod.rs:2638-2656 test_broadcast_scalar_with_complex_negative_slice
        auto a = Tensor<int32_t>::from_buf(cuda, iota<int32_t>(1, 10), {10});
        auto sliced = a.slice(0, Slice{8, 2, -2});
        ASSERT_EQ((sliced + 100).cpu(), (std::vector<int32_t>{109, 107, 105}));
    }
    {  // backend/cpu.rs:1174-1196 reduce total max / min / prod; backend/cuda.rs:2304-2309 total sum
        auto t = Tensor<double>::from_buf(cuda, {0.2, 0.3, 0.1, 0.3, 0.3, -0.1, -0.3, 0.3}, {4, 2});
        ASSERT_EQ(t.max().item(), 0.3);
        ASSERT_EQ(t.sum().item(), 1.1);
        auto u = Tensor<double>::from_buf(cuda, {0.2, 0.3, 0.1, -0.9, 0.3, -0.1, -0.3, 0.3}, {4, 2});
        ASSERT_EQ(u.min().item(), -0.9);
        auto p = Tensor<double>::from_buf(cuda, {1, 2, 3, 4, 5, 6, 7, 8}, {4, 2});
        ASSERT_EQ(p.prod().item(), 40320.0);
    }
    {  // backend/cpu.rs:1199-1278 axis reductions keep the reduced dim as size 1
        auto t = Tensor<double>::from_buf(cuda, {3, 5, 6, 8, 1, 2, -1, 4}, {4, 2});
        ASSERT_EQ(t.max_at(0).cpu(), (std::vector<double>{6, 8}));
        ASSERT_EQ(t.max_at(0).shape(), (std::vector<size_t>{1, 2}));
        ASSERT_EQ(t.min_at(0).cpu(), (std::vector<double>{-1, 2}));
        ASSERT_EQ(t.prod_at(0).cpu(), (std::vector<double>{-18, 320}));
        auto m = Tensor<double>::from_buf(cuda, {1, 2, 3, 4, 5, 6, 7, 8}, {4, 2});
        ASSERT_EQ(m.mean_at(0).cpu(), (std::vector<double>{4, 5}));
        ASSERT_EQ(m.mean_at(1).cpu(), (std::vector<double>{1.5, 3.5, 5.5, 7.5}));
        ASSERT_EQ(m.mean_at(1).shape(), (std::vector<size_t>{4, 1}));
    }
    {  // backend/cuda.rs:2320-2590: the reductions only the reference's CUDA backend has
        auto near = [](double a, double b) { return std::fabs(a - b) <= 1e-14 * std::fabs(b); };
        auto m = Tensor<double>::from_buf(cuda, {1, 2, 3, 4, 5, 6, 7, 8}, {4, 2});
        ASSERT_EQ(m.var().item(), 6.0);
        ASSERT_EQ(m.pop_var().item(), 5.25);
        ASSERT_TRUE(near(m.std(true).item(), 2.449489742783178));
        ASSERT_TRUE(near(m.std(false).item(), 2.29128784747792));
        ASSERT_EQ(m.l1_norm().item(), 36.0);
        ASSERT_TRUE(near(m.l2_norm().item(), 14.2828568570857));
        ASSERT_EQ(m.pop_var_at(0).cpu(), (std::vector<double>{5, 5}));
        ASSERT_EQ(m.var_at(0).shape(), (std::vector<size_t>{1, 2}));
        ASSERT_TRUE(near(m.var_at(0).cpu()[1], 6.666666666666667));
        ASSERT_TRUE(near(m.std_at(0, true).cpu()[0], 2.581988897471611));
        ASSERT_TRUE(near(m.logsumexp_at(0).cpu()[0], 7.145077938960783));
        ASSERT_TRUE(near(m.logsumexp_at(0).cpu()[1], 8.145077938960782));
        ASSERT_EQ(m.l1_norm_at(0).cpu(), (std::vector<double>{16, 20}));
        ASSERT_TRUE(near(m.l2_norm_at(0).cpu()[0], 9.16515138991168));
        auto am = Tensor<double>::from_buf(cuda, {1, 4, 3, 2, 9, 6, 7, 1}, {4, 2});
        ASSERT_EQ(am.argmax_at(0).cpu(), (std::vector<uint64_t>{2, 2}));
        auto an = Tensor<double>::from_buf(cuda, {1, -4, 3, 2, 9, 6, -7, 1}, {4, 2});
        ASSERT_EQ(an.argmin_at(0).cpu(), (std::vector<uint64_t>{3, 0}));
        auto t = Tensor<double>::from_buf(cuda, {0.2, 0.3, 0.1, 0.7, 0.3, -0.1, -0.3, 0.3}, {4, 2});
        ASSERT_EQ(t.argmax().item(), (uint64_t)3);
        ASSERT_EQ(t.argmin().item(), (uint64_t)6);
        // a transposed view reduces without a copy and counts positions in the view's own order
        ASSERT_EQ(am.permute({1, 0}).argmax_at(1).cpu(), (std::vector<uint64_t>{2, 2}));
    }
    {  // ops/unary/mod.rs:442-451 relu on the N-d strided fixture (testing/mod.rs:159-195)
        std::vector<double> def = {-1.0, 1.0, 0.0, 2.0, 1.0, 2.3, -0.3, 0.4, 0.0, -0.3, 0.4, 0.5, -0.2, 0.1, 0.2, -0.5};
        auto t = Tensor<double>::from_buf(cuda, def, {4, 4, 1});
        auto l2 = t.slice(0, Slice::full().step(2)).slice(1, Slice::full().step(2));
        l2.relu_inplace();
        auto got = cuda.dump(*t.buf);
        for (size_t i = 0; i < 4; ++i)
            for (size_t j = 0; j < 4; ++j) {
                double x = def[i * 4 + j];
                double want = (i % 2 == 0 && j % 2 == 0) ? std::fmax(x, 0.0) : x;
                ASSERT_EQ(got[i * 4 + j], want);
            }
    }
    {  // mean_l1_loss (ops/broadcast/l1.rs:79-84); no reference test pins a value: small exact case
        auto a = Tensor<float>::from_buf(cuda, {1, 2, 3, 4}, {2, 2});
        auto b = Tensor<float>::from_buf(cuda, {2, 2, 1, 8}, {2, 2});
        ASSERT_EQ(mean_l1_loss(a, b).item(), 1.75f);
    }
    {  // into_dtype (core/primitives.rs:527-538; values of backend/remote/remote_tests.rs:816-825),
       // row / column (core/primitives.rs:428-444), view_as / reshape / transpose (core/tensor.rs:238-243,328-355)
        auto t = Tensor<float>::from_buf(cuda, {1.7f, -2.2f, 3.0f}, {3});
        ASSERT_EQ(t.into_dtype<int64_t>().cpu(), (std::vector<int64_t>{2, -2, 3}));
        ASSERT_EQ(t.into_dtype<uint8_t>().cpu(), (std::vector<uint8_t>{2, 0, 3}));
        ASSERT_EQ(t.into_dtype<double>().cpu(), (std::vector<double>{(double)1.7f, (double)-2.2f, 3.0}));
        auto r = Tensor<int32_t>::row(cuda, {1, 2, 3, 4, 5, 6});
        ASSERT_EQ(r.shape(), (std::vector<size_t>{1, 6}));
        ASSERT_EQ(Tensor<int32_t>::column(cuda, {1, 2, 3}).shape(), (std::vector<size_t>{3}));
        auto m = r.view_as({2, 3});
        ASSERT_EQ(m.transpose().shape(), (std::vector<size_t>{3, 2}));
        ASSERT_EQ(m.transpose().cpu(), (std::vector<int32_t>{1, 4, 2, 5, 3, 6}));
        bool threw = false;
        try { m.transpose().view_as({6}); } catch (const TensorError &) { threw = true; }
        ASSERT_TRUE(threw);
        auto flat = m.transpose().reshape({6});
        ASSERT_EQ(flat.cpu(), (std::vector<int32_t>{1, 4, 2, 5, 3, 6}));
        ASSERT_TRUE(flat.buf.get() != m.buf.get());
        auto f = m.slice(1, Slice::full().step(2));
        f.fill(9);
        ASSERT_EQ(r.cpu(), (std::vector<int32_t>{9, 2, 9, 9, 5, 9}));
        ASSERT_EQ(f.into_dtype<float>().cpu(), (std::vector<float>{9, 9, 9, 9}));
    }
    {  // buffer-level trait methods (backend/mod.rs:227-233) with the CPU backend's checks (backend/cpu.rs:151-207)
        auto a = cuda.alloc_from_slice<int32_t>({1, 2, 3, 4, 5, 6});
        auto b = cuda.alloc<int32_t>(6);
        cuda.copy_from_slice(*b, std::vector<int32_t>{10, 20, 30, 40, 50, 60});
        cuda.copy_range_within(*b, *a, 1, 3, 2);
        ASSERT_EQ(cuda.dump(*b), (std::vector<int32_t>{10, 4, 5, 40, 50, 60}));
        ASSERT_EQ(cuda.len(*b), (size_t)6);
        ASSERT_EQ(cuda.read(*b, 2), 5);
        cuda.write(*b, 5, 7);
        ASSERT_EQ(cuda.read(*b, 5), 7);
        int errors = 0;
        try { cuda.read(*b, 6); } catch (const TensorError &e) { errors += e.code == RTB_ERR_BOUNDS; }
        try { cuda.write(*b, 6, 1); } catch (const TensorError &e) { errors += e.code == RTB_ERR_BOUNDS; }
        try { cuda.copy_range_within(*b, *a, 5, 0, 2); } catch (const TensorError &e) { errors += e.code == RTB_ERR_BOUNDS; }
        try { cuda.copy_from_slice(*b, std::vector<int32_t>{1}); } catch (const TensorError &e) { errors += e.code == RTB_ERR_SHAPE; }
        ASSERT_EQ(errors, 4);
    }
    {  // gradient maps of relu and abs (ops/unary/mod.rs:213-252): > 0 -> 1, else 0 / -1
        auto t = Tensor<float>::from_buf(cuda, {-1.0f, 0.0f, 2.0f, 3.0f, -0.5f, 0.25f}, {2, 3});
        ASSERT_EQ(t.relu_grad_map().cpu(), (std::vector<float>{0, 0, 1, 1, 0, 1}));
        ASSERT_EQ(t.abs_grad_map().cpu(), (std::vector<float>{-1, -1, 1, 1, -1, 1}));
        ASSERT_EQ(t.transpose().relu_grad_map().cpu(), (std::vector<float>{0, 1, 0, 0, 1, 1}));
        ASSERT_EQ(t.leaky_relu_grad_map(0.125f).cpu(), (std::vector<float>{0.125f, 0.125f, 1, 1, 0.125f, 1}));
        ASSERT_EQ(t.slice(1, Slice::range(2, 3)).reciprocal_map().cpu(), (std::vector<float>{0.5f, 4.0f}));
        auto u = Tensor<uint8_t>::from_buf(cuda, {0, 5}, {2});
        ASSERT_EQ(u.relu_grad_map().cpu(), (std::vector<uint8_t>{0, 1}));
        bool threw = false;
        try { u.abs_grad_map(); } catch (const TensorError &e) { threw = e.code == RTB_ERR_DTYPE; }
        ASSERT_TRUE(threw);
    }
    {  // tensors in host memory: `a + b.T` and column sums without a resident copy, against host loops
        const size_t R = 37, Cn = 53;
        Cuda::HostVec<float> a(R * Cn), b(R * Cn), out(R * Cn), cols(Cn);
        Cuda::HostVec<uint64_t> arg(R);
        for (size_t i = 0; i < R * Cn; ++i) { a[i] = (float)((i * 7) % 31) - 15.f; b[i] = (float)((i * 5) % 17) * 0.25f; }
        MetaTensor am = MetaTensor::contiguous({R, Cn}), bt = MetaTensor::contiguous({Cn, R}).transpose();
        check(rtb_host_set_stage_bytes(cuda.ctx(), Cn * sizeof(float) * 4));  // four rows per stage: the ring is reused
        cuda.host_broadcast(a, am, b, bt, BinaryOpType::Add, out, 0, R);
        cuda.host_reduce_view<float, float>(a, am, 0, ReductionOpTypes::Sum, cols);
        cuda.host_reduce_view<float, uint64_t>(a, am, 1, ReductionOpTypes::ArgMax, arg);
        cuda.host_wait();
        check(rtb_host_set_stage_bytes(cuda.ctx(), size_t(64) << 20));
        for (size_t i = 0; i < R; ++i)
            for (size_t j = 0; j < Cn; ++j) ASSERT_EQ(out[i * Cn + j], a[i * Cn + j] + b[j * R + i]);
        for (size_t j = 0; j < Cn; ++j) {
            float want = 0;
            for (size_t i = 0; i < R; ++i) want += a[i * Cn + j];   // small integers: exact in any order
            ASSERT_EQ(cols[j], want);
        }
        for (size_t i = 0; i < R; ++i) {
            size_t best = 0;
            for (size_t j = 1; j < Cn; ++j)
                if (a[i * Cn + j] > a[i * Cn + best]) best = j;
            ASSERT_EQ(arg[i], (uint64_t)best);
        }
        // the primitives: upload, scale on the device, copy out, give the block back
        float *blk = cuda.host_stage_in(a);
        cuda.host_ready(blk);
        float two = 2.f;
        check(rtb_scalar_op(cuda.ctx(), RTB_F32, (int)BinaryOpType::Mul, blk, &two, am.rank(), am.shape.data(), am.strides.data(), 0));
        cuda.host_stage_out(blk, out, R * Cn);
        cuda.host_release(blk);
        cuda.host_join();
        cuda.sync();
        for (size_t i = 0; i < R * Cn; ++i) ASSERT_EQ(out[i], a[i] * 2.f);
    }
    std::printf("ok: %d checks\n", g_checks);
    return 0;
}
