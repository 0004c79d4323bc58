// The tape of include/rtensors_b200_grad.hpp: analytic gradient checks, then the first four models of the
// reference's own autograd test (src/grad/mod.rs:607-790 of the reference) trained with SGD in both modes.
// Exit code 0 = all passed; prints the first failure otherwise.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <vector>

#include "rtensors_b200_grad.hpp"

using namespace rtb200;
using namespace rtb200::grad;
using V = Var<float>;
using Tn = TensorBase<float>;

static int g_checks = 0;
#define ASSERT_TRUE(x)                                                                            \
    do {                                                                                         \
        ++g_checks;                                                                              \
        if (!(x)) { std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #x); std::exit(1); }      \
    } while (0)

static V ones(const Cuda &c, std::vector<size_t> s) { return V{Tn::ones(c, std::move(s))}; }
static V zeros(const Cuda &c, std::vector<size_t> s) { return V{Tn::zeros(c, std::move(s))}; }

// trains `model` over `params` and returns {initial loss, final loss}
static std::pair<float, float> train(bool quirks, std::vector<V> params, float lr, int steps,
                                     const std::function<V(GradContext<float> &, std::vector<V> &)> &model) {
    GradContext<float> ctx(quirks);
    SGD<float> opt(lr);
    for (V &p : params) opt.register_parameter(ctx, p);
    const float initial = model(ctx, params).t.item();
    for (int i = 0; i < steps; ++i) {
        V loss = model(ctx, params);
        ctx.backwards(loss);
        opt.step();
    }
    const float final_loss = model(ctx, params).t.item();
    return {initial, final_loss};
}

int main() {
    Cuda cuda(0);

    {  // d/dw, d/db of mean|x*w + b - 0| with b broadcast over the rows: sign/N summed over the rows
        GradContext<float> ctx(false);
        V w{Tn::from_buf(cuda, {1, -2, 3, -4, 5, -6}, {2, 3})}, b{Tn::from_buf(cuda, {0.5f, 0.25f, -0.5f}, {3})};
        V x{Tn::from_buf(cuda, {2, 2, 2, 3, 3, 3}, {2, 3})}, target = zeros(cuda, {2, 3});
        ctx.param(w);
        ctx.param(b);
        V loss = mean_l1_loss(ctx, add(ctx, mul(ctx, x, w), b), target);
        // x*w + b = {2.5, -3.75, 5.5, -11.5, 15.25, -18.5}
        ASSERT_TRUE(std::fabs(loss.t.item() - (2.5f + 3.75f + 5.5f + 11.5f + 15.25f + 18.5f) / 6) < 1e-6f);
        ctx.backwards(loss);
        ASSERT_TRUE(w.grad->has && b.grad->has);
        const std::vector<float> gw = w.grad->value.cpu(), gb = b.grad->value.cpu();
        const std::vector<float> want_w{2 / 6.f, -2 / 6.f, 2 / 6.f, -3 / 6.f, 3 / 6.f, -3 / 6.f};
        for (size_t i = 0; i < 6; ++i) ASSERT_TRUE(std::fabs(gw[i] - want_w[i]) < 1e-6f);
        ASSERT_TRUE(b.grad->value.shape() == (std::vector<size_t>{3}));
        const std::vector<float> want_b{0.f, 0.f, 0.f};  // +1/6 - 1/6 per column
        for (size_t i = 0; i < 3; ++i) ASSERT_TRUE(std::fabs(gb[i] - want_b[i]) < 1e-6f);
        ASSERT_TRUE(ctx.nodes.size() == 2);  // only the two leaves are left on the tape
    }
    {  // the same graph as the reference computes it: seed = loss value, b's gradient = the first 3 upstream elements
        GradContext<float> ctx(true);
        V w{Tn::from_buf(cuda, {1, -2, 3, -4, 5, -6}, {2, 3})}, b{Tn::from_buf(cuda, {0.5f, 0.25f, -0.5f}, {3})};
        V x{Tn::from_buf(cuda, {2, 2, 2, 3, 3, 3}, {2, 3})}, target = zeros(cuda, {2, 3});
        ctx.param(w);
        ctx.param(b);
        V loss = mean_l1_loss(ctx, add(ctx, mul(ctx, x, w), b), target);
        const float l = loss.t.item();
        ctx.backwards(loss);
        const std::vector<float> gb = b.grad->value.cpu();
        const std::vector<float> want{l / 6, -l / 6, l / 6};
        for (size_t i = 0; i < 3; ++i) ASSERT_TRUE(std::fabs(gb[i] - want[i]) < 1e-6f);
    }
    {  // a parameter used twice accumulates both paths; a second backward pass adds to the kept gradient
        GradContext<float> ctx(false);
        V p = ones(cuda, {4});
        ctx.param(p);
        V target = zeros(cuda, {4});
        for (int pass = 1; pass <= 2; ++pass) {
            V loss = mean_l1_loss(ctx, add(ctx, p, mul_scalar(ctx, p, 3.f)), target);
            ctx.backwards(loss);
            for (float g : p.grad->value.cpu()) ASSERT_TRUE(std::fabs(g - pass * 1.0f) < 1e-6f);  // (1 + 3) / 4 per pass
        }
    }
    {  // untracked operands put nothing on the tape, and a root without a loss is refused
        GradContext<float> ctx(false);
        V a = ones(cuda, {2}), b = ones(cuda, {2});
        V c = add(ctx, a, b);
        ASSERT_TRUE(c.op == 0 && ctx.nodes.empty());
        bool threw = false;
        try { ctx.backwards(c); } catch (const std::runtime_error &) { threw = true; }
        ASSERT_TRUE(threw);
    }

    for (bool quirks : {true, false}) {
        const int steps = quirks ? 10 : 1;  // the reference's thresholds are tuned to its loss-scaled gradients
        auto drop = [&](std::pair<float, float> r, float threshold) {
            ASSERT_TRUE(std::isfinite(r.second));
            if (quirks) ASSERT_TRUE(r.first - r.second > threshold);
            else ASSERT_TRUE(r.second < r.first);
        };
        // src/grad/mod.rs:613-617, 689-708: scalar + matrix
        drop(train(quirks, {V{Tn::scalar(cuda, 1.f)}, ones(cuda, {2, 2})}, 1.f, steps,
                   [&](GradContext<float> &c, std::vector<V> &p) { return mean_l1_loss(c, add(c, p[0], p[1]), zeros(cuda, {2, 2})); }),
             0.1f);
        // :619-630, 712-728: a + (b + c)
        drop(train(quirks, {ones(cuda, {2, 2}), ones(cuda, {2, 2}), ones(cuda, {2, 2})}, 1.f, steps,
                   [&](GradContext<float> &c, std::vector<V> &p) {
                       return mean_l1_loss(c, add(c, p[0], add(c, p[1], p[2])), zeros(cuda, {2, 2}));
                   }),
             0.5f);
        // :632-645, 732-749: permute then abs
        drop(train(quirks, {ones(cuda, {2, 3}), ones(cuda, {3, 2})}, 1.f, steps,
                   [&](GradContext<float> &c, std::vector<V> &p) {
                       V inner = abs(c, permute(c, add(c, ones(cuda, {2, 3}), p[0]), {1, 0}));
                       return mean_l1_loss(c, add(c, p[1], inner), zeros(cuda, {3, 2}));
                   }),
             0.5f);
        // :647-658, 754-769: permute then relu
        drop(train(quirks, {ones(cuda, {2, 3}), ones(cuda, {3, 2})}, 1.f, steps,
                   [&](GradContext<float> &c, std::vector<V> &p) {
                       V inner = relu(c, permute(c, add(c, ones(cuda, {2, 3}), p[0]), {1, 0}));
                       return mean_l1_loss(c, add(c, p[1], inner), zeros(cuda, {3, 2}));
                   }),
             0.5f);
    }
    std::printf("ok: %d checks\n", g_checks);
    return 0;
}
