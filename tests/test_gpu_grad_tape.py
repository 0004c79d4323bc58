"""The autograd tape (rtensors_b200.grad) and the fused dense-layer kernel on the GPU: the MLP step
written with tensors and operators, as a user of the reference writes it, must equal the fused
fixed-graph step bit for bit in both modes, and the CPU oracle's step within the GEMM tolerance."""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def _b():
    from cuda_engine import backend
    return backend()


@pytest.mark.parametrize("dt", [np.float32, np.float64], ids=["f32", "f64"])
@pytest.mark.parametrize("rows,cols", [(1, 4), (7, 10), (64, 1024), (33, 1028), (513, 250), (9, 3)])
def test_bias_relu_mask_equals_add_then_relu_with_mask(dt, rows, cols):
    rng = np.random.default_rng(rows * 1000 + cols)
    z = rng.uniform(-1, 1, rows * cols).astype(dt)
    bias = rng.uniform(-0.5, 0.5, cols).astype(dt)
    z[::13] = 0.0
    bias[::5] = 0.0
    z[5 % z.size] = np.nan
    want = z.copy()
    zm = O.Meta.contiguous((rows, cols))
    shape, sa, sb = O.broadcast_params(zm, O.Meta.contiguous((1, cols)))
    O.broadcast(want, O.Meta(shape, sa, 0), bias, O.Meta(shape, sb, 0), want, O.Meta(shape, sa, 0), O.ADD)
    pre = want.copy()
    O.unary_op(want, O.RELU, O.Meta.contiguous((want.size,)))
    wmask = (pre > 0).astype(dt)
    be = _b()
    d = be.alloc_from_slice(z)
    mask = be.bias_relu_mask(d, be.alloc_from_slice(bias), rows, cols)
    assert d.cpu().numpy().tobytes() == want.tobytes()
    assert mask.cpu().numpy().tobytes() == wmask.tobytes()


@pytest.mark.parametrize("ref_quirks", [False, True], ids=["intended", "ref_quirks"])
def test_tape_step_equals_the_fused_step_bit_for_bit_and_the_oracle(ref_quirks):
    from mlp_oracle import mlp_step
    from rtensors_b200.meta import Meta
    from rtensors_b200.mlp import DenseMlp, synthetic_batch, tape_step
    from rtensors_b200.tensor import Tensor
    torch.backends.cuda.matmul.allow_tf32 = False
    be = _b()
    sizes = (784, 128, 64, 10)
    model = DenseMlp(be, sizes, lr=0.01, ref_quirks=ref_quirks)
    img, tgt, img_h, tgt_h = synthetic_batch(96, "cuda:0")
    host0 = model.host_params()
    host0[1][:] = np.linspace(-0.05, 0.05, host0[1].size, dtype=np.float32).reshape(host0[1].shape)  # non-zero biases
    host0[3][:] = 0.01
    model.load_params(host0)
    params = [Tensor(be, be.alloc_from_slice(p.reshape(-1)), Meta.contiguous(p.shape)) for p in host0]
    ref_params = [p.copy() for p in host0]
    for step in range(3):
        l_fused = model.step(img, tgt)
        l_tape = tape_step(be, params, img, tgt, 0.01, ref_quirks)
        assert l_fused.cpu().numpy().tobytes() == l_tape.buf.cpu().numpy()[:1].tobytes(), step
        for a, t in zip(model.host_params(), params):
            assert a.tobytes() == t.cpu().tobytes(), step
        l_ref, ref_params, _ = mlp_step(ref_params, sizes, img_h, tgt_h, 0.01, ref_quirks)
        assert abs(float(l_fused.item()) - l_ref) <= 1e-4 * abs(l_ref)
        for a, r in zip(model.host_params(), ref_params):
            assert np.max(np.abs(a - r)) <= 1e-4 * max(float(np.max(np.abs(r))), 1e-6)


def test_gradients_reaching_a_node_twice_are_summed_and_leaves_accumulate():
    """z = (x*w) + (x*w) used twice, loss = mean_l1_loss(z, t): dL/dw collects both paths; a second
    backward pass without an optimizer step adds into the same leaf gradient."""
    from rtensors_b200 import grad
    from rtensors_b200.tensor import Tensor, mean_l1_loss_tracked
    be = _b()
    rng = np.random.default_rng(5)
    xh = rng.uniform(0.5, 1.5, (4, 6)).astype(np.float32)
    wh = rng.uniform(0.5, 1.5, (1, 6)).astype(np.float32)
    th = np.zeros((4, 6), dtype=np.float32)
    x, w, t = Tensor.from_buf(xh, xh.shape, backend=be), Tensor.from_buf(wh, wh.shape, backend=be), Tensor.from_buf(th, th.shape, backend=be)
    with grad.enabled() as ctx:
        w.param()
        for rep in (1, 2):
            y = x * w
            z = y + y
            loss = mean_l1_loss_tracked(z, t)
            ctx.backwards(loss)
            # z > 0 everywhere: dL/dz = 1/24, dL/dy = 2/24, dL/dw[j] = sum_i x[i,j] * 2/24
            want = rep * (xh * np.float32(2.0 / 24.0)).sum(axis=0, dtype=np.float64)
            got = w.grad.value.cpu().reshape(-1)
            assert np.allclose(got, want, rtol=1e-5), rep
        assert len(ctx.nodes) == 2          # the sentinel and the leaf: every other node was consumed


def test_linear_model_loss_decreases_under_sgd():
    """What the reference's own autograd tests assert (src/grad/mod.rs:607-1586): the loss goes down."""
    from rtensors_b200 import grad
    from rtensors_b200.tensor import Tensor, mean_l1_loss_tracked
    be = _b()
    rng = np.random.default_rng(6)
    xh = rng.uniform(-1, 1, (64, 8)).astype(np.float32)
    true_w = rng.uniform(-1, 1, (8, 3)).astype(np.float32)
    yh = xh @ true_w + 0.25
    x, y = Tensor.from_buf(xh, xh.shape, backend=be), Tensor.from_buf(yh, yh.shape, backend=be)
    w = Tensor.zeros((8, 3), backend=be)
    b = Tensor.zeros((1, 3), backend=be)
    losses = []
    for _ in range(40):
        with grad.enabled() as ctx:
            opt = grad.SGD(0.2)
            opt.register_parameters([w, b])
            loss = mean_l1_loss_tracked(x.matmul(w) + b, y)
            ctx.backwards(loss)
            opt.step()
        losses.append(float(loss.item()))
    assert losses[-1] < 0.5 * losses[0]
    with grad.no_grad():
        assert not grad.is_enabled()


_UNARY_CASES = {
    # name: (f, f', domain)
    "sigmoid": (lambda x: 1 / (1 + np.exp(-x)), lambda x: (1 / (1 + np.exp(-x))) * (1 - 1 / (1 + np.exp(-x))), (-2, 2)),
    "tanh": (np.tanh, lambda x: 1 - np.tanh(x) ** 2, (-2, 2)),
    "sqrt": (np.sqrt, lambda x: 0.5 / np.sqrt(x), (0.5, 3)),
    "exp": (np.exp, np.exp, (-1, 1)),
    "reciprocal": (lambda x: 1 / x, lambda x: -1 / x ** 2, (0.5, 2)),
    "rsqrt": (lambda x: x ** -0.5, lambda x: -0.5 * x ** -1.5, (0.5, 2)),
    "ln": (np.log, lambda x: 1 / x, (0.5, 3)),
    "sin": (np.sin, np.cos, (-2, 2)),
    "cos": (np.cos, lambda x: -np.sin(x), (-2, 2)),
    "tan": (np.tan, lambda x: 1 / np.cos(x) ** 2, (-1, 1)),
    "square": (lambda x: x * x, lambda x: 2 * x, (-2, 2)),
    "cube": (lambda x: x ** 3, lambda x: 3 * x * x, (-2, 2)),
    "sinh": (np.sinh, np.cosh, (-2, 2)),
    "cosh": (np.cosh, np.sinh, (-2, 2)),
    "expm1": (np.expm1, np.exp, (-1, 1)),
    "ln1p": (np.log1p, lambda x: 1 / (1 + x), (0.0, 2)),
    "abs": (np.abs, np.sign, (-2, 2)),
    "neg": (lambda x: -x, lambda x: -np.ones_like(x), (-2, 2)),
}


@pytest.mark.parametrize("name", sorted(_UNARY_CASES))
def test_unary_nodes_backpropagate_the_analytic_derivative(name):
    """loss = mean_l1_loss(f(x), t) with t far below f(x): dL/dx = f'(x) / N (src/grad/backwards.rs:240-510)."""
    from rtensors_b200 import grad
    from rtensors_b200.tensor import Tensor, mean_l1_loss_tracked
    be = _b()
    f, df, (lo, hi) = _UNARY_CASES[name]
    rng = np.random.default_rng(len(name))
    xh = rng.uniform(lo, hi, (6, 50)).astype(np.float64)
    xh[np.abs(xh) < 0.05] = 0.3
    x = Tensor.from_buf(xh, xh.shape, dtype=np.float64, backend=be)
    t = Tensor.full(xh.shape, -100.0, dtype=np.float64, backend=be)
    with grad.enabled() as ctx:
        x.param()
        y = getattr(x, name)()
        assert np.allclose(y.cpu(), f(xh), rtol=1e-12, atol=1e-12)
        loss = mean_l1_loss_tracked(y, t)
        ctx.backwards(loss)
    assert np.allclose(x.grad.value.cpu(), df(xh) / xh.size, rtol=1e-10, atol=1e-14), name


def test_division_scalar_division_and_view_nodes():
    """z = ((a / b).permute(1,0) / 2).unsqueeze(0).squeeze().reshape(-1): gradients flow back through
    BroadcastDiv (with b broadcast over the rows), DivScalar, Permute, Unsqueeze, Squeeze and Reshape."""
    from rtensors_b200 import grad
    from rtensors_b200.tensor import Tensor, mean_l1_loss_tracked
    be = _b()
    rng = np.random.default_rng(9)
    ah = rng.uniform(1, 2, (5, 7)).astype(np.float64)
    bh = rng.uniform(1, 2, (1, 7)).astype(np.float64)
    a = Tensor.from_buf(ah, ah.shape, dtype=np.float64, backend=be)
    b = Tensor.from_buf(bh, bh.shape, dtype=np.float64, backend=be)
    t = Tensor.full((35,), -100.0, dtype=np.float64, backend=be)
    with grad.enabled() as ctx:
        a.param(); b.param()
        z = ((a / b).permute((1, 0)) / 2.0).unsqueeze(0).squeeze().reshape((35,))
        assert np.allclose(z.cpu(), ((ah / bh).T / 2).reshape(-1))
        loss = mean_l1_loss_tracked(z, t)
        ctx.backwards(loss)
    n = 35.0
    assert np.allclose(a.grad.value.cpu(), (1 / bh) / 2 / n * np.ones_like(ah), rtol=1e-12)
    assert np.allclose(b.grad.value.cpu().reshape(-1), (-(ah / bh ** 2) / 2 / n).sum(axis=0), rtol=1e-12)
