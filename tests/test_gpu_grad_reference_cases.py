"""The reference's own autograd tests (src/grad/mod.rs:607-1290), restated on the tape of
rtensors_b200.grad: small models trained for ten SGD steps; the reference asserts only that the loss
drops by more than a threshold.  In `ref_quirks` mode (the reference's observable behaviour: backward
seeded with the loss value, broadcast gradients re-labelled instead of summed) the reference's own
thresholds must hold.  In intended mode (seed 1, true sums) ten steps at the reference's learning rates
overshoot in some of these models -- its thresholds were tuned to its loss-scaled gradients -- so there
the check is that ONE step lowers the loss."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _b():
    from cuda_engine import backend
    return backend()


def _T():
    from rtensors_b200.tensor import Tensor
    return Tensor


def _loss(a, b):
    from rtensors_b200.tensor import mean_l1_loss_tracked
    return mean_l1_loss_tracked(a, b)


def ones(shape): return _T().ones(shape, backend=_b())
def zeros(shape): return _T().zeros(shape, backend=_b())


# (name, source lines, parameter shapes (None = rank-0 scalar 1.0), fixed inputs, model, learning rate, threshold)
CASES = [
    ("scalar plus matrix", "613-617, 689-708", [None, (2, 2)], lambda: (zeros((2, 2)),), lambda p, f: _loss(p[0] + p[1], f[0]), 1.0, 0.1),
    ("three way add", "619-630, 712-728", [(2, 2), (2, 2), (2, 2)], lambda: (zeros((2, 2)),),
     lambda p, f: _loss(p[0] + (p[1] + p[2]), f[0]), 1.0, 0.5),
    ("permute then abs", "632-645, 732-749", [(2, 3), (3, 2)], lambda: (ones((2, 3)), zeros((3, 2))),
     lambda p, f: _loss(p[1] + (f[0] + p[0]).permute((1, 0)).abs(), f[1]), 1.0, 0.5),
    ("permute then relu", "647-658, 754-769", [(2, 3), (3, 2)], lambda: (ones((2, 3)), zeros((3, 2))),
     lambda p, f: _loss(p[1] + (f[0] + p[0]).permute((1, 0)).relu(), f[1]), 1.0, 0.5),
    ("negated sqrt against a transposed target", "660-666, 774-790", [(2, 3)], lambda: (zeros((3, 2)),),
     lambda p, f: _loss(p[0].sqrt().neg(), f[0].transpose()), 1.0, 0.5),
    ("sin + tanh(cos)", "1031-1049, 1062-1078", [(2, 3)], lambda: (ones((2, 3)), zeros((2, 3))),
     lambda p, f: (lambda x: _loss(x.sin() + x.cos().tanh(), f[1]))(f[0] + p[0]), 0.1, 0.01),
    ("sinh + cosh", "1051-1059, 1080-1095", [(2, 3)], lambda: (ones((2, 3)), zeros((2, 3))),
     lambda p, f: (lambda x: _loss(x.sinh() + x.cosh(), f[1]))(f[0] + p[0]), 0.1, 0.5),
    ("exp", "1101-1109, 1121-1137", [(2, 3)], lambda: (ones((2, 3)), ones((2, 3))),
     lambda p, f: _loss((f[0] + p[0]).exp(), f[1]), 0.01, 0.1),
    ("square + cube", "1111-1119, 1139-1153", [(2, 3)], lambda: (ones((2, 3)), ones((2, 3))),
     lambda p, f: (lambda x: _loss(x.square() + x.cube(), f[1]))(f[0] + p[0]), 0.01, 0.1),
    ("reciprocal", "1161-1169", [(2, 3)], lambda: (ones((2, 3)), ones((2, 3))),
     lambda p, f: _loss((f[0] + p[0]).reciprocal(), f[1]), 0.1, 0.001),
    ("rsqrt", "1170-1178", [(2, 3)], lambda: (ones((2, 3)), ones((2, 3))),
     lambda p, f: _loss((f[0] + p[0]).rsqrt(), f[1]), 0.1, 0.001),
    ("square, tanh, add, sinh, reciprocal", "1223-1234", [(2, 3), (2, 3)], lambda: (ones((2, 3)), zeros((2, 3))),
     lambda p, f: _loss(((f[0] + p[0]).square().tanh() + p[1]).sinh().reciprocal(), f[1]), 0.1, 0.001),
    ("sin, exp, rsqrt chain", "1235-1243", [(2, 3)], lambda: (ones((2, 3)), zeros((2, 3))),
     lambda p, f: _loss((f[0] + p[0]).sin().exp().rsqrt(), f[1]), 0.1, 0.0001),
]


@pytest.mark.parametrize("ref_quirks", [True, False], ids=["ref_quirks", "intended"])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_reference_autograd_case(case, ref_quirks):
    from rtensors_b200 import grad
    name, _lines, shapes, fixed, model, lr, threshold = case
    T = _T()
    with grad.enabled(ref_quirks=ref_quirks) as ctx:
        params = [T.scalar(1.0, backend=_b()) if s is None else ones(s) for s in shapes]
        f = fixed()
        opt = grad.SGD(lr)
        opt.register_parameters(params)
        initial = float(model(params, f).item())
        for _ in range(10 if ref_quirks else 1):
            loss = model(params, f)
            ctx.backwards(loss)
            opt.step()
        final = float(model(params, f).item())
    assert np.isfinite(final)
    if ref_quirks:
        assert initial - final > threshold, (name, initial, final)
    else:
        assert final < initial, (name, initial, final)
