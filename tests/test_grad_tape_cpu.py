"""Host logic of the autograd tape that needs no device: attach rules, the topological order and
cycle detection of `graph_toposort` (src/grad/mod.rs:291-360)."""
import pytest

from rtensors_b200 import grad


class _T:
    """Stand-in for a Tensor: the tape only touches `.op`."""

    def __init__(self):
        self.op = None
        self.grad = None


def test_attach_skips_nodes_whose_parents_are_all_untracked():
    ctx = grad.GradContext()
    a, b, out = _T(), _T(), _T()
    ctx.attach(out, grad.GradNode("BroadcastAdd", [a.op, b.op]))
    assert out.op is None                      # no parent is tracked: nothing goes on the tape
    a.op = ctx._insert(grad.GradNode("Leaf", [], {"grad": grad.GradHolder()}))
    ctx.attach(out, grad.GradNode("BroadcastAdd", [a.op, b.op]))
    assert out.op is not None and ctx.nodes[out.op].parents == [a.op, None]
    stale = _T()
    stale.op = 10 ** 9                         # a key from some other context
    o2 = _T()
    ctx.attach(o2, grad.GradNode("ReLU", [stale.op]))
    assert o2.op is None


def test_toposort_puts_every_parent_before_its_consumers():
    ctx = grad.GradContext()
    leaf = ctx._insert(grad.GradNode("Leaf", [], {"grad": grad.GradHolder()}))
    y = ctx._insert(grad.GradNode("MulScalar", [leaf]))
    z1 = ctx._insert(grad.GradNode("ReLU", [y]))
    z2 = ctx._insert(grad.GradNode("Negate", [y]))
    root = _T()
    root.op = ctx._insert(grad.GradNode("BroadcastAdd", [z1, z2]))
    order = ctx.graph_toposort(root)
    pos = {k: i for i, k in enumerate(order)}
    assert pos[leaf] < pos[y] < min(pos[z1], pos[z2]) < pos[root.op]
    assert order.count(y) == 1                 # the diamond's shared node appears once


def test_toposort_reports_a_cycle():
    ctx = grad.GradContext()
    a = ctx._insert(grad.GradNode("ReLU", []))
    b = ctx._insert(grad.GradNode("ReLU", [a]))
    ctx.nodes[a].parents = [b]
    root = _T()
    root.op = b
    with pytest.raises(RuntimeError, match="cycle"):
        ctx.graph_toposort(root)


def test_sgd_needs_a_context_and_a_leaf():
    opt = grad.SGD(0.1)
    with pytest.raises(RuntimeError, match="without a grad context"):
        opt.register_parameter(_T())
    assert not grad.is_enabled()
    with grad.enabled() as ctx:
        assert grad.is_enabled()
        with grad.no_grad():
            assert not grad.is_enabled()
        assert grad.is_enabled() and isinstance(ctx, grad.GradContext)
    assert not grad.is_enabled()
