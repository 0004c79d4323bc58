"""Tape autograd over `Tensor`, the way the reference does it (src/grad/mod.rs, src/grad/backwards.rs,
src/grad/optim.rs): a `GradContext` holds the nodes, every tracked op attaches one node with its
parents and whatever it must keep for the backward pass, `backwards(loss)` sorts the graph
topologically and walks it in reverse, leaves accumulate with `+=`, `SGD.step` applies
`p -= grad * lr`.  Every node's arithmetic is one of the library's `rtb_*` calls (GEMMs stay on
cuBLAS through torch.matmul); nothing here computes on the host.

Two modes.  `ref_quirks=True` reproduces what the reference's code does: the backward pass is seeded
with the loss VALUE (src/grad/mod.rs:441-447) and the gradient of a broadcast operand is the first
slab of the upstream, because `inverse_broadcast_gradient` keeps only the meta of its `sum_at`
(src/grad/backwards.rs:527).  `ref_quirks=False` is what that code means to do: seed 1 and a true
sum over the broadcast dims.

    with grad.enabled(ref_quirks=False) as ctx:
        w.param(); b.param()
        loss = mean_l1_loss((x.matmul(w) + b).relu(), target)
        ctx.backwards(loss)
        opt.step()
"""
from __future__ import annotations

import itertools
import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from . import _lib as L
from .meta import Meta, broadcast_params

_keys = itertools.count(1)   # node keys are unique across contexts, so a key left on a tensor by an
                             # earlier context can never name a node of a later one
_state = threading.local()   # the reference keeps its context in a thread-local too (src/grad/mod.rs:503-506)


def _ctx() -> Optional["GradContext"]:
    if getattr(_state, "disabled", False):
        return None
    return getattr(_state, "ctx", None)


def is_enabled() -> bool:
    return _ctx() is not None


class no_grad:
    """Disables tracking inside the block and restores the previous state after it (grad::no_grad)."""

    def __enter__(self):
        self.prev = getattr(_state, "disabled", False)
        _state.disabled = True

    def __exit__(self, *exc):
        _state.disabled = self.prev


class enabled:
    """grad::with: runs the block with a thread-local GradContext (created on first use)."""

    def __init__(self, ref_quirks: bool = False):
        self.ref_quirks = ref_quirks

    def __enter__(self) -> "GradContext":
        self.prev = getattr(_state, "ctx", None)
        if self.prev is None:
            _state.ctx = GradContext(self.ref_quirks)
        return _state.ctx

    def __exit__(self, *exc):
        _state.ctx = self.prev


@dataclass
class GradNode:
    """One variant of the reference's GradNode enum (src/grad/mod.rs:27-123): kind, parent keys
    (None = an untracked input) and the tensors saved for the backward pass."""
    kind: str
    parents: List[Optional[int]] = field(default_factory=list)
    saved: Dict[str, object] = field(default_factory=dict)

    def is_leaf(self) -> bool:
        return self.kind == "Leaf"


class GradHolder:
    """The shared cell a leaf's gradient accumulates in (`Grad`, src/core/primitives.rs:47-66)."""

    def __init__(self):
        self.value = None


class GradContext:
    def __init__(self, ref_quirks: bool = False):
        self.ref_quirks = ref_quirks
        self.nodes: Dict[int, GradNode] = {}
        self.none_node = self._insert(GradNode("None"))

    def _insert(self, node: GradNode) -> int:
        k = next(_keys)
        self.nodes[k] = node
        return k

    def attach(self, tensor, node: GradNode) -> None:
        """Tracks `node` as the producer of `tensor` unless every parent is untracked
        (src/grad/mod.rs:291-305)."""
        node.parents = [p if p is not None and p in self.nodes and p != self.none_node else None for p in node.parents]
        if node.parents and all(p is None for p in node.parents):
            return
        tensor.op = self._insert(node)

    def _resolve(self, key: Optional[int]) -> int:
        # a key from an earlier context names nothing here: the tensor counts as an untracked input
        return key if key is not None and key in self.nodes else self.none_node

    def graph_toposort(self, root) -> List[int]:
        """Iterative depth-first post-order with cycle detection (src/grad/mod.rs:319-360)."""
        order: List[int] = []
        marks: Dict[int, bool] = {}
        stack = [("enter", self._resolve(root.op))]
        while stack:
            what, k = stack.pop()
            if what == "exit":
                marks[k] = True
                order.append(k)
                continue
            seen = marks.get(k)
            if seen is True:
                continue
            if seen is False:
                raise RuntimeError("Graph contains a cycle.")
            marks[k] = False
            stack.append(("exit", k))
            node = self.nodes.get(k)
            if node is None:
                raise RuntimeError("Node not found during backward pass.")
            for p in node.parents:
                stack.append(("enter", self._resolve(p)))
        return order

    def backwards(self, root) -> None:
        """src/grad/mod.rs:432-495: reverse topological walk; the gradients a node receives from its
        consumers are summed, handed to the node's backward function, and its results queued for its
        parents; leaves keep theirs in their GradHolder."""
        from .tensor import Tensor
        order = self.graph_toposort(root)
        if root.op is None or root.op not in self.nodes:
            raise RuntimeError("Root node must have an associated GradNode.")
        rnode = self.nodes[root.op]
        loss = rnode.saved.get("loss")
        if loss is None:
            raise RuntimeError("Root node does not contain a loss.")
        with no_grad():
            seed = loss.owned() if self.ref_quirks else Tensor.full(loss.shape, 1.0, loss.np_dtype, loss.backend)
            acc: Dict[int, list] = {root.op: [seed]}
            for k in reversed(order):
                if k == self.none_node:
                    continue
                ups = acc.pop(k)
                dldy = ups[0]
                for g in ups[1:]:
                    dldy = dldy + g
                node = self.nodes[k]
                grads = _BACKWARD[node.kind](self, node, dldy)
                for p, g in zip(node.parents, grads):
                    if p is not None:
                        acc.setdefault(p, []).append(g)
                if node.kind not in ("None", "Leaf"):
                    acc.pop(k, None)
                    del self.nodes[k]


# ---- backward functions (src/grad/backwards.rs) -------------------------------------------------
def _accumulate_grad(ctx, node, upstream):
    holder: GradHolder = node.saved["grad"]
    if holder.value is not None:
        holder.value += upstream                      # `*existing_grad += upstream`, :17-19
    else:
        holder.value = upstream.owned()
    return [upstream]


def _inverse_broadcast_gradient(ctx, grad, strides: Sequence[int], shape: Sequence[int]):
    """src/grad/backwards.rs:512-538: collapse the upstream over the dims the operand was broadcast
    along (stride 0), then squeeze the dims the operand did not have."""
    from .tensor import Tensor
    if not any(s == 0 for s in strides):
        return grad
    g = grad if grad.is_contiguous() and grad.offset == 0 else grad.contiguous()
    be = g.backend
    diff = len(g.shape) - len(shape)
    oshape = tuple(1 if s == 0 else n for n, s in zip(g.shape, strides))
    if ctx.ref_quirks:
        # the reference runs the sums but keeps only their META: the un-reduced buffer is re-labelled
        # with the reduced shape, so what is read afterwards is its first prod(reduced shape) elements
        out = Tensor(be, g.buf, Meta.contiguous(oshape))
    else:
        buf, got = be.reduce_to_shape(g.buf, g.shape, tuple(strides))
        assert tuple(got) == oshape
        out = Tensor(be, buf, Meta.contiguous(oshape))
    for d in reversed(range(len(strides))):
        if strides[d] == 0 and (d < diff or shape[d - diff] != 1):
            out = out.squeeze(d)
    return out


def _backwards_add(ctx, node, upstream):
    sv = node.saved
    return [_inverse_broadcast_gradient(ctx, upstream, sv["lhs_strides"], sv["lhs_shape"]),
            _inverse_broadcast_gradient(ctx, upstream, sv["rhs_strides"], sv["rhs_shape"])]


def _backwards_sub(ctx, node, upstream):
    sv = node.saved
    return [_inverse_broadcast_gradient(ctx, upstream, sv["lhs_strides"], sv["lhs_shape"]),
            _inverse_broadcast_gradient(ctx, upstream.neg(), sv["rhs_strides"], sv["rhs_shape"])]


def _backwards_mul(ctx, node, upstream):
    sv = node.saved
    return [_inverse_broadcast_gradient(ctx, sv["rhs"] * upstream, sv["lhs_strides"], sv["lhs_shape"]),
            _inverse_broadcast_gradient(ctx, sv["lhs"] * upstream, sv["rhs_strides"], sv["rhs_shape"])]


def _backwards_l1(ctx, node, upstream):
    t = node.saved["grad_map"]                         # sign(a - b) [/ N]
    return [t * upstream, t.neg() * upstream]          # :148-161, upstream is the rank-0 seed


def _backwards_relu(ctx, node, upstream):
    return [node.saved["grad_map"] * upstream]         # :229-239


def _backwards_matmul(ctx, node, upstream):
    left, right = node.saved["left_input"], node.saved["right_input"]   # :493-510
    return [upstream.matmul(right.transpose()), left.transpose().matmul(upstream)]


def _backwards_add_scalar(ctx, node, upstream):
    return [upstream]


def _backwards_mul_scalar(ctx, node, upstream):
    return [upstream * node.saved["scalar"]]


def _backwards_negate(ctx, node, upstream):
    return [upstream.neg()]


def _backwards_div(ctx, node, upstream):
    sv = node.saved                                    # :84-107
    lhs, rr = sv["lhs"], sv["rhs_reciprocal"]
    return [_inverse_broadcast_gradient(ctx, upstream * rr, sv["lhs_strides"], sv["lhs_shape"]),
            _inverse_broadcast_gradient(ctx, upstream * (lhs * rr.square()).neg(), sv["rhs_strides"], sv["rhs_shape"])]


def _backwards_div_scalar(ctx, node, upstream):
    return [upstream / node.saved["scalar"]]


def _backwards_permute(ctx, node, upstream):
    dims = node.saved["dims"]                          # :163-185: the inverse permutation, meta only
    inverse = [0] * len(dims)
    for i, d in enumerate(dims):
        inverse[d] = i
    return [upstream.permute(inverse)]


def _backwards_unsqueeze(ctx, node, upstream):
    return [upstream.squeeze(node.saved["dim"]).owned()]


def _backwards_reshape(ctx, node, upstream):          # Squeeze and Reshape both go back by reshape
    return [upstream.reshape(node.saved["original_shape"])]


# unary nodes: name -> (what the forward op saves, d/dx as a function of that tensor); :240-510
_UNARY_BACKWARD = {
    "Abs": ("grad_map", lambda t: t),
    "Sigmoid": ("result", lambda r: r * (r.neg() + 1.0)),
    "Sqrt": ("result", None),                          # upstream / (output * 2): divides instead of multiplying
    "Ln": ("x_reciprocal", lambda t: t),
    "Sin": ("input", lambda x: x.cos()),
    "Cos": ("input", lambda x: x.sin().neg()),
    "Tan": ("input", lambda x: x.cos().square().reciprocal()),
    "Tanh": ("result", lambda r: r.square().neg() + 1.0),
    "Exp": ("result", lambda r: r),
    "Square": ("input", lambda x: x * 2.0),
    "Cube": ("input", lambda x: x.square() * 3.0),
    "Reciprocal": ("result", lambda r: r.square().neg()),
    "Rsqrt": ("result", lambda r: r.cube() * -0.5),
    "Sinh": ("input", lambda x: x.cosh()),
    "Cosh": ("input", lambda x: x.sinh()),
    "ExpM1": ("input", lambda x: x.exp()),
    "Ln1p": ("input", lambda x: (x + 1.0).reciprocal()),
}


def _unary_backward(kind):
    key, dfdx = _UNARY_BACKWARD[kind]

    def run(ctx, node, upstream):
        t = node.saved[key]
        if kind == "Sqrt":
            return [upstream / (t * 2.0)]
        return [dfdx(t) * upstream]
    return run


_BACKWARD = {
    "Leaf": _accumulate_grad, "None": lambda ctx, node, up: [],
    "BroadcastAdd": _backwards_add, "BroadcastSub": _backwards_sub, "BroadcastMul": _backwards_mul,
    "BroadcastDiv": _backwards_div,
    "L1": _backwards_l1, "ReLU": _backwards_relu, "MatMul": _backwards_matmul,
    "AddScalar": _backwards_add_scalar, "MulScalar": _backwards_mul_scalar, "DivScalar": _backwards_div_scalar,
    "Negate": _backwards_negate, "Permute": _backwards_permute, "Unsqueeze": _backwards_unsqueeze,
    "Squeeze": _backwards_reshape, "Reshape": _backwards_reshape,
}
_BACKWARD.update({k: _unary_backward(k) for k in _UNARY_BACKWARD})


# ---- attach helpers called by the Tensor operators -------------------------------------------------
def attach_broadcast(kind: str, out, a, b) -> None:
    ctx = _ctx()
    if ctx is None:
        return
    shape, sa, sb = broadcast_params(a.meta, b.meta)
    saved = {"lhs_strides": tuple(sa), "rhs_strides": tuple(sb), "lhs_shape": tuple(a.shape), "rhs_shape": tuple(b.shape)}
    if kind == "BroadcastMul":
        saved["lhs"], saved["rhs"] = a, b            # read in place; the reference copies both operands
    if kind == "BroadcastDiv":
        with no_grad():                               # the reciprocal map in one kernel (reference: a get / set loop)
            saved["lhs"], saved["rhs_reciprocal"] = a, b.reciprocal_map()
    ctx.attach(out, GradNode(kind, [a.op, b.op], saved))


def attach_unary(kind: str, out, src, **saved) -> None:
    ctx = _ctx()
    if ctx is not None:
        ctx.attach(out, GradNode(kind, [src.op], dict(saved)))


def attach_matmul(out, a, b) -> None:
    ctx = _ctx()
    if ctx is not None:
        ctx.attach(out, GradNode("MatMul", [a.op, b.op], {"left_input": a, "right_input": b}))


def attach_l1(loss, a, b, grad_map) -> None:
    ctx = _ctx()
    if ctx is not None:
        ctx.attach(loss, GradNode("L1", [a.op, b.op], {"grad_map": grad_map, "loss": loss}))


def make_leaf(t) -> None:
    """TensorBase::param: the tensor becomes a leaf whose gradient is kept (src/core/primitives.rs)."""
    ctx = _ctx()
    if ctx is None:
        raise RuntimeError("Cannot mark a parameter without a grad context.")
    if t.op is not None and t.op in ctx.nodes and ctx.nodes[t.op].is_leaf():
        return
    t.grad = GradHolder()
    t.op = ctx._insert(GradNode("Leaf", [], {"grad": t.grad}))


class SGD:
    """src/grad/optim.rs:14-64."""

    def __init__(self, learning_rate: float):
        self.learning_rate = float(learning_rate)
        self.parameters: list = []

    def register_parameter(self, param) -> None:
        ctx = _ctx()
        if ctx is None:
            raise RuntimeError("Cannot register a parameter without a grad context.")
        param.param()
        node = ctx.nodes.get(ctx._resolve(param.op))
        if node is None:
            raise RuntimeError("Parameter not found in grad context.")
        if not node.is_leaf():
            raise RuntimeError("Only leaf tensors can be registered as parameters.")
        self.parameters.append(param)

    def register_parameters(self, params) -> None:
        for p in params:
            self.register_parameter(p)

    def step(self) -> None:
        with no_grad():
            for p in self.parameters:
                g = p.grad.value if p.grad is not None else None
                if g is None:
                    continue
                update = g * self.learning_rate       # owned copy + scalar multiply (one rounding)
                p.grad.value = None
                v = p.view()
                v -= update                           # in-place broadcast subtract (second rounding)
