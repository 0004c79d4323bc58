// rtensors_b200_grad.hpp -- the reference's tape autograd (src/grad/mod.rs, src/grad/backwards.rs,
// src/grad/optim.rs) restated over the C++ mirror's TensorBase<T>: a GradContext that holds the nodes,
// graph_toposort + backwards, leaf accumulation with `+=`, and SGD.  Every node's arithmetic is a call
// into librt_b200.so through TensorBase's operators; nothing is computed on the host.
//
// Node types: Leaf, BroadcastAdd / BroadcastSub / BroadcastMul, AddScalar, MulScalar, ReLU, Abs, Negate,
// Permute, L1 -- the ones the reference's own `_playground` autograd test uses.  MatMul is not here: the
// header-only mirror carries no GEMM (the reference's matmul is a cuBLAS call and stays one).
//
// ref_quirks = true reproduces what the reference's code does -- the backward pass is seeded with the
// loss VALUE (src/grad/mod.rs:441-447) and the gradient of a broadcast operand is the un-reduced upstream
// re-labelled with the reduced shape, i.e. its first prod(reduced shape) elements
// (src/grad/backwards.rs:527 keeps only the meta of its `sum_at`); false = seed 1 and a true sum.
//
// A tracked tensor is a `Var<T>`: the TensorBase plus the key of the node that produced it (the Rust
// TensorBase carries that key and the gradient cell in its own fields).
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <vector>

#include "rtensors_b200.hpp"

namespace rtb200 {
namespace grad {

using NodeKey = uint64_t;  // 0 = no node (an untracked input)

template <typename T> struct GradCell {  // `Grad` of the reference: where a leaf's gradient accumulates
    bool has = false;
    TensorBase<T> value;
};

template <typename T> struct Var {
    TensorBase<T> t;
    NodeKey op = 0;
    std::shared_ptr<GradCell<T>> grad;  // set for leaves
    Var() = default;
    Var(TensorBase<T> tensor) : t(std::move(tensor)) {}  // an untracked tensor
};

template <typename T> struct GradNode {
    const char *kind = "None";
    std::vector<NodeKey> parents;
    // dL/d(parents) from dL/d(this); `quirks` = the context's ref_quirks
    std::function<std::vector<TensorBase<T>>(const TensorBase<T> &, bool)> backward;
    std::shared_ptr<GradCell<T>> leaf;   // Leaf only
    bool has_loss = false;
    TensorBase<T> loss;                  // L1 only: the value the reference seeds the backward pass with
};

template <typename T> class GradContext {
  public:
    explicit GradContext(bool ref_quirks = false) : ref_quirks(ref_quirks) {}
    const bool ref_quirks;
    std::map<NodeKey, GradNode<T>> nodes;

    NodeKey insert(GradNode<T> n) {
        const NodeKey k = ++next_;
        nodes.emplace(k, std::move(n));
        return k;
    }
    // src/grad/mod.rs:291-305: a node whose parents are all untracked is not put on the tape
    NodeKey attach(GradNode<T> n) {
        bool any = n.parents.empty();
        for (NodeKey &p : n.parents) {
            if (p && !nodes.count(p)) p = 0;
            any = any || p != 0;
        }
        return any ? insert(std::move(n)) : 0;
    }
    // TensorBase::param: the tensor becomes a leaf whose gradient is kept
    void param(Var<T> &v) {
        if (v.op && nodes.count(v.op) && nodes[v.op].leaf) return;
        v.grad = std::make_shared<GradCell<T>>();
        GradNode<T> n;
        n.kind = "Leaf";
        n.leaf = v.grad;
        v.op = insert(std::move(n));
    }
    // iterative depth-first post-order with cycle detection, src/grad/mod.rs:319-360
    std::vector<NodeKey> graph_toposort(NodeKey root) const {
        std::vector<NodeKey> order;
        std::map<NodeKey, bool> marks;
        std::vector<std::pair<bool, NodeKey>> stack{{false, root}};
        while (!stack.empty()) {
            auto [leaving, k] = stack.back();
            stack.pop_back();
            if (leaving) {
                marks[k] = true;
                order.push_back(k);
                continue;
            }
            auto m = marks.find(k);
            if (m != marks.end()) {
                if (m->second) continue;
                throw std::runtime_error("Graph contains a cycle.");
            }
            marks[k] = false;
            stack.push_back({true, k});
            auto it = nodes.find(k);
            if (it == nodes.end()) throw std::runtime_error("Node not found during backward pass.");
            for (NodeKey p : it->second.parents)
                if (p) stack.push_back({false, p});
        }
        return order;
    }
    // src/grad/mod.rs:432-495
    void backwards(const Var<T> &root) {
        auto rit = nodes.find(root.op);
        if (!root.op || rit == nodes.end()) throw std::runtime_error("Root node must have an associated GradNode.");
        if (!rit->second.has_loss) throw std::runtime_error("Root node does not contain a loss.");
        const std::vector<NodeKey> order = graph_toposort(root.op);
        const TensorBase<T> &loss = rit->second.loss;
        std::map<NodeKey, std::vector<TensorBase<T>>> acc;
        acc[root.op].push_back(ref_quirks ? loss.owned() : TensorBase<T>::full(*loss.backend, loss.shape(), T(1)));
        for (auto k = order.rbegin(); k != order.rend(); ++k) {
            std::vector<TensorBase<T>> ups = std::move(acc[*k]);
            acc.erase(*k);
            TensorBase<T> dldy = ups.at(0);
            for (size_t i = 1; i < ups.size(); ++i) dldy = dldy + ups[i];
            GradNode<T> &node = nodes.at(*k);
            if (node.leaf) {  // accumulate_grad, src/grad/backwards.rs:7-25
                if (node.leaf->has) node.leaf->value += dldy;
                else { node.leaf->value = dldy.owned(); node.leaf->has = true; }
                continue;
            }
            std::vector<TensorBase<T>> grads = node.backward(dldy, ref_quirks);
            for (size_t i = 0; i < node.parents.size() && i < grads.size(); ++i)
                if (node.parents[i]) acc[node.parents[i]].push_back(grads[i]);
            nodes.erase(*k);  // consumed
        }
    }

  private:
    NodeKey next_ = 0;
};

// src/grad/backwards.rs:512-538: collapse the upstream over the dims the operand was broadcast along,
// then squeeze the dims the operand did not have
template <typename T>
TensorBase<T> inverse_broadcast_gradient(const TensorBase<T> &grad, const std::vector<ptrdiff_t> &strides,
                                         const std::vector<size_t> &shape, bool quirks) {
    bool any = false;
    for (ptrdiff_t s : strides) any = any || s == 0;
    if (!any) return grad;
    TensorBase<T> g = (grad.is_contiguous() && grad.offset() == 0) ? grad : grad.contiguous();
    std::vector<size_t> oshape(g.shape().size());
    for (size_t d = 0; d < oshape.size(); ++d) oshape[d] = strides[d] == 0 ? 1 : g.shape()[d];
    TensorBase<T> out;
    if (quirks) {
        out = g.view_of(MetaTensor::contiguous(oshape));  // the un-reduced buffer under the reduced meta
    } else {
        MetaTensor om = MetaTensor::contiguous(oshape);
        out = TensorBase<T>{g.backend, g.backend->template alloc<T>(om.size()), om};
        std::vector<size_t> got(oshape.size() ? oshape.size() : 1);
        check(rtb_reduce_to_shape(g.backend->ctx(), DTypeOf<T>::value, g.buf->ptr, g.shape().size(), g.shape().data(), strides.data(),
                                  out.buf->ptr, got.data()));
    }
    const size_t diff = strides.size() - shape.size();
    std::vector<size_t> keep_shape;
    std::vector<ptrdiff_t> keep_strides;
    for (size_t d = 0; d < strides.size(); ++d) {
        const bool squeeze = strides[d] == 0 && (d < diff || shape[d - diff] != 1);
        if (!squeeze) { keep_shape.push_back(out.meta.shape[d]); keep_strides.push_back(out.meta.strides[d]); }
    }
    return out.view_of(MetaTensor{keep_shape, keep_strides, out.meta.offset});
}

// ---- tracked operators ---------------------------------------------------------------------------
template <typename T> Var<T> broadcast_op(GradContext<T> &ctx, const Var<T> &a, const Var<T> &b, BinaryOpType op) {
    Var<T> out{a.t.binary(b.t, op)};
    std::vector<size_t> shape;
    std::vector<ptrdiff_t> sa, sb;
    broadcast_params(a.t.meta, b.t.meta, shape, sa, sb);
    const std::vector<size_t> sha = a.t.shape(), shb = b.t.shape();
    GradNode<T> n;
    n.parents = {a.op, b.op};
    const TensorBase<T> ta = a.t, tb = b.t;
    if (op == BinaryOpType::Add) {
        n.kind = "BroadcastAdd";
        n.backward = [=](const TensorBase<T> &up, bool q) {
            return std::vector<TensorBase<T>>{inverse_broadcast_gradient(up, sa, sha, q), inverse_broadcast_gradient(up, sb, shb, q)};
        };
    } else if (op == BinaryOpType::Sub) {
        n.kind = "BroadcastSub";
        n.backward = [=](const TensorBase<T> &up, bool q) {
            return std::vector<TensorBase<T>>{inverse_broadcast_gradient(up, sa, sha, q), inverse_broadcast_gradient(up.neg(), sb, shb, q)};
        };
    } else if (op == BinaryOpType::Mul) {
        n.kind = "BroadcastMul";
        n.backward = [=](const TensorBase<T> &up, bool q) {
            return std::vector<TensorBase<T>>{inverse_broadcast_gradient(up * tb, sa, sha, q), inverse_broadcast_gradient(up * ta, sb, shb, q)};
        };
    } else {
        throw std::runtime_error("division is not on the C++ tape");
    }
    out.op = ctx.attach(std::move(n));
    return out;
}
template <typename T> Var<T> add(GradContext<T> &c, const Var<T> &a, const Var<T> &b) { return broadcast_op(c, a, b, BinaryOpType::Add); }
template <typename T> Var<T> sub(GradContext<T> &c, const Var<T> &a, const Var<T> &b) { return broadcast_op(c, a, b, BinaryOpType::Sub); }
template <typename T> Var<T> mul(GradContext<T> &c, const Var<T> &a, const Var<T> &b) { return broadcast_op(c, a, b, BinaryOpType::Mul); }

template <typename T> Var<T> add_scalar(GradContext<T> &ctx, const Var<T> &a, T v) {
    Var<T> out{a.t + v};
    GradNode<T> n;
    n.kind = "AddScalar";
    n.parents = {a.op};
    n.backward = [](const TensorBase<T> &up, bool) { return std::vector<TensorBase<T>>{up}; };
    out.op = ctx.attach(std::move(n));
    return out;
}
template <typename T> Var<T> mul_scalar(GradContext<T> &ctx, const Var<T> &a, T v) {
    Var<T> out{a.t * v};
    GradNode<T> n;
    n.kind = "MulScalar";
    n.parents = {a.op};
    n.backward = [v](const TensorBase<T> &up, bool) { return std::vector<TensorBase<T>>{up * v}; };
    out.op = ctx.attach(std::move(n));
    return out;
}
// relu / abs keep the gradient map of their INPUT (one kernel; the reference fills it element by element)
template <typename T> Var<T> relu(GradContext<T> &ctx, const Var<T> &a) {
    Var<T> out{a.t.relu()};
    const TensorBase<T> map = a.t.relu_grad_map();
    GradNode<T> n;
    n.kind = "ReLU";
    n.parents = {a.op};
    n.backward = [map](const TensorBase<T> &up, bool) { return std::vector<TensorBase<T>>{map * up}; };
    out.op = ctx.attach(std::move(n));
    return out;
}
template <typename T> Var<T> abs(GradContext<T> &ctx, const Var<T> &a) {
    Var<T> out{a.t.abs()};
    const TensorBase<T> map = a.t.abs_grad_map();
    GradNode<T> n;
    n.kind = "Abs";
    n.parents = {a.op};
    n.backward = [map](const TensorBase<T> &up, bool) { return std::vector<TensorBase<T>>{map * up}; };
    out.op = ctx.attach(std::move(n));
    return out;
}
template <typename T> Var<T> neg(GradContext<T> &ctx, const Var<T> &a) {
    Var<T> out{a.t.neg()};
    GradNode<T> n;
    n.kind = "Negate";
    n.parents = {a.op};
    n.backward = [](const TensorBase<T> &up, bool) { return std::vector<TensorBase<T>>{up.neg()}; };
    out.op = ctx.attach(std::move(n));
    return out;
}
template <typename T> Var<T> permute(GradContext<T> &ctx, const Var<T> &a, const std::vector<size_t> &dims) {
    Var<T> out{a.t.permute(dims)};
    std::vector<size_t> inverse(dims.size());
    for (size_t i = 0; i < dims.size(); ++i) inverse[dims[i]] = i;
    GradNode<T> n;
    n.kind = "Permute";
    n.parents = {a.op};
    n.backward = [inverse](const TensorBase<T> &up, bool) { return std::vector<TensorBase<T>>{up.permute(inverse)}; };
    out.op = ctx.attach(std::move(n));
    return out;
}
// mean_l1_loss with its gradient map sign(a - b) / N from one fused kernel (attach_l1_grad, src/ops/broadcast/l1.rs:16-46)
template <typename T> Var<T> mean_l1_loss(GradContext<T> &ctx, const Var<T> &a, const Var<T> &b) {
    if (a.t.shape() != b.t.shape()) throw TensorError(RTB_ERR_SHAPE, "mean_l1_loss needs equal shapes");
    const TensorBase<T> ca = a.t.is_contiguous() ? a.t : a.t.contiguous(), cb = b.t.is_contiguous() ? b.t : b.t.contiguous();
    const Cuda *be = a.t.backend;
    TensorBase<T> loss{be, be->template alloc<T>(1), MetaTensor::contiguous({})};
    TensorBase<T> map{be, be->template alloc<T>(ca.size()), MetaTensor::contiguous(a.t.shape())};
    check(rtb_l1_loss(be->ctx(), DTypeOf<T>::value, ca.buf->ptr + ca.meta.offset, cb.buf->ptr + cb.meta.offset, ca.size(), 0, loss.buf->ptr,
                      map.buf->ptr));
    Var<T> out{loss};
    GradNode<T> n;
    n.kind = "L1";
    n.parents = {a.op, b.op};
    n.has_loss = true;
    n.loss = loss;
    n.backward = [map](const TensorBase<T> &up, bool) { return std::vector<TensorBase<T>>{map * up, map.neg() * up}; };  // backwards.rs:148-161
    out.op = ctx.attach(std::move(n));
    return out;
}

// src/grad/optim.rs:14-64
template <typename T> class SGD {
  public:
    explicit SGD(T learning_rate) : learning_rate_(learning_rate) {}
    void register_parameter(GradContext<T> &ctx, Var<T> &p) {
        ctx.param(p);
        params_.push_back(&p);
    }
    void step() {
        for (Var<T> *p : params_) {
            if (!p->grad || !p->grad->has) continue;
            TensorBase<T> update = p->grad->value * learning_rate_;  // owned copy + scalar multiply: one rounding
            p->grad->has = false;
            p->t -= update;                                          // in-place broadcast subtract: the second rounding
        }
    }

  private:
    T learning_rate_;
    std::vector<Var<T> *> params_;
};

}  // namespace grad
}  // namespace rtb200
