"""The dense-MLP SGD step composed from the CPU oracle's pieces (test infrastructure).  GEMMs use
the oracle's f64-accumulating GEMM in place of OpenBLAS; everything else is the restated CPU
backend.  Data flow and quirks: the docstring of rtensors_b200/mlp.py."""
import numpy as np

import oracle as O


def mlp_step(params, sizes, img_u8, targets, lr, ref_quirks):
    """params: list [W1, b1, W2, b2, ...] of float32 arrays (updated copies are returned).
    -> (loss, new_params, grads)"""
    b = img_u8.shape[0]
    n_layers = len(sizes) - 1
    x = O.u8_to_f32_div(img_u8.reshape(-1), 255.0)
    acts, masks = [x], []
    h = x
    for li in range(n_layers):
        fi, fo = sizes[li], sizes[li + 1]
        z = O.gemm(h, params[2 * li].reshape(-1), b, fi, fo)
        zm = O.Meta.contiguous((b, fo))
        shape, sa, sb = O.broadcast_params(zm, O.Meta.contiguous((1, fo)))
        O.broadcast(z, O.Meta(shape, sa, 0), params[2 * li + 1].reshape(-1), O.Meta(shape, sb, 0), z, O.Meta(shape, sa, 0), O.ADD)
        if li != n_layers - 1:
            masks.append(O.relu_mask(z))
        acts.append(z)
        h = z
    out = acts[-1]
    n_out = sizes[-1]
    loss, gmap = O.l1_loss(out, targets.reshape(-1).astype(np.float32), 0, True)  # gmap = sign/N
    if ref_quirks:
        O.scalar_op(gmap, O.MUL, loss[0], O.Meta.contiguous((gmap.size,)))
    up = gmap
    grads = [None] * (2 * n_layers)
    for li in reversed(range(n_layers)):
        fi, fo = sizes[li], sizes[li + 1]
        grads[2 * li] = O.gemm(acts[li], up, fi, b, fo, ta=True)           # x^T . U
        if ref_quirks:
            grads[2 * li + 1] = up[:fo].copy()
        else:
            grads[2 * li + 1], _ = O.reduce_to_shape(up, (b, fo), (0, 1), intended=True)
        if li > 0:
            dh = O.gemm(up, params[2 * li].reshape(-1), b, fo, fi, tb=True)  # U . W^T
            m = O.Meta.contiguous((dh.size,))
            O.broadcast(dh, m, masks[li - 1], m, dh, m, O.MUL)
            up = dh
    new_params = []
    for p, g in zip(params, grads):
        q = p.reshape(-1).copy()
        O.sgd_update(q, g.reshape(-1), lr)
        new_params.append(q.reshape(p.shape))
    return float(loss[0]), new_params, grads
