"""One autograd SGD step of the dense MLP (784 -> 1024 -> 1024 -> 10, ReLU, mean_l1_loss, SGD), the
way the reference's tape computes it (examples/mnist/src/main.rs:17-46 for the model,
src/grad/mod.rs:432-495 and src/grad/backwards.rs for the backward pass, src/grad/optim.rs:30-50 for
the update), with every non-GEMM op on this library's kernels:

  u8 -> f32 / 255            rtb_u8_to_f32_div
  x @ W                      cuBLAS through torch.matmul (matmul stays on cuBLAS by design)
  + bias (1,out) in place    rtb_broadcast, in-place form
  relu + gradient mask       rtb_relu_mask_f32          (reference: per-element get/set loop)
  mean_l1_loss + grad map    rtb_l1_loss                 (reference: 5 launches, 2 temporaries)
  grad_map * seed            rtb_scalar_op (scalar multiply in place)
  mask * upstream            rtb_broadcast (same-shape multiply, in place)
  bias gradient              rtb_reduce_to_shape         (column sum of the upstream)
  p -= g * lr                rtb_sgd_update_f32 over one flat parameter buffer

Two modes.  intended: backward seed 1 and the bias gradient is the batch sum.  ref_quirks: the
reference's observable behaviour -- the seed is the loss VALUE (src/grad/mod.rs:441-447) and the
bias "gradient" is row 0 of the upstream (src/grad/backwards.rs:527 keeps only the meta of the sum).

Data parallel: each rank holds batch/world rows; the loss partial sums are all-reduced (the seed
needs the global loss in ref_quirks mode), gradients live in ONE flat bucket that is all-reduced
once, and every rank applies the same update.  Parameters live in one flat buffer with the same
layout as the bucket.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from . import _lib as L
from .backend import CudaB200
from .meta import Meta


class DenseMlp:
    def __init__(self, be: CudaB200, sizes: Sequence[int] = (784, 1024, 1024, 10), lr: float = 0.01,
                 ref_quirks: bool = False, seed: int = 0x5EED + 5):
        self.be, self.sizes, self.lr, self.ref_quirks = be, tuple(sizes), float(lr), ref_quirks
        dev = f"cuda:{be.device}"
        self.shapes = []
        for fi, fo in zip(sizes[:-1], sizes[1:]):
            self.shapes += [(fi, fo), (1, fo)]
        # 16-byte aligned segments so every view is vector-aligned
        self.offsets, total = [], 0
        for shp in self.shapes:
            self.offsets.append(total)
            total += (shp[0] * shp[1] + 3) // 4 * 4
        self.n_flat = total
        self.params = torch.zeros(total, device=dev, dtype=torch.float32)
        self.grads = torch.zeros(total, device=dev, dtype=torch.float32)
        rng = np.random.default_rng(seed)
        for k, (shp, off) in enumerate(zip(self.shapes, self.offsets)):
            if k % 2 == 0:  # weight: uniform +-1/sqrt(fan_in); biases stay zero
                bound = 1.0 / np.sqrt(shp[0])
                w = rng.uniform(-bound, bound, shp[0] * shp[1]).astype(np.float32)
                self.params[off: off + w.size] = torch.from_numpy(w).to(dev)

    def _view(self, flat: torch.Tensor, k: int) -> torch.Tensor:
        shp, off = self.shapes[k], self.offsets[k]
        return flat[off: off + shp[0] * shp[1]].view(shp)

    def weight(self, layer: int): return self._view(self.params, 2 * layer)
    def bias(self, layer: int): return self._view(self.params, 2 * layer + 1)
    def grad_weight(self, layer: int): return self._view(self.grads, 2 * layer)
    def grad_bias(self, layer: int): return self._view(self.grads, 2 * layer + 1)

    def host_params(self) -> List[np.ndarray]:
        return [self._view(self.params, k).detach().cpu().numpy().copy() for k in range(len(self.shapes))]

    def load_params(self, arrays: Sequence[np.ndarray]):
        for k, a in enumerate(arrays):
            self._view(self.params, k).copy_(torch.from_numpy(np.ascontiguousarray(a)).view(self.shapes[k]))

    # ------------------------------------------------------------------------------------------
    def step(self, images_u8: torch.Tensor, targets: torch.Tensor, global_batch: Optional[int] = None):
        """images_u8: (b, 784) uint8 on the device; targets: (b, 10) f32.  Returns the (global) loss
        as a 1-element device tensor.  b is this rank's share of global_batch."""
        be = self.be
        world = dist.get_world_size() if dist.is_initialized() else 1
        b = images_u8.shape[0]
        gb = global_batch or b * world
        n_layers = len(self.sizes) - 1
        x = be.u8_to_f32_div(images_u8.reshape(-1), 255.0).view(b, self.sizes[0])
        acts, masks = [x], []
        h = x
        for li in range(n_layers):
            z = torch.matmul(h, self.weight(li))              # cuBLAS
            fo = self.sizes[li + 1]
            be.binary_assign(z.view(-1), Meta.contiguous((b, fo)), self.bias(li).view(-1), Meta.contiguous((1, fo)), L.ADD)
            if li != n_layers - 1:
                masks.append(be.relu_mask(z.view(-1)).view(b, fo))
            acts.append(z)
            h = z
        out = acts[-1]
        n_out = self.sizes[-1]
        # loss: local sum of |out - target| and the map sign(out - target); both scaled by N_global
        lsum, gmap = be.l1_loss(out.view(-1), targets.reshape(-1), 1, True)
        if world > 1:
            dist.all_reduce(lsum, op=dist.ReduceOp.SUM)
        n_global = np.float32(gb * n_out)
        loss = lsum / float(n_global)                                   # mean = sum / (f32)N
        m_all = Meta.contiguous((gmap.numel(),))
        be.scalar_apply(gmap, L.DIV, float(n_global), m_all)            # grad_map = sign / N
        if self.ref_quirks:
            be.scalar_apply(gmap, L.MUL, float(loss.item()), m_all)     # seed = the loss value
        up = gmap.view(b, n_out)
        for li in reversed(range(n_layers)):
            fo = self.sizes[li + 1]
            a_in = acts[li]
            torch.matmul(a_in.t(), up, out=self.grad_weight(li))        # dW = x^T . U   (cuBLAS)
            gb_view = self.grad_bias(li).view(-1)
            if self.ref_quirks:
                rank = dist.get_rank() if dist.is_initialized() else 0
                if rank == 0:
                    gb_view.copy_(up[0])                                # row 0 of the upstream
                else:
                    gb_view.zero_()
            else:
                red, _ = be.reduce_to_shape(up.reshape(-1), (b, fo), (0, 1))
                gb_view.copy_(red[:fo])
            if li > 0:
                dh = torch.matmul(up, self.weight(li).t())              # dx = U . W^T   (cuBLAS)
                fi = self.sizes[li]
                mm = Meta.contiguous((b * fi,))
                be.broadcast((dh.view(-1), mm), (masks[li - 1].view(-1), mm), (dh.view(-1), mm), L.MUL)
                up = dh
        if world > 1:
            dist.all_reduce(self.grads, op=dist.ReduceOp.SUM)           # one flat bucket
        be.sgd_update(self.params, self.grads, self.lr)
        return loss


    # ------------------------------------------------------------------------------------------
    def step_graphed(self, images_u8: torch.Tensor, targets: torch.Tensor, global_batch: Optional[int] = None):
        """The same step replayed from a CUDA graph: about thirty launches (library kernels and
        cuBLAS GEMMs) become one graph launch.  The first call for a batch shape runs the step eagerly
        (that sizes the library's workspace and allocator cache) and records the graph; later calls
        copy the inputs into the graph's static buffers and replay it.  Single-GPU, intended-semantics
        mode only -- with several ranks or the reference-quirks seed (which reads the loss back to the
        host) it falls through to step()."""
        world = dist.get_world_size() if dist.is_initialized() else 1
        if world > 1 or self.ref_quirks:
            return self.step(images_u8, targets, global_batch)
        key = (tuple(images_u8.shape), tuple(targets.shape), global_batch)
        if getattr(self, "_graph_key", None) != key:
            loss = self.step(images_u8, targets, global_batch)
            self._g_img, self._g_tgt = images_u8.clone(), targets.clone()
            be = self.be
            cur = torch.cuda.current_stream(be.device)
            side = torch.cuda.Stream(device=f"cuda:{be.device}")
            side.wait_stream(cur)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    be.sync_stream()
                    self._g_loss = self.step(self._g_img, self._g_tgt, global_batch)
            cur.wait_stream(side)
            be.sync_stream()
            self._graph, self._graph_key = graph, key
            return loss
        self._g_img.copy_(images_u8, non_blocking=True)
        self._g_tgt.copy_(targets, non_blocking=True)
        self._graph.replay()
        return self._g_loss


def synthetic_batch(batch: int, device: str, seed: int = 0x5EED + 50, rank: int = 0):
    """Seeded stand-in for MNIST-shaped data: u8 pixels uniform[0,255], one-hot targets."""
    rng = np.random.default_rng(seed + rank)
    img = rng.integers(0, 256, (batch, 784), dtype=np.uint8)
    lab = rng.integers(0, 10, batch)
    tgt = np.zeros((batch, 10), dtype=np.float32)
    tgt[np.arange(batch), lab] = 1.0
    return torch.from_numpy(img).to(device), torch.from_numpy(tgt).to(device), img, tgt
