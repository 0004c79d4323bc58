"""One autograd SGD step of the dense MLP (784 -> 1024 -> 1024 -> 10, ReLU, mean_l1_loss, SGD), the
way the reference's tape computes it (examples/mnist/src/main.rs:17-46 for the model,
src/grad/mod.rs:432-495 and src/grad/backwards.rs for the backward pass, src/grad/optim.rs:30-50 for
the update), with every non-GEMM op on this library's kernels:

  u8 -> f32 / 255              rtb_u8_to_f32_div
  x @ W                        cuBLAS through torch.matmul (matmul stays on cuBLAS by design)
  + bias, relu, gradient mask  rtb_bias_relu_mask, ONE pass (reference: broadcast add, relu, and a
                               per-element get/set loop for the mask); the last layer's plain
                               `+ bias` is rtb_broadcast in place
  mean_l1_loss + grad map      rtb_l1_loss / rtb_mg_l1_loss (reference: 5 launches, 2 temporaries)
  grad_map * seed              rtb_broadcast with the rank-0 loss tensor as right operand (no host
                               read of the loss), as backwards_l1 does (src/grad/backwards.rs:148-161)
  mask * upstream              rtb_broadcast (same-shape multiply, in place)
  bias gradient                rtb_reduce_to_shape, written straight into the gradient bucket
  p -= g * lr                  rtb_sgd_update_f32 over one flat parameter buffer

This class is the fused, fixed-graph form of the step; `rtensors_b200.grad` runs the same step
through a tape with the reference's node types, and the two agree bit for bit.

Two modes.  intended: backward seed 1 and the bias gradient is the batch sum.  ref_quirks: the
reference's observable behaviour -- the seed is the loss VALUE (src/grad/mod.rs:441-447) and the
bias "gradient" is row 0 of the upstream (src/grad/backwards.rs:527 keeps only the meta of the sum).

Data parallel (the engine owns a communicator, `CudaB200.mg_init`): each rank holds batch/world
rows; the loss is combined inside the L1 kernel's last CTA over peer memory (the seed needs the
global loss in ref_quirks mode); every layer's gradients (dW, db -- adjacent in the flat bucket) are
all-reduced with NCCL on the communicator's side stream as soon as they exist, overlapping the
next layer's backward GEMMs; every rank applies the same update.  The whole step, collectives
included, can be captured in a CUDA graph (`step_graphed`).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib as L
from ._lib import lib
from .backend import CudaB200
from .meta import Meta


class DenseMlp:
    def __init__(self, be: CudaB200, sizes: Sequence[int] = (784, 1024, 1024, 10), lr: float = 0.01,
                 ref_quirks: bool = False, seed: int = 0x5EED + 5):
        self.be, self.sizes, self.lr, self.ref_quirks = be, tuple(sizes), float(lr), ref_quirks
        # any engine with the Backend-mirror methods this class calls works (the CPU tests drive the
        # same step logic through an engine made of the oracle's pieces); CudaB200 is the product's
        dev = getattr(be, "torch_device", None) or f"cuda:{be.device}"
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

    def layer_bucket(self, layer: int) -> torch.Tensor:
        """dW and db of one layer: adjacent in the flat gradient buffer, all-reduced as one message."""
        lo = self.offsets[2 * layer]
        hi = self.offsets[2 * layer + 2] if 2 * layer + 2 < len(self.offsets) else self.n_flat
        return self.grads[lo:hi]

    def host_params(self) -> List[np.ndarray]:
        return [self._view(self.params, k).detach().cpu().numpy().copy() for k in range(len(self.shapes))]

    def load_params(self, arrays: Sequence[np.ndarray]):
        for k, a in enumerate(arrays):
            self._view(self.params, k).copy_(torch.from_numpy(np.ascontiguousarray(a)).view(self.shapes[k]))

    # ------------------------------------------------------------------------------------------
    def step(self, images_u8: torch.Tensor, targets: torch.Tensor, global_batch: Optional[int] = None):
        """images_u8: (b, 784) uint8 on the device; targets: (b, 10) f32.  Returns the (global) loss
        as a 1-element device tensor.  b is this rank's share of global_batch.  Nothing in the step
        reads the device from the host."""
        be = self.be
        world, rank = be.mg_world, be.mg_rank
        b = images_u8.shape[0]
        gb = global_batch or b * world
        n_layers = len(self.sizes) - 1
        x = be.u8_to_f32_div(images_u8.reshape(-1), 255.0).view(b, self.sizes[0])
        acts, masks = [x], []
        h = x
        for li in range(n_layers):
            z = torch.matmul(h, self.weight(li))              # cuBLAS
            fo = self.sizes[li + 1]
            if li != n_layers - 1:
                masks.append(be.bias_relu_mask(z.view(-1), self.bias(li).view(-1), b, fo).view(b, fo))
            else:
                be.binary_assign(z.view(-1), Meta.contiguous((b, fo)), self.bias(li).view(-1), Meta.contiguous((1, fo)), L.ADD)
            acts.append(z)
            h = z
        out = acts[-1]
        n_out = self.sizes[-1]
        # loss = sum |out - target| / (f32)N over the GLOBAL batch, map = sign(out - target) / (f32)N
        if world > 1:
            loss, gmap = be.mg_l1_loss(out.view(-1), targets.reshape(-1), gb * n_out, 0, True)
        else:
            loss, gmap = be.l1_loss(out.view(-1), targets.reshape(-1), 0, True)
        if self.ref_quirks:                                             # seed = the loss value
            shp = (gmap.numel(),)
            mg_ = Meta.contiguous(shp)
            be.broadcast((gmap, mg_), (loss, Meta(shp, (0,), 0)), (gmap, mg_), L.MUL)
        up = gmap.view(b, n_out)
        for li in reversed(range(n_layers)):
            fo = self.sizes[li + 1]
            a_in = acts[li]
            torch.matmul(a_in.t(), up, out=self.grad_weight(li))        # dW = x^T . U   (cuBLAS)
            gb_view = self.grad_bias(li).view(-1)
            if self.ref_quirks:
                if rank == 0:
                    gb_view.copy_(up[0])                                # row 0 of the (global) upstream
                else:
                    gb_view.zero_()
            else:
                be.reduce_to_shape(up.reshape(-1), (b, fo), (0, 1), out=gb_view)
            if world > 1:                                               # this layer's bucket, overlapped
                be.mg_allreduce(self.layer_bucket(li), L.SUM, overlap=True)
            if li > 0:
                dh = torch.matmul(up, self.weight(li).t())              # dx = U . W^T   (cuBLAS)
                fi = self.sizes[li]
                mm = Meta.contiguous((b * fi,))
                be.broadcast((dh.view(-1), mm), (masks[li - 1].view(-1), mm), (dh.view(-1), mm), L.MUL)
                up = dh
        if world > 1:
            be.mg_allreduce_join()
        be.sgd_update(self.params, self.grads, self.lr)
        return loss

    # ------------------------------------------------------------------------------------------
    def step_graphed(self, images_u8: torch.Tensor, targets: torch.Tensor, global_batch: Optional[int] = None):
        """The same step replayed from a CUDA graph: about thirty launches (library kernels, cuBLAS
        GEMMs and, with several ranks, the peer exchange and the NCCL all-reduces) become one graph
        launch.  The first call for a batch shape runs the step eagerly (that sizes the library's
        workspace and allocator cache) and records the graph; later calls copy the inputs into the
        graph's static buffers and replay it.  The graph is recorded again when the library reports
        that device memory it may hold has moved (rtb_ctx_workspace_generation)."""
        be = self.be
        key = (tuple(images_u8.shape), tuple(targets.shape), global_batch)
        gen = int(lib().rtb_ctx_workspace_generation(be._ctx))
        if getattr(self, "_graph_key", None) != key or getattr(self, "_graph_gen", None) != gen:
            loss = self.step(images_u8, targets, global_batch)
            self._g_img, self._g_tgt = images_u8.clone(), targets.clone()
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
            self._graph_gen = int(lib().rtb_ctx_workspace_generation(be._ctx))
            # the capture ran no kernel: the eager step above is this call's step
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


def tape_step(be: CudaB200, params, images_u8: torch.Tensor, targets: torch.Tensor, lr: float, ref_quirks: bool):
    """The same SGD step written the way a user of the reference writes it -- tensors, operators,
    `grad.enabled`, `ctx.backwards(loss)`, `SGD.step` (examples/mnist/src/main.rs:17-46) -- on the
    tape of rtensors_b200.grad.  params: [W1, b1, W2, b2, ...] as Tensors, updated in place.
    -> loss Tensor (rank 0)."""
    from . import grad
    from .tensor import Tensor, mean_l1_loss_tracked
    b = images_u8.shape[0]
    with grad.enabled(ref_quirks=ref_quirks) as ctx:
        opt = grad.SGD(lr)
        opt.register_parameters(params)
        x = Tensor(be, be.u8_to_f32_div(images_u8.reshape(-1), 255.0), Meta.contiguous((b, images_u8.shape[1])))
        t = Tensor(be, targets.reshape(-1), Meta.contiguous(tuple(targets.shape)))
        h = x
        n_layers = len(params) // 2
        for li in range(n_layers):
            h = h.matmul(params[2 * li]) + params[2 * li + 1]
            if li != n_layers - 1:
                h = h.relu()
        loss = mean_l1_loss_tracked(h, t)
        ctx.backwards(loss)
        opt.step()
    return loss
