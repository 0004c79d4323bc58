"""Host-buffer front end: hot-path work whose inputs and outputs live in pinned HOST memory, over the
library's own host-buffer operations (`rtb_host_*`: an upload lane, a download lane and a pool of device
blocks inside the context, ordered by events).  A tensor's upload, the kernels and the copy-out of the
results of neighbouring pieces overlap (PCIe is full duplex) -- the reference does the same transfers
whole-tensor and synchronously (`alloc_from_slice` / `dump`, src/backend/cuda.rs:668-680, 770-788).
This module only cuts the work into pieces; every transfer and every wait is a library call.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

import torch

from .backend import CudaB200
from .meta import Meta


class HostPipeline:
    def __init__(self, be: CudaB200, chunk_elems: int = 1 << 24):
        self.be = be
        self.chunk = int(chunk_elems)

    def run(self, n: int, inputs: Dict[str, torch.Tensor], outputs: Dict[str, Tuple[torch.Tensor, torch.dtype]],
            compute: Callable[[Dict[str, torch.Tensor], int], None]):
        """Flat elementwise work over n elements, chunk by chunk.  inputs: name -> pinned host tensor;
        outputs: name -> (pinned host tensor, dtype).  An output named like an input is that input's
        block after the kernels ran (in-place work); any other output gets a block of its own.
        compute(blocks, length) enqueues the kernels for one chunk on the context's stream.  Chunk k's
        copy-out and chunk k+1's upload run while chunk k+1's / k's kernels do.  Returns after
        enqueueing; `be.host_wait()` (or `be.sync()`) completes it."""
        be = self.be
        be.sync_stream()
        for lo in range(0, n, self.chunk):
            hi = min(lo + self.chunk, n)
            blocks = {k: be.host_stage_in(h[lo:hi]) for k, h in inputs.items()}
            for k, (h, dtype) in outputs.items():
                if k not in blocks:
                    blocks[k] = be.host_scratch(hi - lo, dtype)
            for k in inputs:
                be.host_ready(blocks[k])
            compute(blocks, hi - lo)
            for k, (h, _) in outputs.items():
                be.host_stage_out(blocks[k], h[lo:hi])
            for b in blocks.values():
                be.host_release(b)

    def broadcast_to_host(self, a_host: torch.Tensor, am: Meta, b_host: torch.Tensor, bm: Meta, op: int,
                          out_host: torch.Tensor, dim_range: Optional[tuple] = None):
        """`a op b` with operand buffers in pinned host memory and the result written to out_host
        (row-major over this call's part of the output: dim_range = (begin, end) of the outermost
        output dim, a rank's share).  One library call (rtb_host_broadcast): the output is produced in
        stages into a ring of device blocks, a stage's copy-out running behind the next stage's kernel.
        Enqueues only."""
        self.be.sync_stream()
        self.be.host_broadcast(a_host, am, b_host, bm, op, out_host, dim_range)

    def reduce_to_host(self, host: torch.Tensor, meta: Meta, axis: Optional[int], op: int, out_host: torch.Tensor, **settings):
        """Reduction of a host tensor into out_host (rtb_host_reduce_view).  Enqueues only: the upload
        runs on the upload lane while whatever was enqueued before keeps the other lanes busy."""
        self.be.sync_stream()
        self.be.host_reduce_view(host, meta, axis, op, out_host, **settings)
