"""Host-buffer front end: run hot-path work whose inputs and outputs live in pinned HOST memory.
Tensors are cut into chunks along the outermost dimension; a chunk's host->device copy, its kernels
and its device->host copy run on three streams, so the copies of neighbouring chunks overlap the
kernels and each other (PCIe is full duplex).  This is what a caller uses when the data does not
fit, or does not live, on the device -- the reference does the same transfers whole-tensor and
synchronously (`alloc_from_slice` / `dump`, src/backend/cuda.rs:668-680, 770-788).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence

import torch

from . import _lib as L
from .backend import CudaB200
from .meta import Meta, broadcast_params, shard_range


class HostPipeline:
    def __init__(self, be: CudaB200, chunk_elems: int = 1 << 24):
        self.be = be
        self.chunk = int(chunk_elems)
        dev = f"cuda:{be.device}"
        self.s_in = torch.cuda.Stream(device=dev)
        self.s_run = torch.cuda.Stream(device=dev)
        self.s_out = torch.cuda.Stream(device=dev)

    def run(self, n: int, inputs: Dict[str, tuple], outputs: Dict[str, tuple],
            compute: Callable[[Dict[str, torch.Tensor], int], None]):
        """inputs / outputs: name -> (pinned host tensor, device tensor), all of n elements.
        compute(dev_chunks, length) enqueues the kernels for one chunk on the current stream; it
        gets chunk views of every device tensor by name."""
        be = self.be
        cur = torch.cuda.current_stream(be.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        for lo in range(0, n, self.chunk):
            hi = min(lo + self.chunk, n)
            ev_in, ev_run = torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(self.s_in):
                for host, dev in inputs.values():
                    dev[lo:hi].copy_(host[lo:hi], non_blocking=True)
                ev_in.record()
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(ev_in)
                be.sync_stream()
                views = {k: d[lo:hi] for k, (_, d) in {**inputs, **outputs}.items()}
                compute(views, hi - lo)
                ev_run.record()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_run)
                for host, dev in outputs.values():
                    host[lo:hi].copy_(dev[lo:hi], non_blocking=True)
        for s in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(s)
        be.sync_stream()

    # ---- out-of-place broadcast op whose (large) result goes to the host ------------------------
    def broadcast_to_host(self, a_host: torch.Tensor, am: Meta, b_host: torch.Tensor, bm: Meta, op: int,
                          out_host: torch.Tensor, staging: Sequence[torch.Tensor], a_dev: torch.Tensor, b_dev: torch.Tensor,
                          dim_range: Optional[tuple] = None):
        """`a op b` with operand buffers in pinned host memory and the result written to out_host
        (row-major over this call's part of the output).  The output is produced one outermost-dim
        slab at a time into a ring of device staging buffers; slab k's device->host copy overlaps
        slab k+1's kernel.  dim_range = (begin, end) restricts the call to a range of the outermost
        output dim (a rank's share).  Enqueues only; the caller synchronises."""
        be = self.be
        shape, sa, sb = broadcast_params(am, bm)
        lo, hi = dim_range if dim_range is not None else (0, shape[0])
        per = 1
        for n in shape[1:]:
            per *= n
        cur = torch.cuda.current_stream(be.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            a_dev.copy_(a_host, non_blocking=True)
            b_dev.copy_(b_host, non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record()
        sshape = (1,) + tuple(shape[1:])
        dm = Meta.contiguous(sshape)
        free_ev = [None] * len(staging)
        for k, i in enumerate(range(lo, hi)):
            st = staging[k % len(staging)]
            with torch.cuda.stream(self.s_run):
                if k == 0:
                    self.s_run.wait_event(ev_in)
                if free_ev[k % len(staging)] is not None:
                    self.s_run.wait_event(free_ev[k % len(staging)])   # the slab's previous copy-out is done
                be.sync_stream()
                be.broadcast((a_dev, Meta(sshape, sa, am.offset + i * sa[0])), (b_dev, Meta(sshape, sb, bm.offset + i * sb[0])),
                             (st, dm), op)
                ev_run = torch.cuda.Event()
                ev_run.record()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_run)
                out_host[(i - lo) * per:(i - lo + 1) * per].copy_(st[:per], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                free_ev[k % len(staging)] = ev
        for s in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(s)
        be.sync_stream()

    def upload_chunked(self, host: torch.Tensor, dev: torch.Tensor, chunks: int = 8) -> torch.cuda.Event:
        """Host->device copy of a whole tensor on the input stream in `chunks` pieces (so that it
        interleaves with other traffic); returns the event that marks its end."""
        n = host.numel()
        with torch.cuda.stream(self.s_in):
            for c in range(chunks):
                lo, hi = shard_range(n, chunks, c)
                if hi > lo:
                    dev[lo:hi].copy_(host[lo:hi], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        return ev
