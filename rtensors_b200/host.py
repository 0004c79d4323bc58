"""Host-buffer front end: run elementwise / broadcast work whose inputs and outputs live in pinned
HOST memory.  The tensors are cut into chunks along the flat (outermost) dimension; chunk k's
host->device copy, its kernels and its device->host copy run on three streams, so the copies of
neighbouring chunks overlap the kernels and each other (PCIe is full duplex).  This is what a
caller uses when the data does not fit, or does not live, on the device -- the reference does the
same transfers whole-tensor and synchronously (`alloc_from_slice` / `dump`,
src/backend/cuda.rs:668-680, 770-788).
"""
from __future__ import annotations

from typing import Callable, Dict, Sequence

import torch

from .backend import CudaB200


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
