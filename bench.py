#!/usr/bin/env python
"""Benchmark of the tensor hot path on B200.

    python bench.py --gpus N --steps K --warmup W          # this repository's CUDA path
    python bench.py --impl reference ...                   # the reference CPU algorithm on host cores

A "step" is one pass of the headline workload over resident inputs: the contiguous scalar chain
a*=3; a+=2; a-=1 on an f32 tensor of 2^28 elements plus the i32 tensor+tensor add of two
2^28-element tensors (4 kernel launches, 9 GiB of algorithmic HBM traffic).  With N > 1 every rank
owns one outer-dimension slab of that size (weak scaling, no data-path collective); the timed
region is bracketed by a barrier + synchronize and the slowest rank's device time is used.
Rank 0 prints ONE JSON line.  The line also carries, under "ops", the achieved GB/s, elements/s and
roofline fraction of every other named op (broadcast add, strided/negative-step broadcast, axis and
full reductions, mean_l1_loss, reduce-to-shape) measured the same way.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_ELEMS = 1 << 28
METRIC = "achieved HBM GB/s & elements/s for broadcast-add and axis-sum at 1/2/4/8 B200"
WORKLOAD = ("configs[1]: f32 scalar chain a*=3; a+=2; a-=1 on 2^28 elements + i32 tensor+tensor add of two "
            "2^28-element tensors, per GPU slab")
STEP_BYTES = 3 * 2 * 4 * N_ELEMS + 3 * 4 * N_ELEMS  # three in-place passes + one 3-stream add
STEP_ELEMS = 4 * N_ELEMS
FALLBACK_PEAK_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the in-place f32 kernel, from the ncu
# capture summarised under profiles/ (captured at 2^27 elements, scaled by 2: traffic is linear in n)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 2.026e9  # at 2^28 elements: 2 x (536.9 MB read + 476.1 MB written) measured at 2^27


def peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_PEAK_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self, wait_s: float = 4.0):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
            t0 = time.time()
            while not self.lines and time.time() - t0 < wait_s:  # nvidia-smi needs a moment to start
                time.sleep(0.05)
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark(self):
        return time.time()

    def stop(self, t_from: float = 0.0, t_to: float = float("inf")):
        """Summary of the samples taken in [t_from, t_to] (all samples if that window holds none)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        window = [ln for t, ln in self.lines if t_from <= t <= t_to] or [ln for _, ln in self.lines]
        for ln in window:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU algorithm (oracle port) on the host
# ------------------------------------------------------------------------------------------------
def cpu_step(O, a, ia, ib, iout, meta, imeta):
    O.scalar_op(a, O.MUL, 3.0, meta, fast=True)
    O.scalar_op(a, O.ADD, 2.0, meta, fast=True)
    O.scalar_op(a, O.SUB, 1.0, meta, fast=True)
    O.broadcast(ia, imeta, ib, imeta, iout, imeta, O.ADD, fast=True)


def cpu_baseline(sample_elems: int, steps: int, warmup: int):
    """Times the CPU oracle (C port of the reference CPU backend; single-threaded, as the reference
    is for this path) on a bounded sample of the same workload.  -> (GB/s, ms per step)."""
    import oracle as O
    rng = np.random.default_rng(0x5EED + 1)
    a = rng.uniform(-1, 1, sample_elems).astype(np.float32)
    ia = rng.integers(-(1 << 20), 1 << 20, sample_elems, endpoint=True).astype(np.int32)
    ib = rng.integers(-(1 << 20), 1 << 20, sample_elems, endpoint=True).astype(np.int32)
    iout = np.zeros_like(ia)
    meta = O.Meta.contiguous((sample_elems,))
    for _ in range(warmup):
        cpu_step(O, a, ia, ib, iout, meta, meta)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(O, a, ia, ib, iout, meta, meta)
    dt = time.perf_counter() - t0
    step_bytes = STEP_BYTES * sample_elems / N_ELEMS
    return step_bytes * steps / dt / 1e9, dt / steps * 1e3


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 1 << 24
    gbs, ms = cpu_baseline(sample, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32+i32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"each step = the same chain + add on 2^24 elements per tensor "
                                                     f"(1/16 of the per-GPU slab) on the host"},
        "elements_per_s": STEP_ELEMS * (sample / N_ELEMS) / (ms / 1e3),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "port",
                         "sample": "2^24 elements per tensor per step; C port of the reference CPU backend "
                                   "(single-threaded like the reference; the Rust crate cannot be built here)"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# this repository's arm
# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-ops", action="store_true", help="skip the per-op table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--e2e-chunk-log2", type=int, default=23, help="elements per chunk of the host pipeline")
    ap.add_argument("--elems-log2", type=int, default=28, help="per-GPU slab size (for small profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    import rtensors_b200 as rt
    from rtensors_b200 import _lib as L
    from rtensors_b200.backend import CudaB200
    from rtensors_b200.meta import Meta, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    be = CudaB200(local)
    dev = f"cuda:{local}"
    n = 1 << args.elems_log2
    scale = n / N_ELEMS
    # the global tensors have world*n elements; this rank's outer-dim slab is [lo, hi)
    lo, hi = shard_range(world * n, world, rank)
    assert hi - lo == n

    g = torch.Generator(device=dev)
    g.manual_seed(0x5EED + 1 + rank)
    a = torch.rand(n, device=dev, generator=g, dtype=torch.float32) * 2 - 1
    ia = torch.randint(-(1 << 20), (1 << 20) + 1, (n,), device=dev, generator=g, dtype=torch.int32)
    ib = torch.randint(-(1 << 20), (1 << 20) + 1, (n,), device=dev, generator=g, dtype=torch.int32)
    iout = torch.empty_like(ia)
    m = Meta.contiguous((n,))

    def step():
        be.scalar_apply(a, L.MUL, 3.0, m)
        be.scalar_apply(a, L.ADD, 2.0, m)
        be.scalar_apply(a, L.SUB, 1.0, m)
        be.broadcast((ia, m), (ib, m), (iout, m), L.ADD)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = be.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = be.launches - launches0
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_step = ms_total / args.steps
    step_bytes = STEP_BYTES * scale
    value = world * step_bytes / (ms_step * 1e-3) / 1e9

    # dominant kernel: the in-place f32 flat kernel, timed launch by launch with events
    peak, peak_kind = peak_gbs()
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(12)]
    for s, e in kev:
        s.record()
        be.scalar_apply(a, L.ADD, 0.5, m)
        e.record()
    torch.cuda.synchronize()
    k_ms = float(np.mean([s.elapsed_time(e) for s, e in kev[2:]]))
    k_gbs = 2 * 4 * n / (k_ms * 1e-3) / 1e9
    # clocks under load: the timed region above is short, so sample while the same step keeps running
    t_load0 = sampler.mark()
    t_end = time.time() + 1.5
    while time.time() < t_end:
        for _ in range(20):
            step()
        torch.cuda.synchronize()
    t_load1 = sampler.mark()
    clocks = sampler.stop(t_load0 + 0.2, t_load1) if rank == 0 else None

    roofline = {"bound": "hbm", "kernel": "flat_kernel<f32, scalar op> (in place, 2^%d elements)" % args.elems_log2,
                "achieved": k_gbs, "peak": peak, "unit": "GB/s", "frac": k_gbs / peak, "peak_kind": peak_kind,
                "ms_per_launch": k_ms,
                "traffic": None if NCU_TRAFFIC_BYTES_PER_LAUNCH is None else NCU_TRAFFIC_BYTES_PER_LAUNCH * scale}

    # end to end through the public API with HOST buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e:
        ha = torch.empty(n, dtype=torch.float32).pin_memory()
        hia = torch.empty(n, dtype=torch.int32).pin_memory()
        hib = torch.empty(n, dtype=torch.int32).pin_memory()
        ha.copy_(a.cpu().clamp_(-1, 1)); hia.copy_(ia.cpu()); hib.copy_(ib.cpu())
        ra = torch.empty(n, dtype=torch.float32).pin_memory()
        ri = torch.empty(n, dtype=torch.int32).pin_memory()
        esteps = max(1, min(args.steps, 5))

        from rtensors_b200.host import HostPipeline
        pipe = HostPipeline(be, chunk_elems=1 << args.e2e_chunk_log2)

        def chunk_compute(v, length):
            mc = Meta.contiguous((length,))
            be.scalar_apply(v["a"], L.MUL, 3.0, mc)
            be.scalar_apply(v["a"], L.ADD, 2.0, mc)
            be.scalar_apply(v["a"], L.SUB, 1.0, mc)
            be.broadcast((v["ia"], mc), (v["ib"], mc), (v["iout"], mc), L.ADD)

        def e2e_step():
            # public host-buffer API: chunked H2D -> kernels -> D2H over three streams
            pipe.run(n, {"a": (ha, a), "ia": (hia, ia), "ib": (hib, ib)},
                     {"a": (ra, a), "iout": (ri, iout)}, chunk_compute)
        e2e_step()
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(esteps):
            e2e_step()
        e.record()
        barrier()
        tt = torch.tensor([s.elapsed_time(e)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e_ms = float(tt.item()) / esteps
        e2e = {"value": world * step_bytes / (e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e_ms,
               "h2d_bytes_per_step": 3 * 4 * n, "d2h_bytes_per_step": 2 * 4 * n, "steps": esteps,
               "how": f"HostPipeline: 2^{args.e2e_chunk_log2}-element chunks, H2D / kernels / D2H on three streams, pinned host buffers"}
        del ha, hia, hib, ra, ri

    ops = None
    if not args.no_ops:
        del a, ia, ib, iout
        torch.cuda.empty_cache()
        from rtensors_b200 import opbench
        ops = opbench.run(be, peak, world, rank, quick=args.elems_log2 < 28)

    cpu = None
    if rank == 0 and not args.no_cpu and world == 1:
        sample = 1 << 26
        reps = 32
        c_gbs, c_ms = cpu_baseline(sample, reps, 1)
        cpu = {"value": c_gbs, "unit": "GB/s", "cores": 1, "kind": "port",
               "sample": f"{reps} steps of the same chain + add on 2^26 elements per tensor (1/4 slab), "
                         f"{c_ms * reps / 1e3:.1f} s of CPU work; C port of the single-threaded reference CPU backend"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32+i32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "elements_per_tensor_per_gpu": n, "parallelism": f"slab x{world}",
                       "l2": "inputs larger than L2 (1 GiB per tensor)"},
            "elements_per_s": world * STEP_ELEMS * scale / (ms_step * 1e-3),
            "frac_of_peak": value / world / peak, "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks, "ops": ops,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
