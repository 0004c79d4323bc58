#!/usr/bin/env python
"""Benchmark of the tensor hot path on B200.

    python bench.py --gpus N --steps K --warmup W          # this repository's CUDA path
    python bench.py --impl reference ...                   # the reference CPU algorithm on host cores
    python bench.py --case NAME                            # one small profiling case (see --help)

A "step" is one pass of the ops the metric names over resident inputs:

  * the strided / negative-step broadcast add of BASELINE config 3,
    A(16,1,1024,1) [a permuted view] + B(1,64,1,1024) [step -1 on its last dim] -> (16,64,1024,1024) f32;
  * the axis sums of config 4: (8192,8192) over axis 0 and over axis 1, (64,4096,1024) over axis 1;
  * the full sum of 2^30 elements.

With N > 1 the SAME global tensors are cut into slabs (strong scaling): the broadcast along its
outermost output dim, every axis sum along a KEPT dim (each rank owns its outputs, no exchange), the
full sum along its flat range with the per-GPU totals exchanged inside the reduction's last CTA over
NVLink peer memory -- that exchange is inside the timed region.  The timed region is bracketed by a
barrier + synchronize; the slowest rank's device time is used.  Rank 0 prints ONE JSON line; under
"ops" it carries every other named op (scalar chain and i32 add of config 2, config 1, mean_l1_loss,
MLP step ...) measured the same way.
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

METRIC = "achieved HBM GB/s & elements/s for broadcast-add and axis-sum at 1/2/4/8 B200"
FALLBACK_PEAK_GBS = 6650.0
# independent probes measured on this pool's B200s (streaming read / fill of 4 GiB); the copy figure
# of MEASURED_PEAKS.json sits below both, which is why fractions "of measured" can exceed 1
PROBE_READ_GBS, PROBE_WRITE_GBS, NOMINAL_GBS = 7300.0, 7450.0, 8000.0
CPU_SAMPLE_LOG2 = 6      # the CPU legs run the same op list at 1/64 of every tensor


def sig(x, n=4):
    """Rounded to n significant digits (keeps the JSON line short)."""
    if x is None or not isinstance(x, float) or x == 0 or not math.isfinite(x):
        return x
    return round(x, n - 1 - int(math.floor(math.log10(abs(x)))))


class Shapes:
    """The step's tensors at 1 / 2^s of BASELINE's sizes (s = 0 for the bench itself)."""

    def __init__(self, s: int = 0):
        self.s = s
        self.k3 = 1024 >> s
        self.c3 = (16, 64, self.k3, 1024)
        self.m = (8192 >> ((s + 1) // 2), 8192 >> (s // 2))
        self.t = (64, 4096 >> s, 1024)
        self.f = 1 << (30 - s)
        self.n_a, self.n_b = self.k3 * 16, 64 * 1024
        self.c3_out = 16 * 64 * self.k3 * 1024

    def bytes_by_op(self):
        m, t = self.m, self.t
        return {
            "broadcast_add": 4 * (self.c3_out + self.n_a + self.n_b),
            "sum_at(0) matrix": 4 * (m[0] * m[1] + m[1]),
            "sum_at(1) matrix": 4 * (m[0] * m[1] + m[0]),
            "sum_at(1) cube": 4 * (t[0] * t[1] * t[2] + t[0] * t[2]),
            "sum (full)": 4 * self.f + 4,
        }

    def step_bytes(self):
        return sum(self.bytes_by_op().values())

    def step_elems(self):
        m, t = self.m, self.t
        return self.c3_out + 2 * m[0] * m[1] + t[0] * t[1] * t[2] + self.f

    def describe(self):
        return (f"configs[2]+[3]: f32 broadcast add A(16,1,{self.k3},1) permuted view + B(1,64,1,1024) step -1 -> {self.c3}; "
                f"sum over axis 0 and axis 1 of {self.m}; sum over axis 1 of {self.t}; full sum of 2^{30 - self.s}")


def peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_PEAK_GBS, "fallback"


def ncu_traffic(kernel: str):
    """dram bytes per launch of the roofline kernel, from the tracked capture summary next to the
    profile it came from; scaled by the caller to the launch it times."""
    try:
        with open(os.path.join(ROOT, "profiles", "roofline_traffic.json")) as f:
            return json.load(f)[kernel]
    except Exception:
        return None


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
# host side of the step: seeded inputs and the reference CPU algorithm (oracle port)
# ------------------------------------------------------------------------------------------------
def host_inputs(sh: Shapes, seed: int = 0x5EED + 3, with_reduction_inputs: bool = True):
    rng = np.random.default_rng(seed)
    bufa = rng.uniform(-1, 1, sh.n_a).astype(np.float32)
    bufb = rng.uniform(-1, 1, sh.n_b).astype(np.float32)
    red = None
    if with_reduction_inputs:
        red = rng.standard_normal(max(sh.f, sh.t[0] * sh.t[1] * sh.t[2]), dtype=np.float32)
    return bufa, bufb, red


def c3_views(M, sh: Shapes):
    """A = permute([2,0,1,3]) of a (K,16,1,1) buffer viewed as (1,K,16,1); B = step -1 on the last dim."""
    A = M.contiguous((sh.k3, 16, 1, 1)).view_as((1, sh.k3, 16, 1)).permute((2, 0, 1, 3))
    B = M.contiguous((1, 64, 1, 1024)).slice(3, None, None, -1)
    return A, B


def cpu_step(O, sh: Shapes, bufa, bufb, red):
    """The same op list on the host: Backend::broadcast and the axis / flat reductions of the
    reference CPU backend (C port, single-threaded as the reference is for this path)."""
    A, B = c3_views(O.Meta, sh)
    out, _ = O.binary(bufa, A, bufb, B, O.ADD, fast=True)
    mm = O.Meta.contiguous(sh.m)
    r0, _ = O.reduce_axis(red, mm, 0, O.SUM, fast=True)
    r1, _ = O.reduce_axis(red, mm, 1, O.SUM, fast=True)
    r2, _ = O.reduce_axis(red, O.Meta.contiguous(sh.t), 1, O.SUM, fast=True)
    r3 = O.reduce_flat(red, 0, sh.f, O.SUM, fast=True)
    return out, r0, r1, r2, r3


def cpu_baseline(steps: int, warmup: int):
    import oracle as O
    sh = Shapes(CPU_SAMPLE_LOG2)
    bufa, bufb, red = host_inputs(sh)
    for _ in range(warmup):
        cpu_step(O, sh, bufa, bufb, red)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(O, sh, bufa, bufb, red)
    dt = time.perf_counter() - t0
    return sh, sh.step_bytes() * steps / dt / 1e9, dt / steps * 1e3


def sample_text(sh: Shapes):
    return (f"the same five ops at 1/{1 << sh.s} of every tensor ({sh.c3}; {sh.m}; {sh.t}; 2^{30 - sh.s}) on one host core")


def config_block():
    """The same in both arms: the workload, and which sample of it each arm times."""
    return {"workload": Shapes(0).describe(),
            "sample": "GPU arm: the full tensors, cut into slabs over the N GPUs (strong scaling); reference arm and cpu_baseline: "
                      + sample_text(Shapes(CPU_SAMPLE_LOG2)) + " -- rates (GB/s of algorithmic bytes) are compared",
            "l2": "every tensor is larger than L2 (0.27 - 4.3 GB per op on the GPU, 4 - 67 MB per op on the host sample)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sh, gbs, ms = cpu_baseline(args.steps, max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": sig(gbs), "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sig(ms), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_block(),
        "elements_per_s": sig(sh.step_elems() / (ms / 1e3)),
        "cpu_baseline": {"value": sig(gbs), "unit": "GB/s", "cores": 1, "kind": "port",
                         "sample": "each step = " + sample_text(sh) + "; C port of the reference CPU backend "
                                   "(single-threaded like the reference; the Rust crate cannot be built here)"},
        "e2e": {"value": sig(gbs), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
    ap.add_argument("--no-verify", action="store_true", help="skip the oracle check of the timed buffers")
    ap.add_argument("--no-ref-cuda", action="store_true", help="skip timing the reference's own CUDA kernels")
    ap.add_argument("--scale-log2", type=int, default=0, help="run the step at 1/2^s of every tensor (small profiling runs)")
    ap.add_argument("--case", default=None, help="run one small profiling case and exit: " + ", ".join(
        ("flat", "c3", "red", "ext", "convert", "transpose", "mid", "sum", "host", "l1", "mlp")))
    ap.add_argument("--case-arg", type=int, default=None)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    import rtensors_b200 as rt
    from rtensors_b200 import _lib as L
    from rtensors_b200 import sharding
    from rtensors_b200.backend import CudaB200
    from rtensors_b200.meta import Meta, broadcast_params, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if args.case:
        from rtensors_b200 import opbench
        return opbench.small_case(CudaB200(local), args.case, args.case_arg)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    be = CudaB200(local)
    if world > 1:
        sharding.init_communicator(be)
    dev = f"cuda:{local}"
    sh = Shapes(args.scale_log2)
    f32 = torch.float32

    # ---- the global tensors (same seed on every rank), each rank works on its slabs ------------------
    bufa_h, bufb_h, _ = host_inputs(sh, with_reduction_inputs=False)
    bufa, bufb = be.alloc_from_slice(bufa_h), be.alloc_from_slice(bufb_h)
    g = torch.Generator(device=dev)
    g.manual_seed(0x5EED + 4)
    n_t = sh.t[0] * sh.t[1] * sh.t[2]
    Mx = torch.randn(sh.m[0] * sh.m[1], device=dev, generator=g, dtype=f32)
    Tx = torch.randn(n_t, device=dev, generator=g, dtype=f32)
    Fx = torch.randn(sh.f, device=dev, generator=g, dtype=f32)
    Am, Bm = c3_views(Meta, sh)
    slab = sharding.binary_slab(Am, Bm, world, rank)
    sdm = Meta.contiguous(slab.shape)
    out3 = be.alloc(max(sdm.size, 1), f32)
    mm, tm = Meta.contiguous(sh.m), Meta.contiguous(sh.t)

    def cut(meta, axis):
        d = sharding.pick_reduce_dim(meta.shape, axis, world) if world > 1 else None
        if d is None:
            return meta, None, 0, meta.shape[0]
        assert d != axis
        b, e = shard_range(meta.shape[d], world, rank)
        return meta.slice(d, b, e, 1), d, b, e
    m0, m0_dim, m0_b, m0_e = cut(mm, 0)       # columns cut: a strided window, reduced in place
    m1, m1_dim, m1_b, m1_e = cut(mm, 1)       # rows cut
    t1, t1_dim, t1_b, t1_e = cut(tm, 1)       # outermost dim cut
    f_lo, f_hi = shard_range(sh.f, world, rank)
    r_m0 = be.alloc(m0.shape[1], f32)
    r_m1 = be.alloc(m1.shape[0], f32)
    r_t1 = be.alloc(t1.shape[0] * t1.shape[2], f32)
    r_f = be.alloc(1, f32)

    def op_c3():
        be.broadcast((bufa, slab.left), (bufb, slab.right), (out3, sdm), L.ADD)

    def op_full_sum():
        if world > 1:
            be.mg_reduce_flat(Fx, f_lo, f_hi - f_lo, sh.f, L.SUM, dst=r_f)
        else:
            be.apply_reduce_contiguous_flat(Fx, r_f, 0, sh.f, L.SUM)

    def step():
        op_c3()
        be.reduce_view(Mx, m0, 0, L.SUM, out=r_m0)
        be.reduce_view(Mx, m1, 1, L.SUM, out=r_m1)
        be.reduce_view(Tx, t1, 1, L.SUM, out=r_t1)
        op_full_sum()

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
    ms_step = float(t.item()) / args.steps
    value = sh.step_bytes() / (ms_step * 1e-3) / 1e9
    mg_status = be.mg_status() if world > 1 else 0

    # ---- per-op device time inside the step (events around each op, slowest rank) and the roofline kernel
    peak, peak_kind = peak_gbs()

    def timed(fn, reps=12):
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        for s, e in ev:
            s.record(); fn(); e.record()
        torch.cuda.synchronize()
        tt = torch.tensor([float(np.mean([s.elapsed_time(e) for s, e in ev[2:]]))], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())
    by = sh.bytes_by_op()
    split = {}
    for name, fn in (("broadcast_add", op_c3), ("sum_at(0) matrix", lambda: be.reduce_view(Mx, m0, 0, L.SUM, out=r_m0)),
                     ("sum_at(1) matrix", lambda: be.reduce_view(Mx, m1, 1, L.SUM, out=r_m1)),
                     ("sum_at(1) cube", lambda: be.reduce_view(Tx, t1, 1, L.SUM, out=r_t1)), ("sum (full)", op_full_sum)):
        ms = timed(fn)
        split[name] = {"ms": sig(ms), "gbs": sig(by[name] / (ms * 1e-3) / 1e9), "frac": sig(by[name] / (ms * 1e-3) / 1e9 / (peak * world))}
    k_ms = split["broadcast_add"]["ms"]
    k_bytes = by["broadcast_add"] / world
    k_gbs = k_bytes / (k_ms * 1e-3) / 1e9
    traffic = ncu_traffic("rows_lean_kernel")
    roofline = {"bound": "hbm", "kernel": "rows_lean_kernel<f32 add; A broadcast scalar per row, B reversed vector> "
                                          f"(config-3 broadcast add, this rank's slab {slab.shape})",
                "achieved": sig(k_gbs), "peak": peak, "unit": "GB/s", "frac": sig(k_gbs / peak), "peak_kind": peak_kind,
                "frac_of_probe": sig(k_gbs / PROBE_WRITE_GBS), "frac_of_nominal": sig(k_gbs / NOMINAL_GBS),
                "ms_per_launch": sig(k_ms),
                "traffic": None if traffic is None else sig(max(4.0 * sdm.size * (1.0 + traffic["read_bytes_per_output_byte"])
                                                                - traffic["dirty_bytes_left_in_l2"], 0.0)),
                "traffic_source": None if traffic is None else "profiles/roofline_traffic.json: " + traffic["rule"]}

    # clocks under load: the timed region above is short, so sample while the same step keeps running
    t_load0 = sampler.mark()
    t_end = time.time() + 1.5
    while time.time() < t_end:
        for _ in range(20):
            step()
        torch.cuda.synchronize()
    t_load1 = sampler.mark()
    clocks = sampler.stop(t_load0 + 0.2, t_load1) if rank == 0 else None

    # ---- the timed buffers against the CPU oracle (outside the timed region) ------------------------
    verified = None
    if not args.no_verify:
        verified = verify(be, sh, world, rank, dict(bufa=bufa_h, bufb=bufb_h, out3=out3, slab=slab, Mx=Mx, Tx=Tx, Fx=Fx,
                                                    r_m0=r_m0, r_m1=r_m1, r_t1=r_t1, r_f=r_f, m0=(m0_b, m0_e), m1=(m1_b, m1_e),
                                                    t1=(t1_b, t1_e)))
        if world > 1:
            vt = torch.tensor([1 if verified else 0], device=dev)
            dist.all_reduce(vt, op=dist.ReduceOp.MIN)
            verified = bool(vt.item())

    # ---- end to end through the public API with HOST buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, be, sh, world, rank, dev, barrier, dict(bufa_h=bufa_h, bufb_h=bufb_h, bufa=bufa, bufb=bufb, Am=Am, Bm=Bm,
                                                                    slab=slab, Mx=Mx, Tx=Tx, Fx=Fx, m0=m0, m1=m1, t1=t1,
                                                                    cuts=((m0_b, m0_e), (m1_b, m1_e), (t1_b, t1_e), (f_lo, f_hi)),
                                                                    outs=(r_m0, r_m1, r_t1, r_f)))

    ops = None
    if not args.no_ops:
        del out3, Mx, Tx, Fx
        torch.cuda.empty_cache()
        from rtensors_b200 import opbench
        ops = opbench.run(be, peak, world, rank, quick=args.scale_log2 > 0)

    # the reference's own CUDA kernels on the same GPU, beside the rows they correspond to
    ref_note = None
    if ops is not None and world == 1 and rank == 0 and not args.no_ref_cuda:
        rc = ref_cuda_times(dev, args.scale_log2 > 0)
        if rc is None:
            ref_note = "baseline/_ref/libref_cuda.so absent (built from the reference checkout by __graft_entry__.build())"
        else:
            for row in ops:
                ms = rc.get((row["op"], row.get("shape")))
                if ms is not None:
                    row["ref_cuda_ms"] = sig(ms)
            for name, key in (("broadcast_add", ("broadcast_add f32 permuted A, step -1 B", str(tuple(sh.c3)))),
                              ("sum_at(0) matrix", ("sum_at(0) f32", f"({sh.m[0]},{sh.m[1]})")),
                              ("sum_at(1) matrix", ("sum_at(1) f32", f"({sh.m[0]},{sh.m[1]})")),
                              ("sum_at(1) cube", ("sum_at(1) f32", str(sh.t))), ("sum (full)", ("sum (full) f32", f"2^{30 - sh.s}"))):
                if key in rc:
                    split[name]["ref_cuda_ms"] = sig(rc[key])
            if all("ref_cuda_ms" in v for v in split.values()):
                ref_ms = sum(v["ref_cuda_ms"] for v in split.values())
                ref_note = {"step_ms": sig(ref_ms), "step_gbs": sig(sh.step_bytes() / (ref_ms * 1e-3) / 1e9),
                            "what": "the reference's own CUDA kernels recompiled for sm_100a with its release flags, kernel time only "
                                    "(its host-side zero upload and per-call index-array allocations excluded)"}

    cpu = None
    if rank == 0 and not args.no_cpu and world == 1:
        reps = 120
        csh, c_gbs, c_ms = cpu_baseline(reps, 1)
        cpu = {"value": sig(c_gbs), "unit": "GB/s", "cores": 1, "kind": "port",
               "sample": f"{reps} steps, {c_ms * reps / 1e3:.1f} s of CPU work; each step = " + sample_text(csh) +
                         "; C port of the single-threaded reference CPU backend"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": sig(value, 5), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": sig(ms_step, 5), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_block() if sh.s == 0 else {"workload": sh.describe(), "sample": f"1/{1 << sh.s} of every tensor"},
            "parallel": {"slabs": world,
                         "collective": None if world == 1 else "full sum: per-GPU totals exchanged over NVLink peer memory inside the "
                                                                "reduction kernel's last CTA (rtb_mg_reduce_flat), inside the timed region",
                         "peer_mapped": bool(be.mg_peer_mapped) if world > 1 else None},
            "elements_per_s": sig(sh.step_elems() / (ms_step * 1e-3), 5),
            "frac_of_peak": sig(value / world / peak), "peaks": {"measured_copy": peak, "probe_read": PROBE_READ_GBS,
                                                                  "probe_write": PROBE_WRITE_GBS, "nominal": NOMINAL_GBS},
            "step_ops": split, "ref_cuda": ref_note, "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "verified": verified,
            "gpu_launches": int(launches), "mg_status": mg_status, "clocks": clocks, "ops": ops,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        be.mg_finalize()
        dist.destroy_process_group()


def ref_cuda_times(dev: str, quick: bool):
    """Device time of the REFERENCE's own CUDA kernels (recompiled for sm_100a with its release flags,
    baseline/_ref/libref_cuda.so) on the ops of configs 1-4, launched the way its Rust host launches
    them: block 256, index arrays in device memory, legacy default stream.  Kernel time only -- the
    host-side costs of the reference (zero upload of every output, per-call cudaMalloc of the index
    arrays) are not included, so this is a lower bound on what the reference spends.
    -> {(op name, shape string): ms} keyed like the rows of the op table."""
    import torch
    from baseline import ref_cuda as R
    from rtensors_b200 import opbench
    from rtensors_b200.meta import Meta, broadcast_params
    if not R.available():
        return None
    f32 = torch.float32
    out = {}
    g = torch.Generator(device=dev)
    g.manual_seed(0x5EED)

    def t(fn, flush=False):
        return opbench._time(fn, reps=5, rounds=3, warm=1, flush=flush, dev=dev)[0]
    # config 1
    A, B = torch.rand(4096, device=dev, generator=g), torch.rand(4096, device=dev, generator=g)
    am, bm = Meta.contiguous((4096, 1)), Meta.contiguous((1, 4096))
    shape, sa, sb = broadcast_params(am, bm)
    dm = Meta.contiguous(shape)
    o1 = torch.empty(dm.size, device=dev)
    out[("broadcast_add f32", "(4096,1)+(1,4096)")] = t(R.Broadcast(A, Meta(shape, sa, 0), B, Meta(shape, sb, 0), o1, dm, R.ADD), True)
    r1 = torch.empty(8192, device=dev)
    out[("sum_at(1) f32", "(4096,4096)")] = t(lambda: R.reduce_nd(o1, r1, 0, 4096, 4096, 1, R.SUM), True)
    del o1
    # config 2
    n2 = 1 << (24 if quick else 28)
    lg = int(math.log2(n2))
    x = torch.rand(n2, device=dev, generator=g)
    out[("scalar_mul f32 in place", f"2^{lg}")] = t(lambda: R.scalar_contiguous(x, "mul", 1.0001))
    ia = torch.randint(-(1 << 20), 1 << 20, (n2,), device=dev, generator=g, dtype=torch.int32)
    io = torch.empty_like(ia)
    m2 = Meta.contiguous((n2,))
    out[("tensor_add i32", f"2^{lg}")] = t(R.Broadcast(ia, m2, ia, m2, io, m2, R.ADD))
    del ia, io, x
    # config 3
    sh = Shapes(4 if quick else 0)
    bufa = torch.rand(sh.n_a, device=dev, generator=g)
    bufb = torch.rand(sh.n_b, device=dev, generator=g)
    Am, Bm = c3_views(Meta, sh)
    shape3, sa3, sb3 = broadcast_params(Am, Bm)
    dm3 = Meta.contiguous(shape3)
    o3 = torch.empty(dm3.size, device=dev)
    out[("broadcast_add f32 permuted A, step -1 B", str(tuple(shape3)))] = t(
        R.Broadcast(bufa, Meta(shape3, sa3, Am.offset), bufb, Meta(shape3, sb3, Bm.offset), o3, dm3, R.ADD))
    # config 4 (o3 re-used as the normal(0,1) source)
    o3.normal_(generator=g)
    S = 2048 if quick else 8192
    rs = torch.empty(64 * 1024, device=dev)
    out[("sum_at(0) f32", f"({S},{S})")] = t(lambda: R.reduce_nd(o3, rs, 0, 1, S, S, R.SUM), S * S * 4 < (200 << 20))
    out[("sum_at(1) f32", f"({S},{S})")] = t(lambda: R.reduce_nd(o3, rs, 0, S, S, 1, R.SUM), S * S * 4 < (200 << 20))
    d3 = (64, 512, 1024) if quick else (64, 4096, 1024)
    out[("sum_at(1) f32", str(d3))] = t(lambda: R.reduce_nd(o3, rs, 0, d3[0], d3[1], d3[2], R.SUM))
    nf = dm3.size
    out[("sum (full) f32", f"2^{int(math.log2(nf))}")] = t(lambda: R.reduce_flat(o3, rs, 0, nf, R.SUM))
    torch.cuda.synchronize()
    assert not R.alloc_failed()
    return out


def verify(be, sh, world, rank, d) -> bool:
    """Compares what the timed region left in the output buffers with the CPU oracle on the same
    inputs: one outermost slab of the broadcast result bit for bit, every reduction output within
    1e-5 * log2(n) * sum|x| of the oracle's sequential sums."""
    import oracle as O
    ok = True
    slab = d["slab"]
    if slab.end > slab.begin:
        i = slab.begin + (slab.end - slab.begin) // 2
        A, B = c3_views(O.Meta, sh)
        want, _ = O.binary(d["bufa"], A.slice(0, i, i + 1, 1), d["bufb"], B, O.ADD, fast=True)
        per = want.size
        got = d["out3"][(i - slab.begin) * per:(i - slab.begin + 1) * per].cpu().numpy()
        ok &= got.tobytes() == want.tobytes()

    def close(got, want, scale, n):
        return bool(np.all(np.abs(got.astype(np.float64) - want.astype(np.float64)) <= 1e-5 * math.log2(max(n, 2)) * scale))
    M = d["Mx"].cpu().numpy().reshape(sh.m)
    absM = np.abs(M)
    w0, _ = O.reduce_axis(M.reshape(-1), O.Meta.contiguous(sh.m), 0, O.SUM, fast=True)
    b, e = d["m0"]
    ok &= close(d["r_m0"].cpu().numpy(), w0.reshape(-1)[b:e] if world > 1 else w0.reshape(-1), (absM.sum(axis=0, dtype=np.float64)[b:e] if world > 1 else absM.sum(axis=0, dtype=np.float64)), sh.m[0])
    w1, _ = O.reduce_axis(M.reshape(-1), O.Meta.contiguous(sh.m), 1, O.SUM, fast=True)
    b, e = d["m1"]
    ok &= close(d["r_m1"].cpu().numpy(), w1.reshape(-1)[b:e] if world > 1 else w1.reshape(-1), (absM.sum(axis=1, dtype=np.float64)[b:e] if world > 1 else absM.sum(axis=1, dtype=np.float64)), sh.m[1])
    del M, absM
    b, e = d["t1"] if world > 1 else (0, sh.t[0])
    T = d["Tx"].cpu().numpy().reshape(sh.t)[b:e]
    w2, _ = O.reduce_axis(np.ascontiguousarray(T).reshape(-1), O.Meta.contiguous(T.shape), 1, O.SUM, fast=True)
    ok &= close(d["r_t1"].cpu().numpy(), w2.reshape(-1), np.abs(T).sum(axis=1, dtype=np.float64).reshape(-1), sh.t[1])
    del T
    F = d["Fx"].cpu().numpy()
    w3 = O.reduce_flat(F, 0, sh.f, O.SUM, fast=True)
    truth = float(O.sum_f64(F))
    scale = float(O.abs_sum_f64(F))
    got = float(d["r_f"].cpu().numpy()[0])
    tol = 1e-5 * math.log2(sh.f) * scale
    ok &= abs(got - float(w3[0])) <= tol and abs(got - truth) <= tol
    return bool(ok)


def run_e2e(args, be, sh, world, rank, dev, barrier, d):
    """The same step through the host-buffer API: every step uploads the reduction inputs and the
    broadcast operands from pinned host memory and brings every result back (the 4.3 GB broadcast
    output slab by slab while the next slab is computed)."""
    import torch
    import torch.distributed as dist
    from rtensors_b200 import _lib as L
    from rtensors_b200.host import HostPipeline
    from rtensors_b200.meta import Meta
    pipe = HostPipeline(be)
    slab = d["slab"]
    n_slabs = max(slab.end - slab.begin, 1)
    per = 1
    for n in slab.shape[1:]:
        per *= n
    (m0b, m0e), (m1b, m1e), (t1b, t1e), (flo, fhi) = d["cuts"]
    cols = sh.m[1]
    # host copies of this rank's share of every input, pinned.  The column window of the matrix (the
    # axis-0 sum's share at N > 1) is a dense (rows, e - b) block on the host.
    h_a = torch.from_numpy(d["bufa_h"]).reshape(-1).pin_memory()
    h_b = torch.from_numpy(d["bufb_h"]).reshape(-1).pin_memory()
    Mfull = d["Mx"].view(sh.m)
    h_m0 = (Mfull[:, m0b:m0e] if world > 1 else Mfull).contiguous().reshape(-1).cpu().pin_memory()
    h_m1 = Mfull[m1b:m1e].contiguous().reshape(-1).cpu().pin_memory() if world > 1 else None   # N = 1: one matrix serves both sums
    Tfull = d["Tx"].view(sh.t)
    h_t = (Tfull[t1b:t1e] if world > 1 else Tfull).contiguous().reshape(-1).cpu().pin_memory()
    h_f = d["Fx"][flo:fhi].cpu().pin_memory()
    h_out = torch.empty(n_slabs * per, dtype=torch.float32).pin_memory()
    r_m0, r_m1, r_t1, r_f = d["outs"]
    h_res = [torch.empty_like(r, device="cpu").pin_memory() for r in (r_m0, r_m1, r_t1, r_f)]
    rows = sh.m[0]
    m0_meta = Meta.contiguous((rows, m0e - m0b) if world > 1 else sh.m)
    m1_meta = Meta.contiguous((m1e - m1b, cols) if world > 1 else sh.m)
    t_meta = Meta.contiguous(((t1e - t1b) if world > 1 else sh.t[0], sh.t[1], sh.t[2]))
    h2d = 4 * (h_a.numel() + h_b.numel() + h_m0.numel() + (h_m1.numel() if h_m1 is not None else 0) + h_t.numel() + h_f.numel())
    d2h = 4 * (h_out.numel() + sum(h.numel() for h in h_res))

    def e2e_step():
        be.sync_stream()
        # the broadcast first: its kernels start at once and are paced by the copy-out of its stages, while
        # the uploads below run on the upload lane; each reduction waits for its own input only
        pipe.broadcast_to_host(h_a, d["Am"], h_b, d["Bm"], L.ADD, h_out, (slab.begin, slab.end))
        b_m0 = be.host_stage_in(h_m0)
        b_m1 = be.host_stage_in(h_m1) if h_m1 is not None else b_m0
        b_t = be.host_stage_in(h_t)
        b_f = be.host_stage_in(h_f)
        be.host_ready(b_m0)
        be.reduce_view(b_m0, m0_meta, 0, L.SUM, out=r_m0)
        if h_m1 is not None:
            be.host_ready(b_m1)
        be.reduce_view(b_m1, m1_meta, 1, L.SUM, out=r_m1)
        be.host_ready(b_t)
        be.reduce_view(b_t, t_meta, 1, L.SUM, out=r_t1)
        be.host_ready(b_f)
        if world > 1:
            be.mg_reduce_flat(b_f, 0, h_f.numel(), sh.f, L.SUM, dst=r_f)
        else:
            be.apply_reduce_contiguous_flat(b_f, r_f, 0, h_f.numel(), L.SUM)
        for h, r in zip(h_res, (r_m0, r_m1, r_t1, r_f)):
            be.host_stage_out(r, h)                                  # the step's results, read back
        for blk in ((b_m0, b_t, b_f) if h_m1 is None else (b_m0, b_m1, b_t, b_f)):
            be.host_release(blk)
        be.host_join()                                               # the stream the step is timed on waits for both lanes
    esteps = max(1, min(args.steps, 5))
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
    # the results that came back through the host must be the resident arm's
    same = all(np.array_equal(h.numpy(), r.cpu().numpy()) for h, r in zip(h_res, (r_m0, r_m1, r_t1, r_f)))
    return {"value": sig(sh.step_bytes() / (e_ms * 1e-3) / 1e9), "unit": "GB/s", "ms_per_step": sig(e_ms),
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": esteps, "results_read_back": bool(same),
            "how": "the library's host-buffer operations (rtb_host_*): broadcast result produced in stages (about 64 MiB, at least one index of the outermost dim) into a ring of "
                   "three device blocks and copied out behind the next stage's kernel, reduction inputs uploaded on the upload lane, "
                   "each reduction waiting for its own input only; pinned host buffers; bytes are this rank's"}


if __name__ == "__main__":
    main()
