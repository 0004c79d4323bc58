"""Per-op timing table used by bench.py: every named op of the hot path, timed with CUDA events on
the launching stream (10 back-to-back launches per event pair, median of 5 pairs), with the
algorithmic HBM bytes that define its roofline.

Algorithmic bytes (s = element size): in-place scalar/unary op 2*s*n; same-shape binary 3*s*n;
broadcast binary s*(n_out + n_A + n_B) (each operand's unique elements once); axis reduce
s*(outer*R*inner + outer*inner); flat reduce s*n + s; fused mean_l1_loss 2*s*n + s; reduce-to-shape
s*(rows*cols + cols); relu with mask 3*s*n; SGD update 3*s*n.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib as L
from .meta import Meta, broadcast_params

_FLUSH = None


def _flush_l2(dev):
    global _FLUSH
    if _FLUSH is None or _FLUSH.device != torch.device(dev):
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    _FLUSH.add_(1)


def _span(fn, reps):
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e)


def _time(fn, reps=10, rounds=5, warm=3, flush=False, dev=None):
    """Device time per call in ms: `reps` calls are enqueued back to back between one pair of CUDA
    events, so the host-side enqueue cost of a call is not counted as kernel time.  With
    flush=True every call is preceded by a write of a 256 MiB buffer (larger than L2) and the
    time of the same number of flushes alone is subtracted."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(rounds):
        if flush:
            def both():
                _flush_l2(dev)
                fn()
            t1 = _span(both, reps)
            t0 = _span(lambda: _flush_l2(dev), reps)
            ts.append(max(t1 - t0, 1e-6) / reps)
        else:
            ts.append(_span(fn, reps) / reps)
    return float(np.median(ts)), float(np.min(ts))


def run(be, peak_gbs: float, world: int = 1, rank: int = 0, quick: bool = False):
    dev = f"cuda:{be.device}"
    rows = []

    def add(name, shape, nbytes, elems, fn, flush=False, note=None):
        med, best = _time(fn, flush=flush, dev=dev)
        gbs = nbytes / (med * 1e-3) / 1e9
        row = {"op": name, "shape": shape, "ms": med, "ms_best": best, "gbs": gbs, "elements_per_s": elems / (med * 1e-3),
               "frac": gbs / peak_gbs, "bytes": nbytes}
        if flush:
            row["l2"] = "flushed between iterations (working set could sit in L2)"
        if note:
            row["note"] = note
        rows.append(row)

    g = torch.Generator(device=dev)
    g.manual_seed(0x5EED)
    f32 = torch.float32

    # ---- config 1: (4096,1) + (1,4096) -> (4096,4096), then sum over axis 1
    A = torch.rand(4096, device=dev, generator=g) * 2 - 1
    B = torch.rand(4096, device=dev, generator=g) * 2 - 1
    am, bm = Meta.contiguous((4096, 1)), Meta.contiguous((1, 4096))
    shape, sa, sb = broadcast_params(am, bm)
    dm = Meta.contiguous(shape)
    out = be.alloc(dm.size, f32)
    add("broadcast_add f32", "(4096,1)+(1,4096)", 4 * (dm.size + 8192), dm.size,
        lambda: be.broadcast((A, Meta(shape, sa, 0)), (B, Meta(shape, sb, 0)), (out, dm), L.ADD), flush=True)
    red = be.alloc(4096, f32)
    add("sum_at(1) f32", "(4096,4096)", 4 * (dm.size + 4096), dm.size,
        lambda: be.apply_reduce((out, dm), red, 1, L.SUM), flush=True)
    del out
    add("broadcast_add + sum_at(1) fused f32 (no 64 MiB intermediate)", "(4096,1)+(1,4096) -> (4096,1)",
        4 * (4096 + 4096 + 4096), 4096 * 4096, lambda: be.broadcast_reduce(A, am, B, bm, L.ADD, 1, L.SUM), flush=True,
        note="bytes = the three small vectors actually touched; compare its time with the two rows above")
    add("broadcast_add + sum_at(0) fused f32 (k cut into chunks, partial rows folded)", "(4096,1)+(1,4096) -> (1,4096)",
        4 * (4096 + 4096 + 4096), 4096 * 4096, lambda: be.broadcast_reduce(A, am, B, bm, L.ADD, 0, L.SUM), flush=True)

    # ---- config 2 parts
    n2 = 1 << (24 if quick else 28)
    x = torch.rand(n2, device=dev, generator=g) * 2 - 1
    m2 = Meta.contiguous((n2,))
    add("scalar_mul f32 in place", f"2^{int(np.log2(n2))}", 8 * n2, n2, lambda: be.scalar_apply(x, L.MUL, 1.0001, m2))
    add("relu f32 in place", f"2^{int(np.log2(n2))}", 8 * n2, n2, lambda: be.apply_unary(x, L.RELU, m2))
    ia = torch.randint(-(1 << 20), 1 << 20, (n2,), device=dev, generator=g, dtype=torch.int32)
    ib = torch.randint(-(1 << 20), 1 << 20, (n2,), device=dev, generator=g, dtype=torch.int32)
    io = torch.empty_like(ia)
    add("tensor_add i32", f"2^{int(np.log2(n2))}", 12 * n2, n2, lambda: be.broadcast((ia, m2), (ib, m2), (io, m2), L.ADD))
    add("fill f32", f"2^{int(np.log2(n2))}", 4 * n2, n2, lambda: be.fill(x, 1.5, m2), note="pure-write probe")
    del ia, ib, io
    # other element sizes through the same kernels (1-byte and 8-byte lanes of the 128-bit vectors)
    nb = n2 * 4
    ua = torch.randint(0, 255, (nb,), device=dev, generator=g, dtype=torch.uint8)
    ub = torch.randint(0, 255, (nb,), device=dev, generator=g, dtype=torch.uint8)
    uo = torch.empty_like(ua)
    mb = Meta.contiguous((nb,))
    add("tensor_add u8", f"2^{int(np.log2(nb))}", 3 * nb, nb, lambda: be.broadcast((ua, mb), (ub, mb), (uo, mb), L.ADD))
    del ua, ub, uo
    xd = torch.rand(n2 // 2, device=dev, generator=g, dtype=torch.float64)
    md = Meta.contiguous((n2 // 2,))
    add("scalar_mul f64 in place", f"2^{int(np.log2(n2 // 2))}", 16 * (n2 // 2), n2 // 2,
        lambda: be.scalar_apply(xd, L.MUL, 1.0001, md))
    rd = be.alloc(1, torch.float64)
    add("sum (full) f64", f"2^{int(np.log2(n2 // 2))}", 8 * (n2 // 2) + 8, n2 // 2,
        lambda: be.apply_reduce_contiguous_flat(xd, rd, 0, n2 // 2, L.SUM))
    del xd
    # dtype conversion (Backend::convert): one streaming kernel per type pair
    for dt, label in ((torch.float64, "f64"), (torch.int32, "i32"), (torch.uint8, "u8")):
        co = be.alloc(n2, dt)
        add(f"convert f32 -> {label}", f"2^{int(np.log2(n2))}", (4 + co.element_size()) * n2, n2,
            lambda co=co, dt=dt: be.convert(x, dt, out=co))
        if dt is torch.uint8:
            add("convert u8 -> f32", f"2^{int(np.log2(n2))}", 5 * n2, n2, lambda co=co: be.convert(co, f32, out=x))
        del co

    # ---- config 3: strided / negative-step broadcast add -> (16,64,K,1024)
    K = 64 if quick else 1024
    bufa = torch.rand(K * 16, device=dev, generator=g) * 2 - 1
    bufb = torch.rand(64 * 1024, device=dev, generator=g) * 2 - 1
    Am = Meta.contiguous((K, 16, 1, 1)).view_as((1, K, 16, 1)).permute((2, 0, 1, 3))
    Bm = Meta.contiguous((1, 64, 1, 1024)).slice(3, None, None, -1)
    shape3, sa3, sb3 = broadcast_params(Am, Bm)
    dm3 = Meta.contiguous(shape3)
    out3 = be.alloc(dm3.size, f32)
    add("broadcast_add f32 permuted A, step -1 B", str(shape3), 4 * (dm3.size + K * 16 + 65536), dm3.size,
        lambda: be.broadcast((bufa, Meta(shape3, sa3, Am.offset)), (bufb, Meta(shape3, sb3, Bm.offset)), (out3, dm3), L.ADD))

    # ---- config 4: reductions (reuse out3's storage as normal(0,1) input)
    n4 = dm3.size
    src = out3
    src.normal_(generator=g)
    S = 2048 if quick else 8192
    msq = Meta.contiguous((S, S))
    r1 = be.alloc(S, f32)
    for opn, op in (("sum", L.SUM), ("mean", L.MEAN), ("max", L.MAX), ("min", L.MIN)):
        for axis in (0, 1):
            add(f"{opn}_at({axis}) f32", f"({S},{S})", 4 * (S * S + S), S * S,
                (lambda op=op, axis=axis: be.apply_reduce((src, msq), r1, axis, op)), flush=S * S * 4 < (200 << 20))
    # reductions over a strided view: an (S,S) window of an (S,2S) matrix, reduced in place, against
    # the reference's recipe for non-contiguous tensors (copy the view contiguous, then reduce)
    win = Meta.contiguous((S, 2 * S)).slice(1, S // 2, S // 2 + S, 1)
    for axis in (0, 1):
        add(f"sum_at({axis}) f32 over a strided window, no copy", f"({S},{S}) window of ({S},{2 * S})", 4 * (S * S + S), S * S,
            (lambda axis=axis: be.reduce_view(src, win, axis, L.SUM)), flush=S * S * 4 < (200 << 20))

    # elementwise ops in place on the same window (rows of S elements with a pitch of 2S)
    add("scalar_add f32 in place on a strided window", f"({S},{S}) window of ({S},{2 * S})", 8 * S * S, S * S,
        lambda: be.scalar_apply(src, L.ADD, 1.0, win), flush=S * S * 8 < (200 << 20))
    add("fill f32 on a strided window", f"({S},{S}) window of ({S},{2 * S})", 4 * S * S, S * S,
        lambda: be.fill(src, 0.25, win), flush=S * S * 4 < (200 << 20))
    src.normal_(generator=g)

    def copy_then_reduce():
        tmp = be.contiguous(src, win)
        be.apply_reduce((tmp, msq), r1, 1, L.SUM)
    add("sum_at(1) f32 over the same window, copy first (reference recipe)", f"({S},{S}) window of ({S},{2 * S})",
        4 * (S * S + S), S * S, copy_then_reduce, flush=S * S * 4 < (200 << 20),
        note="algorithmic bytes of the reduction alone; the copy moves 2x more")
    # transposed views: contiguous() (the transposing tile kernel), a reduction along the view's
    # strided-then-dense dims in place, and a binary op with one transposed operand
    tview = msq.permute((1, 0))
    tmp_t = be.alloc(S * S, f32)
    add("contiguous() of a transposed matrix f32", f"({S},{S}) strides (1,{S})", 8 * S * S, S * S,
        lambda: be.contiguous(src, tview))
    for axis in (0, 1):
        add(f"sum_at({axis}) f32 over the transposed view, no copy", f"({S},{S}) strides (1,{S})", 4 * (S * S + S), S * S,
            (lambda axis=axis: be.reduce_view(src, tview, axis, L.SUM)), flush=S * S * 4 < (200 << 20))
    add("a.T + b f32", f"({S},{S})", 12 * S * S, S * S,
        lambda: be.broadcast((src, tview), (src[S * S:], msq), (tmp_t, msq), L.ADD))
    del tmp_t

    d3 = (64, 512, 1024) if quick else (64, 4096, 1024)
    m3 = Meta.contiguous(d3)
    r3 = be.alloc(d3[0] * d3[2], f32)
    for opn, op in (("sum", L.SUM), ("mean", L.MEAN), ("max", L.MAX), ("min", L.MIN)):
        add(f"{opn}_at(1) f32", str(d3), 4 * (m3.size + d3[0] * d3[2]), m3.size,
            (lambda op=op: be.apply_reduce((src, m3), r3, 1, op)))
    # state-merging reductions (variance / std, logsumexp, L2 norm, argmax) on the same tensors
    ri = be.alloc(max(S, d3[0] * d3[2]), torch.int64)
    ext = (("var", L.VARIANCE, (True, False, 2), r1, r3), ("std", L.VARIANCE, (True, True, 2), r1, r3),
           ("logsumexp", L.LOGSUMEXP, (True, False, 2), r1, r3), ("l2_norm", L.NORM, (True, False, 2), r1, r3),
           ("argmax", L.ARGMAX, (True, False, 2), ri, ri))
    for opn, op, args, o1, o3 in ext:
        for axis in (0, 1):
            add(f"{opn}_at({axis}) f32", f"({S},{S})", 4 * (S * S + S), S * S,
                (lambda op=op, axis=axis, args=args, o1=o1: be.apply_reduce_ex((src, msq), o1, axis, op, *args)),
                flush=S * S * 4 < (200 << 20))
        add(f"{opn}_at(1) f32", str(d3), 4 * (m3.size + d3[0] * d3[2]), m3.size,
            (lambda op=op, args=args, o3=o3: be.apply_reduce_ex((src, m3), o3, 1, op, *args)))
    mflat = Meta.contiguous((n4,))
    for opn, op, args, o1, o3 in ext:
        add(f"{opn} (full) f32", f"2^{int(np.log2(n4))}", 4 * n4 + 4, n4,
            (lambda op=op, args=args, o1=o1: be.apply_reduce_ex((src, mflat), o1, 0, op, *args)))
    r0 = be.alloc(1, f32)
    nflat = n4
    if world == 1:
        add("sum (full) f32", f"2^{int(np.log2(nflat))}", 4 * nflat + 4, nflat,
            lambda: be.apply_reduce_contiguous_flat(src, r0, 0, nflat, L.SUM))
    else:
        import torch.distributed as dist
        per = nflat // world

        def sharded_sum():
            be.apply_reduce_contiguous_flat(src, r0, 0, per, L.SUM)
            dist.all_reduce(r0, op=dist.ReduceOp.SUM)
        add("sum (full) f32, per-GPU partial + NCCL allreduce", f"2^{int(np.log2(nflat))} over {world} GPUs",
            4 * nflat + 4, nflat, sharded_sum, note=f"aggregate bytes over all GPUs / this rank's time; frac is of {world} x peak")
        rows[-1]["frac"] = rows[-1]["gbs"] / (peak_gbs * world)
    nl = (1024 if quick else 4096) ** 2
    ta, tb = src[:nl], src[nl:2 * nl]
    add("mean_l1_loss f32", f"two ({int(nl ** 0.5)},{int(nl ** 0.5)})", 8 * nl + 4, nl,
        lambda: be.l1_loss(ta, tb, 0, False), flush=True)
    add("mean_l1_loss f32 + grad map", f"two ({int(nl ** 0.5)},{int(nl ** 0.5)})", 12 * nl + 4, nl,
        lambda: be.l1_loss(ta, tb, 0, True), flush=True)

    # ---- config 5 pieces: bias add, relu+mask, bias-grad reduce-to-shape, SGD update
    Bt, H = 4096, 1024
    act = src[: Bt * H]
    bias = torch.zeros(H, device=dev)
    ma, mb = Meta.contiguous((Bt, H)), Meta.contiguous((1, H))
    shp, s_a, s_b = broadcast_params(ma, mb)
    add("bias add in place f32", "(4096,1024)+=(1,1024)", 4 * (2 * Bt * H + H), Bt * H,
        lambda: be.binary_assign(act, ma, bias, mb, L.ADD), flush=True)
    add("relu + mask f32", "(4096,1024)", 12 * Bt * H, Bt * H, lambda: be.relu_mask(act), flush=True)
    add("reduce_to_shape (bias grad) f32", "(4096,1024)->(1,1024)", 4 * (Bt * H + H), Bt * H,
        lambda: be.reduce_to_shape(act, (Bt, H), (0, 1)), flush=True)
    nw = 784 * 1024 + 1024 * 1024 + 1024 * 10 + 2058
    nw -= nw % 4
    w, gw = src[:nw], src[nw:2 * nw]
    add("sgd_update f32", f"{nw} params", 12 * nw, nw, lambda: be.sgd_update(w, gw, 0.0), flush=True)
    # ---- multi-GPU (strong scaling of single ops): slab-sharded view broadcast with no collective,
    # axis sum over the sharded dim with one all-reduce of the partial vector
    if world > 1:
        import torch.distributed as dist
        from . import sharding

        def add_sharded(name, shape, nbytes, elems, fn):
            med, best = _time(fn)
            t = torch.tensor([med], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)  # slowest rank
            med = float(t.item())
            gbs = nbytes / (med * 1e-3) / 1e9
            rows.append({"op": name, "shape": shape, "ms": med, "ms_best": best, "gbs": gbs,
                         "elements_per_s": elems / (med * 1e-3), "frac": gbs / (peak_gbs * world), "bytes": nbytes,
                         "note": f"aggregate over {world} GPUs / slowest rank's time; frac is of {world} x peak"})
        slab = sharding.binary_slab(Am, Bm, world, rank)
        sdm = Meta.contiguous(slab.shape)
        sout = out3[: sdm.size]
        add_sharded("broadcast_add f32 permuted A, step -1 B, slab-sharded", f"{shape3} over {world} GPUs",
                    4 * (dm3.size + K * 16 + 65536), dm3.size,
                    lambda: be.broadcast((bufa, slab.left), (bufb, slab.right), (sout, sdm), L.ADD))
        lo, hi = sharding.scalar_slab(S, world, rank)
        part_rows = src[lo * S: hi * S]
        add_sharded("sum_at(0) f32, rows sharded + all-reduce of the partial vector", f"({S},{S}) over {world} GPUs",
                    4 * (S * S + S), S * S,
                    lambda: sharding.sharded_reduce_axis(be, part_rows, 1, hi - lo, S, L.SUM, "r", S))
        add_sharded("sum_at(1) f32, rows sharded, no collective", f"({S},{S}) over {world} GPUs", 4 * (S * S + S), S * S,
                    lambda: sharding.sharded_reduce_axis(be, part_rows, hi - lo, S, 1, L.SUM, "outer", S))

    # ---- a launch-bound chain of small calls, eager and replayed from a CUDA graph (config-1 sized
    # pieces: outer-product add, two in-place passes, column sum, row variance, fused add + row sum)
    cr, cc = 512, 1024
    ca = torch.rand(cr, device=dev, generator=g)
    cb = torch.rand(cc, device=dev, generator=g)
    cam, cbm = Meta.contiguous((cr, 1)), Meta.contiguous((1, cc))
    cshape, csa, csb = broadcast_params(cam, cbm)
    cdm = Meta.contiguous(cshape)
    cml, cmr = Meta(cshape, csa, 0), Meta(cshape, csb, 0)
    cout, ccol, cvar = be.alloc(cr * cc, f32), be.alloc(cc, f32), be.alloc(cr, f32)

    def chain():
        be.broadcast((ca, cml), (cb, cmr), (cout, cdm), L.ADD)
        be.scalar_apply(cout, L.MUL, 1.5, cdm)
        be.apply_unary(cout, L.RELU, cdm)
        be.apply_reduce((cout, cdm), ccol, 0, L.SUM)
        be.apply_reduce_ex((cout, cdm), cvar, 1, L.VARIANCE)
        be.broadcast_reduce(ca, cam, cb, cbm, L.ADD, 1, L.SUM)
    med_e, best_e = _time(chain, reps=10, rounds=5)
    cur = torch.cuda.current_stream(be.device)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        be.sync_stream()
        chain()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            be.sync_stream()
            chain()
        med_g, best_g = _time(graph.replay, reps=10, rounds=5)
    cur.wait_stream(side)
    be.sync_stream()
    rows.append({"op": "chain of 6 small calls (2 MiB tensor): eager from Python / replayed from a CUDA graph",
                 "shape": f"({cr},1)+(1,{cc}), *=, relu, sum_at(0), var_at(1), fused add+sum_at(1)", "ms": med_g, "ms_best": best_g,
                 "ms_eager": med_e, "note": "same kernels, same results; the graph removes the host cost of six enqueues"})

    # ---- config 5 as a whole: one SGD step of the 784-1024-1024-10 MLP, global batch 4096 split
    # across the ranks (data parallel: loss all-reduce + one flat gradient bucket all-reduce)
    from .mlp import DenseMlp, synthetic_batch
    torch.backends.cuda.matmul.allow_tf32 = False
    model = DenseMlp(be, (784, 1024, 1024, 10), lr=0.01)
    local_b = 4096 // world
    img, tgt, _, _ = synthetic_batch(local_b, dev, rank=rank)
    med, best = _time(lambda: model.step(img, tgt, 4096), reps=5, rounds=5)
    gemm_flops = 2 * 4096 * (784 * 1024 + 1024 * 1024 + 1024 * 10) * 3 - 2 * 4096 * 784 * 1024
    rows.append({"op": "MLP SGD step 784-1024-1024-10 (GEMMs on cuBLAS, rest on this library)",
                 "shape": f"global batch 4096, {local_b} per GPU x {world}", "ms": med, "ms_best": best,
                 "samples_per_s": 4096 / (med * 1e-3), "gemm_tflops": gemm_flops / (med * 1e-3) / 1e12,
                 "note": "whole step incl. cuBLAS GEMMs and, at N>1, two NCCL all-reduces (loss, 7.45 MB gradient bucket)"})
    if world == 1:
        model.step_graphed(img, tgt, 4096)  # eager step + capture
        med_g, best_g = _time(lambda: model.step_graphed(img, tgt, 4096), reps=5, rounds=5)
        rows.append({"op": "MLP SGD step, replayed from a CUDA graph", "shape": "global batch 4096, 1 GPU", "ms": med_g,
                     "ms_best": best_g, "samples_per_s": 4096 / (med_g * 1e-3), "gemm_tflops": gemm_flops / (med_g * 1e-3) / 1e12,
                     "note": "same kernels as the row above, one graph launch per step"})
    torch.cuda.synchronize()
    return rows
