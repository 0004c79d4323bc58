"""Per-op timing table used by bench.py: every named op of the hot path, timed with CUDA events on
the launching stream (10 back-to-back launches per event pair, median of 5 pairs), with the
algorithmic HBM bytes that define its roofline.

L2 between launches: read-only ops below 1 GiB run with the L2 flushed before every launch (a 268 MB input
is only twice the L2, and what a back-to-back repetition finds there depends on the view); in-place and
write-only ops on more than the L2 run back to back instead, so that every launch pays the write-back of
its predecessor's dirty lines -- flushed, up to 126 MB of a launch's own writes would drain after its end
and go uncharged.

Algorithmic bytes (s = element size): in-place scalar/unary op 2*s*n; same-shape binary 3*s*n;
broadcast binary s*(n_out + n_A + n_B) (each operand's unique elements once); axis reduce
s*(outer*R*inner + outer*inner); flat reduce s*n + s; fused mean_l1_loss 2*s*n + s; reduce-to-shape
s*(rows*cols + cols); relu with mask 3*s*n; SGD update 3*s*n.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import _lib as L
from .meta import Meta, broadcast_params

_FLUSH = None
_FLUSH_READ = None


def _flush_l2(dev):
    """Evicts the timed op's data from L2: a 256 MiB buffer is WRITTEN (larger than L2), then a second
    256 MiB buffer is READ.  The read pass matters: L2 is write-back, so after the write alone about
    126 MB of dirty lines would be written out during the op that follows, charging it up to ~18 us of
    DRAM traffic that is not its own.  After the read pass L2 holds clean lines of unrelated data."""
    global _FLUSH, _FLUSH_READ
    if _FLUSH is None or _FLUSH.device != torch.device(dev):
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        _FLUSH_READ = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    _FLUSH.add_(1)
    torch.max(_FLUSH_READ)


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
    flush=True every call is preceded by an L2 flush (_flush_l2: a 256 MiB write, then a 256 MiB read
    so that no dirty lines are left) and the time of the same number of flushes alone is subtracted."""
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


def _sig(x, n=4):
    if not isinstance(x, float) or x == 0 or not math.isfinite(x):
        return x
    return round(x, n - 1 - int(math.floor(math.log10(abs(x)))))


def run(be, peak_gbs: float, world: int = 1, rank: int = 0, quick: bool = False):
    """-> rows {op, shape, ms, gbs, frac (of the measured copy peak), bytes [, l2: "flushed"] [, note]};
    elements/s = elements of `shape` / ms."""
    dev = f"cuda:{be.device}"
    rows = []

    def add(name, shape, nbytes, elems, fn, flush=False, note=None):
        med, best = _time(fn, flush=flush, dev=dev)
        gbs = nbytes / (med * 1e-3) / 1e9
        row = {"op": name, "shape": shape, "ms": _sig(med), "gbs": _sig(gbs), "frac": _sig(gbs / peak_gbs), "bytes": nbytes}
        if flush:
            row["l2"] = "flushed"
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

    def config2_step():
        be.scalar_apply(x, L.MUL, 3.0, m2)
        be.scalar_apply(x, L.ADD, 2.0, m2)
        be.scalar_apply(x, L.SUB, 1.0, m2)
        be.broadcast((ia, m2), (ib, m2), (io, m2), L.ADD)
    add("configs[1] step: f32 a*=3; a+=2; a-=1 and i32 a+b", f"2^{int(np.log2(n2))} per tensor", (3 * 8 + 12) * n2, 4 * n2,
        config2_step, note="four launches back to back")
    x.uniform_(-1, 1, generator=g)
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
                (lambda op=op, axis=axis: be.apply_reduce((src, msq), r1, axis, op)), flush=S * S * 4 < (1 << 30))
    # reductions over a strided view: an (S,S) window of an (S,2S) matrix, reduced in place, against
    # the reference's recipe for non-contiguous tensors (copy the view contiguous, then reduce)
    win = Meta.contiguous((S, 2 * S)).slice(1, S // 2, S // 2 + S, 1)
    for axis in (0, 1):
        add(f"sum_at({axis}) f32 over a strided window, no copy", f"({S},{S}) window of ({S},{2 * S})", 4 * (S * S + S), S * S,
            (lambda axis=axis: be.reduce_view(src, win, axis, L.SUM)), flush=S * S * 4 < (1 << 30))

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
        4 * (S * S + S), S * S, copy_then_reduce, flush=S * S * 4 < (1 << 30),
        note="algorithmic bytes of the reduction alone; the copy moves 2x more")
    # transposed views: contiguous() (the transposing tile kernel), a reduction along the view's
    # strided-then-dense dims in place, and a binary op with one transposed operand
    tview = msq.permute((1, 0))
    tmp_t = be.alloc(S * S, f32)
    add("contiguous() of a transposed matrix f32", f"({S},{S}) strides (1,{S})", 8 * S * S, S * S,
        lambda: be.contiguous(src, tview))
    for axis in (0, 1):
        add(f"sum_at({axis}) f32 over the transposed view, no copy", f"({S},{S}) strides (1,{S})", 4 * (S * S + S), S * S,
            (lambda axis=axis: be.reduce_view(src, tview, axis, L.SUM)), flush=S * S * 4 < (1 << 30))
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
                flush=S * S * 4 < (1 << 30))
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
        from . import sharding
        lo_f, hi_f = sharding.scalar_slab(nflat, world, rank)

        def sharded_sum_nccl():
            be.apply_reduce_contiguous_flat(src, r0, lo_f, hi_f - lo_f, L.SUM)
            be.mg_allreduce(r0, L.SUM)
        for name, fn in (("sum (full) f32, per-GPU partial + peer-memory exchange in the last CTA (rtb_mg_reduce_flat)",
                          lambda: be.mg_reduce_flat(src, lo_f, hi_f - lo_f, nflat, L.SUM, dst=r0)),
                         ("sum (full) f32, per-GPU partial + ncclAllReduce of one element", sharded_sum_nccl)):
            add(name, f"2^{int(np.log2(nflat))} over {world} GPUs", 4 * nflat + 4, nflat, fn,
                note=f"aggregate bytes / this rank's time; frac is of {world} x peak")
            rows[-1]["frac"] = _sig(rows[-1]["gbs"] / (peak_gbs * world))
        one = torch.ones(1, device=dev)
        t_peer, _ = _time(lambda: be.mg_combine(one, L.MAX), reps=20)
        t_nccl, _ = _time(lambda: be.mg_allreduce(one, L.MAX), reps=20)
        vec = torch.ones(8192, device=dev)
        t_peer_v, _ = _time(lambda: be.mg_combine(vec, L.MAX), reps=20)
        t_nccl_v, _ = _time(lambda: be.mg_allreduce(vec, L.MAX), reps=20)
        rows.append({"op": "combine of per-GPU partials alone: peer-memory exchange kernel vs ncclAllReduce", "shape": f"{world} GPUs",
                     "us_peer_4B": _sig(t_peer * 1e3), "us_nccl_4B": _sig(t_nccl * 1e3), "us_peer_32KiB": _sig(t_peer_v * 1e3),
                     "us_nccl_32KiB": _sig(t_nccl_v * 1e3), "peer_mapped": bool(be.mg_peer_mapped)})
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
    add("bias add + relu + mask in one pass f32 (rtb_bias_relu_mask)", "(4096,1024)+(1,1024)", 4 * (3 * Bt * H + H), Bt * H,
        lambda: be.bias_relu_mask(act, bias, Bt, H), flush=True)
    add("reduce_to_shape (bias grad) f32", "(4096,1024)->(1,1024)", 4 * (Bt * H + H), Bt * H,
        lambda: be.reduce_to_shape(act, (Bt, H), (0, 1)), flush=True)
    nw = 784 * 1024 + 1024 * 1024 + 1024 * 10 + 2058
    nw -= nw % 4
    w, gw = src[:nw], src[nw:2 * nw]
    add("sgd_update f32", f"{nw} params", 12 * nw, nw, lambda: be.sgd_update(w, gw, 0.0), flush=True)
    # ---- multi-GPU (strong scaling of single ops): an axis sum whose kept dim is cut needs no exchange;
    # the same sum with the REDUCED dim cut (data that already lives row-sharded) combines 32 KiB partials
    if world > 1:
        import torch.distributed as dist
        from . import sharding

        def add_sharded(name, shape, nbytes, elems, fn, note=None):
            med, best = _time(fn, flush=True, dev=dev)
            t = torch.tensor([med], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)  # slowest rank
            med = float(t.item())
            gbs = nbytes / (med * 1e-3) / 1e9
            rows.append({"op": name, "shape": shape, "ms": _sig(med), "gbs": _sig(gbs), "frac": _sig(gbs / (peak_gbs * world)),
                         "bytes": nbytes, "l2": "flushed",
                         "note": (note + "; " if note else "") + f"aggregate over {world} GPUs / slowest rank; frac is of {world} x peak"})
        for axis in (0, 1):
            add_sharded(f"sum_at({axis}) f32, kept dim cut by the partitioner, no exchange", f"({S},{S}) over {world} GPUs",
                        4 * (S * S + S), S * S, (lambda axis=axis: sharding.sharded_reduce_view(be, src, msq, axis, L.SUM, world, rank)))
        lo, hi = sharding.scalar_slab(S, world, rank)
        add_sharded("sum_at(0) f32, rows resident per GPU: partial vector + peer-memory combine (rtb_mg_reduce_axis)",
                    f"({S},{S}) over {world} GPUs", 4 * (S * S + S), S * S,
                    lambda: be.mg_reduce_axis(src, lo * S, 1, hi - lo, S, S, L.SUM))
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
                 "shape": f"({cr},1)+(1,{cc}), *=, relu, sum_at(0), var_at(1), fused add+sum_at(1)", "ms": _sig(med_g),
                 "ms_eager": _sig(med_e), "note": "same kernels, same results; the graph removes the host cost of six enqueues"})

    # ---- config 5 as a whole: one SGD step of the 784-1024-1024-10 MLP, global batch 4096 split
    # across the ranks (data parallel: loss all-reduce + one flat gradient bucket all-reduce)
    from .mlp import DenseMlp, synthetic_batch
    torch.backends.cuda.matmul.allow_tf32 = False
    sizes = (784, 1024, 1024, 10)
    model = DenseMlp(be, sizes, lr=0.01)
    local_b = 4096 // world
    img, tgt, _, _ = synthetic_batch(local_b, dev, rank=rank)
    med, best = _time(lambda: model.step(img, tgt, 4096), reps=5, rounds=5)
    gemm_flops = 2 * 4096 * (784 * 1024 + 1024 * 1024 + 1024 * 10) * 3 - 2 * 4096 * 784 * 1024
    # the step's library GEMMs alone (same shapes and operand layouts), and its gradient all-reduces alone
    xs = [torch.randn(local_b, n, device=dev) for n in sizes]

    def gemms():
        for li in range(3):
            torch.matmul(xs[li], model.weight(li))
            torch.matmul(xs[li].t(), xs[li + 1], out=model.grad_weight(li))
            if li:
                torch.matmul(xs[li + 1], model.weight(li).t())
    t_gemm, _ = _time(gemms, reps=5, rounds=5)
    t_ar = 0.0
    if world > 1:
        def buckets():
            for li in reversed(range(3)):
                be.mg_allreduce(model.layer_bucket(li), L.SUM)
        t_ar, _ = _time(buckets, reps=5, rounds=5)
    model.step_graphed(img, tgt, 4096)  # eager step + capture (all ranks capture the same sequence)
    med_g, best_g = _time(lambda: model.step_graphed(img, tgt, 4096), reps=5, rounds=5)
    for v in (med, med_g, t_gemm, t_ar):
        pass
    if world > 1:
        import torch.distributed as dist
        tt = torch.tensor([med, med_g, t_gemm, t_ar], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        med, med_g, t_gemm, t_ar = [float(v) for v in tt.tolist()]
    rows.append({"op": "MLP SGD step 784-1024-1024-10 (GEMMs on cuBLAS, rest on this library)",
                 "shape": f"global batch 4096, {local_b} per GPU x {world}", "ms": _sig(med), "ms_graph": _sig(med_g),
                 "ms_gemms_alone": _sig(t_gemm), "ms_allreduce_alone": _sig(t_ar),
                 "ms_rest": _sig(max(med_g - t_gemm, 0.0)), "samples_per_s": _sig(4096 / (med_g * 1e-3)),
                 "gemm_tflops": _sig(gemm_flops / world / (t_gemm * 1e-3) / 1e12),
                 "note": "ms = eager from Python, ms_graph = one CUDA-graph launch per step (collectives captured); ms_rest = ms_graph - "
                         "GEMMs alone = this library's kernels plus whatever of the gradient all-reduces (three per-layer buckets on a "
                         "side stream) is not hidden behind the backward GEMMs"})
    # ---- how time grows with size for three bandwidth-bound kernels: the fixed part (launch, ramp to full DRAM
    #      throughput, tail, the last CTA's fold) is what separates a 134 MB op from a 4 GB op of the same kernel
    if not quick and world == 1:
        curve = []
        big = torch.empty(1 << 28, device=dev, dtype=f32).normal_(generator=g)
        dst = torch.empty(1 << 27, device=dev, dtype=f32)
        one = be.alloc(1, f32)
        for lg in (23, 25, 26, 28):
            n = 1 << lg
            mflat = Meta.contiguous((n,))
            t_sum, _ = _time(lambda: be.apply_reduce_contiguous_flat(big, one, 0, n, L.SUM), flush=True, dev=dev)
            t_fill, _ = _time(lambda: be.fill(big, 1.0, mflat), flush=True, dev=dev)
            entry = {"bytes": 4 * n, "us_full_sum": _sig(t_sum * 1e3), "us_fill": _sig(t_fill * 1e3)}
            if n <= dst.numel():
                t_copy, _ = _time(lambda: dst[:n].copy_(big[:n]), flush=True, dev=dev)
                entry["us_torch_copy_of_the_same_bytes_read"] = _sig(t_copy * 1e3)
            curve.append(entry)
        # least-squares line t = t0 + bytes / bw through the full-sum points
        xs = np.array([c["bytes"] for c in curve], dtype=np.float64)
        ys = np.array([c["us_full_sum"] for c in curve], dtype=np.float64)
        slope, t0 = np.polyfit(xs, ys, 1)
        rows.append({"op": "time against size: full sum (read), fill (write), torch device copy (read + write of the same element count)",
                     "shape": "2^23 .. 2^28 f32", "points": curve, "full_sum_fit_us": _sig(float(t0)),
                     "full_sum_fit_gbs": _sig(1e-3 / float(slope)), "l2": "flushed",
                     "note": "full_sum_fit_us = the size-independent part of a one-wave reduction's time; every op of a few "
                             "hundred MB carries it, which is why their fractions sit below the multi-GB ops'; the fill points are optimistic by up "
                             "to 126 MB of write-back that drains from L2 after the kernel has ended"})
        del big, dst
    torch.cuda.synchronize()
    return rows


def small_case(be, which: str, arg=None):
    """Small cases of the hot-path kernels for profiling (a few hundred MB -- larger than L2 -- and a
    handful of launches, so that an `ncu` capture ends by itself in a minute or two).  Run as
    `python bench.py --case NAME [--case-arg K]`:
      flat       the config-2 chain (f32 a*=3; a+=2; a-=1 and i32 a+b) on 2^K elements per tensor (default 26), 5 times
      c3         strided / negative-step broadcast add with K rows in dim 2 (default 64), 4 launches
      red        axis sums of (8192,8192) over both axes and of (16,4096,1024) over axis 1, 3 launches each
      ext        variance / logsumexp / L2 norm / argmax of (8192,8192) over both axes, twice each
      convert    dtype conversion of 2^26 elements: f32->f64, f32->i32, u8->f32, f32->u8, twice each
      transpose  contiguous() of a transposed (8192,8192) f32 matrix and a.T + b, twice each
      host       the host-buffer lanes: 4 GiB copied out, 4 GiB uploaded and reduced, and both at once (prints ms)
      sum        full sums of 2^25 .. 2^28 f32, twice each, L2 flushed between
      l1         mean_l1_loss of two (4096,4096) without and with the gradient map, 3 times, L2 flushed between
      mid        mid-size ops (L1 loss, config-1 add and fused add+sum, bias add, reduce-to-shape) with L2 flushes
      mlp        the fused bias+relu+mask kernel, reduce-to-shape and SGD update at MLP sizes, L2 flushed between"""
    dev = f"cuda:{be.device}"
    f32 = torch.float32
    if which == "flat":
        n = 1 << (arg or 26)
        x = torch.rand(n, device=dev) * 2 - 1
        ia = torch.randint(-(1 << 20), 1 << 20, (n,), device=dev, dtype=torch.int32)
        ib = torch.randint(-(1 << 20), 1 << 20, (n,), device=dev, dtype=torch.int32)
        io = torch.empty_like(ia)
        m = Meta.contiguous((n,))
        for _ in range(5):
            be.scalar_apply(x, L.MUL, 3.0, m)
            be.scalar_apply(x, L.ADD, 2.0, m)
            be.scalar_apply(x, L.SUB, 1.0, m)
            be.broadcast((ia, m), (ib, m), (io, m), L.ADD)
    elif which == "c3":
        K = arg or 64
        bufa = torch.rand(K * 16, device=dev) * 2 - 1
        bufb = torch.rand(64 * 1024, device=dev) * 2 - 1
        Am = Meta.contiguous((K, 16, 1, 1)).view_as((1, K, 16, 1)).permute((2, 0, 1, 3))
        Bm = Meta.contiguous((1, 64, 1, 1024)).slice(3, None, None, -1)
        shape, sa, sb = broadcast_params(Am, Bm)
        dm = Meta.contiguous(shape)
        out = be.alloc(dm.size, f32)
        for _ in range(4):
            be.broadcast((bufa, Meta(shape, sa, Am.offset)), (bufb, Meta(shape, sb, Bm.offset)), (out, dm), L.ADD)
    elif which == "red":
        S = 8192
        src = torch.randn(S * S, device=dev)
        m = Meta.contiguous((S, S))
        r1 = be.alloc(S, f32)
        for _ in range(3):
            be.apply_reduce((src, m), r1, 0, L.SUM)
            be.apply_reduce((src, m), r1, 1, L.SUM)
        m3 = Meta.contiguous((16, 4096, 1024))
        r3 = be.alloc(16 * 1024, f32)
        for _ in range(3):
            be.apply_reduce((src, m3), r3, 1, L.SUM)
    elif which == "ext":
        S = 8192
        src = torch.randn(S * S, device=dev)
        m = Meta.contiguous((S, S))
        r1, ri = be.alloc(S, f32), be.alloc(S, torch.int64)
        for op, out in ((L.VARIANCE, r1), (L.LOGSUMEXP, r1), (L.NORM, r1), (L.ARGMAX, ri)):
            for axis in (0, 1):
                for _ in range(2):
                    be.apply_reduce_ex((src, m), out, axis, op, True, False, 2)
    elif which == "convert":
        n = 1 << 26
        x = torch.randn(n, device=dev) * 100
        u = torch.randint(0, 255, (n,), device=dev, dtype=torch.uint8)
        o64, o32, o8 = be.alloc(n, torch.float64), be.alloc(n, torch.int32), be.alloc(n, torch.uint8)
        for _ in range(2):
            be.convert(x, torch.float64, out=o64)
            be.convert(x, torch.int32, out=o32)
            be.convert(u, f32, out=x)
            be.convert(x, torch.uint8, out=o8)
    elif which == "transpose":
        S = 8192
        a, b = torch.randn(S * S, device=dev), torch.randn(S * S, device=dev)
        out = be.alloc(S * S, f32)
        m = Meta.contiguous((S, S))
        for _ in range(2):
            be.contiguous(a, m.permute((1, 0)))
            be.broadcast((a, m.permute((1, 0))), (b, m), (out, m), L.ADD)
    elif which == "host":
        # the host-buffer lanes alone: 4 GiB result copied out by rtb_host_broadcast, a 4 GiB input uploaded and
        # reduced, and both in either order (CUDA events over 3 repetitions each; prints one line of ms)
        import json
        n0, per = 64, 1 << 24
        h_a, h_b = torch.randn(per).pin_memory(), torch.randn(per).pin_memory()
        am, bm = Meta((n0, per), (0, 1), 0), Meta.contiguous((per,))
        h_out = torch.empty(n0 * per).pin_memory()
        h_f = torch.randn(1 << 30).pin_memory()
        h_r = torch.empty(1).pin_memory()
        r = be.alloc(1, f32)

        def bc():
            be.host_broadcast(h_a, am, h_b, bm, L.ADD, h_out)

        def red():
            blk = be.host_stage_in(h_f)
            be.host_ready(blk)
            be.apply_reduce_contiguous_flat(blk, r, 0, h_f.numel(), L.SUM)
            be.host_stage_out(r, h_r)
            be.host_release(blk)

        def timed(fn, reps=3):
            fn()
            be.host_join()
            torch.cuda.synchronize()
            s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_.record()
            for _ in range(reps):
                fn()
                be.host_join()
            e_.record()
            torch.cuda.synchronize()
            return round(s_.elapsed_time(e_) / reps, 1)
        be.sync_stream()
        print(json.dumps({"case": "host", "bytes_each_way": 4 << 30,
                          "ms_broadcast_to_host_alone": timed(bc), "ms_upload_and_reduce_alone": timed(red),
                          "ms_broadcast_then_reduce": timed(lambda: (bc(), red())),
                          "ms_reduce_then_broadcast": timed(lambda: (red(), bc()))}))
    elif which == "sum":
        # full sums of 2^25, 2^26 and 2^27 f32 (one CTA per 32 KiB block) and of 2^28 (one wave), L2 flushed between
        src = torch.randn(1 << 28, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        one = be.alloc(1, f32)
        for _ in range(2):
            for lg in (25, 26, 27, 28):
                flush.add_(1)
                be.apply_reduce_contiguous_flat(src, one, 0, 1 << lg, L.SUM)
    elif which in ("l1", "mid", "mlp"):
        n = 4096 * 4096
        src = torch.randn(2 * n, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        A, B = torch.rand(4096, device=dev), torch.rand(4096, device=dev)
        am, bm = Meta.contiguous((4096, 1)), Meta.contiguous((1, 4096))
        shape, sa, sb = broadcast_params(am, bm)
        dm = Meta.contiguous(shape)
        bias = torch.zeros(1024, device=dev)
        act = src[:4096 * 1024]
        for _ in range(3):
            flush.add_(1)
            be.l1_loss(src[:n], src[n:], 0, False)
            flush.add_(1)
            be.l1_loss(src[:n], src[n:], 0, True)
            if which == "mid":
                flush.add_(1)
                be.broadcast((A, Meta(shape, sa, 0)), (B, Meta(shape, sb, 0)), (src[:n], dm), L.ADD)
                flush.add_(1)
                be.apply_reduce((src[:n], dm), be.alloc(4096, f32), 1, L.SUM)
                flush.add_(1)
                be.broadcast_reduce(A, am, B, bm, L.ADD, 1, L.SUM)
                flush.add_(1)
                be.broadcast_reduce(A, am, B, bm, L.ADD, 0, L.SUM)
            if which in ("mid", "mlp"):
                flush.add_(1)
                be.binary_assign(act, Meta.contiguous((4096, 1024)), bias, Meta.contiguous((1, 1024)), L.ADD)
                flush.add_(1)
                be.bias_relu_mask(act, bias, 4096, 1024)
                flush.add_(1)
                be.reduce_to_shape(act, (4096, 1024), (0, 1))
                flush.add_(1)
                be.sgd_update(src[:1 << 21], src[1 << 21: 1 << 22], 0.0)
    else:
        raise SystemExit(f"unknown case {which!r}")
    torch.cuda.synchronize()
    print(f"case {which}: {be.launches} launches, done")
