"""Small cases of the hot-path kernels for profiling (a few hundred MB, larger than L2, a handful
of launches), so that an `ncu` capture ends by itself in a minute or two:

    python -m rtensors_b200.profile_cases c3 [K]   strided / negative-step broadcast add, K rows (default 64)
    python -m rtensors_b200.profile_cases red      axis sums of (8192,8192) and (16,4096,1024)
    python -m rtensors_b200.profile_cases ext      variance / logsumexp / L2 norm / argmax of (8192,8192) over both axes
    python -m rtensors_b200.profile_cases convert  dtype conversion of 2^26 elements: f32->f64, f32->i32, u8->f32, f32->u8 (twice each)
    python -m rtensors_b200.profile_cases transpose  contiguous() of a transposed (8192,8192) f32 matrix and a.T + b (twice each)
    python -m rtensors_b200.profile_cases mid      mid-size ops (and the fused broadcast+reduce) with an L2 flush between them
"""
import sys

import numpy as np
import torch

from . import _lib as L
from .backend import CudaB200
from .meta import Meta, broadcast_params


def main():
    which = sys.argv[1]
    be = CudaB200(0)
    dev='cuda:0'
    if which == 'c3':
        K = int(sys.argv[2]) if len(sys.argv) > 2 else 64
        bufa = torch.rand(K*16, device=dev)*2-1
        bufb = torch.rand(64*1024, device=dev)*2-1
        Am = Meta.contiguous((K,16,1,1)).view_as((1,K,16,1)).permute((2,0,1,3))
        Bm = Meta.contiguous((1,64,1,1024)).slice(3,None,None,-1)
        shape, sa, sb = broadcast_params(Am,Bm)
        dm = Meta.contiguous(shape)
        out = be.alloc(dm.size, torch.float32)
        for _ in range(4):
            be.broadcast((bufa, Meta(shape,sa,Am.offset)), (bufb, Meta(shape,sb,Bm.offset)), (out, dm), L.ADD)
    elif which == 'red':
        S = 8192
        src = torch.randn(S*S, device=dev)
        m = Meta.contiguous((S,S))
        r1 = be.alloc(S, torch.float32)
        for _ in range(3):
            be.apply_reduce((src,m), r1, 0, L.SUM)
            be.apply_reduce((src,m), r1, 1, L.SUM)
        m3 = Meta.contiguous((16,4096,1024))
        r3 = be.alloc(16*1024, torch.float32)
        for _ in range(3):
            be.apply_reduce((src,m3), r3, 1, L.SUM)
    elif which == 'ext':
        S = 8192
        src = torch.randn(S*S, device=dev)
        m = Meta.contiguous((S,S))
        r1 = be.alloc(S, torch.float32)
        ri = be.alloc(S, torch.int64)
        for op, args, out in ((L.VARIANCE, (True, False, 2), r1), (L.LOGSUMEXP, (True, False, 2), r1),
                              (L.NORM, (True, False, 2), r1), (L.ARGMAX, (True, False, 2), ri)):
            for axis in (0, 1):
                for _ in range(2):
                    be.apply_reduce_ex((src, m), out, axis, op, *args)
    torch.cuda.synchronize()
    print('done')
    if which == 'mid':
        n = 4096*4096
        src = torch.randn(2*n, device=dev)
        flush = torch.empty(256<<20, dtype=torch.uint8, device=dev)
        for _ in range(3):
            flush.add_(1)
            be.l1_loss(src[:n], src[n:], 0, False)
            flush.add_(1)
            be.l1_loss(src[:n], src[n:], 0, True)
            flush.add_(1)
            r0 = be.alloc(1, torch.float32)
            be.apply_reduce_contiguous_flat(src, r0, 0, 2*n, L.SUM)
            flush.add_(1)
            A = torch.rand(4096, device=dev); B = torch.rand(4096, device=dev)
            am, bm = Meta.contiguous((4096,1)), Meta.contiguous((1,4096))
            shape, sa, sb = broadcast_params(am,bm); dm = Meta.contiguous(shape)
            out = src[:n]
            be.broadcast((A, Meta(shape,sa,0)), (B, Meta(shape,sb,0)), (out, dm), L.ADD)
            flush.add_(1)
            bias = torch.zeros(1024, device=dev)
            act = src[:4096*1024]
            be.binary_assign(act, Meta.contiguous((4096,1024)), bias, Meta.contiguous((1,1024)), L.ADD)
            flush.add_(1)
            be.reduce_to_shape(act, (4096,1024), (0,1))
            flush.add_(1)
            red = be.alloc(4096, torch.float32)
            be.apply_reduce((src[:n], Meta.contiguous((4096,4096))), red, 1, L.SUM)
            flush.add_(1)
            be.broadcast_reduce(A, am, B, bm, L.ADD, 1, L.SUM)   # fused: no (4096,4096) intermediate
            flush.add_(1)
            be.broadcast_reduce(A, am, B, bm, L.ADD, 0, L.SUM)
        torch.cuda.synchronize()
        print('done mid')
    elif which == 'transpose':
        S = 8192
        a = torch.randn(S * S, device=dev)
        b = torch.randn(S * S, device=dev)
        out = be.alloc(S * S, torch.float32)
        m = Meta.contiguous((S, S))
        for _ in range(2):
            be.contiguous(a, m.permute((1, 0)))
            be.broadcast((a, m.permute((1, 0))), (b, m), (out, m), L.ADD)
        torch.cuda.synchronize()
        print('done transpose')
    elif which == 'convert':
        n = 1 << 26
        x = torch.randn(n, device=dev) * 100
        u = torch.randint(0, 255, (n,), device=dev, dtype=torch.uint8)
        o64, o32, o8 = be.alloc(n, torch.float64), be.alloc(n, torch.int32), be.alloc(n, torch.uint8)
        for _ in range(2):
            be.convert(x, torch.float64, out=o64)
            be.convert(x, torch.int32, out=o32)
            be.convert(u, torch.float32, out=x)
            be.convert(x, torch.uint8, out=o8)
        torch.cuda.synchronize()
        print('done convert')


if __name__ == "__main__":
    main()
