"""Builds rtensors_b200/librt_b200.so from csrc/ with nvcc for sm_100a (in-tree, no JIT cache).

    python -m rtensors_b200.build [--force] [--verbose]

Float flags: --fmad=false --prec-div=true --prec-sqrt=true and no fast-math, so every float
elementwise op is the single IEEE operation the reference CPU backend performs (the reference's
own release build uses --use_fast_math --fmad=true, libs/rtensors/build.rs:455-464).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(PKG, "librt_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-std=c++17", "-O3", "-lineinfo", "--fmad=false", "--prec-div=true", "--prec-sqrt=true",
          "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-I", os.path.join(ROOT, "include"), "-I", CSRC]

EW_DTYPES = list(range(13))
PLAIN = ["rtb_planner.cpp", "rtb_context.cpp", "rtb_api.cpp", "rtb_host.cpp", "rtb_abi_v1.cpp", "rtb_reduce.cu", "rtb_reduce_ext.cu", "rtb_noalloc.cu", "rtb_mg.cu",
         "rtb_convert.cu"]


def _units():
    units = []
    for name in PLAIN:
        src = os.path.join(CSRC, name)
        if os.path.exists(src):
            units.append((src, os.path.join(OBJ, name.rsplit(".", 1)[0] + ".o"), []))
    for code in EW_DTYPES:
        units.append((os.path.join(CSRC, "rtb_ew_impl.cu"), os.path.join(OBJ, f"rtb_ew_{code}.o"),
                      [f"-DRTB_EW_DTYPE={code}"]))
    return units


def _newest_header() -> float:
    t = 0.0
    for d in (CSRC, os.path.join(ROOT, "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh", ".inl")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return max(t, os.path.getmtime(os.path.abspath(__file__)))


def _compile(unit, verbose):
    src, obj, extra = unit
    cmd = [NVCC, *ARCH, *COMMON, *extra, "-x", "cu", "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src} {extra}:\n{p.stdout}\n{p.stderr}")
    return p.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr = _newest_header()
    todo = []
    units = _units()
    for u in units:
        src, obj, _ = u
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr):
            todo.append(u)
    if todo:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            for log in ex.map(lambda u: _compile(u, verbose), todo):
                if verbose and log:
                    print(log, file=sys.stderr)
    objs = [u[1] for u in units]
    if todo or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [NVCC, *ARCH, "-shared", "-o", LIB, *objs, "-Xcompiler", "-fPIC", "-ldl"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"link failed:\n{p.stdout}\n{p.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
