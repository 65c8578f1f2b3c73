"""Builds libsage_b200.so (the C-ABI library declared in include/sage_b200.h) for sm_100a, and
libsage_b200_torch.so (the torch operators registered over it, csrc/torch_ops.cpp).

    python sageattention-autotune_b200/build.py [--force]

The C-ABI library is plain nvcc, no torch involved: it depends on the CUDA runtime only and resolves
the one driver entry point it needs (cuTensorMapEncodeTiled) at run time, so it loads on a machine
without a GPU driver too.  The operator library is one C++ file compiled with g++ against torch's
stable-ABI headers; it links libsage_b200.so from its own directory.  Objects are cached under
build/ and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "sageattention", "libsage_b200.so")
TORCH_LIB = os.path.join(HERE, "sageattention", "libsage_b200_torch.so")
# Host compiler of the operator library.  Deliberately not $CXX: the library must share the C++ run time
# (libstdc++.so) with torch, and a relocated toolchain that only ships libstdc++.a links a private
# copy in, after which an exception thrown by an operator kills the process instead of reaching Python.
CXX = os.environ.get("SAGE_B200_CXX", "g++")
SOURCES = ["api.cu", "quant.cu", "attn_fwd.cu", "peer.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-DSAGE_B200_BUILD"]


def _newest_header() -> float:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps.append(os.path.join(HERE, "..", "include", "sage_b200.h"))
    return max(os.path.getmtime(d) for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr = _newest_header()
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            jobs.append([NVCC, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", s, "-o", o])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=4) as ex:
        for log in ex.map(run, jobs):
            if verbose and log:
                print(log)
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in SOURCES]
    if jobs or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        run([NVCC, "-shared", "-o", LIB, *objs, "-cudart", "shared"])
    build_torch_ops(force)
    return LIB


def build_torch_ops(force: bool = False) -> str:
    """g++ on csrc/torch_ops.cpp: stable-ABI headers of the installed torch (target version 2.10, the
    first with the tensor-creation calls used), linked against libsage_b200.so beside it ($ORIGIN)."""
    import torch
    src = os.path.join(CSRC, "torch_ops.cpp")
    hdr = os.path.join(HERE, "..", "include", "sage_b200.h")
    if not force and os.path.exists(TORCH_LIB) and \
            os.path.getmtime(TORCH_LIB) >= max(os.path.getmtime(src), os.path.getmtime(hdr), os.path.getmtime(LIB)):
        return TORCH_LIB
    tdir = os.path.dirname(torch.__file__)
    cmd = [CXX, "-std=c++20", "-O2", "-fPIC", "-shared", "-DUSE_CUDA", "-DTORCH_TARGET_VERSION=0x020a000000000000",
           f"-I{tdir}/include", "-I/usr/local/cuda/include", src, "-o", TORCH_LIB,
           f"-L{os.path.dirname(LIB)}", "-l:libsage_b200.so", f"-L{tdir}/lib", "-ltorch", "-ltorch_cpu", "-lc10",
           "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    syms = subprocess.run(["nm", "-D", "--defined-only", TORCH_LIB], capture_output=True, text=True).stdout
    if " __cxa_throw" in syms:
        os.remove(TORCH_LIB)
        raise RuntimeError(f"{CXX} linked a private copy of the C++ run time into the operator library; "
                           "set SAGE_B200_CXX to a g++ that links libstdc++.so")
    return TORCH_LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
