"""Builds libaspen_b200.so (host library + sm_100a kernels) in-tree with nvcc.

`python -m aspen_b200.build` or `aspen_b200.build.build()`.  The shared library is the product's
C ABI (include/aspen_b200.h); it links the CUDA runtime statically and resolves the one driver
entry point it needs at run time, so it loads on machines without a GPU driver (where only the
host-side graph functions work).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libaspen_b200.so")
SOURCES = ["cfg.cpp", "dnn.cpp", "tiler.cpp", "graph.cpp", "runtime.cpp", "engine.cu", "noalloc.cu"]
HEADERS = ["internal.h", "device_types.h", "tiles_simt.cuh", "tiles_tc.cuh", "scheduler.cuh",
           os.path.join("..", "..", "include", "aspen_b200.h")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-Wall", "-Xcompiler", "-Wno-unused-function", "-cudart", "static"] + os.environ.get("ASPEN_B200_NVCC_FLAGS", "").split()


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    objs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, os.path.splitext(src)[0] + ".o")
        cmd = [NVCC, *FLAGS, "-x", "cu", "-c", os.path.join(CSRC, src), "-o", obj]
        if src.endswith(".cu") and verbose:
            cmd.insert(1, "-Xptxas=-v")
        subprocess.run(cmd, check=True)
        objs.append(obj)
    subprocess.run([NVCC, *FLAGS, "-shared", "-Xlinker", "-Bsymbolic", "-o", LIB, *objs, "-lpthread", "-ldl", "-lrt"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
