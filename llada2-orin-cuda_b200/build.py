"""Builds libllattn.so (the C-ABI library) in-tree with nvcc for sm_100a. nvcc cross-compiles without a GPU."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libllattn.so")

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared", "-I", os.path.join(ROOT, "include")]


def sources():
    return [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh", ".inl"))] + \
           [os.path.join(ROOT, "include", "llattn.h")]


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/llattn.cu -> libllattn.so when any source is newer than the library. Returns the path."""
    srcs = sources()
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(s) for s in srcs):
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    tmp = LIB + ".building"                      # the library appears in one step: a reader never sees half a file
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [os.path.join(CSRC, "llattn.cu"), "-o", tmp]
    subprocess.check_call(cmd)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
