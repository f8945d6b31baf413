"""Compile the CUDA / C++ sources under csrc/ into the in-tree shared library (sm_100a only)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200moe.so")
CLI = os.path.join(HERE, "b2-debug-logits")        # the reference's `aegist debug-logits` over the C ABI
SOURCES = ["engine.cu"]
HEADERS = sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".hpp"))) + ["../../include/b200moe.h"]


def nvcc() -> str:
    for p in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if p and (os.path.isabs(p) and os.path.exists(p) or not os.path.isabs(p)):
            return p
    raise RuntimeError("nvcc not found")


def stale() -> bool:
    if not os.path.exists(LIB) or not os.path.exists(CLI):
        return True
    t = min(os.path.getmtime(LIB), os.path.getmtime(CLI))
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS + ["debug_logits.cpp"])


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not stale():
        return LIB
    cmd = [nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC,-O3", "-Xptxas", "-v" if verbose else "-warn-spills",
           "-I/usr/include", "-ldl", "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed")
    # the command-line parity driver: plain C++ over the C ABI, finds the library beside itself
    cmd = ["g++", "-O2", "-std=c++17", "-o", CLI, os.path.join(CSRC, "debug_logits.cpp"), "-L" + HERE, "-lb200moe",
           "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("g++ failed on debug_logits.cpp")
    return LIB


if __name__ == "__main__":
    build(verbose=True, force=True)
    print(LIB)
