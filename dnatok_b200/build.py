"""Build ``libdnatok_b200.so`` in-tree with nvcc for sm_100a.

    python -m dnatok_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(CSRC, "libdnatok_b200.so")
SOURCES = ["dnatok_abi.cu", "bpe_table.cc"]
DEPS = SOURCES + ["common.cuh", "emit_kernel.cuh", "embed_kernel.cuh", "kmer_kernel.cuh", "bpe_kernel.cuh", "bpe_table.h",
                  os.path.join("..", "..", "include", "dnatok_b200.h")]


def nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def stale() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(os.path.join(CSRC, d)) > t for d in DEPS)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return OUT
    cmd = [nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "--expt-extended-lambda", "-Xcompiler", "-fPIC", "-shared", "-o", OUT] + SOURCES
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    subprocess.check_call(cmd, cwd=CSRC)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
