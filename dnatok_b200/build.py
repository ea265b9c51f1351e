"""Build ``libdnatok_b200.so`` (nvcc, sm_100a) and the host packer ``_pack.so`` (gcc, CPython API) in-tree.

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


PACK_SRC = os.path.join(CSRC, "pack_module.c")
PACK_OUT = os.path.join(HERE, "_pack.so")


def build_packer(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(PACK_OUT) and os.path.getmtime(PACK_OUT) >= os.path.getmtime(PACK_SRC):
        return PACK_OUT
    import sysconfig
    cmd = [os.environ.get("CC", "gcc"), "-O3", "-shared", "-fPIC", "-pthread", "-I", sysconfig.get_paths()["include"],
           "-o", PACK_OUT, PACK_SRC]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return PACK_OUT


def build(force: bool = False, verbose: bool = False) -> str:
    build_packer(force, verbose)
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
