"""Compile the CUDA sources of this package into ``libhapx.so`` (in-tree, sm_100a only).

Usage: ``python hap_b200/csrc/build.py [--force] [--verbose]``.  This file is a stand-alone
script (it does not import the package, which needs the library it builds).  The library
is built with nvcc directly; there is no JIT cache and no fallback when it is missing.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(CSRC)
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libhapx.so")
SOURCES = ["hapx_comm.cu", "hapx_collectives.cu", "hapx_gemm_sm100.cu", "hapx_attention.cu", "hapx_attention_fused.cu", "hapx_sgemm.cu", "hapx_optim.cu", "hapx_loss.cu", "hapx_norm.cu", "hapx_dropout.cu", "hapx_moe.cu", "hapx_sharding.cpp"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def sources():
    extra = [f for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cpp")) and f not in SOURCES]
    return [os.path.join(CSRC, f) for f in SOURCES + extra]


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".h")]
    deps.append(os.path.join(ROOT, "include", "hapx.h"))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Build ``libhapx.so`` if it is missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB
    cmd = [_nvcc(), "-O3", "-std=c++17", *ARCH_FLAGS, "-lineinfo", "-Xcompiler", "-fPIC", "-shared",
           "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-o", LIB, *sources()]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), file=sys.stderr)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libhapx.so")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
