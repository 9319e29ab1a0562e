"""Build the C-ABI library in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libevt_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def lib_sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".cu", ".cuh", ".h")):
                out.append(os.path.join(root, f))
    out.append(os.path.join(HERE, "..", "include", "evt_b200.h"))
    return out


def build_library(force: bool = False, verbose: bool = False) -> str:
    srcs = lib_sources()
    if not force and _newer(LIB, srcs):
        return LIB
    cmd = [NVCC, "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS,
           "-I", CSRC, "-o", LIB, os.path.join(CSRC, "evtb_api.cu"), os.path.join(CSRC, "fixed_kernels.cu"),
           os.path.join(CSRC, "bn_kernels.cu"),
           os.path.join(CSRC, "pool_kernels.cu")]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building libevt_b200.so:\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stderr)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
