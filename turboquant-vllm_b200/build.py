"""Build libtq4_sm100a.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Usage:  python turboquant-vllm_b200/build.py [--force] [--verbose]
The library lands in turboquant-vllm_b200/turboquant_vllm/lib/ where the Python host code
loads it with ctypes.  No torch headers are involved: the ABI is plain C (include/tq4.h).
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "turboquant_vllm", "lib")
OUT = os.path.join(OUT_DIR, "libtq4_sm100a.so")


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def needs_build() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(ROOT, "include", "tq4.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [
        nvcc, "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-I", os.path.join(ROOT, "include"), "-I", CSRC,
        "-o", OUT,
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += sources()
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
