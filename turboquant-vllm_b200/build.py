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


def _deps() -> list[str]:
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + [
        os.path.join(ROOT, "include", "tq4.h")]


def needs_build() -> bool:
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    return any(os.path.getmtime(d) > t for d in sources() + _deps())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu to an object file (in parallel, only those older than their inputs) and
    link the shared library."""
    if not force and not needs_build():
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    flags = ["-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo",
             "-gencode", "arch=compute_100a,code=sm_100a",
             "-I", os.path.join(ROOT, "include"), "-I", CSRC]
    if verbose:
        flags += ["-Xptxas", "-v"]
    hdr_time = max(os.path.getmtime(d) for d in _deps())
    jobs, objs = [], []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        stale = force or verbose or not os.path.exists(obj) or os.path.getmtime(obj) < max(
            os.path.getmtime(src), hdr_time)
        if stale:
            jobs.append((src, subprocess.Popen([nvcc, "-c", *flags, "-o", obj, src])))
    failed = [src for src, p in jobs if p.wait() != 0]
    if failed:
        raise subprocess.CalledProcessError(1, f"nvcc -c {' '.join(failed)}")
    subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", OUT, *objs], check=True)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
