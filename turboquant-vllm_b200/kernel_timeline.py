"""Timelines of the attention and cache-write kernels from a tuning build of the library (B200).

    python turboquant-vllm_b200/kernel_timeline.py decode     # paged decode step, batch 64 x 4096 tokens
    python turboquant-vllm_b200/kernel_timeline.py prefill    # tcgen05 chunked prefill, 8 x 2048 on 8192
    python turboquant-vllm_b200/kernel_timeline.py compress   # tcgen05 cache write, 16 384 tokens x 8 heads

Builds `turboquant_vllm/lib/libtq4_sm100a_trace.so`: the same sources with `-DTQ4_TRACE`, which compiles
time stamps into `attention_mma_kernel` (`%globaltimer` at its phases, lane 0 of every warp of every
CTA), `prefill_tc_kernel` (SM clock at points of the tile loop, four warps of one CTA) and
`compress_tc16_kernel` (SM clock at the hand-overs of its tile pipeline, four warps of CTA 0) and
exports the functions that read them back.  The shipped library has neither.  The workloads are the ones
`bench.py` times; the decode timeline is taken with the prologue inside the attention kernel
(`TQ4_FUSED_PROLOGUE=1`), the form whose single kernel shows every phase of a step.
"""
from __future__ import annotations

import ctypes
import glob
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
TRACE_LIB = os.path.join(HERE, "turboquant_vllm", "lib", "libtq4_sm100a_trace.so")


def build_trace_library() -> str:
    obj_dir = os.path.join(HERE, "build", "trace")
    os.makedirs(obj_dir, exist_ok=True)
    os.makedirs(os.path.dirname(TRACE_LIB), exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    flags = ["-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
             "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-DTQ4_TRACE"]
    deps = glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(ROOT, "include", "tq4.h")]
    newest_dep = max(os.path.getmtime(d) for d in deps)
    jobs, objs = [], []
    for src in sorted(glob.glob(os.path.join(CSRC, "*.cu"))):
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), newest_dep):
            jobs.append((src, subprocess.Popen([nvcc, "-c", *flags, "-o", obj, src])))
    for src, job in jobs:
        if job.wait() != 0:
            raise SystemExit(f"nvcc failed on {src}")
    if jobs or not os.path.exists(TRACE_LIB):
        subprocess.check_call([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", TRACE_LIB, *objs])
    return TRACE_LIB


def _load(kind: str):
    """The package bound to the trace library (before anything else loads the shipped one)."""
    for p in (ROOT, HERE):
        if p not in sys.path:
            sys.path.insert(0, p)
    from turboquant_vllm import _native as nv

    nv._LIB_PATH = build_trace_library()
    reader = {"decode": "tq4_trace_read", "prefill": "tq4_prefill_trace_read", "compress": "tq4_compress_trace_read"}[kind]
    nv._SIGNATURES[reader] = (ctypes.c_int, [ctypes.c_void_p])
    return nv, reader


def decode_timeline() -> None:
    os.environ["TQ4_FUSED_PROLOGUE"] = "1"
    nv, reader = _load("decode")
    import torch

    import bench
    from turboquant_vllm.kernels import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    wl = bench.build_workload(dev, 1, 2)
    batch, hkv, hq = wl["batch"], wl["hkv"], wl["hq"]
    q, k, v = wl["q_host"].to(dev), wl["k_host"].to(dev), wl["v_host"].to(dev)
    out = torch.empty(batch, hq, 128, dtype=torch.bfloat16, device=dev)
    ws = torch.empty(ops.attention_workspace_bytes(batch, hq, hkv, 128), dtype=torch.uint8, device=dev)
    for i in range(5):
        ops.tq4_write_and_attention(k, v, wl["new_slots"], wl["even"], wl["odd"], wl["kb"], wl["vb"], q,
                                    wl["caches"][i % 2], wl["block_table"], wl["seq_lens"], wl["kc"], wl["vc"],
                                    wl["rot"], hkv, 16, None, out=out, workspace=ws)
    torch.cuda.synchronize()
    buf = np.zeros(160 * 16 * 16, dtype=np.int64)
    assert getattr(nv.lib(), reader)(buf.ctypes.data) == 0
    t = buf.reshape(160, 16, 16)[:148].astype(np.float64)
    t = (t - t[:, :, 0].min()) / 1e3  # us since the first warp entered the kernel
    names = {0: "kernel entry", 1: "tile plan in registers", 2: "Pi and the CTA's vectors staged",
             8: "last rotation task of the warp starts", 9: "... and ends", 3: "rotated, written, block barrier",
             4: "dequantisation table built", 5: "first tile pair consumed", 6: "last segment streamed",
             7: "partials stored"}
    print("us since kernel entry over all warps of the 148 CTAs:   min / median / max")
    for i, name in names.items():
        x = t[:, :, i]
        x = x[x > -1e6]
        if x.size:
            print(f"  {name:40s} {x.min():7.2f} {np.median(x):7.2f} {x.max():7.2f}")


def prefill_timeline() -> None:
    nv, reader = _load("prefill")
    import torch

    import bench
    from turboquant_vllm.kernels import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    r = bench.prefill_case(dev, ops, hq=32, hkv=8, d=128, window=None, modes=(("tcgen05", 3, 2),))
    print("config 4a on the traced build:", r["tcgen05"])
    torch.cuda.synchronize()
    buf = np.zeros(4 * 64 * 16, dtype=np.int64)
    assert getattr(nv.lib(), reader)(buf.ctypes.data) == 0
    t = buf.reshape(4, 64, 16).astype(np.float64)
    warps = ["softmax warp 0", "softmax warp 4", "first dequantising warp (issues the MMAs)",
             "last dequantising warp (issues copies)"]
    softmax = ["top", "S ready", "scores", "row maximum exchanged", "PV of the previous tile done",
               "P in tensor memory", None, "block barrier passed", "end of iteration"]
    dequant = ["top", "packed stage landed", "keys dequantised", "S of the next tile issued",
               "PV of the previous tile done", "values dequantised", None, "block barrier passed",
               "PV issued / end of iteration"]
    for w in range(4):
        events = softmax if w < 2 else dequant
        rows = [[t[w, j, e] - t[w, j, 0] for e in range(9)] + [t[w, j + 1, 0] - t[w, j, 0]] for j in range(20, 50)]
        m = np.mean(np.array(rows), axis=0)
        print(f"== {warps[w]}: SM cycles since the top of the iteration (mean of iterations 20..49)")
        for e in range(9):
            if events[e] is not None and abs(m[e]) < 1e9:
                print(f"   {events[e]:32s} {m[e]:8.0f}")
        print(f"   {'next top':32s} {m[9]:8.0f}")


def compress_timeline() -> None:
    nv, reader = _load("compress")
    import torch

    from turboquant_vllm.kernels import ops
    from turboquant_vllm.quantizer import TurboQuantMSE

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    nt, hkv, d, bs = 16384, 8, 128, 16
    rot, even, odd, kc, kb = TurboQuantMSE(d, 4, seed=42).device_primitives(dev)
    g = torch.Generator(device=dev).manual_seed(3)
    k = torch.randn(nt, hkv, d, device=dev, generator=g).bfloat16()
    v = torch.randn(nt, hkv, d, device=dev, generator=g).bfloat16()
    cache = torch.zeros(nt // bs, bs, hkv * 256, dtype=torch.uint8, device=dev)
    slots = torch.randperm(nt, device=dev, generator=g)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        e0.record()
        ops.tq4_write_paged(k, v, cache, slots, even, odd, kb, kb)
        e1.record()
    torch.cuda.synchronize()
    print(f"write of {nt} tokens x {hkv} heads, K and V: {e0.elapsed_time(e1) * 1e3:.1f} us on the traced build")
    buf = np.zeros(4 * 32 * 8, dtype=np.int64)
    assert getattr(nv.lib(), reader)(buf.ctypes.data) == 0
    t = buf.reshape(4, 32, 8).astype(np.float64)
    t0 = t[0, 31, 6]
    print(f"CTA 0, SM cycles since kernel entry; set-up (Pi converted, tensor memory allocated) done at {t[0, 31, 7] - t0:.0f}")
    print("tile | stage free, copy issued | rows landed + accumulator free, MMAs issued | group: rows landed, norm done, "
          "product ready, tile stored")
    for i in range(14):
        p, m, e = t[0, i] - t0, t[1, i] - t0, t[2 + (i & 1), i] - t0
        ep = "  ".join(f"{x:7.0f}" for x in e[:4]) if abs(e[0]) < 1e9 else "(group not traced)"
        print(f"{i:4d} | {p[0]:7.0f} | {m[0]:7.0f} {m[1]:7.0f} | {ep}")


if __name__ == "__main__":
    modes = {"decode": decode_timeline, "prefill": prefill_timeline, "compress": compress_timeline}
    if len(sys.argv) != 2 or sys.argv[1] not in modes:
        raise SystemExit(__doc__)
    modes[sys.argv[1]]()
