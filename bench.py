"""Benchmark of the TQ4 hot path: cache write of one new token per sequence + fused paged
TQ4 decode over the packed cache, one transformer layer per step.

Workload (N = 1): Llama-3.1-8B-shaped single-layer paged decode — batch 64, context 4096
each, 32 query / 8 KV heads, head_dim 128, block_size 16 with a seeded shuffled block table,
K4/V4 packed cache (vLLM padded rows) filled by the fused write kernel from N(0,1) K/V with
four outlier channels scaled x8, bf16 queries.  Several layer caches are rotated so the
working set is far larger than L2.
N > 1: KV heads are sharded across ranks (tensor parallel, no collective inside attention);
the global batch grows with N so per-GPU work is fixed (weak scaling).  The headline is the
CUDA-graph replay of the step; a block of --steps steps is repeated until the timed region is at
least --min-region seconds and the median block is reported.

After the headline the same line carries side measurements (each its own key):
`serving_mix` (K4/V3, batch 256, contexts ~U[512, 32768], heads divided over the N GPUs: strong
scaling), at N = 1 `long_context` (batch 8 x 131 072, head_dim 96) and `prefill` (chunked prefill,
head_dim 128 and 256), at N > 1 `split_kv` (the same long-context batch split by sequence over the
N GPUs, NCCL all-gather of partials + merge, with a parity check against the single-rank kernel
that fails the run if it does not hold) and `dense_rows` (the headline step on unpadded token rows).

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the
reference's PyTorch path (oracle/) on the host cores instead.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "turboquant-vllm_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

BATCH_PER_GPU_UNIT, CTX, HQ, HKV, D, BS = 64, 4096, 32, 8, 128, 16
K_BITS = V_BITS = 4
SEED = 0
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant (attention) kernel on
# the N = 1 workload.  A STORED figure from an ncu capture (the timed run cannot measure DRAM
# traffic): it is reported together with the name of the capture it comes from and only while the
# kernel build named there is the one that runs; otherwise `traffic` is null.
NCU_TRAFFIC = {"bytes": 308781824,  # dram__bytes_read.sum 304 016 384 + dram__bytes_write.sum 4 765 440
               "capture": "profiles/attention_mma_kernel_b64_ctx4096_ncu_full.md (form A: attention kernel "
                          "behind the prologue kernel, one launch, ncu --set full)"}


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_peak_tflops():
    """Burst bf16 GEMM peak of this pool's B200s (MEASURED_PEAKS.json), else the fallback 1590."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops"])
    except Exception:
        return 1590.0


# ----------------------------------------------------------------------------------------
# clocks sampling (read-only NVML)
# ----------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        names = {
            0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
            0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self._nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=1.0)
        med = int(statistics.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------
# workload
# ----------------------------------------------------------------------------------------
def primitives():
    from turboquant_vllm.quantizer import TurboQuantMSE

    kq = TurboQuantMSE(D, K_BITS, seed=42)
    vq = kq if V_BITS == K_BITS else TurboQuantMSE(D, V_BITS, seed=42)
    return kq, vq


def synth_kv_gpu(n, h, gen, device):
    k = torch.randn(n, h, D, device=device, generator=gen)
    v = torch.randn(n, h, D, device=device, generator=gen)
    for ch in (3, 17, 64, 101):
        k[..., ch] *= 8.0
        v[..., ch] *= 8.0
    return k.bfloat16(), v.bfloat16()


def build_workload(device, world, layers, row_bytes=0):
    """Per-rank state: `layers` packed caches filled through the fused write kernel."""
    from turboquant_vllm.kernels import ops

    batch = BATCH_PER_GPU_UNIT * world
    hkv, hq = HKV // world, HQ // world
    kq, vq = primitives()
    rot, even, odd, kc, kb = kq.device_primitives(device)
    _, _, _, vc, vb = vq.device_primitives(device)
    nblk = batch * CTX // BS
    slot = 1 << ((D + 8) - 1).bit_length()  # vLLM padded per-head slot (256 B at D=128)
    width = row_bytes or hkv * slot  # row_bytes: a denser token row than vLLM's padded page format
    gen = torch.Generator(device=device).manual_seed(SEED)
    perm = torch.randperm(nblk, device=device, generator=gen)
    block_table = perm.view(batch, CTX // BS).to(torch.int32).contiguous()
    seq_lens = torch.full((batch,), CTX, dtype=torch.int32, device=device)
    pos = torch.arange(CTX, device=device)
    caches = []
    chunk_seqs = max(1, 16384 // CTX)
    for _ in range(layers):
        cache = torch.zeros(nblk, BS, width, dtype=torch.uint8, device=device)
        for s0 in range(0, batch, chunk_seqs):
            s1 = min(batch, s0 + chunk_seqs)
            slots = (block_table[s0:s1].long()[:, pos // BS] * BS + (pos % BS)).reshape(-1)
            k, v = synth_kv_gpu(slots.numel(), hkv, gen, device)
            ops.tq4_write_paged(k, v, cache, slots, even, odd, kb, vb)
        caches.append(cache)
    # the token appended each step lives at position CTX-1 of every sequence
    new_slots = (block_table[:, (CTX - 1) // BS].long() * BS + (CTX - 1) % BS).contiguous()
    cpu_gen = torch.Generator().manual_seed(SEED + 1)
    q_host = torch.randn(batch, hq, D, generator=cpu_gen).bfloat16().pin_memory()
    k_host = torch.randn(batch, hkv, D, generator=cpu_gen).bfloat16().pin_memory()
    v_host = torch.randn(batch, hkv, D, generator=cpu_gen).bfloat16().pin_memory()
    return dict(batch=batch, hkv=hkv, hq=hq, rot=rot, even=even, odd=odd, kc=kc, kb=kb, vc=vc, vb=vb,
                caches=caches, block_table=block_table, seq_lens=seq_lens, new_slots=new_slots,
                q_host=q_host, k_host=k_host, v_host=v_host, width=width, nblk=nblk)


def run_ours(args, rank, world, device):
    from turboquant_vllm import _native as nv
    from turboquant_vllm.kernels import ops

    wl = build_workload(device, args.emulate_world or world, args.layers, args.row_bytes)
    batch, hkv, hq = wl["batch"], wl["hkv"], wl["hq"]
    q = wl["q_host"].to(device)
    k_new, v_new = wl["k_host"].to(device), wl["v_host"].to(device)
    out = torch.empty(batch, hq, D, dtype=torch.bfloat16, device=device)
    ws = torch.empty(ops.attention_workspace_bytes(batch, hq, hkv, D), dtype=torch.uint8, device=device)

    sm_scale = 1.0 / (D ** 0.5)

    def make_step(wl_):
        def step(i, q_=q, k_=k_new, v_=v_new, slots_=wl_["new_slots"], bt_=wl_["block_table"],
                 sl_=wl_["seq_lens"], out=out):
            cache = wl_["caches"][i % args.layers]
            if args.separate_write:
                ops.tq4_write_paged(k_, v_, cache, slots_, wl_["even"], wl_["odd"], wl_["kb"], wl_["vb"])
                ops.fused_paged_tq4_decode(q_, cache, bt_, sl_, wl_["kc"], wl_["rot"], hkv, D, BS, None, out,
                                           v_centroids=wl_["vc"], workspace=ws, mode=args.mode)
            else:  # one call: the cache write and the attention of the step
                ops.tq4_write_and_attention(k_, v_, slots_, wl_["even"], wl_["odd"], wl_["kb"], wl_["vb"],
                                            q_, cache, bt_, sl_, wl_["kc"], wl_["vc"], wl_["rot"], hkv, BS,
                                            sm_scale, out=out, workspace=ws, mode=args.mode)
        return step

    step = make_step(wl)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def graphed(fn):
        """fn(i) for i in range(steps) as CUDA-graph replays of `layers` consecutive steps (one per
        rotating layer cache) plus an eager remainder: the launch-bound inner loop is captured
        once, as a serving engine does for decode.  Returns (callable(steps), used_graph)."""
        if args.no_graph:
            return (lambda n: [fn(i) for i in range(n)]), False
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(args.layers):
                    fn(i)
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(args.layers):
                    fn(i)
        except Exception as e:  # noqa: BLE001
            print(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); running eagerly",
                  file=sys.stderr)
            torch.cuda.synchronize()
            return (lambda n: [fn(i) for i in range(n)]), False

        def run(n):
            for _ in range(n // args.layers):
                g.replay()
            for i in range(n % args.layers):
                fn(i)
        return run, True

    for i in range(max(args.warmup, 3)):
        step(i)
    sampler = ClockSampler(device.index or 0)  # clocks over every timed block (graph and eager)
    sampler.start()
    run_steps, used_graph = graphed(step)
    run_steps(max(args.warmup, 3))

    def timed_blocks(run_block):
        """One BLOCK = exactly --steps steps between barrier + synchronize on both sides, timed with
        CUDA events, max over ranks.  Blocks repeat until the timed region is at least --min-region
        seconds (the driver's 20 steps are under 2 ms: one block is noise); the result is the
        median block."""
        first = timed(lambda i: run_block(args.steps) if i == 0 else None, 1)
        n = int(min(args.max_blocks, max(1, -(-args.min_region * 1e3 // max(first, 1e-3)))))
        if world > 1:  # every rank must run the same number of blocks
            t = torch.tensor([n], dtype=torch.int64, device=device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            n = int(t.item())
        blocks = [first] + [timed(lambda i: run_block(args.steps) if i == 0 else None, 1) for _ in range(n - 1)]
        return statistics.median(blocks), blocks

    # Headline launch style: CUDA-graph replay (how a serving engine issues uniform decode steps);
    # the eager time of the same steps is reported beside it, never substituted.
    ms_total, blocks_ms = timed_blocks(run_steps)
    ms_step = ms_total / args.steps
    ms_eager_total, _ = timed_blocks(lambda n: [step(i) for i in range(n)])
    ms_eager = ms_eager_total / args.steps
    clocks = sampler.stop()
    ms_graph = ms_step if used_graph else None
    launch_style = f"CUDA graph of {args.layers} steps, replayed" if used_graph else "eager"
    value = batch * args.steps / (ms_total * 1e-3)

    # ---- per-kernel durations: an identical second pass with event brackets per kernel ------
    nsamp = min(args.steps, 2000)
    nv.profile_start(nsamp)
    timed(step, nsamp)
    nv.profile_stop()
    prof = {name: nv.profile_read(kind, nsamp) for name, kind in
            (("write", nv.PROF_WRITE), ("prologue", nv.PROF_PROLOGUE), ("attention", nv.PROF_ATTENTION),
             ("combine", nv.PROF_COMBINE))}
    avg = {k: (sum(v) / len(v) if v else None) for k, v in prof.items()}
    alg_bytes = batch * CTX * hkv * (D + 8)  # 136 B per token per KV head at D=128
    peak, peak_kind = measured_peak_gbs()
    achieved = alg_bytes / (avg["attention"] * 1e-3) / 1e9
    # kernels per step: write + prologue + attention + combine as separate calls; prologue + attention +
    # combine while rows x KV heads <= 512; attention (prologue inside) + combine above that
    forced = os.environ.get("TQ4_FUSED_PROLOGUE")
    fused_step = (forced != "0" and not os.environ.get("TQ4_NO_FUSED_PROLOGUE")) and (forced == "1" or batch * hkv > 512) and batch <= 512
    launches_per_step = 4 if args.separate_write else (2 if fused_step else 3)
    # the stored capture is of the 8-heads-per-GPU layout with the prologue kernel in front (what the
    # library picks at 64 query rows x 8 KV heads)
    traffic_known = (alg_bytes == 285212672 and world == 1 and not args.emulate_world and not args.separate_write
                     and not fused_step and not args.row_bytes)
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4),
                "traffic": NCU_TRAFFIC["bytes"] if traffic_known else None,
                "traffic_source": NCU_TRAFFIC["capture"] if traffic_known else None,
                "kernel": "paged TQ4 attention (streaming) kernel", "peak_kind": f"of {peak_kind}",
                "algorithmic_bytes_per_launch": alg_bytes,
                "kernel_ms": {k: (round(v, 5) if v is not None else None) for k, v in avg.items()},
                "frac_of_nominal_8TBs": round(achieved / 8000.0, 4)}

    # ---- compress throughput (prefill-sized write: 16384 tokens, K and V) -----------------------
    gen = torch.Generator(device=device).manual_seed(7)
    nt = 16384
    kc_, vc_ = synth_kv_gpu(nt, hkv, gen, device)
    cslots = torch.arange(nt, device=device)

    def wstep(i):
        ops.tq4_write_paged(kc_, vc_, wl["caches"][i % args.layers], cslots, wl["even"], wl["odd"],
                            wl["kb"], wl["vb"])

    for i in range(3):
        wstep(i)
    wms = timed(wstep, 20) / 20
    compress_mtok_s = nt / (wms * 1e-3) / 1e6
    # restore the rows the compress timing overwrote is unnecessary: bytes stay valid TQ4 rows

    # ---- end to end through the public API with host buffers ------------------------------------
    # Every step copies its six inputs from pinned host memory and its output back.  The copies of
    # step i+1 run on a second stream while step i computes (two sets of device input buffers), as a
    # serving engine stages the next step's inputs; the join at the end of a step orders them before
    # the next step.  --e2e-serial puts everything on one stream.
    slots_h = wl["new_slots"].cpu().pin_memory()
    bt_h = wl["block_table"].cpu().pin_memory()
    sl_h = wl["seq_lens"].cpu().pin_memory()
    host_in = (wl["q_host"], wl["k_host"], wl["v_host"], slots_h, bt_h, sl_h)
    dev_in = [tuple(torch.empty_like(x, device=device) for x in host_in) for _ in range(2)]
    out_h = torch.empty(batch, hq, D, dtype=torch.bfloat16).pin_memory()
    copy_stream = torch.cuda.Stream()

    def h2d(bufs):
        for d_, h_ in zip(bufs, host_in):
            d_.copy_(h_, non_blocking=True)

    def e2e_step(i):
        cur_bufs, next_bufs = dev_in[i % 2], dev_in[(i + 1) % 2]
        if args.e2e_serial:
            h2d(cur_bufs)
            step(i, *cur_bufs)
            out_h.copy_(out, non_blocking=True)
            return
        cur = torch.cuda.current_stream()
        copy_stream.wait_stream(cur)  # fork: step i - 1 (it read next_bufs, wrote outs[(i - 1) % 2]) is done
        with torch.cuda.stream(copy_stream):
            out_h.copy_(outs[(i + 1) % 2], non_blocking=True)  # result of step i - 1
            h2d(next_bufs)                                      # inputs of step i + 1
        step(i, *cur_bufs, out=outs[i % 2])  # inputs of step i were staged during step i - 1
        cur.wait_stream(copy_stream)  # join

    outs = [out, torch.empty_like(out)]
    h2d(dev_in[0])
    for i in range(3):
        e2e_step(i)
    run_e2e, e2e_graph = graphed(e2e_step)
    run_e2e(3)
    e2e_ms, _ = timed_blocks(run_e2e)
    h2d_bytes = sum(x.numel() * x.element_size() for x in host_in)
    d2h = out_h.numel() * out_h.element_size()
    e2e = {"value": round(batch * args.steps / (e2e_ms * 1e-3), 1), "unit": "tok/s",
           "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h,
           "ms_per_step": round(e2e_ms / args.steps, 5), "cuda_graph": e2e_graph,
           "copies": "serial" if args.e2e_serial else
           "second stream: inputs of step i+1 in, result of step i-1 out, while step i computes"}

    # ---- chunked prefill: 8 sequences x 2048 new tokens on an 8192-token packed prefix, causal
    #      (head_dim 128: tcgen05 kernel and, beside it, the streaming kernel; head_dim 256 with a
    #      sliding window of 4096) ---------------------------------------------------------------
    prefill = None
    if rank == 0 and world == 1 and not args.no_prefill:
        try:
            prefill = prefill_measurement(device, wl, ops)
        except Exception as e:  # noqa: BLE001
            prefill = {"error": f"{type(e).__name__}: {e}"[:200]}

    line = {
        "metric": "paged_tq4_decode_tok_per_s", "value": round(value, 1), "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_step, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {
            "workload": "Llama-3.1-8B-shaped single-layer paged TQ4 decode: cache write of 1 token/seq + "
                        "fused paged decode; batch 64/GPU x ctx 4096, 32q/8kv heads (sharded over GPUs), "
                        "head_dim 128, block 16 shuffled, K4/V4, bf16 q",
            "global_batch": batch, "seq_len": CTX, "kv_heads_per_gpu": hkv, "q_heads_per_gpu": hq,
            "parallelism": f"tp{world} head-sharded, no collective",
            "l2": f"inputs>L2: {args.layers} rotating layer caches of {wl['nblk'] * BS * wl['width'] / 1e6:.0f} MB",
            "kernel_mode": args.mode,
            "row_bytes": wl["width"],
            "launch": launch_style,
            "ms_per_step_eager": round(ms_eager, 5),
            "ms_per_step_graph": round(ms_graph, 5) if used_graph else None,
            "timed_blocks": len(blocks_ms),
            "timed_region_s": round(sum(blocks_ms) * 1e-3, 4),
            "block_ms_min_median_max": [round(min(blocks_ms), 5), round(statistics.median(blocks_ms), 5),
                                        round(max(blocks_ms), 5)],
        },
        "hbm_gbs": round(alg_bytes / (ms_step * 1e-3) / 1e9, 1),
        "compress_mtok_s": round(compress_mtok_s, 3),
        "compress_config": f"{nt} tokens x {hkv} KV heads, K and V, bf16 -> paged cache, one launch",
        "prefill": prefill,
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_bf16_baseline:
        del wl["caches"][1:]  # free HBM for the bf16 copies
        line["bf16_paged_decode"] = bf16_paged_decode_baseline(device, batch, hq, hkv)
        if "ms" in line["bf16_paged_decode"]:
            line["bf16_paged_decode"]["tq4_attention_path_ms"] = round(
                sum(avg[k] or 0.0 for k in ("prologue", "attention", "combine")), 5)
    eff_world = args.emulate_world or world
    if eff_world > 1 and not args.no_dense_rows and not args.row_bytes:
        # the same step on dense token rows (kv_heads * 136 bytes rounded up to 16) instead of vLLM's
        # power-of-two slots: what the TQ4_DENSE_ROWS=1 backend option allocates
        try:
            del wl["caches"][:]
            torch.cuda.empty_cache()
            wl_d = build_workload(device, eff_world, args.layers, (hkv * (D + 8) + 15) & ~15)
            step_d = make_step(wl_d)
            for i in range(3):
                step_d(i)
            run_d, graph_d = graphed(step_d)
            run_d(3)
            ms_d, _ = timed_blocks(run_d)
            nv.profile_start(200)
            timed(step_d, 200)
            nv.profile_stop()
            att_d = nv.profile_read(nv.PROF_ATTENTION, 200)
            att_d = sum(att_d) / len(att_d)
            line["dense_rows"] = {
                "row_bytes": wl_d["width"], "ms_per_step": round(ms_d / args.steps, 5),
                "value": round(batch * args.steps / (ms_d * 1e-3), 1), "unit": "tok/s", "cuda_graph": graph_d,
                "frac": round(alg_bytes / (att_d * 1e-3) / 1e9 / peak, 4),
                "step_frac": round(alg_bytes / (ms_d / args.steps * 1e-3) / 1e9 / peak, 4)}
            del wl_d["caches"][:]
        except Exception as e:  # noqa: BLE001
            line["dense_rows"] = {"error": f"{type(e).__name__}: {e}"[:200]}
    line["step_frac"] = round(alg_bytes / (ms_step * 1e-3) / 1e9 / peak, 4)
    if not args.no_side_configs and not args.emulate_world:
        del wl["caches"][:]  # free HBM: the side caches are several GB each
        torch.cuda.empty_cache()
        side = {}

        def guarded(name, fn):
            # every rank takes part (collectives inside); a failure is reported, and fails the run
            try:
                side[name] = fn()
            except Exception as e:  # noqa: BLE001
                side[name] = {"error": f"{type(e).__name__}: {e}"[:300]}

        guarded("serving_mix", lambda: serving_mix_measurement(device, world, rank))
        if world > 1:
            guarded("serving_mix_dense_rows", lambda: serving_mix_measurement(device, world, rank, dense_rows=True))
            guarded("split_kv", lambda: split_kv_measurement(device, world, rank))
        else:
            guarded("long_context", lambda: ragged_decode_measurement(
                device, "batch 8 x 131072, 32q/32kv, D=96, K4/V4 (one GPU holds the whole sequences)",
                lens=[131072] * 8, hq=32, hkv=32, d=96, k_bits=4, v_bits=4, iters=10))
        line.update(side)
    if rank == 0 and world == 1 and args.extra:
        del wl["caches"][:]
        torch.cuda.empty_cache()
        try:
            line["extra_decode_configs"] = extra_decode_configs(device, args.extra.split(","))
        except Exception as e:  # noqa: BLE001
            line["extra_decode_configs"] = {"error": f"{type(e).__name__}: {e}"[:200]}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(budget_s=args.cpu_budget)
    return line


def device_time_ms(fn, iters, world, device, warmup=3):
    """Mean milliseconds of fn() over `iters` calls: CUDA events on the current stream, barrier +
    synchronize on both sides, max over ranks."""
    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / iters
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def prefill_case(device, ops, *, hq, hkv, d, window, modes, nseq=8, prefix=8192, new=2048):
    """`nseq` sequences x `new` new tokens attending causally (optionally inside a sliding window)
    over a `prefix`-token packed prefix + themselves, shuffled 16-token pages, vLLM's padded page
    format.  Reports ms, TFLOP/s (4 * visible keys * head_dim * q_heads) and new tokens/s per mode."""
    from turboquant_vllm.quantizer import TurboQuantMSE

    kq = TurboQuantMSE(d, 4, seed=42)
    rot, even, odd, kc, kb = kq.device_primitives(device)
    total = prefix + new
    nblk = nseq * total // BS
    gen = torch.Generator(device=device).manual_seed(11)
    width = hkv * (1 << ((d + 8) - 1).bit_length())
    cache = torch.zeros(nblk, BS, width, dtype=torch.uint8, device=device)
    bt = torch.randperm(nblk, device=device, generator=gen).view(nseq, total // BS).to(torch.int32)
    slots = (bt.long()[:, :, None] * BS + torch.arange(BS, device=device)[None, None, :]).reshape(-1)
    chunk = 16384
    for t0 in range(0, nseq * total, chunk):
        k = torch.randn(chunk, hkv, d, device=device, generator=gen).bfloat16()
        v = torch.randn(chunk, hkv, d, device=device, generator=gen).bfloat16()
        ops.tq4_write_paged(k, v, cache, slots[t0:t0 + chunk], even, odd, kb, kb)
    del k, v
    q = torch.randn(nseq * new, hq, d, device=device, generator=gen).bfloat16()
    qsl = (torch.arange(nseq + 1, device=device) * new).to(torch.int32)
    sl = torch.full((nseq,), total, dtype=torch.int32, device=device)
    keys = nseq * sum(min(prefix + i + 1, window or (prefix + i + 1)) for i in range(new))
    flops = 4.0 * keys * d * hq
    res = {"config": f"{nseq} seqs x {new} new tokens on {prefix}-token packed prefix, causal, "
                     f"{hq}q/{hkv}kv, D={d}" + (f", sliding window {window}" if window else ""),
           "visible_pairs": keys, "flops": flops}
    precise = None
    for name, mode, iters in modes:
        def run():
            return ops.paged_tq4_attention(q, cache, bt, sl, kc, kc, rot, hkv, BS, query_start_loc=qsl,
                                           sliding_window=window, mode=mode, out_dtype=torch.float32)
        try:
            out = run()
        except NotImplementedError as e:
            res[name] = {"unsupported": str(e)[:120]}
            continue
        ms = device_time_ms(run, iters, 1, device, warmup=1)
        res[name] = {"ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 1),
                     "frac_of_bf16_burst_peak": round(flops / ms / 1e9 / measured_peak_tflops(), 4),
                     "tokens_per_s": round(nseq * new / (ms * 1e-3), 1)}
        if precise is None:
            precise = out  # the first mode listed is the one parity-tested against the oracle
        else:  # how far this mode's fp32 output is from the first one's
            res[name]["vs_" + modes[0][0]] = {
                "max_abs": float(f"{float((out - precise).abs().max()):.3e}"),
                "cos": round(float(torch.nn.functional.cosine_similarity(
                    out.flatten().double(), precise.flatten().double(), dim=0)), 8)}
        del out
    return res


def prefill_measurement(device, wl, ops):
    """Chunked prefill on packed keys: (a) Llama shape 32 q / 8 KV heads, head_dim 128; (b) Gemma-2-2B
    shape 8 q / 4 KV heads, head_dim 256, sliding window 4096.  `mode 0` is what the backend picks,
    `mode 2` the streaming kernel."""
    a = prefill_case(device, ops, hq=32, hkv=8, d=128, window=None,
                     modes=(("tcgen05", 0, 5), ("tcgen05_fast_single_term", 4, 5), ("streaming", 2, 2)))
    try:
        b = prefill_case(device, ops, hq=8, hkv=4, d=256, window=4096, modes=(("auto", 0, 3),))
    except Exception as e:  # noqa: BLE001
        b = {"error": f"{type(e).__name__}: {e}"[:200]}
    a["head_dim_256_window_4096"] = b
    return a


def ragged_decode_measurement(device, name, *, lens, hq, hkv, d, k_bits, v_bits, iters=20, world=1,
                              dense_rows=False):
    """Side measurement of one decode step (cache write of a token per sequence + fused paged decode)
    on a ragged batch: `lens` tokens already held per sequence, shuffled 16-token pages, vLLM's padded
    page format.  The cache is filled through the write kernel from one 65 536-token block of
    N(0,1)+outlier K/V that is reused for every chunk (contents do not change the timing).  Reports
    ms per step, algorithmic GB/s (sum(lens) * hkv * (d + 8)) and tok/s.  `hq` / `hkv` are THIS
    rank's heads; with world > 1 the time is the max over ranks (strong scaling: the batch is fixed,
    the heads are divided).  `dense_rows`: token rows of hkv * (d + 8) bytes rounded up to 16 instead
    of the power-of-two slots of vLLM's page format."""
    from turboquant_vllm.kernels import ops
    from turboquant_vllm.quantizer import TurboQuantMSE

    kq = TurboQuantMSE(d, k_bits, seed=42)
    vq = kq if v_bits == k_bits else TurboQuantMSE(d, v_bits, seed=42)
    rot, even, odd, kc, kb = kq.device_primitives(device)
    _, _, _, vc, vb = vq.device_primitives(device)
    gen = torch.Generator(device=device).manual_seed(23)
    lens_t = torch.as_tensor(lens, dtype=torch.int64, device=device)
    batch, total = lens_t.numel(), int(lens_t.sum())
    blocks = (lens_t + BS - 1) // BS
    nblk, max_blocks = int(blocks.sum()), int(blocks.max())
    width = (hkv * (d + 8) + 15) & ~15 if dense_rows else hkv * (1 << ((d + 8) - 1).bit_length())
    cache = torch.empty(nblk, BS, width, dtype=torch.uint8, device=device)
    perm = torch.randperm(nblk, device=device, generator=gen).to(torch.int32)
    first = torch.cumsum(blocks, 0) - blocks
    col = torch.arange(max_blocks, device=device)[None, :]
    block_table = perm[(first[:, None] + col).clamp_(max=nblk - 1)].masked_fill_(col >= blocks[:, None], 0)
    block_table = block_table.contiguous()
    seq_of = torch.repeat_interleave(torch.arange(batch, device=device), lens_t)
    pos = torch.arange(total, device=device) - (torch.cumsum(lens_t, 0) - lens_t)[seq_of]
    slots = block_table[seq_of, pos // BS].long() * BS + pos % BS
    chunk = 65536
    k = torch.randn(chunk, hkv, d, device=device, generator=gen)
    v = torch.randn(chunk, hkv, d, device=device, generator=gen)
    for ch in (3, 17, 64, 101):
        if ch < d:
            k[..., ch] *= 8.0
            v[..., ch] *= 8.0
    k, v = k.bfloat16(), v.bfloat16()
    for t0 in range(0, total, chunk):
        n = min(chunk, total - t0)
        ops.tq4_write_paged(k[:n], v[:n], cache, slots[t0 : t0 + n], even, odd, kb, vb)
    new_slots = slots[torch.cumsum(lens_t, 0) - 1].contiguous()  # the step rewrites each last token
    seq_lens = lens_t.to(torch.int32)
    q = torch.randn(batch, hq, d, device=device, generator=gen).bfloat16()
    out = torch.empty_like(q)
    ws = torch.empty(ops.attention_workspace_bytes(batch, hq, hkv, d), dtype=torch.uint8, device=device)

    def step():
        ops.tq4_write_and_attention(k[:batch], v[:batch], new_slots, even, odd, kb, vb, q, cache, block_table,
                                    seq_lens, kc, vc, rot, hkv, BS, None, out=out, workspace=ws)
    ms = device_time_ms(step, iters, world, device)
    alg = total * hkv * (d + 8)
    peak, _ = measured_peak_gbs()
    gbs = alg / (ms * 1e-3) / 1e9
    return {"config": name, "batch": batch, "tokens_held": total, "cache_mb": round(cache.numel() / 1e6),
            "kv_heads_per_gpu": hkv, "row_bytes": width,
            "ms_per_step": round(ms, 4), "hbm_gbs_per_gpu": round(gbs, 1), "frac": round(gbs / peak, 4),
            "tok_per_s": round(batch / (ms * 1e-3), 1)}


def serving_mix_measurement(device, world, rank, dense_rows=False, iters=20):
    """Asymmetric K4/V3 serving mix, one layer: batch 256 with context lengths ~U[512, 32768]
    (seeded), cache write of one new token per sequence + paged decode, 32 q / 8 KV heads of
    head_dim 128 divided over `world` ranks (strong scaling: the batch is fixed)."""
    import random

    rng = random.Random(7)
    lens = [rng.randint(512, 32768) for _ in range(256)]
    r = ragged_decode_measurement(
        device, f"batch 256, ctx~U[512,32768], 32q/8kv heads over {world} GPU(s), D=128, K4/V3, "
                + ("dense rows" if dense_rows else "vLLM padded pages"),
        lens=lens, hq=HQ // world, hkv=HKV // world, d=D, k_bits=4, v_bits=3, iters=iters, world=world,
        dense_rows=dense_rows)
    r["scaling"] = "strong"
    r["hbm_gbs_all_gpus"] = round(r["hbm_gbs_per_gpu"] * world, 1)
    return r


def build_split_kv_case(device, world, rank, *, batch, ctx, hq, hkv, d, seed):
    """This rank's token slice of `batch` sequences of `ctx` tokens (contiguous, block aligned;
    turboquant_vllm.parallel.split_sequence), written through the write kernel into a local paged
    cache with shuffled pages.  K/V come from ONE seeded 32 768-token block of N(0,1)+outlier rows
    reused cyclically by absolute position, so any rank can rebuild any slice."""
    from turboquant_vllm import parallel
    from turboquant_vllm.kernels import ops
    from turboquant_vllm.quantizer import TurboQuantMSE

    kq = TurboQuantMSE(d, 4, seed=42)
    rot, even, odd, kc, kb = kq.device_primitives(device)
    gen = torch.Generator(device=device).manual_seed(seed)
    period = 32768
    k = torch.randn(period, hkv, d, device=device, generator=gen)
    v = torch.randn(period, hkv, d, device=device, generator=gen)
    for ch in (3, 17, 64, 101):
        if ch < d:
            k[..., ch] *= 8.0
            v[..., ch] *= 8.0
    k, v = k.bfloat16(), v.bfloat16()
    start, end = parallel.split_sequence(ctx, world, BS)[rank]
    local = end - start
    nb_seq = (local + BS - 1) // BS
    nblk = max(1, batch * nb_seq)
    width = hkv * (1 << ((d + 8) - 1).bit_length())
    cache = torch.zeros(nblk, BS, width, dtype=torch.uint8, device=device)
    gen2 = torch.Generator(device=device).manual_seed(seed + 1 + rank)
    bt = torch.randperm(nblk, device=device, generator=gen2).view(batch, max(nb_seq, 1)).to(torch.int32).contiguous()
    pos = torch.arange(local, device=device)
    for b in range(batch):
        for t0 in range(0, local, period):
            n = min(period, local - t0)
            p_ = pos[t0:t0 + n]
            slots = bt[b].long()[p_ // BS] * BS + p_ % BS
            src = (start + t0 + b * 977) % period  # sequences differ by a cyclic shift
            idx = (torch.arange(n, device=device) + src) % period
            ops.tq4_write_paged(k[idx], v[idx], cache, slots, even, odd, kb, kb)
    seq_lens = torch.full((batch,), local, dtype=torch.int32, device=device)
    g = torch.Generator().manual_seed(seed + 100)
    q = torch.randn(batch, hq, d, generator=g).bfloat16().to(device)
    return dict(cache=cache, bt=bt, seq_lens=seq_lens, q=q, rot=rot, kc=kc, local=local, width=width)


def split_kv_measurement(device, world, rank, *, iters=20):
    """Long-context sequence-split decode (Phi-3-mini shape: 32 q / 32 KV heads, head_dim 96, batch 8
    x 131 072 tokens, K4/V4): every rank holds 1/world of every sequence, attends over its slice,
    all ranks exchange (output, log-sum-exp) partials with one NCCL all-gather and merge locally
    (turboquant_vllm.parallel.split_kv_decode).  Before timing, a small case checks that the
    world-rank result equals the single-rank kernel run on the whole sequences."""
    from turboquant_vllm import parallel
    from turboquant_vllm.kernels import ops

    hq = hkv = 32
    d = 96
    # ---- parity on a small case: N ranks vs one rank over the whole sequences ---------------------
    small = dict(batch=4, ctx=2048, hq=hq, hkv=hkv, d=d, seed=41)
    mine = build_split_kv_case(device, world, rank, **small)
    got = parallel.split_kv_decode(mine["q"], mine["cache"], mine["bt"], mine["seq_lens"], mine["kc"], mine["kc"],
                                   mine["rot"], hkv, BS, out_dtype=torch.float32)
    whole = build_split_kv_case(device, 1, 0, **small)
    want = ops.paged_tq4_attention(whole["q"], whole["cache"], whole["bt"], whole["seq_lens"], whole["kc"],
                                   whole["kc"], whole["rot"], hkv, BS, out_dtype=torch.float32)
    torch.cuda.synchronize()
    cos = float(torch.nn.functional.cosine_similarity(got.flatten().double(), want.flatten().double(), dim=0))
    max_abs = float((got - want).abs().max())
    parity = {"case": "4 seqs x 2048 tokens", "cos": round(cos, 7), "max_abs": float(f"{max_abs:.3e}"),
              "ok": bool(cos >= 0.99999 and max_abs <= 1e-4)}
    del mine, whole
    # ---- the timed case ---------------------------------------------------------------------------
    batch, ctx = 8, 131072
    c = build_split_kv_case(device, world, rank, batch=batch, ctx=ctx, hq=hq, hkv=hkv, d=d, seed=43)
    events: list = []

    def step():
        parallel.split_kv_decode(c["q"], c["cache"], c["bt"], c["seq_lens"], c["kc"], c["kc"], c["rot"], hkv, BS,
                                 exchange_events=events)
    ms = device_time_ms(step, iters, world, device)
    ex = [a.elapsed_time(b) for a, b in events[-iters:]]
    ex_ms = sum(ex) / len(ex)
    if world > 1:
        t = torch.tensor([ex_ms], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ex_ms = float(t.item())
    alg_rank = batch * c["local"] * hkv * (d + 8)
    peak, _ = measured_peak_gbs()
    gbs = alg_rank / (ms * 1e-3) / 1e9
    return {"config": f"batch {batch} x {ctx} tokens, 32q/32kv, D=96, K4/V4, sequence split over {world} GPU(s), "
                      "NCCL all-gather of (O, LSE) partials + local merge",
            "tokens_per_rank_per_seq": c["local"], "ms_per_step": round(ms, 4),
            "per_rank_gbs": round(gbs, 1), "frac": round(gbs / peak, 4),
            "all_ranks_gbs": round(gbs * world, 1), "tok_per_s": round(batch / (ms * 1e-3), 1),
            "allgather_us": round(ex_ms * 1e3, 1), "allgather_share": round(ex_ms / ms, 4),
            "exchange_bytes": batch * hq * (d + 1) * 4, "scaling": "strong", "parity_vs_single_rank": parity}


def hf_fused_measurement(device, batch=8, ctx=32768, hq=32, hkv=8, d=128, iters=50):
    """One decode step of a layer on the HuggingFace side: `CompressedDynamicCache.update` of one
    token per sequence in fused mode (token rows) + the `triton_fa_tq4_kv` backend's forward, on a
    cache that already holds `ctx` tokens per sequence (same packed bytes as the headline workload)."""
    import types

    from transformers import DynamicCache

    from turboquant_vllm.kv_cache import CompressedDynamicCache
    from turboquant_vllm.triton.attention_interface import triton_fa_tq4_kv_forward

    gen = torch.Generator(device=device).manual_seed(31)
    cache = DynamicCache()
    cc = CompressedDynamicCache(cache, head_dim=d, bits=4)
    cc.fused_mode = True
    module = types.SimpleNamespace(layer_idx=0, _tq4_cache=cc, is_causal=True)
    for s0 in range(0, ctx, 4096):  # prefill in chunks
        k = torch.randn(batch, hkv, 4096, d, device=device, generator=gen).bfloat16()
        cache.update(k, -k, 0)
    k1 = torch.randn(batch, hkv, 1, d, device=device, generator=gen).bfloat16()
    q = torch.randn(batch, hq, 1, d, device=device, generator=gen).bfloat16()
    store = cc.get_token_rows(0)
    store._reserve(ctx + iters + 8)  # keep capacity growth out of the timed steps

    def step():
        cache.update(k1, k1, 0)
        return triton_fa_tq4_kv_forward(module, q, k1, k1, None)[0]
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    alg = batch * ctx * hkv * (d + 8)
    return {"config": f"HF fused mode: batch {batch} x {ctx} tokens held, {hq}q/{hkv}kv, D={d}, K4/V4, "
                      "update of 1 token/seq + attention forward",
            "ms_per_step": round(ms, 4), "hbm_gbs": round(alg / (ms * 1e-3) / 1e9, 1),
            "tok_per_s": round(batch / (ms * 1e-3), 1)}


def extra_decode_configs(device, which):
    """`serving_mix`: batch 256, contexts ~U[512, 32768] (seeded), 32q/8kv, head_dim 128, K4/V3.
    `long_context`: batch 8 x 131 072 tokens, 32q/32kv, head_dim 96, K4/V4 (one rank's view of the
    sequence-split case with W = 1)."""
    import random

    res = {}
    if "serving_mix" in which:
        rng = random.Random(7)
        lens = [rng.randint(512, 32768) for _ in range(256)]
        res["serving_mix"] = ragged_decode_measurement(
            device, "batch 256, ctx~U[512,32768], 32q/8kv, D=128, K4/V3", lens=lens, hq=32, hkv=8, d=128,
            k_bits=4, v_bits=3)
    if "hf_fused" in which:
        res["hf_fused"] = hf_fused_measurement(device)
    if "long_context_small" in which:  # the long_context shape at a size suited to a profiler capture
        res["long_context_small"] = ragged_decode_measurement(
            device, "batch 2 x 65536, 32q/32kv, D=96, K4/V4", lens=[65536] * 2, hq=32, hkv=32, d=96,
            k_bits=4, v_bits=4, iters=3)
    if "long_context" in which and "long_context_small" not in which:
        res["long_context"] = ragged_decode_measurement(
            device, "batch 8 x 131072, 32q/32kv, D=96, K4/V4", lens=[131072] * 8, hq=32, hkv=32, d=96,
            k_bits=4, v_bits=4, iters=10)
    return res


# ----------------------------------------------------------------------------------------
# comparison point: bf16 paged decode of the SAME (uncompressed) cache with a library kernel
# ----------------------------------------------------------------------------------------
def bf16_paged_decode_baseline(device, batch, hq, hkv, steps=50):
    """FlashAttention-style paged decode on a bf16 cache of the same shape (library kernels:
    vLLM's flash-attn build or FlashInfer).  Returns {"ms", "impl"} or {"error"}.  This is a
    reference point for the compressed path, not part of the product."""
    nblk = batch * CTX // BS
    try:
        gen = torch.Generator(device=device).manual_seed(3)
        kc = torch.randn(nblk, BS, hkv, D, device=device, generator=gen).bfloat16()
        vc = torch.randn(nblk, BS, hkv, D, device=device, generator=gen).bfloat16()
        kc2, vc2 = kc.clone(), vc.clone()  # rotate two copies: working set 4.3 GB >> L2
        q = torch.randn(batch, hq, D, device=device, generator=gen).bfloat16()
        bt = torch.randperm(nblk, device=device, generator=gen).view(batch, CTX // BS).to(torch.int32)
        sl = torch.full((batch,), CTX, dtype=torch.int32, device=device)
        cu = torch.arange(batch + 1, dtype=torch.int32, device=device)
        out = torch.empty_like(q)
    except Exception as e:  # noqa: BLE001
        return {"error": f"setup: {type(e).__name__}: {e}"[:200]}
    errors = []

    def time_it(fn):
        for i in range(5):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    try:
        from vllm.vllm_flash_attn import flash_attn_varlen_func

        def fa(i):
            k_, v_ = (kc, vc) if i % 2 == 0 else (kc2, vc2)
            flash_attn_varlen_func(q=q, k=k_, v=v_, out=out, cu_seqlens_q=cu, max_seqlen_q=1,
                                   seqused_k=sl, max_seqlen_k=CTX, softmax_scale=D ** -0.5, causal=True,
                                   block_table=bt, fa_version=2)

        return {"ms": round(time_it(fa), 5), "impl": "vllm flash_attn_varlen_func (FA2, paged bf16)"}
    except Exception as e:  # noqa: BLE001
        errors.append(f"vllm-fa: {type(e).__name__}: {e}"[:160])
    try:
        import flashinfer

        ws = torch.empty(128 << 20, dtype=torch.uint8, device=device)
        w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
        indptr = torch.arange(batch + 1, dtype=torch.int32, device=device) * (CTX // BS)
        last = torch.full((batch,), BS, dtype=torch.int32, device=device)
        w.plan(indptr, bt.reshape(-1).contiguous(), last, hq, hkv, D, BS, q_data_type=torch.bfloat16,
               kv_data_type=torch.bfloat16)

        def fi(i):
            k_, v_ = (kc, vc) if i % 2 == 0 else (kc2, vc2)
            w.run(q, (k_, v_), out=out)

        return {"ms": round(time_it(fi), 5), "impl": "flashinfer BatchDecodeWithPagedKVCacheWrapper (bf16)"}
    except Exception as e:  # noqa: BLE001
        errors.append(f"flashinfer: {type(e).__name__}: {e}"[:160])
    return {"error": " | ".join(errors)}


# ----------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's PyTorch path
# ----------------------------------------------------------------------------------------
def cpu_workload(n_seqs, hkv=HKV, hq=HQ):
    from oracle import tq4_oracle as O

    cents, bounds = O.solve_lloyd_max(D, K_BITS)
    rot = O.rotation_matrix(D, 42)
    nblk = n_seqs * CTX // BS
    cache = torch.zeros(nblk, BS, O.row_layout(hkv, D)[3], dtype=torch.uint8)
    g = torch.Generator().manual_seed(SEED)
    perm = torch.randperm(nblk, generator=g)
    bt = perm.view(n_seqs, CTX // BS).to(torch.int32)
    pos = torch.arange(CTX)
    for s in range(n_seqs):
        k, v = O.synthetic_kv(CTX, hkv, D, seed=SEED + s, dtype=torch.bfloat16)
        slots = bt[s].long()[pos // BS] * BS + pos % BS
        kp, kn = O.compress_rows(k, rot, bounds)
        vp, vn = O.compress_rows(v, rot, bounds)
        cache.view(-1, cache.shape[-1])[slots] = O.assemble_rows(kp, kn, vp, vn)
    q = torch.randn(n_seqs, hq, D, generator=g).bfloat16()
    k_new, v_new = O.synthetic_kv(n_seqs, hkv, D, seed=99, dtype=torch.bfloat16)
    new_slots = bt[:, (CTX - 1) // BS].long() * BS + (CTX - 1) % BS
    return dict(O=O, cents=cents, bounds=bounds, rot=rot, cache=cache, bt=bt, q=q, k_new=k_new,
                v_new=v_new, new_slots=new_slots, n_seqs=n_seqs, hkv=hkv)


def cpu_step(w):
    O = w["O"]
    O.write_paged(w["k_new"], w["v_new"], w["cache"], w["new_slots"], w["rot"], w["bounds"], w["bounds"])
    return O.paged_decode_fp32(w["q"], w["cache"], w["bt"], [CTX] * w["n_seqs"], w["cents"], w["cents"],
                               w["rot"], w["hkv"])


def cpu_baseline(budget_s=15.0):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = cpu_workload(2)
    cpu_step(w)
    t0 = time.perf_counter()
    cpu_step(w)
    per = (time.perf_counter() - t0) / 2
    reps = max(1, min(50, int(budget_s / max(per * 2, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        cpu_step(w)
    dt = time.perf_counter() - t0
    return {"value": round(2 * reps / dt, 2), "unit": "tok/s", "cores": cores, "kind": "port",
            "sample": f"{reps} steps of 2 of the 64 sequences (ctx 4096, 8 KV heads): write 1 token/seq + fp32 "
                      "decode with the CPU restatement of the reference's PyTorch path"}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n_seqs = 2
    w = cpu_workload(n_seqs)
    warm = max(args.warmup, 3)  # the same rule as the GPU arm
    for _ in range(warm):
        cpu_step(w)
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(w)
    dt = time.perf_counter() - t0
    val = round(n_seqs * steps / dt, 2)
    sample = (f"each step = 2 of the {BATCH_PER_GPU_UNIT * world} sequences (ctx 4096, 8 KV heads): cache write of "
              "1 token/seq + fp32 paged decode, CPU restatement of the reference's PyTorch path (oracle/), "
              f"{steps} timed steps")
    return {
        "impl": "reference", "metric": "paged_tq4_decode_tok_per_s", "value": val, "unit": "tok/s",
        "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": round(dt / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "Llama-3.1-8B-shaped single-layer paged TQ4 decode (CPU sample)",
                   "global_batch": BATCH_PER_GPU_UNIT * world, "seq_len": CTX},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", type=int, default=0, help="0 auto, 1 fp32 CUDA-core kernel, 2 tensor-core LUT kernel")
    ap.add_argument("--layers", type=int, default=4, help="distinct layer caches rotated per step")
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-bf16-baseline", action="store_true")
    ap.add_argument("--separate-write", action="store_true",
                    help="tq4_write_paged + attention as two calls (4 launches) instead of the fused step")
    ap.add_argument("--e2e-serial", action="store_true",
                    help="end-to-end: copies and kernels of a step on one stream (no staging of the next step)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the chunked-prefill measurement")
    ap.add_argument("--no-side-configs", action="store_true",
                    help="skip the serving-mix / long-context / sequence-split measurements after the headline")
    ap.add_argument("--no-dense-rows", action="store_true",
                    help="N > 1: skip the second timing of the headline step on dense token rows")
    ap.add_argument("--extra", default="", help="comma list of side measurements run after the timed region: "
                                                "serving_mix, long_context, long_context_small, hf_fused")
    ap.add_argument("--row-bytes", type=int, default=0,
                    help="token-row stride of the cache in bytes (>= kv_heads*(head_dim+8), multiple of 16); "
                         "0 = vLLM's padded page format, which the reference uses")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly (no CUDA graph)")
    ap.add_argument("--min-region", type=float, default=0.5,
                    help="repeat the block of --steps timed steps until the timed region is this many seconds")
    ap.add_argument("--max-blocks", type=int, default=2000)
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="tuning aid: run ONE rank's share of a W-GPU head-sharded job on this GPU")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # stdout carries the JSON line and nothing else: libraries that print from C (NCCL's version banner)
    # write to file descriptor 1, so that descriptor points at stderr while the bench runs
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(line):
        os.write(json_fd, (json.dumps(line) + "\n").encode())

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            emit(line)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback of the product path)")
    if HKV % world:
        raise SystemExit(f"{HKV} KV heads cannot be sharded over {world} GPUs")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    line = run_ours(args, rank, world, device)
    if rank == 0:
        emit(line)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    par = (line.get("split_kv") or {}).get("parity_vs_single_rank") if isinstance(line, dict) else None
    if par is not None and not par.get("ok", False):
        raise SystemExit(f"sequence-split decode disagrees with the single-rank kernel: {par}")


if __name__ == "__main__":
    main()
