"""Generate golden vectors by importing the reference implementation (CPU).

Run where the reference source tree is available::

    python tests/golden/make_golden.py --reference-src <path-to-reference>/src

It writes ``tests/golden/*.npz``.  The fixtures are committed; the tests and the benchmark
never need the reference tree.  Nothing here imports this repository's product package
(the product reuses the reference's top-level module name on purpose, so the two must not
be mixed in one process).
"""

from __future__ import annotations

import argparse
import math
import os
import random
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
OUTLIERS = (3, 17, 64, 101)


def synth(n, h, d, seed):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(n, h, d, generator=g)
    v = torch.randn(n, h, d, generator=g)
    for ch in OUTLIERS:
        k[..., ch % d] *= 8.0
        v[..., ch % d] *= 8.0
    return k, v


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-src", required=True)
    args = ap.parse_args()
    sys.path.insert(0, args.reference_src)

    from turboquant_vllm.kv_cache import CompressedDynamicCache
    from turboquant_vllm.lloyd_max import solve_lloyd_max
    from turboquant_vllm.quantizer import TurboQuantMSE, _generate_rotation_matrix
    from turboquant_vllm.triton.tq4_compress import _tq4_compress_cpu
    from turboquant_vllm.triton.tq4_decompress import _tq4_decompress_cpu

    torch.manual_seed(42)

    # ---- 1. codebooks -------------------------------------------------------------
    cb = {}
    for d in (64, 96, 128, 256):
        for bits in (2, 3, 4, 5):
            c, b = solve_lloyd_max(d, bits)
            cb[f"c_{d}_{bits}"] = c.numpy()
            cb[f"b_{d}_{bits}"] = b.numpy()
    np.savez_compressed(os.path.join(HERE, "codebooks.npz"), **cb)

    # ---- 2. rotations ---------------------------------------------------------------
    rot = {}
    for d in (64, 96, 128, 256):
        for seed in (42, 7):
            r = _generate_rotation_matrix(d, seed)
            rot[f"row0_{d}_{seed}"] = r[0].numpy()
            rot[f"diag_{d}_{seed}"] = torch.diag(r).numpy()
            rot[f"colsum_{d}_{seed}"] = r.double().sum(0).numpy()
    rot["full_64_42"] = _generate_rotation_matrix(64, 42).numpy()
    np.savez_compressed(os.path.join(HERE, "rotations.npz"), **rot)

    # ---- 3. compress rows -----------------------------------------------------------
    comp = {}
    for d in (64, 96, 128, 256):
        qz = TurboQuantMSE(d, 4, seed=42)
        rt = qz.rotation.T.contiguous()
        even, odd = rt[:, 0::2].contiguous(), rt[:, 1::2].contiguous()
        k, _ = synth(24, 4, d, seed=100 + d)
        x = k.bfloat16()  # model dtype; values exactly representable
        x[5, 2] = 0  # an all-zero vector hits the boundary tie at 0.0
        x[7, 1] *= 1e-3
        x[9, 0] *= 1e3
        packed, norms = _tq4_compress_cpu(x, even, odd, qz.codebook.boundaries)
        idx, norms2 = qz.quantize(x)
        flat = x.reshape(-1, d).float()
        nrm = torch.norm(flat, dim=-1, keepdim=True)
        rotated = (flat / (nrm + 1e-10)) @ qz.rotation.T
        assert torch.equal(norms.reshape(-1), norms2.reshape(-1))
        dec = _tq4_decompress_cpu(packed, norms, qz.codebook.centroids, torch.float32)
        deq = qz.dequantize(idx, norms2)
        comp[f"x_{d}"] = x.float().numpy()
        comp[f"rotated_{d}"] = rotated.numpy()
        comp[f"packed_{d}"] = packed.numpy()
        comp[f"norms_{d}"] = norms.numpy()
        comp[f"idx_{d}"] = idx.to(torch.uint8).numpy()
        comp[f"dec_{d}"] = dec.numpy()
        comp[f"deq_{d}"] = deq.numpy()
    # fp32 (not bf16-representable) input and a 3-bit codebook at D=128
    qz3 = TurboQuantMSE(128, 3, seed=42)
    k, v = synth(16, 2, 128, seed=5)
    rt = qz3.rotation.T.contiguous()
    p3, n3 = _tq4_compress_cpu(v, rt[:, 0::2].contiguous(), rt[:, 1::2].contiguous(),
                               qz3.codebook.boundaries)
    comp["x_f32_128"] = v.numpy()
    comp["packed_f32_128_b3"] = p3.numpy()
    comp["norms_f32_128_b3"] = n3.numpy()
    np.savez_compressed(os.path.join(HERE, "compress.npz"), **comp)

    # ---- 4. paged write through the reference vLLM impl -------------------------------
    from turboquant_vllm.vllm.tq4_backend import (
        TQ4AttentionBackend,
        TQ4AttentionImpl,
        _padded_slot_bytes,
        _tq4_bytes_per_token,
        _tq4_bytes_per_token_kv,
    )

    def make_impl(h_kv, h_q, d, kq, vq):
        impl = object.__new__(TQ4AttentionImpl)
        impl.head_size, impl.num_kv_heads, impl.num_heads = d, h_kv, h_q
        impl._tq4_rotation = kq.rotation.clone()
        impl._k_centroids = kq.codebook.centroids.clone()
        impl._k_boundaries = kq.codebook.boundaries.clone()
        impl._v_centroids = vq.codebook.centroids.clone()
        impl._v_boundaries = vq.codebook.boundaries.clone()
        rt = kq.rotation.T.contiguous()
        impl._tq4_rot_T_even = rt[:, 0::2].contiguous()
        impl._tq4_rot_T_odd = rt[:, 1::2].contiguous()
        impl._cg_buffers_ready = False
        impl._k_idx_size = impl._v_idx_size = d // 2
        impl._k_idx_end = h_kv * (d // 2)
        impl._k_norm_end = impl._k_idx_end + h_kv * 4
        impl._v_idx_end = impl._k_norm_end + h_kv * (d // 2)
        impl._total_bytes = impl._v_idx_end + h_kv * 4
        return impl

    paged = {}
    bs = 16
    for tag, d, h_kv, h_q, vbits, padded in (
        ("k4v4", 128, 2, 8, 4, False),
        ("k4v3", 128, 2, 8, 3, True),
        ("d96", 96, 4, 4, 4, False),
        ("d64g7", 64, 1, 7, 4, False),
        # K/V regions on 16-byte boundaries (KV heads a multiple of 4): the layout the tcgen05
        # chunked-prefill kernel accepts
        ("k4v4h4", 128, 4, 16, 4, True),
    ):
        kq = TurboQuantMSE(d, 4, seed=42)
        vq = kq if vbits == 4 else TurboQuantMSE(d, vbits, seed=42)
        impl = make_impl(h_kv, h_q, d, kq, vq)
        seq_lens = [32, 17, 48, 1]
        total_blocks = sum((s + bs - 1) // bs for s in seq_lens) + 2
        width = h_kv * _padded_slot_bytes(d) if padded else impl._total_bytes
        cache = torch.zeros(total_blocks, bs, width, dtype=torch.uint8)
        order = list(range(total_blocks))
        random.Random(42).shuffle(order)
        max_blocks = max((s + bs - 1) // bs for s in seq_lens)
        bt = torch.zeros(len(seq_lens), max_blocks, dtype=torch.int32)
        slots, bi = [], 0
        for i, s in enumerate(seq_lens):
            for b in range((s + bs - 1) // bs):
                bt[i, b] = order[bi]
                bi += 1
            for t in range(s):
                slots.append(int(bt[i, t // bs]) * bs + t % bs)
        n = sum(seq_lens)
        k, v = synth(n, h_kv, d, seed=11 + d + vbits)
        k, v = k.bfloat16(), v.bfloat16()
        slot_mapping = torch.tensor(slots, dtype=torch.int64)
        impl._compress_and_store(k, v, cache, slot_mapping)

        # fp32 reference attention composed from the reference's own functions
        g = torch.Generator().manual_seed(77 + d)
        q_dec = torch.randn(len(seq_lens), h_q, d, generator=g).bfloat16()
        q_lens = [8, 17, 5, 1]  # prefill chunk lengths (<= seq_len), bottom-right aligned
        q_pre = torch.randn(sum(q_lens), h_q, d, generator=g).bfloat16()
        rot = kq.rotation
        scale = 1.0 / math.sqrt(d)

        def attend(qrows, i, s, window=None):
            flat = cache.reshape(-1, cache.shape[-1])
            rows = torch.stack(
                [flat[int(bt[i, t // bs]) * bs + t % bs] for t in range(s)]
            )
            a, b_, c_, tot = impl._k_idx_end, impl._k_norm_end, impl._v_idx_end, impl._total_bytes
            kp = rows[:, :a].contiguous().reshape(s, h_kv, d // 2)
            kn = rows[:, a:b_].contiguous().view(torch.float32).reshape(s, h_kv, 1)
            vp = rows[:, b_:c_].contiguous().reshape(s, h_kv, d // 2)
            vn = rows[:, c_:tot].contiguous().view(torch.float32).reshape(s, h_kv, 1)
            kd = _tq4_decompress_cpu(kp, kn, impl._k_centroids, torch.float32)
            vd = _tq4_decompress_cpu(vp, vn, impl._v_centroids, torch.float32)
            grp = h_q // h_kv
            kd = kd.permute(1, 0, 2).repeat_interleave(grp, 0)
            vd = vd.permute(1, 0, 2).repeat_interleave(grp, 0)
            qr = (qrows.float() @ rot.T).permute(1, 0, 2)
            ql = qrows.shape[0]
            qpos = (s - ql) + torch.arange(ql).unsqueeze(1)
            kpos = torch.arange(s).unsqueeze(0)
            mask = kpos <= qpos
            if window is not None:
                mask &= kpos > qpos - window
            o = torch.nn.functional.scaled_dot_product_attention(
                qr, kd, vd, attn_mask=mask.unsqueeze(0), scale=scale
            )
            return (o.permute(1, 0, 2) @ rot)

        dec_out = torch.stack(
            [attend(q_dec[i : i + 1], i, s)[0] for i, s in enumerate(seq_lens)]
        )
        pre_out, pre_out_w, off = [], [], 0
        for i, (s, ql) in enumerate(zip(seq_lens, q_lens)):
            pre_out.append(attend(q_pre[off : off + ql], i, s))
            pre_out_w.append(attend(q_pre[off : off + ql], i, s, window=9))
            off += ql
        paged[f"{tag}_key"] = k.float().numpy()
        paged[f"{tag}_value"] = v.float().numpy()
        paged[f"{tag}_slot_mapping"] = slot_mapping.numpy()
        paged[f"{tag}_block_table"] = bt.numpy()
        paged[f"{tag}_seq_lens"] = np.array(seq_lens, dtype=np.int32)
        paged[f"{tag}_q_lens"] = np.array(q_lens, dtype=np.int32)
        paged[f"{tag}_cache"] = cache.numpy()
        paged[f"{tag}_q_dec"] = q_dec.float().numpy()
        paged[f"{tag}_q_pre"] = q_pre.float().numpy()
        paged[f"{tag}_dec_out"] = dec_out.numpy()
        paged[f"{tag}_pre_out"] = torch.cat(pre_out).numpy()
        paged[f"{tag}_pre_out_w9"] = torch.cat(pre_out_w).numpy()
        paged[f"{tag}_meta"] = np.array([d, h_kv, h_q, 4, vbits, bs], dtype=np.int32)
    np.savez_compressed(os.path.join(HERE, "paged.npz"), **paged)

    # ---- 5. byte-size known answers ----------------------------------------------------
    kat = {
        "bytes_per_token_128_4": _tq4_bytes_per_token(128, 4),
        "bytes_per_token_64_4": _tq4_bytes_per_token(64, 4),
        "bytes_per_token_128_3": _tq4_bytes_per_token(128, 3),
        "bytes_per_token_kv_128": _tq4_bytes_per_token_kv(128),
        "bytes_per_token_kv_64": _tq4_bytes_per_token_kv(64),
        "padded_slot_64": _padded_slot_bytes(64),
        "padded_slot_96": _padded_slot_bytes(96),
        "padded_slot_128": _padded_slot_bytes(128),
        "padded_slot_256": _padded_slot_bytes(256),
        "cache_shape_100_16_8_128": np.array(
            TQ4AttentionBackend.get_kv_cache_shape(100, 16, 8, 128), dtype=np.int64
        ),
    }
    np.savez_compressed(os.path.join(HERE, "sizes.npz"), **{k: np.asarray(v) for k, v in kat.items()})

    # ---- 6. round trip + decode on the CPU-reference configuration ----------------------
    d, h_kv, h_q, n = 128, 8, 32, 1024
    qz = TurboQuantMSE(d, 4, seed=42)
    k, v = synth(n, h_kv, d, seed=0)
    g = torch.Generator().manual_seed(1)
    q = torch.randn(h_q, d, generator=g).bfloat16()
    ki, kn = qz.quantize(k)
    vi, vn = qz.quantize(v)
    kpk = CompressedDynamicCache._nibble_pack(ki.to(torch.uint8))
    vpk = CompressedDynamicCache._nibble_pack(vi.to(torch.uint8))
    kd = qz.dequantize(CompressedDynamicCache._nibble_unpack(kpk), kn)
    vd = qz.dequantize(CompressedDynamicCache._nibble_unpack(vpk), vn)

    def sdpa(kk, vv):
        grp = h_q // h_kv
        kk = kk.permute(1, 0, 2).repeat_interleave(grp, 0)
        vv = vv.permute(1, 0, 2).repeat_interleave(grp, 0)
        return torch.nn.functional.scaled_dot_product_attention(
            q.float().unsqueeze(1), kk, vv
        ).squeeze(1)

    out_c = sdpa(kd, vd)
    out_u = sdpa(k, v)
    np.savez_compressed(
        os.path.join(HERE, "config1.npz"),
        q=q.float().numpy(),
        k_packed=kpk.numpy(),
        v_packed=vpk.numpy(),
        k_norms=kn.numpy(),
        v_norms=vn.numpy(),
        out_compressed=out_c.numpy(),
        out_uncompressed=out_u.numpy(),
    )

    # ---- 7. HF cache wrapper -------------------------------------------------------------
    from transformers import DynamicCache

    hf = {}
    for tag, kb, vb in (("b4", 4, 4), ("k4v3", 4, 3)):
        cache = DynamicCache()
        cc = CompressedDynamicCache(cache, head_dim=64, k_bits=kb, v_bits=vb, seed=42)
        g = torch.Generator().manual_seed(9)
        k1 = torch.randn(1, 2, 5, 64, generator=g).bfloat16()
        v1 = torch.randn(1, 2, 5, 64, generator=g).bfloat16()
        k2 = torch.randn(1, 2, 1, 64, generator=g).bfloat16()
        v2 = torch.randn(1, 2, 1, 64, generator=g).bfloat16()
        cache.update(k1, v1, 0)
        ok, ov = cache.update(k2, v2, 0)
        kpk_, knm_, vpk_, vnm_ = cc.get_compressed(0)
        hf[f"{tag}_k1"], hf[f"{tag}_v1"] = k1.float().numpy(), v1.float().numpy()
        hf[f"{tag}_k2"], hf[f"{tag}_v2"] = k2.float().numpy(), v2.float().numpy()
        hf[f"{tag}_kidx"], hf[f"{tag}_knorm"] = kpk_.numpy(), knm_.numpy()
        hf[f"{tag}_vidx"], hf[f"{tag}_vnorm"] = vpk_.numpy(), vnm_.numpy()
        hf[f"{tag}_out_k"], hf[f"{tag}_out_v"] = ok.float().numpy(), ov.float().numpy()
        hf[f"{tag}_seq_len"] = np.array(cache.get_seq_length(0))
        hf[f"{tag}_vram"] = np.array(cc.vram_bytes())
        hf[f"{tag}_baseline"] = np.array(cc.baseline_vram_bytes())
    np.savez_compressed(os.path.join(HERE, "hf_cache.npz"), **hf)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
