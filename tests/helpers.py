"""Shared helpers for the parity tests: primitives, seeded paged caches, error metrics."""

from __future__ import annotations

import random

import numpy as np
import torch

from oracle import tq4_oracle as O


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


class Prims:
    """Rotation + codebooks for (head_dim, k_bits, v_bits, seed), on CPU and (lazily) on GPU."""

    def __init__(self, d: int, k_bits: int = 4, v_bits: int = 4, seed: int = 42):
        self.d = d
        self.kc, self.kb = O.solve_lloyd_max(d, k_bits)
        self.vc, self.vb = O.solve_lloyd_max(d, v_bits)
        self.rot = O.rotation_matrix(d, seed)
        rt = self.rot.T.contiguous()
        self.even = rt[:, 0::2].contiguous()
        self.odd = rt[:, 1::2].contiguous()

    def cuda(self):
        dev = "cuda"
        return dict(
            rot=self.rot.to(dev), even=self.even.to(dev), odd=self.odd.to(dev),
            kc=self.kc.to(dev), kb=self.kb.to(dev), vc=self.vc.to(dev), vb=self.vb.to(dev),
        )


def build_paged_case(seq_lens, h_kv, d, bs, prims: Prims, seed=0, padded=False, extra_blocks=2,
                     dtype=torch.bfloat16):
    """Seeded K/V (outlier channels), shuffled physical blocks, cache written by the ORACLE."""
    nblk = [(s + bs - 1) // bs for s in seq_lens]
    total_blocks = sum(nblk) + extra_blocks
    if padded == "dense":  # the tight row rounded up to 16 bytes (the backend's TQ4_DENSE_ROWS format)
        width = (O.row_layout(h_kv, d)[3] + 15) & ~15
    else:
        width = h_kv * O.padded_slot_bytes(d) if padded else O.row_layout(h_kv, d)[3]
    cache = torch.zeros(total_blocks, bs, width, dtype=torch.uint8)
    order = list(range(total_blocks))
    random.Random(seed).shuffle(order)
    bt = torch.zeros(len(seq_lens), max(max(nblk), 1), dtype=torch.int32)
    slots, bi = [], 0
    for i, s in enumerate(seq_lens):
        for b in range(nblk[i]):
            bt[i, b] = order[bi]
            bi += 1
        for tok in range(s):
            slots.append(int(bt[i, tok // bs]) * bs + tok % bs)
    n = sum(seq_lens)
    k, v = O.synthetic_kv(max(n, 1), h_kv, d, seed=seed + 1)
    k, v = k[:n].to(dtype), v[:n].to(dtype)
    slot_mapping = torch.tensor(slots, dtype=torch.int64)
    if n:
        O.write_paged(k, v, cache, slot_mapping, prims.rot, prims.kb, prims.vb)
    return dict(cache=cache, block_table=bt, seq_lens=torch.tensor(seq_lens, dtype=torch.int32),
                slot_mapping=slot_mapping, key=k, value=v)


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    den = a.norm() * b.norm()
    return 1.0 if den == 0 else float((a @ b) / den)


def index_mismatch(packed_a: torch.Tensor, packed_b: torch.Tensor) -> float:
    a = O.nibble_unpack(packed_a.cpu())
    b = O.nibble_unpack(packed_b.cpu())
    return float((a != b).float().mean())


def ulp_diff(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in units of the last place between two positive fp32 tensors."""
    ia = a.cpu().contiguous().view(torch.int32).long()
    ib = b.cpu().contiguous().view(torch.int32).long()
    return (ia - ib).abs()
