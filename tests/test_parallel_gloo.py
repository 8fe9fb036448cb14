"""N > 1 host logic on CPU: two gloo ranks run the sequence-split decode wiring
(per-rank partial attention -> one all-gather -> log-sum-exp merge) with the oracle standing in
for the CUDA kernels, and must reproduce single-process attention.  Also the head-sharding and
sequence-splitting helpers."""

from __future__ import annotations

import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, ret):
    sys.path[:0] = [ROOT, os.path.join(ROOT, "turboquant-vllm_b200")]
    import torch.distributed as dist

    from oracle import tq4_oracle as O
    from tests.helpers import Prims
    from turboquant_vllm import parallel

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d, h_kv, h_q, bs = 96, 4, 8, 16
        pr = Prims(d)
        seq_lens = [70, 16, 130]
        g = torch.Generator().manual_seed(0)
        q = torch.randn(len(seq_lens), h_q, d, generator=g).bfloat16()
        # the full cache (identical on both ranks, built from the same seeds) ...
        n = sum(seq_lens)
        k, v = O.synthetic_kv(n, h_kv, d, seed=5, dtype=torch.bfloat16)
        width = O.row_layout(h_kv, d)[3]
        nblk = [(s + bs - 1) // bs for s in seq_lens]
        full_cache = torch.zeros(sum(nblk), bs, width, dtype=torch.uint8)
        bt = torch.zeros(len(seq_lens), max(nblk), dtype=torch.int32)
        slots, b = [], 0
        for i, s in enumerate(seq_lens):
            for j in range(nblk[i]):
                bt[i, j] = b
                b += 1
            slots += [int(bt[i, t // bs]) * bs + t % bs for t in range(s)]
        O.write_paged(k, v, full_cache, torch.tensor(slots), pr.rot, pr.kb, pr.vb)
        full = O.paged_decode_fp32(q, full_cache, bt, seq_lens, pr.kc, pr.vc, pr.rot, h_kv)
        # ... and this rank's slice of every sequence: a shifted block table + local lengths
        local_len, local_bt = [], torch.zeros_like(bt)
        for i, s in enumerate(seq_lens):
            st, en = parallel.split_sequence(s, world, bs)[rank]
            local_len.append(en - st)
            nb_loc = (en - st + bs - 1) // bs
            local_bt[i, :nb_loc] = bt[i, st // bs: st // bs + nb_loc]
        eye = torch.eye(d)

        def attend(q_, lse_):  # oracle stand-in for the fused kernel (rotated output + LSE)
            o, l = O.paged_attention_fp32(q_.float() @ pr.rot.T, full_cache, local_bt, local_len,
                                          torch.arange(len(seq_lens) + 1), pr.kc, pr.vc, eye, h_kv,
                                          None, False, None, True)
            lse_.copy_(l)
            return o

        def combine(po, pl):
            return O.lse_combine(po, pl) @ pr.rot

        out = parallel.split_kv_decode(q, full_cache, local_bt, torch.tensor(local_len, dtype=torch.int32),
                                       pr.kc, pr.vc, pr.rot, h_kv, bs, attend=attend, combine=combine)
        ret[rank] = bool(torch.allclose(out, full, rtol=1e-4, atol=1e-5))
    finally:
        dist.destroy_process_group()


def test_split_kv_decode_two_gloo_ranks():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_shard_heads_and_split_sequence():
    sys.path[:0] = [os.path.join(ROOT, "turboquant-vllm_b200")]
    from turboquant_vllm import parallel

    qh, kvh = parallel.shard_heads(1, 4, 32, 8)
    assert list(kvh) == [2, 3] and list(qh) == list(range(8, 16))
    allq = [h for r in range(8) for h in parallel.shard_heads(r, 8, 32, 8)[0]]
    assert allq == list(range(32))
    with pytest.raises(ValueError):
        parallel.shard_heads(0, 3, 32, 8)
    for s, w in ((131072, 8), (70, 2), (16, 4), (0, 2), (17, 8)):
        parts = parallel.split_sequence(s, w, 16)
        assert parts[0][0] == 0 and parts[-1][1] == s
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        assert all(st % 16 == 0 for st, _ in parts if st < s)
