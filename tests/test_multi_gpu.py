"""Sequence-split decode on two GPUs over NCCL: every rank runs the CUDA attention kernel on its
token slice (rotated output + log-sum-exp), one all-gather, the CUDA merge kernel; the result
must match the fp32 oracle run on the whole sequences.  Skipped on boxes with fewer than 2 GPUs."""

from __future__ import annotations

import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _worker(rank: int, world: int, port: int, ret):
    sys.path[:0] = [ROOT, os.path.join(ROOT, "turboquant-vllm_b200")]
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.distributed as dist

    from oracle import tq4_oracle as O
    from tests.helpers import Prims, build_paged_case, cosine
    from turboquant_vllm import parallel

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        d, h_kv, h_q, bs = 128, 8, 32, 16
        pr = Prims(d)
        seq_lens = [700, 16, 1300, 33]
        case = build_paged_case(seq_lens, h_kv, d, bs, pr, seed=11, padded=True)
        g = torch.Generator().manual_seed(3)
        q = torch.randn(len(seq_lens), h_q, d, generator=g).bfloat16()
        full = O.paged_decode_fp32(q, case["cache"], case["block_table"], seq_lens, pr.kc, pr.vc,
                                   pr.rot, h_kv)
        bt = case["block_table"]
        local_len, local_bt = [], torch.zeros_like(bt)
        for i, s in enumerate(seq_lens):
            st, en = parallel.split_sequence(s, world, bs)[rank]
            local_len.append(en - st)
            nb_loc = (en - st + bs - 1) // bs
            local_bt[i, :nb_loc] = bt[i, st // bs: st // bs + nb_loc]
        out = parallel.split_kv_decode(
            q.to(dev), case["cache"].to(dev), local_bt.to(dev),
            torch.tensor(local_len, dtype=torch.int32, device=dev),
            pr.kc.to(dev), pr.vc.to(dev), pr.rot.to(dev).contiguous(), h_kv, bs,
            out_dtype=torch.float32)
        torch.cuda.synchronize()
        o = out.float().cpu()
        ret[rank] = (cosine(o, full), float((o - full).abs().max()))
    finally:
        dist.destroy_process_group()


def test_split_kv_decode_two_gpus_nccl():
    world = 2
    port = 29700 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        res = dict(ret)
    assert set(res) == {0, 1}
    for r, (cos, err) in res.items():
        assert cos >= 0.9999 and err <= 2e-3, (r, cos, err)  # fp32-oracle tolerance of the path
