"""The allocation-free attention entry point (collected last on purpose).

`tq4_paged_attention_static` serves callers that cannot allocate device memory when they reach
the attention call (all HBM already handed to the KV cache, a frozen memory pool, a loop that must
not hit cudaMalloc's implicit synchronisation): its scratch is a fixed array inside the library.
Checked here through the C ABI: same output as the regular entry point (which takes a
caller-provided workspace), on two calls in a row that share the built-in scratch, for decode and
for a chunked-prefill call; oversized requests are refused with a clear error.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from tests.helpers import Prims, build_paged_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(cuda_lib):
    from turboquant_vllm.kernels import ops as _ops

    return _ops


def _case(seed, seq_lens, h_kv=8, h_q=32, d=128, bs=16):
    pr = Prims(d)
    case = build_paged_case(seq_lens, h_kv, d, bs, pr, seed=seed, padded=True)
    q = torch.randn(len(seq_lens), h_q, d, generator=torch.Generator().manual_seed(seed)).bfloat16()
    return pr.cuda(), case, q


@pytest.mark.parametrize("mode", [1, 2])
def test_static_scratch_matches_workspace_entry_point(ops, mode):
    outs = []
    for seed, seq_lens in ((3, [130, 17, 64, 1]), (4, [48, 300, 0, 95])):  # two calls in a row
        p, case, q = _case(seed, seq_lens)
        kw = dict(q=q.cuda(), kv_cache=case["cache"].cuda(), block_table=case["block_table"].cuda(),
                  seq_lens=case["seq_lens"].cuda(), k_centroids=p["kc"], v_centroids=p["vc"],
                  rotation=p["rot"].contiguous(), num_kv_heads=8, block_size=16)
        ref = ops.paged_tq4_attention(out_dtype=torch.float32, mode=mode, **kw)
        out = torch.full_like(ref, float("nan"))
        got = ops.paged_tq4_attention_static(out=out, mode=mode, **kw)
        assert got is out
        assert torch.equal(out, ref)  # same kernels, same arithmetic: bit-identical
        outs.append(out)
    assert not torch.equal(outs[0], outs[1])


def test_static_scratch_prefill_and_repeat(ops):
    pr = Prims(128)
    p = pr.cuda()
    seq_lens, q_lens = [150, 33], [22, 33]
    case = build_paged_case(seq_lens, 2, 128, 16, pr, seed=12)
    q = torch.randn(sum(q_lens), 8, 128, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    qsl = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32).cuda()
    kw = dict(q=q, kv_cache=case["cache"].cuda(), block_table=case["block_table"].cuda(),
              seq_lens=case["seq_lens"].cuda(), k_centroids=p["kc"], v_centroids=p["vc"],
              rotation=p["rot"].contiguous(), num_kv_heads=2, block_size=16, query_start_loc=qsl,
              sliding_window=48)
    ref = ops.paged_tq4_attention(out_dtype=torch.float32, **kw)
    out = torch.empty_like(ref)
    for _ in range(2):  # the scratch keeps the previous call's contents; the result must not care
        out.fill_(7.0)
        ops.paged_tq4_attention_static(out=out, **kw)
        assert torch.equal(out, ref)


def test_static_scratch_rejects_oversized_request(ops):
    pr = Prims(128)
    p = pr.cuda()
    rows = 2048  # needs far more than the built-in 32 MiB
    q = torch.zeros(rows, 32, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(rows, 32, 128, dtype=torch.float32, device="cuda")
    cache = torch.zeros(4, 16, 8 * 256, dtype=torch.uint8, device="cuda")
    bt = torch.zeros(rows, 1, dtype=torch.int32, device="cuda")
    sl = torch.zeros(rows, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="static"):
        ops.paged_tq4_attention_static(q, cache, bt, sl, p["kc"], p["vc"], p["rot"].contiguous(), 8, 16, out)
