"""GPU parity: decompress rows / whole-cache decompress."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import tq4_oracle as O
from tests.helpers import Prims, build_paged_case, t

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(cuda_lib):
    from turboquant_vllm.kernels import ops as _ops

    return _ops


@pytest.mark.parametrize("d", [64, 96, 128, 256])
def test_decompress_fp32_bit_exact(ops, golden, d):
    g = golden("compress.npz")
    p = Prims(d).cuda()
    out = ops.tq4_decompress(t(g[f"packed_{d}"]).cuda(), t(g[f"norms_{d}"]).cuda(), p["kc"], torch.float32)
    assert np.array_equal(out.cpu().numpy(), g[f"dec_{d}"])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decompress_16bit_equals_rounded_oracle(ops, golden, dtype):
    g = golden("compress.npz")
    pr = Prims(128)
    p = pr.cuda()
    packed, norms = t(g["packed_128"]), t(g["norms_128"])
    out = ops.tq4_decompress(packed.cuda(), norms.cuda(), p["kc"], dtype)
    ref = O.decompress_rows(packed, norms, pr.kc, dtype)
    assert out.dtype == dtype and torch.equal(out.cpu(), ref)


def test_decompress_out_contract(ops, golden):
    g = golden("compress.npz")
    p = Prims(128).cuda()
    packed, norms = t(g["packed_128"]).cuda(), t(g["norms_128"]).cuda()
    a = ops.tq4_decompress(packed, norms, p["kc"], torch.bfloat16)
    buf = torch.full((24, 4, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    r = ops.tq4_decompress(packed, norms, p["kc"], torch.bfloat16, out=buf)
    assert r is buf and torch.equal(buf, a)
    big = torch.zeros(100, 4, 128, dtype=torch.bfloat16, device="cuda")
    r2 = ops.tq4_decompress(packed, norms, p["kc"], torch.bfloat16, out=big[:24])
    assert torch.equal(r2, a) and not big[24:].any()


@pytest.mark.parametrize("padded", [False, True])
def test_decompress_cache(ops, padded):
    pr = Prims(128, 4, 3)
    p = pr.cuda()
    case = build_paged_case([40, 9], 8, 128, 16, pr, seed=4, padded=padded)
    cache = case["cache"]
    k, v = ops.tq4_decompress_cache(cache.cuda(), 8, 128, p["kc"], p["vc"], torch.float32)
    kp, kn, vp, vn = O.split_rows(cache.reshape(-1, cache.shape[-1]), 8, 128)
    assert torch.equal(k.cpu(), O.decompress_rows(kp, kn, pr.kc))
    assert torch.equal(v.cpu(), O.decompress_rows(vp, vn, pr.vc))
