"""HuggingFace-side fused TQ4 attention: contiguous K/V tensors and the fused-mode cache, against
the fp32 oracle.  Shapes follow the reference's matrix (tests/test_flash_attention_tq4_kv.py:45-53)."""

from __future__ import annotations

import math
import types

import pytest
import torch

from oracle import tq4_oracle as O

pytestmark = pytest.mark.gpu

CHANNELS = (3, 17, 64, 101)  # outlier channels of the synthetic K/V


def _kv(b, h, s, d, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(b, h, s, d, generator=g)
    for c in CHANNELS:
        if c < d:
            x[..., c] *= 8
    return x.to(dtype)


def _prims(d, seed=42):
    from turboquant_vllm.quantizer import TurboQuantMSE

    qz = TurboQuantMSE(d, 4, seed=seed)
    return qz, qz.rotation.clone(), qz.codebook.centroids.clone(), qz.codebook.boundaries.clone()


def _oracle_attention(q, k_packed, k_norms, v_packed, v_norms, cents, rot, causal, sm_scale=None):
    """fp32, top-left causal rule of the reference kernel, everything on CPU -> [B, Hq, Sq, D]."""
    b, hq, sq, d = q.shape
    hkv, s = k_packed.shape[1], k_packed.shape[2]
    k = O.decompress_rows(k_packed.reshape(-1, 1, d // 2), k_norms.reshape(-1, 1, 1), cents).reshape(b, hkv, s, d)
    v = O.decompress_rows(v_packed.reshape(-1, 1, d // 2), v_norms.reshape(-1, 1, 1), cents).reshape(b, hkv, s, d)
    k = k.repeat_interleave(hq // hkv, dim=1)
    v = v.repeat_interleave(hq // hkv, dim=1)
    q_rot = q.float() @ rot.T
    scores = q_rot @ k.transpose(-1, -2) * (sm_scale or 1.0 / math.sqrt(d))
    if causal and sq > 1:
        m = torch.arange(sq)[:, None] >= torch.arange(s)[None, :]
        scores = scores.masked_fill(~m, float("-inf"))
    return torch.softmax(scores, dim=-1) @ v @ rot


def _check(actual, expected):
    a, e = actual.float().cpu().flatten(), expected.flatten()
    cos = torch.nn.functional.cosine_similarity(a, e, dim=0).item()
    assert cos >= 0.9999, cos
    assert (a - e).abs().max().item() <= 2e-3, (a - e).abs().max().item()


SHAPES = [
    pytest.param(1, 4, 4, 32, 32, 128, False, torch.float16, id="mha_basic"),
    pytest.param(1, 32, 8, 64, 64, 128, False, torch.float16, id="gqa_4to1"),
    pytest.param(1, 28, 4, 64, 64, 128, False, torch.float16, id="gqa_7to1"),
    pytest.param(1, 32, 8, 1, 512, 128, False, torch.float16, id="decode"),
    pytest.param(1, 4, 4, 64, 64, 128, True, torch.float16, id="causal"),
    pytest.param(1, 32, 8, 512, 512, 128, True, torch.bfloat16, id="long_causal"),
    pytest.param(4, 32, 8, 64, 64, 128, False, torch.float16, id="batched"),
    pytest.param(2, 8, 4, 5, 300, 128, True, torch.bfloat16, id="causal_fewer_queries_than_keys"),
    pytest.param(2, 8, 4, 40, 333, 96, False, torch.bfloat16, id="d96"),
    pytest.param(1, 8, 4, 3, 70, 256, True, torch.float16, id="d256"),
    pytest.param(3, 6, 2, 1, 257, 64, False, torch.float16, id="d64_two_kv_heads"),
]


@pytest.mark.parametrize(("b", "hq", "hkv", "sq", "skv", "d", "causal", "dtype"), SHAPES)
def test_contiguous_kv_matches_oracle(cuda_lib, b, hq, hkv, sq, skv, d, causal, dtype):
    from turboquant_vllm.token_rows import TokenRowStore
    from turboquant_vllm.triton.flash_attention_tq4_kv import triton_flash_attention_tq4_kv

    qz, rot, cents, _ = _prims(d)
    q = torch.randn(b, hq, sq, d, generator=torch.Generator().manual_seed(1)).to(dtype)
    k_packed, k_norms = qz.quantize_packed(_kv(b, hkv, skv, d, 2, dtype).cuda())
    v_packed, v_norms = qz.quantize_packed(_kv(b, hkv, skv, d, 3, dtype).cuda())
    expected = _oracle_attention(q, k_packed.cpu(), k_norms.cpu(), v_packed.cpu(), v_norms.cpu(), cents, rot, causal)
    # fp32 output for the parity bound
    store = TokenRowStore.from_tensors(k_packed, k_norms.squeeze(-1), v_packed, v_norms)
    views = store.views()
    assert torch.equal(views[0], k_packed) and torch.equal(views[3], v_norms)
    out32 = store.attention(q.cuda(), cents.cuda(), cents.cuda(), rot.cuda(), None, causal, out_dtype=torch.float32)
    assert out32.shape == (b, sq, hq, d)
    _check(out32.transpose(1, 2), expected)
    # the reference's call: output in q's dtype, [B, Hq, Sq, D]
    out = triton_flash_attention_tq4_kv(q.cuda(), k_packed, k_norms, v_packed, v_norms.squeeze(-1),
                                        cents.cuda(), rot.cuda(), is_causal=causal)
    assert out.shape == q.shape and out.dtype == dtype
    torch.testing.assert_close(out.float().cpu(), expected, atol=1.2e-2, rtol=1.6e-2)


def test_fused_mode_cache_rows_and_forward(cuda_lib):
    from transformers import DynamicCache

    from turboquant_vllm.kv_cache import CompressedDynamicCache
    from turboquant_vllm.triton.attention_interface import triton_fa_tq4_kv_forward

    b, hq, hkv, d = 2, 8, 4, 128
    plain = CompressedDynamicCache(DynamicCache(), head_dim=d, bits=4)
    cache = DynamicCache()
    cc = CompressedDynamicCache(cache, head_dim=d, bits=4)
    cc.fused_mode = True
    module = types.SimpleNamespace(layer_idx=0, _tq4_cache=cc, is_causal=True)
    chunks = (70, 1, 1, 200, 1, 300, 1)  # crosses the 256- and 512-token capacities
    ks, vs = [], []
    total = 0
    for i, n in enumerate(chunks):
        k, v = _kv(b, hkv, n, d, 10 + i, torch.bfloat16).cuda(), _kv(b, hkv, n, d, 50 + i, torch.bfloat16).cuda()
        rk, rv = cache.update(k, v, 0)
        assert rk is k and rv is v  # placeholders
        ks.append(k), vs.append(v)
        total += n
        assert cache.get_seq_length(0) == total
        store = cc.get_token_rows(0)
        assert store is not None and store.len == total and store.capacity % 256 == 0
        if n == 1 or i == 0:  # a decode step, and the first chunk (causal prefill from an empty cache)
            q = torch.randn(b, hq, n, d, generator=torch.Generator().manual_seed(90 + i)).bfloat16()
            kp, kn, vp, vn = (x.cpu() for x in cc.get_compressed(0))
            expected = _oracle_attention(q, kp, kn, vp, vn, cc.centroids, cc.rotation, causal=n > 1)
            out, weights = triton_fa_tq4_kv_forward(module, q.cuda(), k, v, None)
            assert weights is None and out.shape == (b, n, hq, d) and out.dtype == torch.bfloat16
            torch.testing.assert_close(out.float().cpu().transpose(1, 2), expected, atol=1.2e-2, rtol=1.6e-2)
    # the rows hold exactly what the stand-alone compress kernel produces
    k_all, v_all = torch.cat(ks, dim=2), torch.cat(vs, dim=2)
    want_k = plain._compress_tensor(plain.key_compressor, k_all, nibble_packed=True)
    want_v = plain._compress_tensor(plain.value_compressor, v_all, nibble_packed=True)
    kp, kn, vp, vn = cc.get_compressed(0)
    assert kp.shape == (b, hkv, total, d // 2) and kn.shape == (b, hkv, total, 1) and kn.dtype == torch.float32
    assert torch.equal(kp, want_k.indices) and torch.equal(kn, want_k.norms)
    assert torch.equal(vp, want_v.indices) and torch.equal(vn, want_v.norms)
    assert cc.vram_bytes() == 2 * b * hkv * total * (d // 2 + 4)
    assert cc.compression_stats()["seq_len"] == total
    # leaving fused mode: the next update returns dequantised K/V of every token held
    cc.fused_mode = False
    k = _kv(b, hkv, 1, d, 99, torch.bfloat16).cuda()
    out_k, out_v = cache.update(k, k, 0)
    assert cc.get_token_rows(0) is None and out_k.shape == (b, hkv, total + 1, d)
    full = torch.cat([k_all, k], dim=2).float()
    cos = torch.nn.functional.cosine_similarity(out_k.float().flatten(2), full.flatten(2), dim=-1)
    assert cos.min() > 0.98
    assert torch.equal(cc.get_compressed(0)[0][:, :, :total], want_k.indices)
    # and back: tokens stored before fused mode was switched on are carried over
    cc.fused_mode = True
    cache.update(k, k, 0)
    store = cc.get_token_rows(0)
    assert store is not None and store.len == total + 2
    assert torch.equal(cc.get_compressed(0)[0][:, :, :total], want_k.indices)


def test_install_on_a_model_matches_dequantised_path(cuda_lib):
    """Tiny random Llama: greedy logits through the fused backend against the same compressed cache
    read through HuggingFace SDPA on dequantised K/V."""
    from transformers import DynamicCache, LlamaConfig, LlamaForCausalLM

    from turboquant_vllm.kv_cache import CompressedDynamicCache
    from turboquant_vllm.triton.attention_interface import (
        BACKEND_NAME, install_fused_tq4_kv, uninstall_fused_tq4_kv)

    cfg = LlamaConfig(hidden_size=1024, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=4, head_dim=128, vocab_size=256, max_position_embeddings=1024)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).eval().to(device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 256, (2, 37), generator=torch.Generator().manual_seed(5)).cuda()
    steps = torch.randint(0, 256, (2, 4), generator=torch.Generator().manual_seed(6)).cuda()

    def run(fused: bool):
        cache = DynamicCache(config=cfg)
        cc = CompressedDynamicCache(cache, head_dim=128, bits=4)
        if fused:
            install_fused_tq4_kv(model, cc)
            assert model.config._attn_implementation == BACKEND_NAME and cc.fused_mode
        logits = []
        with torch.no_grad():
            logits.append(model(ids, past_key_values=cache).logits[:, -1].float())
            for i in range(steps.shape[1]):
                logits.append(model(steps[:, i : i + 1], past_key_values=cache).logits[:, -1].float())
        if fused:
            assert cc.get_token_rows(1) is not None and cache.get_seq_length(0) == 37 + steps.shape[1]
            uninstall_fused_tq4_kv(model)
            assert model.config._attn_implementation == "sdpa" and not cc.fused_mode
            assert not any(hasattr(m, "_tq4_cache") for m in model.modules())
        return torch.stack(logits)

    base, fused = run(False), run(True)
    cos = torch.nn.functional.cosine_similarity(base.flatten(1), fused.flatten(1), dim=-1)
    assert cos.min() > 0.999, cos
    with pytest.raises(AttributeError, match="no config"):
        install_fused_tq4_kv(torch.nn.Linear(2, 2), CompressedDynamicCache(DynamicCache(), head_dim=128, bits=4))
