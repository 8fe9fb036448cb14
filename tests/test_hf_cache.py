"""HF CompressedDynamicCache: host-side contract on CPU, numerics on GPU against the trace the
reference produced (tests/golden/hf_cache.npz)."""

from __future__ import annotations

import types
import warnings

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")
from transformers import DynamicCache  # noqa: E402

from tests.helpers import index_mismatch, t, ulp_diff  # noqa: E402


def _cls():
    from turboquant_vllm.kv_cache import CompressedDynamicCache

    return CompressedDynamicCache


def test_constructor_contract_cpu():
    C = _cls()
    with pytest.raises(ValueError, match="No bit-width"):
        C(DynamicCache(), head_dim=64, bits=None)
    with pytest.raises(ValueError, match="k_bits=4 requires even head_dim"):
        C(DynamicCache(), head_dim=63, bits=4)
    cache = DynamicCache()
    orig_update = cache.update
    cc = C(cache, head_dim=64, k_bits=4, v_bits=3)
    assert (cc.k_bits, cc.v_bits, cc.bits) == (4, 3, 4)
    assert cc.rotation.shape == (64, 64) and cc.centroids.numel() == 16
    assert cc.value_compressor.quantizer.codebook.centroids.numel() == 8
    assert cache.update.__self__ is cc
    with pytest.warns(UserWarning, match="already wrapped"):
        C(cache, head_dim=64, bits=4)
    cc.restore()
    assert cache.update == orig_update
    with C(cache, head_dim=64, bits=4) as c2:
        assert cache.update.__self__ is c2 and c2.vram_bytes() == 0 and c2.compression_stats() == {}
        with pytest.raises(ValueError, match="not yet updated"):
            c2.get_compressed(0)
        assert cache.get_seq_length(0) == 0
    assert cache.update == orig_update
    idx = torch.randint(0, 16, (2, 3, 8), dtype=torch.uint8)
    assert torch.equal(C._nibble_unpack(C._nibble_pack(idx)), idx.long())


def test_mixed_attention_config_and_disabled_passthrough_cpu():
    C = _cls()
    cfg = types.SimpleNamespace(layer_types=["sliding_attention", "full_attention", "sliding_attention"])
    with pytest.warns(UserWarning, match="sliding window layer metadata"):
        cc = C(DynamicCache(), head_dim=64, bits=4, model_config=cfg)
    assert cc._full_attn_bypass == {1}
    k = torch.randn(1, 2, 3, 64)
    # a bypassed (full attention) layer is stored uncompressed by the original cache, even on CPU
    cache = DynamicCache()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        cc = C(cache, head_dim=64, bits=4, model_config=cfg)
    ok, ov = cache.update(k, k, 1)
    assert torch.equal(ok, k) and cache.get_seq_length(1) == 3
    with pytest.raises(ValueError, match="SWA-bypassed"):
        cc.get_compressed(1)
    cc.disable()
    ok, _ = cache.update(k, k, 0)
    assert torch.equal(ok, k)
    cc.enable()
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        cache.update(k, k, 2)  # compression needs a CUDA tensor


@pytest.mark.gpu
@pytest.mark.parametrize("tag,kb,vb", [("b4", 4, 4), ("k4v3", 4, 3)])
def test_update_matches_reference_trace(cuda_lib, golden, tag, kb, vb):
    g = golden("hf_cache.npz")
    C = _cls()
    cache = DynamicCache()
    cc = C(cache, head_dim=64, k_bits=kb, v_bits=vb, seed=42)
    dev = "cuda"
    k1, v1 = t(g[f"{tag}_k1"]).bfloat16().to(dev), t(g[f"{tag}_v1"]).bfloat16().to(dev)
    k2, v2 = t(g[f"{tag}_k2"]).bfloat16().to(dev), t(g[f"{tag}_v2"]).bfloat16().to(dev)
    cache.update(k1, v1, 0)
    ok, ov = cache.update(k2, v2, 0)
    kidx, knorm, vidx, vnorm = cc.get_compressed(0)
    assert kidx.shape == g[f"{tag}_kidx"].shape and vidx.shape == g[f"{tag}_vidx"].shape
    assert kidx.dtype == torch.uint8 and knorm.dtype == torch.float32
    assert index_mismatch(kidx, t(g[f"{tag}_kidx"])) <= 1e-4
    if vb == 4:
        assert index_mismatch(vidx, t(g[f"{tag}_vidx"])) <= 1e-4
    else:  # 3-bit values are stored one index per byte
        assert (vidx.cpu() != t(g[f"{tag}_vidx"])).float().mean() <= 1e-4 and vidx.max() <= 7
    assert ulp_diff(knorm, t(g[f"{tag}_knorm"])).max() <= 4
    assert ulp_diff(vnorm, t(g[f"{tag}_vnorm"])).max() <= 4
    assert ok.shape == (1, 2, 6, 64) and ok.dtype == torch.bfloat16
    assert torch.allclose(ok.float().cpu(), t(g[f"{tag}_out_k"]), atol=2e-2, rtol=2e-2)
    assert torch.allclose(ov.float().cpu(), t(g[f"{tag}_out_v"]), atol=2e-2, rtol=2e-2)
    assert cache.get_seq_length(0) == int(g[f"{tag}_seq_len"]) == 6
    assert cc.vram_bytes() == int(g[f"{tag}_vram"])
    assert cc.baseline_vram_bytes() == int(g[f"{tag}_baseline"])
    stats = cc.compression_stats()
    assert stats["seq_len"] == 6 and stats["k_bits"] == kb and stats["v_bits"] == vb
    assert set(stats) >= {"num_layers", "compressed_mib", "baseline_mib", "compression_ratio",
                          "savings_mib", "vram_estimate", "k_nibble_packed", "v_nibble_packed"}


@pytest.mark.gpu
def test_growth_fused_mode_and_quality(cuda_lib):
    C = _cls()
    cache = DynamicCache()
    cc = C(cache, head_dim=128, bits=4)
    g = torch.Generator().manual_seed(0)
    ks = [torch.randn(2, 4, n, 128, generator=g).bfloat16().cuda() for n in (70, 1, 1, 200, 1)]
    for k in ks:
        out_k, out_v = cache.update(k, -k, 0)
    full = torch.cat(ks, dim=2)
    assert out_k.shape == full.shape and cache.get_seq_length(0) == 273
    cos = torch.nn.functional.cosine_similarity(out_k.float().flatten(2), full.float().flatten(2), dim=-1)
    assert cos.min() > 0.98  # 4-bit reconstruction quality
    # symmetric codebook: V = -K reconstructs to (almost exactly) the negation
    diff = (out_v.float() + out_k.float()).abs()
    assert diff.max() < 0.1 and (diff > 0).float().mean() < 1e-2, (diff.max().item(), (diff > 0).float().mean().item())
    # every append kept the earlier tokens' bytes
    kidx, knorm, _, _ = cc.get_compressed(0)
    first = C(DynamicCache(), head_dim=128, bits=4)._compress_tensor(cc.key_compressor, ks[0], nibble_packed=True)
    assert torch.equal(kidx[:, :, :70], first.indices) and torch.equal(knorm[:, :, :70], first.norms)
    # fused mode: placeholders are returned, compressed storage keeps growing
    cc.fused_mode = True
    k = torch.randn(2, 4, 1, 128, generator=g).bfloat16().cuda()
    rk, _ = cache.update(k, k, 0)
    assert rk is k and cache.get_seq_length(0) == 274
    with pytest.raises(RuntimeError, match="primary head_dim"):
        cache.update(torch.zeros(2, 4, 1, 64, device="cuda").bfloat16(), torch.zeros(2, 4, 1, 64, device="cuda").bfloat16(), 1)


def test_token_rows_layout_cpu():
    """Token-row storage: the four reference tensors are views of one row buffer; growth keeps them."""
    from turboquant_vllm.token_rows import PAGE_TOKENS, TokenRowStore

    g = torch.Generator().manual_seed(3)
    b, h, s, d = 2, 4, 300, 128
    kp = torch.randint(0, 256, (b, h, s, d // 2), dtype=torch.uint8, generator=g)
    vp = torch.randint(0, 256, (b, h, s, d // 2), dtype=torch.uint8, generator=g)
    kn, vn = torch.rand(b, h, s, generator=g), torch.rand(b, h, s, 1, generator=g)
    store = TokenRowStore.from_tensors(kp, kn, vp, vn)
    assert store.len == s and store.capacity == 2 * PAGE_TOKENS and store.row_bytes == h * (d + 8)
    k_idx, k_norm, v_idx, v_norm = store.views()
    assert k_idx.shape == (b, h, s, d // 2) and k_norm.shape == (b, h, s, 1) and k_norm.dtype == torch.float32
    assert torch.equal(k_idx, kp) and torch.equal(v_idx, vp)
    assert torch.equal(k_norm.squeeze(-1), kn) and torch.equal(v_norm, vn)
    assert all(x.untyped_storage().data_ptr() == store.rows.untyped_storage().data_ptr() for x in store.views())
    # one token row = [K idx of all heads | K norms | V idx | V norms]
    row = store.rows[1, 7]
    assert torch.equal(row[: h * d // 2], kp[1, :, 7].reshape(-1))
    assert torch.equal(row[h * d // 2 : h * (d // 2 + 4)].view(torch.float32), kn[1, :, 7])
    assert torch.equal(row[h * (d // 2 + 4) : h * (d + 4)], vp[1, :, 7].reshape(-1))
    # pages of batch b are b*P .. b*P+P-1
    assert store.paged_cache().shape == (b * 2, PAGE_TOKENS, store.row_bytes)
    assert store.block_table().tolist() == [[0, 1], [2, 3]]
    store._reserve(513)  # growth doubles the capacity and keeps the tokens
    assert store.capacity == 4 * PAGE_TOKENS and torch.equal(store.views()[0], kp)
    assert store.block_table().tolist() == [[0, 1, 2, 3], [4, 5, 6, 7]]
    with pytest.raises(ValueError, match="even head_dim"):
        TokenRowStore(1, 4, 63, "cpu")
    with pytest.raises(ValueError, match="multiple of 4"):
        TokenRowStore(1, 1, 6, "cpu")


def test_fused_backend_install_and_fallthrough_cpu():
    """`install_fused_tq4_kv` wiring on a tiny random Llama; a module without a stashed cache is served
    by HuggingFace SDPA."""
    from transformers import LlamaConfig, LlamaForCausalLM
    from transformers.integrations.sdpa_attention import sdpa_attention_forward
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    from turboquant_vllm.triton.attention_interface import (
        BACKEND_NAME, install_fused_tq4_kv, triton_fa_tq4_kv_forward, uninstall_fused_tq4_kv)

    C = _cls()
    cfg = LlamaConfig(hidden_size=64, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=2, head_dim=32, vocab_size=32)
    model = LlamaForCausalLM(cfg).eval()
    cc = C(DynamicCache(config=cfg), head_dim=32, bits=4)
    install_fused_tq4_kv(model, cc)
    assert ALL_ATTENTION_FUNCTIONS[BACKEND_NAME] is triton_fa_tq4_kv_forward
    assert model.config._attn_implementation == BACKEND_NAME and cc.fused_mode
    stashed = [m for m in model.modules() if getattr(m, "_tq4_cache", None) is cc]
    assert len(stashed) >= cfg.num_hidden_layers and all(hasattr(m, "layer_idx") for m in stashed)
    assert cc.get_token_rows(0) is None  # nothing stored yet
    uninstall_fused_tq4_kv(model)
    assert model.config._attn_implementation == "sdpa" and not cc.fused_mode
    assert not any(hasattr(m, "_tq4_cache") for m in model.modules())
    with pytest.raises(AttributeError, match="no config"):
        install_fused_tq4_kv(torch.nn.Linear(2, 2), cc)
    # no stashed cache: the call is HuggingFace SDPA's
    attn = model.model.layers[0].self_attn
    q, k = torch.randn(1, 2, 5, 32), torch.randn(1, 2, 5, 32)
    got, _ = triton_fa_tq4_kv_forward(attn, q, k, k, None, scaling=0.2)
    want, _ = sdpa_attention_forward(attn, q, k, k, None, scaling=0.2)
    assert torch.equal(got, want)
