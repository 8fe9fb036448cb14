"""CPU-only checks: the C-ABI library loads and exports every symbol of include/tq4.h, host-side
byte math / env parsing / registration match the reference's behaviour, product code refuses CPU
tensors instead of falling back."""

from __future__ import annotations

import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(cuda_lib):
    header = open(os.path.join(ROOT, "include", "tq4.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(tq4_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 13
    from turboquant_vllm import _native

    assert declared == set(_native.exported_symbols())
    for name in declared:
        assert hasattr(cuda_lib, name), name
    assert cuda_lib.tq4_version().decode().startswith("tq4-sm100a")
    assert cuda_lib.tq4_status_string(0).decode() == "ok"
    assert cuda_lib.tq4_attention_workspace_bytes(64, 32, 8, 128) > 0
    assert cuda_lib.tq4_attention_workspace_bytes(64, 32, 5, 128) == 0  # 32 % 5 != 0


def test_cpu_tensors_are_rejected(cuda_lib):
    from turboquant_vllm.kernels import ops
    from turboquant_vllm.quantizer import TurboQuantMSE

    q = TurboQuantMSE(64, 4)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        q.quantize(torch.randn(2, 64))
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.tq4_decompress(torch.zeros(1, 1, 32, dtype=torch.uint8), torch.ones(1, 1, 1),
                           q.codebook.centroids)


def test_missing_library_fails_loudly(monkeypatch):
    from turboquant_vllm import _native

    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "_LIB_PATH", "/nonexistent/libtq4.so")
    with pytest.raises(RuntimeError, match="no CPU or Triton fallback"):
        _native.lib()


@pytest.mark.parametrize("d", [64, 96, 128, 256])
@pytest.mark.parametrize("bits", [2, 3, 4, 5])
def test_product_codebook_bit_identical_to_reference(golden, d, bits):
    from turboquant_vllm.lloyd_max import solve_lloyd_max

    g = golden("codebooks.npz")
    c, b = solve_lloyd_max(d, bits)
    assert np.array_equal(c.numpy(), g[f"c_{d}_{bits}"])
    assert np.array_equal(b.numpy(), g[f"b_{d}_{bits}"])
    assert c.dtype == torch.float32 and b.shape == (2**bits - 1,)


def test_product_rotation_matches_reference(golden):
    from turboquant_vllm.quantizer import TurboQuantMSE, _generate_rotation_matrix

    g = golden("rotations.npz")
    assert np.allclose(_generate_rotation_matrix(64, 42).numpy(), g["full_64_42"], atol=1e-6)
    q = TurboQuantMSE(128, 4, seed=7)
    assert np.allclose(q.rotation[0].numpy(), g["row0_128_7"], atol=1e-6)
    assert torch.allclose(q.rotation @ q.rotation.T, torch.eye(128), atol=1e-5)
    with pytest.raises(ValueError, match="does not match"):
        q.quantize_packed(torch.zeros(1, 64))


def test_codebook_quantize_tie_rule():
    from turboquant_vllm.lloyd_max import LloydMaxCodebook, solve_lloyd_max

    c, b = solve_lloyd_max(128, 4)
    cb = LloydMaxCodebook(c, b, 4, 128)
    assert cb.quantize(torch.zeros(3)).tolist() == [7, 7, 7]  # boundary 0.0 is not below 0.0
    assert cb.quantize(torch.tensor([1.0, -1.0])).tolist() == [15, 0]
    assert torch.equal(cb.dequantize(torch.tensor([0, 15])), c[[0, 15]])


# ---- vLLM plugin surface ---------------------------------------------------------------------
vllm = pytest.importorskip("vllm")


@pytest.fixture(scope="module")
def backend():
    from turboquant_vllm.vllm import tq4_backend

    return tq4_backend


def test_byte_math_known_answers(backend, golden):
    g = golden("sizes.npz")
    assert backend._tq4_bytes_per_token(128) == int(g["bytes_per_token_128_4"]) == 68
    assert backend._tq4_bytes_per_token(64) == 36
    assert backend._tq4_bytes_per_token(128, 3) == int(g["bytes_per_token_128_3"]) == 132
    assert backend._tq4_bytes_per_token_kv(128) == 136
    assert backend._tq4_bytes_per_token_kv(64) == 72
    for d in (64, 96, 128, 256):
        assert backend._padded_slot_bytes(d) == int(g[f"padded_slot_{d}"])
    shape = backend.TQ4AttentionBackend.get_kv_cache_shape(100, 16, 8, 128)
    assert shape == tuple(g["cache_shape_100_16_8_128"]) == (100, 16, 2048)
    ratio = (2 * 8 * 128 * 2) / (8 * 136)
    assert round(ratio, 2) == 3.76


def test_backend_class_contract(backend):
    from vllm.v1.attention.backends.flash_attn import (
        FlashAttentionBackend, FlashAttentionImpl, FlashAttentionMetadataBuilder)
    from vllm.v1.kv_cache_interface import FullAttentionSpec

    B = backend.TQ4AttentionBackend
    assert issubclass(B, FlashAttentionBackend)
    assert issubclass(backend.TQ4AttentionImpl, FlashAttentionImpl)
    assert issubclass(backend.TQ4MetadataBuilder, FlashAttentionMetadataBuilder)
    assert issubclass(backend.TQ4FullAttentionSpec, FullAttentionSpec)
    assert B.get_name() == "CUSTOM"
    assert B.get_impl_cls() is backend.TQ4AttentionImpl
    assert B.get_builder_cls() is backend.TQ4MetadataBuilder
    assert B.forward_includes_kv_cache_update is True
    assert B.supports_mm_prefix() is True
    with pytest.raises(NotImplementedError):
        B.get_kv_cache_stride_order()
    spec = backend.TQ4FullAttentionSpec(block_size=16, num_kv_heads=8, head_size=128, dtype=torch.uint8)
    assert spec.real_page_size_bytes == 16 * 8 * 256 == 32768


def test_dense_rows_flag(backend, monkeypatch):
    """TQ4_DENSE_ROWS drops the power-of-two slot padding: same row layout, 16-byte aligned stride."""
    monkeypatch.delenv("TQ4_DENSE_ROWS", raising=False)
    assert backend._row_bytes(8, 128) == 8 * 256 and backend._row_bytes(1, 128) == 256
    monkeypatch.setenv("TQ4_DENSE_ROWS", "1")
    assert backend._row_bytes(8, 128) == 1088 and backend._row_bytes(2, 128) == 272
    assert backend._row_bytes(1, 128) == 144 and backend._row_bytes(1, 64) == 80
    assert backend._row_bytes(32, 96) == 32 * 104
    assert backend.TQ4AttentionBackend.get_kv_cache_shape(100, 16, 1, 128) == (100, 16, 144)
    spec = backend.TQ4FullAttentionSpec(block_size=16, num_kv_heads=1, head_size=128, dtype=torch.uint8)
    assert spec.real_page_size_bytes == 16 * 144
    monkeypatch.setenv("TQ4_DENSE_ROWS", "0")
    assert backend._row_bytes(1, 128) == 256


def test_env_parsing(backend, monkeypatch):
    for k in ("TQ4_K_BITS", "TQ4_V_BITS", "TQ4_USE_FUSED_PAGED", "TQ4_USE_INT8_PREFILL"):
        monkeypatch.delenv(k, raising=False)
    assert backend._parse_kv_bits_env() == (4, 4)
    monkeypatch.setenv("TQ4_K_BITS", "4")
    monkeypatch.setenv("TQ4_V_BITS", "3")
    assert backend._parse_kv_bits_env() == (4, 3)
    monkeypatch.setenv("TQ4_V_BITS", "7")
    with pytest.raises(ValueError, match="TQ4_V_BITS=7"):
        backend._parse_kv_bits_env()
    monkeypatch.setenv("TQ4_V_BITS", "abc")
    with pytest.raises(ValueError, match="expected integer"):
        backend._parse_kv_bits_env()
    assert backend._parse_fused_paged_env() is True  # unset = on (the fused path is the product)
    for val, want in (("1", True), ("TRUE", True), ("yes", True), ("0", False), ("no", False)):
        monkeypatch.setenv("TQ4_USE_FUSED_PAGED", val)
        assert backend._parse_fused_paged_env() is want
    assert backend._parse_int8_prefill_env() is False
    monkeypatch.setenv("TQ4_USE_INT8_PREFILL", "true")
    assert backend._parse_int8_prefill_env() is True


def test_registration_is_idempotent(backend):
    from vllm.model_executor.layers.attention.attention import Attention
    from vllm.v1.attention.backends.registry import AttentionBackendEnum
    from vllm.v1.core.single_type_kv_cache_manager import spec_manager_map
    from vllm.v1.kv_cache_interface import FullAttentionSpec

    original = Attention.get_kv_cache_spec
    try:
        backend.register_tq4_backend()
        first = Attention.get_kv_cache_spec
        backend.register_tq4_backend()
        assert backend.TQ4FullAttentionSpec in spec_manager_map
        assert spec_manager_map[backend.TQ4FullAttentionSpec] is spec_manager_map[FullAttentionSpec]
        assert "TQ4AttentionBackend" in AttentionBackendEnum.CUSTOM.get_path()
        assert backend._original_get_kv_cache_spec is original or backend._original_get_kv_cache_spec is not first
    finally:
        Attention.get_kv_cache_spec = backend._original_get_kv_cache_spec or original


def _bare_impl(backend, **over):
    impl = object.__new__(backend.TQ4AttentionImpl)
    impl.head_size, impl.num_kv_heads, impl.num_heads = 128, 8, 32
    impl.scale = 128**-0.5
    impl.alibi_slopes = impl.sinks = None
    impl.logits_soft_cap = 0
    impl.sliding_window = (-1, -1)
    impl._setup_tq4(over.get("k_bits", 4), over.get("v_bits", 4), torch.device("cpu"),
                    max_prefill_len=2048, max_model_len=6144)
    return impl


def test_impl_layout_and_dispatch_flags(backend, monkeypatch):
    monkeypatch.delenv("TQ4_USE_FUSED_PAGED", raising=False)
    impl = _bare_impl(backend, v_bits=3)
    assert (impl._k_idx_end, impl._k_norm_end, impl._v_idx_end, impl._total_bytes) == (512, 544, 1056, 1088)
    assert impl._tq4_rotation.shape == (128, 128)
    assert impl._tq4_rot_T_even.shape == impl._tq4_rot_T_odd.shape == (128, 64)
    assert torch.equal(impl._tq4_rot_T_even, impl._tq4_rotation.T[:, 0::2])
    assert impl._k_centroids.numel() == 16 and impl._v_centroids.numel() == 8
    assert impl._k_boundaries.numel() == 15 and impl._v_boundaries.numel() == 7
    assert impl._fused_paged_available and not impl._needs_fallback()  # asymmetric K/V stays fused
    assert impl._sliding_window_tokens() == 0
    impl.sliding_window = (4095, 0)
    assert impl._sliding_window_tokens() == 4096
    impl.logits_soft_cap = 30.0
    assert impl._needs_fallback()


def test_forward_guards(backend):
    impl = _bare_impl(backend)
    out = torch.ones(2, 32, 128)
    assert impl.forward(None, None, None, None, None, None, output=out) is out and not out.any()
    out.fill_(1)
    assert not impl.forward(None, None, None, None, torch.zeros(1), None, output=out).any()
    with pytest.raises(NotImplementedError, match="output quantization"):
        impl.forward(None, None, None, None, None, None, output=out, output_scale=torch.ones(1))


def test_cg_buffers_on_cpu_cache_lazy_and_eager(backend):
    """`_init_cg_buffers` is pure allocation, so its shapes can be checked without a GPU: the
    reference-named decompress targets exist after it, eagerly when the FlashAttention fallback is
    reachable and on first access otherwise (reference: vllm/tq4_backend.py:503-514)."""
    cache = torch.zeros(500, 16, 8 * 256, dtype=torch.uint8)
    for fused in (True, False):
        impl = _bare_impl(backend)
        impl._fused_paged_available = fused
        with pytest.raises(AttributeError):
            impl._cg_decompress_k  # noqa: B018  (nothing before _init_cg_buffers)
        impl._init_cg_buffers(cache, compute_dtype=torch.bfloat16)
        assert impl._cg_buffers_ready
        assert ("_cg_decompress_k" in impl.__dict__) is (not fused)
        assert impl._cg_decompress_k.shape == (6144, 8, 128) and impl._cg_decompress_k.dtype == torch.bfloat16
        assert impl._cg_decompress_v.shape == (6144, 8, 128)
        assert impl._cg_prefill_k.shape == impl._cg_prefill_v.shape == (2048, 8, 128)
        assert impl._max_prefill_blocks == 128
        assert impl._cg_compress_row.shape == (1, 1088)
        assert impl._cg_q_rot.shape == (1, 32, 128) and impl._cg_q_rot_cast.dtype == torch.bfloat16
    with pytest.raises(AttributeError):
        impl._not_an_attribute  # noqa: B018


def test_device_error_flag_is_decoded_and_raised():
    """The host layers turn a set device error flag into an exception (fed a fake flag value here)."""
    from turboquant_vllm import _native as nv
    from turboquant_vllm.kernels import ops

    assert nv.describe_device_errors(0) == "no error"
    assert "TQ4_DEV_BAD_SLOT" in nv.describe_device_errors(nv.DEV_BAD_SLOT)
    text = nv.describe_device_errors(nv.DEV_BAD_BLOCK | nv.DEV_TIMEOUT | 64)
    assert "TQ4_DEV_BAD_BLOCK" in text and "TQ4_DEV_TIMEOUT" in text and "0x40" in text
    ops.raise_on_device_errors(torch.device("cpu"), "nowhere", flag=0)  # clean flag: no raise
    with pytest.raises(RuntimeError, match=r"forward: TQ4 kernel reported .*TQ4_DEV_TIMEOUT.*flag 0x4"):
        ops.raise_on_device_errors(torch.device("cpu"), "forward", flag=nv.DEV_TIMEOUT)


def test_error_check_switch(monkeypatch):
    from turboquant_vllm.kernels import ops

    monkeypatch.delenv("TQ4_CHECK_ERRORS", raising=False)
    assert ops.error_checks_enabled() is False
    for val, want in (("1", True), ("true", True), ("0", False), ("", False)):
        monkeypatch.setenv("TQ4_CHECK_ERRORS", val)
        assert ops.error_checks_enabled() is want
