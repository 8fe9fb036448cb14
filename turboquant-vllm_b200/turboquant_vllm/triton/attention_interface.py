"""HuggingFace ``AttentionInterface`` registration of the fused TQ4 K+V attention.

Mirrors the reference's side-channel design
(src/turboquant_vllm/triton/attention_interface.py:142-267): the backend ``triton_fa_tq4_kv`` ignores
the K/V tensors the model passes and reads the packed cache stashed on each attention module as
``_tq4_cache``.  With ``CompressedDynamicCache.fused_mode`` on, a layer is stored as token rows and
the paged sm_100a attention kernels read it in place.  Without a stashed cache the call falls
through to HuggingFace's own SDPA backend (the reference falls through to its vanilla Triton kernel,
which is outside the TQ4 path).
"""

from __future__ import annotations

from typing import TYPE_CHECKING, Optional

import torch

from turboquant_vllm.triton.flash_attention_tq4_kv import triton_flash_attention_tq4_kv

if TYPE_CHECKING:
    from turboquant_vllm.kv_cache import CompressedDynamicCache

BACKEND_NAME = "triton_fa_tq4_kv"


def _causal_flag(module: torch.nn.Module, query: torch.Tensor, attention_mask, kwargs: dict) -> bool:
    """The rule of HuggingFace's SDPA backend: explicit ``is_causal`` wins, else multi-row queries
    without a mask on a causal module."""
    raw = kwargs.pop("is_causal", None)
    if raw is None:
        return bool(query.shape[2] > 1 and attention_mask is None and getattr(module, "is_causal", True))
    return bool(raw)


def triton_fa_tq4_kv_forward(
    module: torch.nn.Module,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    dropout: float = 0.0,
    scaling: Optional[float] = None,
    **kwargs: object,
) -> tuple[torch.Tensor, None]:
    """Attention of ``query [B, Hq, Sq, D]`` over the packed cache of ``module.layer_idx``.

    Returns ``(output [B, Sq, Hq, D], None)``.  ``key`` / ``value`` are placeholders in fused mode and
    are not read; ``attention_mask`` is not applied (only ``is_causal``), as in the reference.
    """
    cache: "CompressedDynamicCache | None" = getattr(module, "_tq4_cache", None)
    layer_idx: int | None = getattr(module, "layer_idx", None)
    if cache is None or layer_idx is None:
        from transformers.integrations.sdpa_attention import sdpa_attention_forward

        return sdpa_attention_forward(module, query, key, value, attention_mask, dropout, scaling, **kwargs)

    is_causal = _causal_flag(module, query, attention_mask, kwargs)
    store = cache.get_token_rows(layer_idx)
    # device-resident copies of the rotation and the codebooks (made once per device)
    rotation, _, _, k_cents, _ = cache.key_compressor.quantizer.device_primitives(query.device)
    if store is not None:
        v_cents = cache.value_compressor.quantizer.device_primitives(query.device)[3]
        out = store.attention(query, k_cents, v_cents, rotation, scaling, is_causal)
        return out, None
    k_packed, k_norms, v_packed, v_norms = cache.get_compressed(layer_idx)
    out = triton_flash_attention_tq4_kv(query, k_packed, k_norms, v_packed, v_norms, k_cents, rotation,
                                        sm_scale=scaling, is_causal=is_causal)
    return out.transpose(1, 2).contiguous(), None


def install_fused_tq4_kv(model: torch.nn.Module, cache: "CompressedDynamicCache") -> None:
    """Register the backend, select it on ``model``, stash ``cache`` on every module that has a
    ``layer_idx`` and switch the cache to fused mode (no dequantised K/V is produced any more).

    Raises:
        AttributeError: ``model`` has no ``config``.
    """
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    ALL_ATTENTION_FUNCTIONS.register(BACKEND_NAME, triton_fa_tq4_kv_forward)
    config = getattr(model, "config", None)
    if config is None:
        raise AttributeError("Model has no config attribute")
    config._attn_implementation = BACKEND_NAME
    cache.fused_mode = True
    for module in model.modules():
        if hasattr(module, "layer_idx"):
            object.__setattr__(module, "_tq4_cache", cache)


def uninstall_fused_tq4_kv(model: torch.nn.Module) -> None:
    """Undo :func:`install_fused_tq4_kv`: drop the stashed cache references, leave fused mode and
    select the ``sdpa`` backend again."""
    config = getattr(model, "config", None)
    if config is not None:
        config._attn_implementation = "sdpa"
    for module in model.modules():
        cache = getattr(module, "_tq4_cache", None)
        if cache is not None and hasattr(cache, "fused_mode"):
            cache.fused_mode = False
        if hasattr(module, "_tq4_cache"):
            delattr(module, "_tq4_cache")


__all__ = ["BACKEND_NAME", "install_fused_tq4_kv", "triton_fa_tq4_kv_forward", "uninstall_fused_tq4_kv"]
