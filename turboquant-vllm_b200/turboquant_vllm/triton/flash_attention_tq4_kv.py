"""Fused attention over contiguous (HuggingFace-side) TQ4 K and V.

Same call as the reference's ``triton_flash_attention_tq4_kv``
(src/turboquant_vllm/triton/flash_attention_tq4_kv.py:251-355): nibble-packed K and V are
dequantised inside the attention kernel, the query is rotated on the way in and the output
un-rotated on the way out.  There is no second kernel family for the contiguous layout: the four
tensors are assembled into token rows (:class:`turboquant_vllm.token_rows.TokenRowStore`) and the
paged sm_100a kernels run over them with an identity block table.  ``CompressedDynamicCache`` in
fused mode already stores token rows, so :mod:`turboquant_vllm.triton.attention_interface` skips the
assembly and reads the cache in place.
"""

from __future__ import annotations

import torch

from turboquant_vllm.token_rows import TokenRowStore


def triton_flash_attention_tq4_kv(
    q: torch.Tensor,
    k_packed: torch.Tensor,
    k_norms: torch.Tensor,
    v_packed: torch.Tensor,
    v_norms: torch.Tensor,
    centroids: torch.Tensor,
    rotation: torch.Tensor,
    sm_scale: float | None = None,
    is_causal: bool = False,
) -> torch.Tensor:
    """``q [B, Hq, Sq, D]`` fp16/bf16 over packed K/V ``[B, Hkv, Skv, D/2]`` u8 with fp32 norms
    ``[B, Hkv, Skv]`` or ``[..., 1]`` -> ``[B, Hq, Sq, D]`` in the original (un-rotated) space.

    ``centroids [16]`` and ``rotation [D, D]`` are shared by K and V.  ``is_causal`` lets query ``i``
    see keys ``0..i`` and is ignored for a single query row, as in the reference.
    """
    b, hq, _, d = q.shape
    _, hkv, _, half_d = k_packed.shape
    assert d % 2 == 0, f"HEAD_DIM must be even, got {d}"
    assert half_d == d // 2
    assert hq % hkv == 0
    assert k_packed.dtype == torch.uint8 and v_packed.dtype == torch.uint8
    assert k_norms.dtype == torch.float32 and v_norms.dtype == torch.float32
    store = TokenRowStore.from_tensors(k_packed, k_norms, v_packed, v_norms)
    cents = centroids.to(device=q.device, dtype=torch.float32)
    out = store.attention(q, cents, cents, rotation.to(device=q.device, dtype=torch.float32),
                          sm_scale, is_causal)
    return out.transpose(1, 2)


__all__ = ["triton_flash_attention_tq4_kv"]
