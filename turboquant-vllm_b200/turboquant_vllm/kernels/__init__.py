"""sm_100a CUDA kernels for the TQ4 hot path (loaded through the C ABI, no Triton)."""

from turboquant_vllm.kernels.ops import (
    attention_workspace_bytes,
    combine_partials,
    fused_paged_tq4_decode,
    fused_paged_tq4_int8_prefill,
    fused_paged_tq4_prefill,
    paged_tq4_attention,
    tq4_compress,
    tq4_decompress,
    tq4_decompress_cache,
    tq4_pack_rotated,
    tq4_write_and_attention,
    tq4_write_paged,
)

__all__ = [
    "attention_workspace_bytes",
    "combine_partials",
    "fused_paged_tq4_decode",
    "fused_paged_tq4_int8_prefill",
    "fused_paged_tq4_prefill",
    "paged_tq4_attention",
    "tq4_compress",
    "tq4_decompress",
    "tq4_decompress_cache",
    "tq4_pack_rotated",
    "tq4_write_and_attention",
    "tq4_write_paged",
]
