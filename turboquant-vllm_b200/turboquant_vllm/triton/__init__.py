"""Import-path compatibility with the reference's ``turboquant_vllm.triton`` package.

The reference implements its kernels in Triton under this module path
(src/turboquant_vllm/triton/__init__.py:50-86).  Here the same names resolve to the
hand-written sm_100a CUDA kernels; nothing in this package imports Triton.
"""

from turboquant_vllm.triton.flash_attention_tq4_kv import triton_flash_attention_tq4_kv
from turboquant_vllm.kernels.ops import (
    fused_paged_tq4_decode,
    fused_paged_tq4_int8_prefill,
    fused_paged_tq4_prefill,
    tq4_compress,
    tq4_decompress,
)

__all__ = [
    "fused_paged_tq4_decode",
    "fused_paged_tq4_int8_prefill",
    "fused_paged_tq4_prefill",
    "tq4_compress",
    "tq4_decompress",
    "triton_flash_attention_tq4_kv",
]
