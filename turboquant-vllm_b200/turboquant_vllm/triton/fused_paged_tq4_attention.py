"""Alias of the reference module path ``turboquant_vllm.triton.fused_paged_tq4_attention``."""
from turboquant_vllm.kernels.ops import fused_paged_tq4_decode

__all__ = ["fused_paged_tq4_decode"]
