"""Alias of the reference module path ``turboquant_vllm.triton.tq4_compress``."""
from turboquant_vllm.kernels.ops import tq4_compress

__all__ = ["tq4_compress"]
