"""Alias of the reference module path ``turboquant_vllm.triton.tq4_decompress``."""
from turboquant_vllm.kernels.ops import tq4_decompress

__all__ = ["tq4_decompress"]
