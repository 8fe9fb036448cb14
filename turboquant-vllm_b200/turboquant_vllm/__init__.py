"""B200-native TQ4 KV-cache compression: drop-in for the hot path of turboquant-vllm.

Public names follow the reference package (src/turboquant_vllm/__init__.py): the quantiser
and codebook holders, the HF ``CompressedDynamicCache`` and the vLLM plugin under
``turboquant_vllm.vllm``.  The arithmetic runs in hand-written sm_100a CUDA kernels behind a
C ABI (include/tq4.h); there is no Triton and no CPU fallback.
"""

from turboquant_vllm.compressors import CompressedValues, TurboQuantCompressorMSE
from turboquant_vllm.lloyd_max import LloydMaxCodebook, solve_lloyd_max
from turboquant_vllm.quantizer import TurboQuantMSE

__version__ = "0.1.0"

__all__ = [
    "CompressedDynamicCache",
    "CompressedValues",
    "LloydMaxCodebook",
    "TurboQuantCompressorMSE",
    "TurboQuantMSE",
    "solve_lloyd_max",
]


def __getattr__(name: str):
    # transformers is imported only when the HF cache wrapper is actually used
    if name == "CompressedDynamicCache":
        from turboquant_vllm.kv_cache import CompressedDynamicCache

        return CompressedDynamicCache
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
