"""Tensor-shaped wrappers used by the HF cache (reference: src/turboquant_vllm/compressors.py:224-285)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from turboquant_vllm.quantizer import TurboQuantMSE


@dataclass
class CompressedValues:
    """Indices (int64, ``[..., D]``) + fp32 norms (``[..., 1]``) + the dtype to restore."""

    indices: torch.Tensor
    norms: torch.Tensor
    original_dtype: torch.dtype = torch.bfloat16


# Keys use the same MSE representation in every path this package serves.
CompressedKeys = CompressedValues


class TurboQuantCompressorMSE:
    """``[batch, heads, seq, head_dim]`` compress / decompress around :class:`TurboQuantMSE`."""

    def __init__(self, head_dim: int, bits: int = 3, *, seed: int = 42) -> None:
        self.head_dim = head_dim
        self.bits = bits
        self.quantizer = TurboQuantMSE(head_dim, bits, seed=seed)

    def compress(self, values: torch.Tensor) -> CompressedValues:
        idx, norms = self.quantizer.quantize(values)
        return CompressedValues(indices=idx, norms=norms, original_dtype=values.dtype)

    def decompress(self, compressed: CompressedValues) -> torch.Tensor:
        out = self.quantizer.dequantize(compressed.indices, compressed.norms)
        return out.to(compressed.original_dtype)
