"""Rotation + Lloyd-Max quantiser (host-side holder of the TQ4 primitives).

Mirrors ``TurboQuantMSE`` and ``_generate_rotation_matrix`` of the reference
(src/turboquant_vllm/quantizer.py:46-191).  Construction is CPU-side and deterministic from
``(dim, bits, seed)``; ``quantize`` / ``dequantize`` on CUDA tensors run the fused sm_100a
kernels (norm + normalise + rotate + bucketize in one launch).  CPU tensors are rejected:
this package has no CPU compute path.
"""

from __future__ import annotations

import torch

from turboquant_vllm.lloyd_max import LloydMaxCodebook, solve_lloyd_max


def _generate_rotation_matrix(dim: int, seed: int = 42) -> torch.Tensor:
    """Haar-distributed orthogonal ``[dim, dim]`` fp32 matrix on CPU.

    QR of a seeded CPU Gaussian; each column is multiplied by the sign of the matching
    diagonal entry of R so the distribution is uniform over O(d).  Uses the same torch CPU
    generator + LAPACK calls as the reference (src/turboquant_vllm/quantizer.py:46-69), so the
    matrix is bit-identical for a given torch build.
    """
    rng = torch.Generator(device="cpu")
    rng.manual_seed(seed)
    g = torch.randn(dim, dim, generator=rng, device="cpu", dtype=torch.float32)
    q, r = torch.linalg.qr(g)
    signs = torch.sign(torch.diagonal(r))
    signs = torch.where(signs == 0, torch.ones_like(signs), signs)
    return q * signs.unsqueeze(0)


def nibble_unpack(packed: torch.Tensor) -> torch.Tensor:
    """u8 ``[..., D/2]`` -> int64 ``[..., D]`` (high nibble first)."""
    hi = (packed >> 4).long()
    lo = (packed & 0x0F).long()
    return torch.stack([hi, lo], dim=-1).flatten(-2)


def nibble_pack(indices: torch.Tensor) -> torch.Tensor:
    """uint8 ``[..., D]`` with values < 16 -> u8 ``[..., D/2]``."""
    u = indices.to(torch.uint8)
    return (u[..., 0::2] << 4) | u[..., 1::2]


class TurboQuantMSE:
    """Rotation + per-coordinate Lloyd-Max quantiser.

    Attributes:
        dim, bits: vector dimension and bits per coordinate.
        codebook: :class:`LloydMaxCodebook` (fp32 CPU tensors).
        rotation: orthogonal ``[dim, dim]`` fp32 CPU tensor (``Pi``).
    """

    def __init__(self, dim: int, bits: int, *, seed: int = 42) -> None:
        self.dim = dim
        self.bits = bits
        cents, bounds = solve_lloyd_max(dim, bits)
        self.codebook = LloydMaxCodebook(centroids=cents, boundaries=bounds, bits=bits, dim=dim)
        self.rotation = _generate_rotation_matrix(dim, seed=seed)
        self._dev: dict[torch.device, tuple[torch.Tensor, ...]] = {}

    def device_primitives(self, device: torch.device):
        """(rotation, rot_T_even, rot_T_odd, centroids, boundaries) resident on ``device``."""
        device = torch.device(device)
        prim = self._dev.get(device)
        if prim is None:
            rot_t = self.rotation.T.contiguous()
            prim = (
                self.rotation.to(device).contiguous(),
                rot_t[:, 0::2].contiguous().to(device),
                rot_t[:, 1::2].contiguous().to(device),
                self.codebook.centroids.to(device),
                self.codebook.boundaries.to(device),
            )
            self._dev[device] = prim
        return prim

    def quantize_packed(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """``[..., dim]`` -> (nibble-packed u8 ``[..., dim/2]``, norms f32 ``[..., 1]``)."""
        from turboquant_vllm.kernels.ops import tq4_compress

        if x.shape[-1] != self.dim:
            raise ValueError(
                f"Input last dimension {x.shape[-1]} does not match quantizer dim {self.dim}. "
                "Ensure the compressor's head_dim matches the model's actual head dimension."
            )
        if self.bits > 4:
            raise NotImplementedError("nibble-packed storage holds at most 4 bits per coordinate")
        _, even, odd, _, bounds = self.device_primitives(x.device)
        lead = x.shape[:-1]
        flat = x.reshape(-1, 1, self.dim)
        packed, norms = tq4_compress(flat, even, odd, bounds)
        return packed.reshape(*lead, self.dim // 2), norms.reshape(*lead, 1)

    def quantize(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """``[..., dim]`` -> (indices int64 ``[..., dim]``, norms f32 ``[..., 1]``)."""
        packed, norms = self.quantize_packed(x)
        return nibble_unpack(packed), norms

    def dequantize_packed(self, packed: torch.Tensor, norms: torch.Tensor,
                          dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """Nibble-packed indices + norms -> reconstructed ``[..., dim]`` in original space."""
        from turboquant_vllm.kernels.ops import tq4_decompress

        rot, _, _, cents, _ = self.device_primitives(packed.device)
        lead = packed.shape[:-1]
        rows = tq4_decompress(
            packed.reshape(-1, 1, self.dim // 2), norms.reshape(-1, 1, 1), cents, torch.float32
        )
        return (rows.reshape(-1, self.dim) @ rot).reshape(*lead, self.dim).to(dtype)

    def dequantize(self, indices: torch.Tensor, norms: torch.Tensor) -> torch.Tensor:
        """``centroids[indices] @ Pi * norm`` (fp32)."""
        if indices.shape[-1] != self.dim:
            raise ValueError(
                f"Indices last dimension {indices.shape[-1]} does not match quantizer dim "
                f"{self.dim}. Check that the same quantizer instance is used for quantize and "
                "dequantize."
            )
        return self.dequantize_packed(nibble_pack(indices), norms)
