"""Lloyd-Max scalar codebooks for the coordinates of a randomly rotated unit vector.

Host-side, init-time only.  Mirrors the interface of the reference's
``src/turboquant_vllm/lloyd_max.py`` (``solve_lloyd_max``, ``LloydMaxCodebook``) and produces
the same fp32 centroids / boundaries, but evaluates the Gaussian cell means in closed form
(``E[X | a<X<b] = s * (phi(a/s) - phi(b/s)) / (Phi(b/s) - Phi(a/s))``) instead of by
numerical quadrature, so a solve takes microseconds rather than seconds.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from functools import lru_cache

import torch

_INV_SQRT_2PI = 1.0 / math.sqrt(2.0 * math.pi)


def _phi(z: float) -> float:
    return _INV_SQRT_2PI * math.exp(-0.5 * z * z)


def _cap_phi(z: float) -> float:
    return 0.5 * (1.0 + math.erf(z / math.sqrt(2.0)))


def _cell_mean_gaussian(a: float, b: float, sigma: float) -> float:
    """Mean of N(0, sigma^2) restricted to [a, b]."""
    za, zb = a / sigma, b / sigma
    mass = _cap_phi(zb) - _cap_phi(za)
    if mass < 1e-15 * 1.0:
        return 0.5 * (a + b)
    return sigma * (_phi(za) - _phi(zb)) / mass


def _cell_mean_beta(a: float, b: float, d: int) -> float:
    """Mean of the exact coordinate law of a uniform point on S^{d-1} restricted to [a, b].

    Density on [-1, 1]: Beta((d-1)/2, (d-1)/2) mapped affinely
    (reference: src/turboquant_vllm/lloyd_max.py:38-60).  Quadrature via scipy, used only
    when ``use_exact=True``.
    """
    from scipy import integrate
    from scipy.stats import beta as beta_dist

    alpha = (d - 1) / 2.0

    def pdf(x: float) -> float:
        return float(beta_dist.pdf((x + 1.0) / 2.0, alpha, alpha) / 2.0)

    num, _ = integrate.quad(lambda x: x * pdf(x), a, b)
    den, _ = integrate.quad(pdf, a, b)
    return 0.5 * (a + b) if den < 1e-15 else num / den


@lru_cache(maxsize=64)
def _solve(d: int, bits: int, use_exact: bool, max_iter: int, tol: float):
    levels = 1 << bits
    sigma = 1.0 / math.sqrt(d)
    lo, hi = -3.0 * sigma, 3.0 * sigma
    width = hi - lo
    cents = [lo + width * (i + 0.5) / levels for i in range(levels)]
    for _ in range(max_iter):
        edges = [lo] + [(cents[i] + cents[i + 1]) / 2.0 for i in range(levels - 1)] + [hi]
        nxt = []
        for i in range(levels):
            a, b = edges[i], edges[i + 1]
            if b - a < 1e-15:
                nxt.append((a + b) / 2.0)
            elif use_exact:
                nxt.append(_cell_mean_beta(a, b, d))
            else:
                nxt.append(_cell_mean_gaussian(a, b, sigma))
        # The law is symmetric about 0: mirror the upper half so that the codebook is exactly
        # antisymmetric and the middle boundary is exactly 0.0 (an all-zero vector rotates to
        # exact zeros, whose bucket is decided by that boundary).
        for i in range(levels // 2):
            nxt[i] = -nxt[levels - 1 - i]
        moved = max(abs(x - y) for x, y in zip(nxt, cents))
        cents = nxt
        if moved < tol:
            break
    bounds = [(cents[i] + cents[i + 1]) / 2.0 for i in range(levels - 1)]
    return (
        torch.tensor(cents, dtype=torch.float32),
        torch.tensor(bounds, dtype=torch.float32),
    )


def solve_lloyd_max(
    d: int,
    bits: int,
    *,
    use_exact: bool = False,
    max_iter: int = 200,
    tol: float = 1e-10,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Centroids ``[2^bits]`` and boundaries ``[2^bits - 1]`` (fp32, CPU) for dimension ``d``.

    Same contract as the reference's ``solve_lloyd_max``
    (src/turboquant_vllm/lloyd_max.py:80-107): N(0, 1/d) truncated to +-3 sigma unless
    ``use_exact``; uniform start; stop when the largest centroid move is below ``tol``.
    Results are cached per argument tuple.
    """
    return _solve(d, bits, use_exact, max_iter, tol)


@dataclass
class LloydMaxCodebook:
    """Centroids + boundaries with the reference's quantize/dequantize methods
    (src/turboquant_vllm/lloyd_max.py:179-234).  ``quantize`` counts boundaries strictly
    below each value (``torch.bucketize`` semantics); these two methods are plain torch ops
    for host-side/unit use — the serving path uses the fused CUDA kernels instead."""

    centroids: torch.Tensor
    boundaries: torch.Tensor
    bits: int
    dim: int

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        return torch.bucketize(x, self.boundaries.to(x.device))

    def dequantize(self, indices: torch.Tensor) -> torch.Tensor:
        return self.centroids.to(indices.device)[indices]
