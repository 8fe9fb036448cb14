"""CPU oracle for the TQ4 KV-cache hot path (TEST INFRASTRUCTURE — NOT A PRODUCT PATH).

This module restates, in plain fp32 torch-CPU / numpy arithmetic, the algorithm of the
reference project's pure-PyTorch path for: codebook solve, rotation generation, the TQ4
compress (norm -> normalise -> rotate -> bucketize -> nibble pack), the packed paged-cache
row layout, decompress, and fp32 attention over the packed cache (decode and chunked
prefill).  Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import it, and only as the checker or the
timed CPU baseline.  Nothing under the product package imports it.

Parity pinning: every function here is checked against golden vectors produced by importing
the reference implementation (see ``tests/golden/make_golden.py`` and
``tests/test_oracle_golden.py``).

Each function cites the reference file:line it follows (paths relative to the reference
project root).
"""

from __future__ import annotations

import math
from functools import lru_cache

import numpy as np
import torch

NORM_BYTES = 4  # one little-endian fp32 norm per (token, head, K-or-V)


# --------------------------------------------------------------------------------------
# Codebook  (src/turboquant_vllm/lloyd_max.py:80-176)
# --------------------------------------------------------------------------------------
@lru_cache(maxsize=64)
def solve_lloyd_max(d: int, bits: int, max_iter: int = 200, tol: float = 1e-10):
    """Lloyd-Max centroids/boundaries for N(0, 1/d) truncated to +-3 sigma.

    Follows src/turboquant_vllm/lloyd_max.py:129-176: uniform initialisation in
    [-3s, 3s], boundaries = midpoints, centroid = E[X | cell] by numerical quadrature
    (scipy.integrate.quad, as the reference does), stop when the largest centroid shift
    is < tol, final boundaries = midpoints of the final centroids, cast to fp32.
    """
    from scipy import integrate
    from scipy.stats import norm

    n_levels = 1 << bits
    sigma = 1.0 / math.sqrt(d)
    lo, hi = -3.0 * sigma, 3.0 * sigma

    def pdf(x: float) -> float:
        return float(norm.pdf(x, loc=0.0, scale=sigma))

    cents = [lo + (hi - lo) * (i + 0.5) / n_levels for i in range(n_levels)]
    for _ in range(max_iter):
        bounds = [(cents[i] + cents[i + 1]) / 2.0 for i in range(n_levels - 1)]
        edges = [lo] + bounds + [hi]
        new = []
        for i in range(n_levels):
            a, b = edges[i], edges[i + 1]
            if b - a < 1e-15:
                new.append((a + b) / 2.0)
                continue
            num, _ = integrate.quad(lambda x: x * pdf(x), a, b)
            den, _ = integrate.quad(pdf, a, b)
            new.append((a + b) / 2.0 if den < 1e-15 else num / den)
        shift = max(abs(new[i] - cents[i]) for i in range(n_levels))
        cents = new
        if shift < tol:
            break
    bounds = [(cents[i] + cents[i + 1]) / 2.0 for i in range(n_levels - 1)]
    return (
        torch.tensor(cents, dtype=torch.float32),
        torch.tensor(bounds, dtype=torch.float32),
    )


# --------------------------------------------------------------------------------------
# Rotation  (src/turboquant_vllm/quantizer.py:46-69)
# --------------------------------------------------------------------------------------
def rotation_matrix(dim: int, seed: int = 42) -> torch.Tensor:
    """Haar rotation: QR of a seeded CPU Gaussian, columns sign-fixed by diag(R)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    gauss = torch.randn(dim, dim, generator=gen, device="cpu", dtype=torch.float32)
    q, r = torch.linalg.qr(gauss)
    sgn = torch.sign(torch.diag(r))
    sgn[sgn == 0] = 1.0
    return q * sgn.unsqueeze(0)


# --------------------------------------------------------------------------------------
# Quantise / pack  (quantizer.py:112-151, lloyd_max.py:208-222, kv_cache.py:537-567)
# --------------------------------------------------------------------------------------
def rotate_rows(x: torch.Tensor, rotation: torch.Tensor):
    """fp32 norm, normalise by (norm + 1e-10), multiply by rotation^T.

    quantizer.py:139-146.  Returns (rotated [M, D], norms [M, 1]).
    """
    flat = x.reshape(-1, x.shape[-1]).float()
    norms = torch.norm(flat, dim=-1, keepdim=True)
    normalized = flat / (norms + 1e-10)
    return normalized @ rotation.float().T, norms


def bucketize(rotated: torch.Tensor, boundaries: torch.Tensor) -> torch.Tensor:
    """Index = number of boundaries strictly below the value (lloyd_max.py:208-222)."""
    return torch.bucketize(rotated, boundaries)


def nibble_pack(idx: torch.Tensor) -> torch.Tensor:
    """High nibble = even coordinate, low nibble = odd coordinate (kv_cache.py:537-551)."""
    u = idx.to(torch.uint8)
    return (u[..., 0::2] << 4) | u[..., 1::2]


def nibble_unpack(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of nibble_pack (kv_cache.py:553-567)."""
    hi = (packed >> 4).long()
    lo = (packed & 0x0F).long()
    return torch.stack([hi, lo], dim=-1).flatten(-2)


def compress_rows(x: torch.Tensor, rotation: torch.Tensor, boundaries: torch.Tensor):
    """x [N, H, D] -> (packed u8 [N, H, D/2], norms f32 [N, H, 1]).

    Restates triton/tq4_compress.py:248-295 (the reference's CPU path), which equals
    quantizer.py:112-151 followed by kv_cache.py:537-551.
    """
    n, h, d = x.shape
    rotated, norms = rotate_rows(x, rotation)
    idx = bucketize(rotated, boundaries).clamp(0, 15)
    packed = nibble_pack(idx)
    return packed.reshape(n, h, d // 2), norms.reshape(n, h, 1)


def pack_from_rotated(rotated: torch.Tensor, boundaries: torch.Tensor) -> torch.Tensor:
    """Bucketize + nibble-pack already-rotated rows [M, D] -> u8 [M, D/2]."""
    return nibble_pack(bucketize(rotated, boundaries).clamp(0, 15))


def decompress_rows(
    packed: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor, dtype=torch.float32
) -> torch.Tensor:
    """Unpack -> centroid gather -> * norm -> cast; stays in rotated space.

    Restates triton/tq4_decompress.py:187-218.
    """
    n, h, half = packed.shape
    idx = nibble_unpack(packed).reshape(n * h, 2 * half)
    out = centroids.float()[idx] * norms.reshape(n * h, 1).float()
    return out.reshape(n, h, 2 * half).to(dtype)


def dequantize(idx: torch.Tensor, norms: torch.Tensor, centroids, rotation) -> torch.Tensor:
    """centroids[idx] @ rotation * norm  (quantizer.py:153-191)."""
    d = idx.shape[-1]
    rec = centroids.float()[idx.reshape(-1, d).long()] @ rotation.float()
    return (rec * norms.reshape(-1, 1).float()).reshape(idx.shape)


# --------------------------------------------------------------------------------------
# Paged row layout  (vllm/tq4_backend.py:409-421, 562-624)
# --------------------------------------------------------------------------------------
def row_layout(num_kv_heads: int, head_dim: int):
    """Byte offsets of [K_idx | K_norm | V_idx | V_norm] within one token row."""
    half = head_dim // 2
    k_idx_end = num_kv_heads * half
    k_norm_end = k_idx_end + num_kv_heads * NORM_BYTES
    v_idx_end = k_norm_end + num_kv_heads * half
    total = v_idx_end + num_kv_heads * NORM_BYTES
    return k_idx_end, k_norm_end, v_idx_end, total


def padded_slot_bytes(head_dim: int) -> int:
    """next_power_of_2(2 * (D/2 + 4)) (vllm/tq4_backend.py:92-106)."""
    raw = 2 * (head_dim // 2 + NORM_BYTES)
    return 1 << (raw - 1).bit_length()


def assemble_rows(k_packed, k_norms, v_packed, v_norms) -> torch.Tensor:
    """[N,H,D/2] u8 + [N,H,1] f32 (x2) -> rows u8 [N, H*(D+8)]."""
    n, h, half = k_packed.shape
    return torch.cat(
        [
            k_packed.reshape(n, h * half),
            k_norms.reshape(n, h).contiguous().view(torch.uint8).reshape(n, h * 4),
            v_packed.reshape(n, h * half),
            v_norms.reshape(n, h).contiguous().view(torch.uint8).reshape(n, h * 4),
        ],
        dim=1,
    )


def write_paged(
    key, value, kv_cache, slot_mapping, rotation, k_boundaries, v_boundaries
) -> None:
    """Compress K and V and scatter the packed rows (vllm/tq4_backend.py:562-624).

    ``slot_mapping`` entries < 0 are skipped (padding convention of vLLM's
    reshape_and_cache kernels; the reference never sees negative slots).
    """
    n, h, d = key.shape
    kp, kn = compress_rows(key, rotation, k_boundaries)
    vp, vn = compress_rows(value, rotation, v_boundaries)
    rows = assemble_rows(kp, kn, vp, vn)
    total = rows.shape[1]
    flat = kv_cache.view(-1, kv_cache.shape[-1])
    num_actual = slot_mapping.shape[0]
    for i in range(num_actual):
        s = int(slot_mapping[i])
        if s >= 0:
            flat[s, :total] = rows[i]


def split_rows(flat_rows: torch.Tensor, num_kv_heads: int, head_dim: int):
    """Rows u8 [T, >=total] -> (k_packed, k_norms, v_packed, v_norms)  (tq4_backend.py:665-687)."""
    half = head_dim // 2
    a, b, c, total = row_layout(num_kv_heads, head_dim)
    t = flat_rows.shape[0]
    kp = flat_rows[:, :a].contiguous().reshape(t, num_kv_heads, half)
    kn = flat_rows[:, a:b].contiguous().view(torch.float32).reshape(t, num_kv_heads, 1)
    vp = flat_rows[:, b:c].contiguous().reshape(t, num_kv_heads, half)
    vn = flat_rows[:, c:total].contiguous().view(torch.float32).reshape(t, num_kv_heads, 1)
    return kp, kn, vp, vn


def gather_sequence_rows(kv_cache, block_table_row, seq_len: int) -> torch.Tensor:
    """Rows of one sequence in logical order, via its block-table row."""
    bs = kv_cache.shape[1]
    t = torch.arange(seq_len)
    phys = block_table_row.long()[t // bs]
    return kv_cache[phys, t % bs]


# --------------------------------------------------------------------------------------
# Attention over the packed cache, fp32 end to end
# (structure of tests/helpers/paged_cache.py:140-234 and tests/helpers/int8_prefill.py:13-78
#  in the reference, kept in fp32; causal alignment follows the FlashAttention call at
#  vllm/tq4_backend.py:1063-1087 — the last query row sees the whole sequence)
# --------------------------------------------------------------------------------------
def paged_attention_fp32(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens,
    query_start_loc,
    k_centroids: torch.Tensor,
    v_centroids: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    sm_scale: float | None = None,
    causal: bool = True,
    sliding_window: int | None = None,
    return_lse: bool = False,
):
    """q [T, H_q, D] -> out fp32 [T, H_q, D] in the original (un-rotated) space.

    Sequence i owns query rows query_start_loc[i]:query_start_loc[i+1]; query row j of a
    chunk of length L sits at absolute position seq_len - L + j.  With L == 1 for every
    sequence this is decode.  ``sliding_window`` = number of most recent keys visible
    (position p sees keys in (p - window, p]); None = unlimited.  A sequence of length 0
    (or a row with no visible key) yields zeros.
    """
    t_total, h_q, d = q.shape
    group = h_q // num_kv_heads
    scale = 1.0 / math.sqrt(d) if sm_scale is None else sm_scale
    rot = rotation.float()
    out = torch.zeros(t_total, h_q, d, dtype=torch.float32)
    lse = torch.full((t_total, h_q), float("-inf"), dtype=torch.float32)
    q_rot = q.float() @ rot.T
    for i, sl in enumerate([int(s) for s in seq_lens]):
        q0, q1 = int(query_start_loc[i]), int(query_start_loc[i + 1])
        ql = q1 - q0
        if ql == 0 or sl == 0:
            continue
        rows = gather_sequence_rows(kv_cache, block_table[i], sl)
        kp, kn, vp, vn = split_rows(rows, num_kv_heads, d)
        k = decompress_rows(kp, kn, k_centroids)  # [sl, H_kv, D]
        v = decompress_rows(vp, vn, v_centroids)
        k = k.permute(1, 0, 2).repeat_interleave(group, dim=0)  # [H_q, sl, D]
        v = v.permute(1, 0, 2).repeat_interleave(group, dim=0)
        qs = q_rot[q0:q1].permute(1, 0, 2)  # [H_q, ql, D]
        s = torch.bmm(qs, k.transpose(1, 2)) * scale  # [H_q, ql, sl]
        qpos = (sl - ql) + torch.arange(ql).unsqueeze(1)
        kpos = torch.arange(sl).unsqueeze(0)
        mask = torch.zeros(ql, sl, dtype=torch.bool)
        if causal:
            mask |= kpos > qpos
        if sliding_window is not None:
            mask |= kpos <= qpos - sliding_window
        s = s.masked_fill(mask.unsqueeze(0), float("-inf"))
        m = s.amax(dim=-1, keepdim=True)
        m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        p = torch.exp(s - m_safe)
        l = p.sum(dim=-1, keepdim=True)
        o = torch.bmm(p, v) / torch.where(l == 0, torch.ones_like(l), l)
        out[q0:q1] = (o @ rot).permute(1, 0, 2)
        lse[q0:q1] = (m_safe + torch.log(l)).squeeze(-1).permute(1, 0)
    return (out, lse) if return_lse else out


def paged_decode_fp32(
    q, kv_cache, block_table, seq_lens, k_centroids, v_centroids, rotation, num_kv_heads,
    sm_scale=None, sliding_window=None,
):
    """One query token per sequence (restates the math of
    triton/fused_paged_tq4_attention.py:255-370 without its 16-bit roundings)."""
    qsl = torch.arange(q.shape[0] + 1)
    return paged_attention_fp32(
        q, kv_cache, block_table, seq_lens, qsl, k_centroids, v_centroids, rotation,
        num_kv_heads, sm_scale, True, sliding_window,
    )


def sdpa_uncompressed_fp32(q, k, v, sm_scale=None):
    """fp32 attention on uncompressed K/V: q [H_q, D], k/v [T, H_kv, D] -> [H_q, D]."""
    h_q, d = q.shape
    group = h_q // k.shape[1]
    scale = 1.0 / math.sqrt(d) if sm_scale is None else sm_scale
    kk = k.float().permute(1, 0, 2).repeat_interleave(group, dim=0)
    vv = v.float().permute(1, 0, 2).repeat_interleave(group, dim=0)
    s = torch.einsum("hd,htd->ht", q.float(), kk) * scale
    return torch.einsum("ht,htd->hd", torch.softmax(s, dim=-1), vv)


# --------------------------------------------------------------------------------------
# Split-KV combine (log-sum-exp merge of per-shard partials; the reference has no
# counterpart — this states the standard identity used by the multi-GPU path)
# --------------------------------------------------------------------------------------
def lse_combine(partials_o: torch.Tensor, partials_lse: torch.Tensor) -> torch.Tensor:
    """partials_o [W, T, H, D] (each normalised), partials_lse [W, T, H] -> [T, H, D]."""
    m = partials_lse.amax(dim=0, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(partials_lse - m)
    den = w.sum(dim=0)
    num = (partials_o * w.unsqueeze(-1)).sum(dim=0)
    return num / torch.where(den == 0, torch.ones_like(den), den).unsqueeze(-1)


# --------------------------------------------------------------------------------------
# Synthetic inputs shared by tests and the benchmark
# --------------------------------------------------------------------------------------
OUTLIER_CHANNELS = (3, 17, 64, 101)


def synthetic_kv(n_tokens: int, num_kv_heads: int, head_dim: int, seed: int, dtype=torch.float32):
    """K, V ~ N(0,1) with four fixed channels scaled x8 (channels folded modulo head_dim)."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(n_tokens, num_kv_heads, head_dim, generator=g)
    v = torch.randn(n_tokens, num_kv_heads, head_dim, generator=g)
    for ch in OUTLIER_CHANNELS:
        k[..., ch % head_dim] *= 8.0
        v[..., ch % head_dim] *= 8.0
    return k.to(dtype), v.to(dtype)


def np_sha(t: torch.Tensor) -> str:
    """sha256 of a tensor's bytes (for compact golden checks)."""
    import hashlib

    return hashlib.sha256(np.ascontiguousarray(t.detach().cpu().numpy()).tobytes()).hexdigest()
