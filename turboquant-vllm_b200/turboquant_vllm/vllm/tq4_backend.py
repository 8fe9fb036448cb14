"""TQ4 packed-KV-cache attention backend for vLLM, B200-native.

Same plugin surface as the reference backend (src/turboquant_vllm/vllm/tq4_backend.py):
``register_tq4_backend`` registers :class:`TQ4AttentionBackend` as the ``CUSTOM`` backend and
rewraps decoder ``FullAttentionSpec`` objects as :class:`TQ4FullAttentionSpec` (uint8 pages
sized for the packed format).  What differs is below the surface:

* the cache write is ONE kernel (compress K and V, scatter into the paged blocks) instead of
  two Triton launches, a row assembly and an ``index_put``
  (reference ``_compress_and_store``, tq4_backend.py:562-624);
* every step whose features the fused kernels cover — causal or not, sliding window,
  asymmetric K/V codebooks, any mix of decode and chunked-prefill rows — goes through one
  fused paged-attention call over the packed cache; nothing is decompressed to HBM
  (reference ``forward`` dispatch, tq4_backend.py:1012-1095);
* ALiBi, logit soft-capping and attention sinks fall back to decompress + FlashAttention,
  exactly like the reference's default path;
* all scratch is allocated once on the first ``forward`` (before CUDA-graph capture).
"""

from __future__ import annotations

import logging
import os
from dataclasses import dataclass
from dataclasses import fields as dc_fields
from typing import TYPE_CHECKING

import torch
from vllm.v1.attention.backends.flash_attn import (
    FlashAttentionBackend,
    FlashAttentionImpl,
    FlashAttentionMetadataBuilder,
)
from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
from vllm.v1.kv_cache_interface import FullAttentionSpec

from turboquant_vllm.kernels import ops
from turboquant_vllm.kernels.ops import tq4_compress, tq4_decompress
from turboquant_vllm.quantizer import TurboQuantMSE

if TYPE_CHECKING:
    from vllm.v1.attention.backend import AttentionCGSupport, AttentionImplBase, AttentionMetadataBuilder

logger = logging.getLogger(__name__)

TQ4_BITS = 4
TQ4_SEED = 42
TQ4_NORM_BYTES = 4  # one fp32 norm per token per head per K-or-V


# --------------------------------------------------------------------------------------
# byte math (reference: tq4_backend.py:64-124)
# --------------------------------------------------------------------------------------
def _packed_index_size(bits: int, head_dim: int) -> int:
    """Index bytes of one token/head in the HF-side format: nibble-packed at 4 bits, else one byte each."""
    return head_dim // 2 if bits == 4 else head_dim


def _tq4_bytes_per_token(head_dim: int, bits: int = TQ4_BITS) -> int:
    """Index bytes + the fp32 norm, for one token, one KV head, one of K or V."""
    return _packed_index_size(bits, head_dim) + TQ4_NORM_BYTES


def _tq4_bytes_per_token_kv(head_dim: int, k_bits: int = TQ4_BITS, v_bits: int = TQ4_BITS) -> int:
    """K + V bytes for one token and one KV head."""
    return _tq4_bytes_per_token(head_dim, k_bits) + _tq4_bytes_per_token(head_dim, v_bits)


def _padded_slot_bytes(head_dim: int) -> int:
    """Per-head slot rounded up to a power of two so TQ4 pages divide evenly against the page
    sizes of other layer types in hybrid models.  The padding bytes are never read."""
    raw = _tq4_bytes_per_token_kv(head_dim)
    return 1 << (raw - 1).bit_length()


def _parse_dense_rows_env() -> bool:
    """``TQ4_DENSE_ROWS`` as a boolean (``1/true/yes``; default off).  No counterpart in the
    reference: drops the power-of-two slot padding, see :func:`_row_bytes`."""
    return os.environ.get("TQ4_DENSE_ROWS", "").lower() in ("1", "true", "yes")


def _row_bytes(num_kv_heads: int, head_dim: int) -> int:
    """Bytes of one token row of the packed cache (all KV heads of this rank).

    Default: ``num_kv_heads`` power-of-two slots, the reference's page format
    (tq4_backend.py:92-106), needed when TQ4 pages must divide evenly against other layer types
    of a hybrid model.  With ``TQ4_DENSE_ROWS=1``: the ``H*(D+8)`` data bytes rounded up to 16.
    The data layout inside a row is the same; only the stride changes.  It matters on
    head-sharded ranks: with one or two KV heads per rank the padded row makes every 128-byte
    line of the cache travel for 136 useful bytes per 256, the dense row streams contiguously.
    """
    if _parse_dense_rows_env():
        return (num_kv_heads * _tq4_bytes_per_token_kv(head_dim) + 15) & ~15
    return num_kv_heads * _padded_slot_bytes(head_dim)


# --------------------------------------------------------------------------------------
# environment knobs (reference: tq4_backend.py:146-215)
# --------------------------------------------------------------------------------------
_VALID_BITS = frozenset({2, 3, 4, 5})
_PACKABLE_BITS = frozenset({2, 3, 4})
_TRUTHY = ("1", "true", "yes")

# The fused kernels are compiled code inside this package, so they are always importable;
# the flags are kept because callers and tests of the reference read them.
_fused_paged_kernel_available = True
_int8_prefill_kernel_available = True
_fused_paged_tq4_decode_fn = ops.fused_paged_tq4_decode
_fused_paged_tq4_int8_prefill_fn = ops.fused_paged_tq4_int8_prefill


def _parse_fused_paged_env() -> bool:
    """``TQ4_USE_FUSED_PAGED`` as a boolean (``1/true/yes``).  The fused path is the only
    fast path here, so an unset variable means *on*; ``0/false/no`` forces the
    decompress + FlashAttention fallback."""
    raw = os.environ.get("TQ4_USE_FUSED_PAGED")
    if raw is None or raw == "":
        return True
    return raw.lower() in _TRUTHY


def _parse_int8_prefill_env() -> bool:
    """``TQ4_USE_INT8_PREFILL`` as a boolean.  Accepted for compatibility: the fused prefill
    kernel of this package is used for prefill whenever the fused path is on."""
    return os.environ.get("TQ4_USE_INT8_PREFILL", "").lower() in _TRUTHY


def _parse_kv_bits_env() -> tuple[int, int]:
    """``(TQ4_K_BITS, TQ4_V_BITS)``, each an integer in {2, 3, 4, 5}; default 4/4.

    Raises:
        ValueError: on a non-integer or out-of-set value.
    """
    raw: dict[str, str] = {}
    try:
        raw["TQ4_K_BITS"] = os.environ.get("TQ4_K_BITS", str(TQ4_BITS))
        k_bits = int(raw["TQ4_K_BITS"])
        raw["TQ4_V_BITS"] = os.environ.get("TQ4_V_BITS", str(TQ4_BITS))
        v_bits = int(raw["TQ4_V_BITS"])
    except ValueError as exc:
        raise ValueError(f"invalid env var value (expected integer): {raw} — {exc}") from exc
    for name, val in (("TQ4_K_BITS", k_bits), ("TQ4_V_BITS", v_bits)):
        if val not in _VALID_BITS:
            raise ValueError(f"{name}={val} is invalid; must be one of {sorted(_VALID_BITS)}")
    return k_bits, v_bits


# --------------------------------------------------------------------------------------
# spec / builder / backend
# --------------------------------------------------------------------------------------
@dataclass(frozen=True, kw_only=True)
class TQ4FullAttentionSpec(FullAttentionSpec):
    """FullAttentionSpec whose page size is that of the packed uint8 rows."""

    @property
    def real_page_size_bytes(self) -> int:  # noqa: D102
        return self.block_size * _row_bytes(self.num_kv_heads, self.head_size)


class TQ4MetadataBuilder(FlashAttentionMetadataBuilder):
    """FlashAttention metadata, plus the CUDA-graph capability of the fused path."""

    @classmethod
    def get_cudagraph_support(cls, vllm_config: object, kv_cache_spec: object) -> AttentionCGSupport:
        """Uniform single-token decode is capturable when the fused path is on (it allocates
        nothing and never reads device data on the host); the fallback path is not."""
        from vllm.v1.attention.backend import AttentionCGSupport

        _parse_kv_bits_env()  # surface bad env values here as the reference does
        if _parse_fused_paged_env() and _fused_paged_kernel_available:
            return AttentionCGSupport.UNIFORM_SINGLE_TOKEN_DECODE
        return AttentionCGSupport.NEVER


class TQ4AttentionBackend(FlashAttentionBackend):
    """CUSTOM backend: 3-D packed cache ``(num_blocks, block_size, H_kv * padded_slot)`` uint8."""

    forward_includes_kv_cache_update = True

    @classmethod
    def supports_mm_prefix(cls) -> bool:
        return True

    @staticmethod
    def get_name() -> str:
        return "CUSTOM"

    @staticmethod
    def get_impl_cls() -> type[AttentionImplBase]:
        return TQ4AttentionImpl

    @staticmethod
    def get_builder_cls() -> type[AttentionMetadataBuilder]:
        return TQ4MetadataBuilder

    @staticmethod
    def get_kv_cache_shape(
        num_blocks: int,
        block_size: int,
        num_kv_heads: int,
        head_size: int,
        cache_dtype_str: str = "auto",
    ) -> tuple[int, ...]:
        return (num_blocks, block_size, _row_bytes(num_kv_heads, head_size))

    @staticmethod
    def get_kv_cache_stride_order(include_num_layers_dimension: bool = False) -> tuple[int, ...]:
        """The 3-D layout wants identity ordering; raising makes vLLM fall back to it."""
        raise NotImplementedError


# --------------------------------------------------------------------------------------
# attention implementation
# --------------------------------------------------------------------------------------
class TQ4AttentionImpl(FlashAttentionImpl):
    """compress -> scatter into the packed cache -> fused paged attention over the packed cache."""

    def __init__(self, *args, **kwargs) -> None:
        super().__init__(*args, **kwargs)
        k_bits, v_bits = _parse_kv_bits_env()
        for name, b in (("TQ4_K_BITS", k_bits), ("TQ4_V_BITS", v_bits)):
            if b not in _PACKABLE_BITS:
                raise ValueError(
                    f"{name}={b}: the packed vLLM cache stores one nibble per coordinate, "
                    f"so at most 4 bits are representable; use one of {sorted(_PACKABLE_BITS)}"
                )
        from vllm.config import get_current_vllm_config_or_none

        cfg = get_current_vllm_config_or_none()
        device = cfg.device_config.device if cfg is not None else torch.device("cpu")
        self._setup_tq4(
            k_bits,
            v_bits,
            device,
            max_prefill_len=cfg.scheduler_config.max_num_batched_tokens if cfg is not None else 2048,
            max_model_len=cfg.model_config.max_model_len if cfg is not None else 6144,
        )

    def _setup_tq4(self, k_bits: int, v_bits: int, device, *, max_prefill_len: int, max_model_len: int) -> None:
        """Build rotation / codebooks on ``device`` and the row byte offsets."""
        d, h = self.head_size, self.num_kv_heads
        self._k_bits, self._v_bits = k_bits, v_bits
        kq = TurboQuantMSE(d, k_bits, seed=TQ4_SEED)
        vq = kq if v_bits == k_bits else TurboQuantMSE(d, v_bits, seed=TQ4_SEED)
        rot_t = kq.rotation.T.contiguous()
        self._tq4_rotation = kq.rotation.contiguous().to(device)
        self._tq4_rot_T_even = rot_t[:, 0::2].contiguous().to(device)
        self._tq4_rot_T_odd = rot_t[:, 1::2].contiguous().to(device)
        self._k_centroids = kq.codebook.centroids.to(device)
        self._k_boundaries = kq.codebook.boundaries.to(device)
        self._v_centroids = vq.codebook.centroids.to(device)
        self._v_boundaries = vq.codebook.boundaries.to(device)
        # row layout: [K_idx | K_norm | V_idx | V_norm]; both components are nibble-packed
        self._k_idx_size = self._v_idx_size = d // 2
        self._k_idx_end = h * self._k_idx_size
        self._k_norm_end = self._k_idx_end + h * TQ4_NORM_BYTES
        self._v_idx_end = self._k_norm_end + h * self._v_idx_size
        self._total_bytes = self._v_idx_end + h * TQ4_NORM_BYTES
        self._cg_buffers_ready = False
        self._fallback_buffers_ready = False
        self._fused_paged_available = _parse_fused_paged_env() and _fused_paged_kernel_available
        self._int8_prefill_available = self._fused_paged_available and _int8_prefill_kernel_available
        self._max_prefill_len = max_prefill_len
        self._max_model_len = max_model_len
        logger.info(
            "TQ4AttentionImpl: %d KV heads, head_size=%d, k_bits=%d, v_bits=%d, "
            "%d bytes/token (%.2fx compression vs FP16)",
            h, d, k_bits, v_bits, self._total_bytes, (2 * h * d * 2) / self._total_bytes,
        )
        logger.info("Fused paged TQ4 attention: %s",
                    "enabled" if self._fused_paged_available else "disabled")

    # ----- scratch -------------------------------------------------------------------
    def _needs_fallback(self) -> bool:
        """Features the fused kernels do not implement."""
        return (
            not self._fused_paged_available
            or getattr(self, "alibi_slopes", None) is not None
            or bool(getattr(self, "logits_soft_cap", 0) or 0)
            or getattr(self, "sinks", None) is not None
        )

    # Decompress targets of the FlashAttention fallback.  The reference allocates them in
    # _init_cg_buffers whatever path is active (tq4_backend.py:503-514); with the fused kernels they
    # are dead weight (up to 2 x max_model_len x H x D elements), so here they come into being on
    # first access: code and tests that read the attributes find them with the reference's shapes,
    # a server that stays on the fused path never pays for them.
    _LAZY_FALLBACK_ATTRS = frozenset(
        {"_cg_decompress_k", "_cg_decompress_v", "_cg_prefill_k", "_cg_prefill_v", "_max_prefill_blocks"}
    )

    def __getattr__(self, name: str):
        if name in TQ4AttentionImpl._LAZY_FALLBACK_ATTRS:
            d = self.__dict__
            if d.get("_cg_buffers_ready") and "_cg_cache_shape" in d:
                self._init_fallback_buffers(None, d["_cg_compute_dtype"])
                return d[name]
        raise AttributeError(f"{type(self).__name__!r} object has no attribute {name!r}")

    def _init_cg_buffers(self, kv_cache: torch.Tensor, compute_dtype: torch.dtype) -> None:
        """One-time scratch allocation, sized from the cache and the scheduler limits."""
        num_blocks, block_size, _ = kv_cache.shape
        device = kv_cache.device
        h, d = self.num_kv_heads, self.head_size
        self._cg_cache_shape = (num_blocks, block_size, device)
        self._cg_compute_dtype = compute_dtype
        self.__dict__.setdefault("_fallback_buffers_ready", False)
        if self._fallback_buffers_ready:  # re-initialisation (e.g. another compute dtype)
            self._fallback_buffers_ready = False
            for name in TQ4AttentionImpl._LAZY_FALLBACK_ATTRS:
                self.__dict__.pop(name, None)
        max_rows = max(1, min(self._max_prefill_len, num_blocks * block_size))
        self._cg_workspace = torch.empty(
            ops.attention_workspace_bytes(max_rows, self.num_heads, h, d),
            dtype=torch.uint8, device=device,
        )
        self._cg_workspace_rows = max_rows
        # small buffers kept for the decompress + FlashAttention fallback
        self._cg_compress_packed = torch.empty(1, h, d // 2, dtype=torch.uint8, device=device)
        self._cg_compress_norms = torch.empty(1, h, 1, dtype=torch.float32, device=device)
        self._cg_q_rot = torch.empty(1, self.num_heads, d, dtype=torch.float32, device=device)
        self._cg_q_rot_cast = torch.empty(1, self.num_heads, d, dtype=compute_dtype, device=device)
        self._cg_compress_row = torch.empty(1, self._total_bytes, dtype=torch.uint8, device=device)
        self._cg_buffers_ready = True
        if self._needs_fallback():
            self._init_fallback_buffers(kv_cache, compute_dtype)
        logger.info("TQ4 scratch allocated: attention workspace %.1f MiB for %d query rows",
                    self._cg_workspace.numel() / 2**20, max_rows)

    def _init_fallback_buffers(self, kv_cache: torch.Tensor | None, compute_dtype: torch.dtype) -> None:
        """Decompress targets of the FlashAttention fallback (reference: tq4_backend.py:480-513).
        ``kv_cache=None`` sizes them from the cache seen by :meth:`_init_cg_buffers`."""
        if kv_cache is not None:
            num_blocks, block_size, device = kv_cache.shape[0], kv_cache.shape[1], kv_cache.device
        else:
            num_blocks, block_size, device = self._cg_cache_shape
        max_tokens = num_blocks * block_size
        h, d = self.num_kv_heads, self.head_size
        dec_tokens = min(self._max_model_len, max_tokens)
        self._cg_decompress_k = torch.empty(dec_tokens, h, d, dtype=compute_dtype, device=device)
        self._cg_decompress_v = torch.empty_like(self._cg_decompress_k)
        pre_tokens = min(self._max_prefill_len, max_tokens)
        self._cg_prefill_k = torch.empty(pre_tokens, h, d, dtype=compute_dtype, device=device)
        self._cg_prefill_v = torch.empty_like(self._cg_prefill_k)
        self._max_prefill_blocks = pre_tokens // block_size
        self._fallback_buffers_ready = True

    # ----- cache write -----------------------------------------------------------------
    def _compress_and_store(
        self,
        key: torch.Tensor,
        value: torch.Tensor,
        kv_cache: torch.Tensor,
        slot_mapping: torch.Tensor,
        *,
        compress_out: tuple[torch.Tensor, torch.Tensor] | None = None,
        row_out: torch.Tensor | None = None,
    ) -> None:
        """Compress ``key``/``value`` ``(N, H, D)`` and write the packed rows at ``slot_mapping``.

        One fused launch; ``compress_out`` / ``row_out`` are accepted for signature
        compatibility and unused (there is no intermediate row to assemble).
        """
        ops.tq4_write_paged(
            key, value, kv_cache, slot_mapping, self._tq4_rot_T_even, self._tq4_rot_T_odd,
            self._k_boundaries, self._v_boundaries,
        )

    # ----- decompress (fallback path and tests) ---------------------------------------------
    def _decompress_cache(
        self,
        kv_cache: torch.Tensor,
        compute_dtype: torch.dtype,
        *,
        apply_rotation: bool = True,
        out_k: torch.Tensor | None = None,
        out_v: torch.Tensor | None = None,
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """Whole cache -> ``(NB, BS, H, D)`` K and V in ``compute_dtype``.

        ``apply_rotation=False`` leaves the tensors in rotated space (the caller rotates Q
        and un-rotates the output instead).
        """
        nb, bs, _ = kv_cache.shape
        h, d = self.num_kv_heads, self.head_size
        k, v = ops.tq4_decompress_cache(
            kv_cache, h, d, self._k_centroids, self._v_centroids, compute_dtype,
            out_k=None if out_k is None else out_k[: nb * bs],
            out_v=None if out_v is None else out_v[: nb * bs],
        )
        if apply_rotation:
            k = (k.float() @ self._tq4_rotation).to(compute_dtype)
            v = (v.float() @ self._tq4_rotation).to(compute_dtype)
        return k.reshape(nb, bs, h, d), v.reshape(nb, bs, h, d)

    def _decompress_cache_paged(
        self,
        kv_cache: torch.Tensor,
        block_table: torch.Tensor,
        seq_lens: torch.Tensor,
        compute_dtype: torch.dtype,
        *,
        out_k: torch.Tensor,
        out_v: torch.Tensor,
    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Decompress only the blocks the batch references; returns a remapped block table.

        Not CUDA-graph safe (data-dependent sizes) — fallback path only.
        """
        nb, bs, _ = kv_cache.shape
        h, d = self.num_kv_heads, self.head_size
        need = (seq_lens + bs - 1) // bs
        cols = torch.arange(block_table.shape[1], device=block_table.device).unsqueeze(0)
        used = torch.unique(block_table[cols < need.unsqueeze(1)], sorted=True)
        n_used = used.numel()
        cap = out_k.shape[0] // bs
        if n_used > cap:
            logger.warning(
                "Paged decompress: %d unique blocks exceed pre-allocated capacity (%d blocks), "
                "using dynamic fallback", n_used, cap,
            )
            out_k = torch.empty(n_used * bs, h, d, dtype=compute_dtype, device=kv_cache.device)
            out_v = torch.empty_like(out_k)
        compact = kv_cache[used.long()].contiguous()
        k, v = ops.tq4_decompress_cache(
            compact, h, d, self._k_centroids, self._v_centroids, compute_dtype,
            out_k=out_k[: n_used * bs], out_v=out_v[: n_used * bs],
        )
        remap = torch.zeros(nb, dtype=block_table.dtype, device=block_table.device)
        remap[used.long()] = torch.arange(n_used, dtype=block_table.dtype, device=block_table.device)
        return k.reshape(n_used, bs, h, d), v.reshape(n_used, bs, h, d), remap[block_table.long()]

    # ----- fallback helpers (reference: tq4_backend.py:824-872) --------------------------------
    def _tq4_decode(self, query, key, value, kv_cache, attn_metadata):
        """Fallback decode: write, rotate Q, decompress referenced blocks."""
        return self._tq4_prefill(query, key, value, kv_cache, attn_metadata, decode=True)

    def _tq4_prefill(self, query, key, value, kv_cache, attn_metadata, decode: bool = False):
        """Fallback prefill: write, rotate Q, decompress referenced blocks."""
        if kv_cache is not None and key is not None and value is not None:
            self._compress_and_store(key, value, kv_cache, attn_metadata.slot_mapping)
        if not self.__dict__.get("_fallback_buffers_ready", False):
            self._init_fallback_buffers(kv_cache, query.dtype)
        q = query[: attn_metadata.num_actual_tokens]
        q_rot = (q.float() @ self._tq4_rotation.T).to(q.dtype)
        kc, vc, bt = self._decompress_cache_paged(
            kv_cache, attn_metadata.block_table, attn_metadata.seq_lens, query.dtype,
            out_k=self._cg_decompress_k if decode else self._cg_prefill_k,
            out_v=self._cg_decompress_v if decode else self._cg_prefill_v,
        )
        return q_rot, kc, vc, bt

    # ----- fused paths ---------------------------------------------------------------------
    def _sliding_window_tokens(self) -> int:
        sw = getattr(self, "sliding_window", None)
        if sw is None:
            return 0
        left = sw[0] if isinstance(sw, (tuple, list)) else sw
        return int(left) + 1 if left is not None and left >= 0 else 0

    def _fused_attention(self, query, kv_cache, attn_metadata, output, *, decode: bool, write=None):
        n = attn_metadata.num_actual_tokens
        ws = self.__dict__.get("_cg_workspace")
        if ws is not None and n > self._cg_workspace_rows:
            ws = None  # more rows than the scheduler limit announced: the shared grow-on-demand scratch
        if write is not None and not kv_cache.is_contiguous():
            self._compress_and_store(write[0], write[1], kv_cache, write[2])  # strided cache view
            write = None
        if write is not None:
            key, value, slot_mapping = write
            write = (key, value, slot_mapping, self._tq4_rot_T_even, self._tq4_rot_T_odd,
                     self._k_boundaries, self._v_boundaries)
        ops.paged_tq4_attention(
            query[:n], kv_cache, attn_metadata.block_table, attn_metadata.seq_lens,
            self._k_centroids, self._v_centroids, self._tq4_rotation, self.num_kv_heads,
            kv_cache.shape[1], self.scale,
            query_start_loc=None if decode else attn_metadata.query_start_loc,
            causal=bool(getattr(attn_metadata, "causal", True)),
            sliding_window=self._sliding_window_tokens(),
            out=output[:n], workspace=ws, write=write,
        )
        # opt-in (TQ4_CHECK_ERRORS=1): surface out-of-range slots / block ids and timed-out device
        # waits as an exception instead of silently skipped rows; never during graph capture
        ops.maybe_raise_on_device_errors(query.device, "TQ4AttentionImpl.forward")
        return output

    def _fused_decode_path(self, query, key, value, kv_cache, attn_metadata, output):
        """Uniform single-token decode in one library call: the cache write of the new tokens rides in
        the kernel that rotates the queries and plans the tiles (three launches), or all of that
        happens inside the attention kernel (two launches; the library picks by batch size)."""
        write = None
        if key is not None and value is not None:
            write = (key, value, attn_metadata.slot_mapping)
        return self._fused_attention(query, kv_cache, attn_metadata, output, decode=True, write=write)

    def _int8_prefill_path(self, query, key, value, kv_cache, attn_metadata, output):
        """Chunked prefill / mixed batches on the fused kernel (multi-sequence, prefix-aware).

        Keeps the reference's method name; there is no INT8 requantisation here.
        """
        if key is not None and value is not None:
            self._compress_and_store(key, value, kv_cache, attn_metadata.slot_mapping)
        return self._fused_attention(query, kv_cache, attn_metadata, output, decode=False)

    # ----- forward ---------------------------------------------------------------------------
    def forward(
        self,
        layer,
        query,
        key,
        value,
        kv_cache,
        attn_metadata,
        output=None,
        output_scale=None,
        output_block_scale=None,
    ):
        """query ``[T, Hq, D]``, key/value ``[T, Hkv, D]``, packed ``kv_cache`` -> ``output``."""
        assert output is not None
        if output_scale is not None or output_block_scale is not None:
            raise NotImplementedError("Fused output quantization is not supported with TQ4 backend")
        if attn_metadata is None or kv_cache is None:  # profiling run / warm-up without a cache
            output.zero_()
            return output

        from vllm.v1.attention.backend import AttentionType

        if self.attn_type in (AttentionType.ENCODER_ONLY, AttentionType.ENCODER):
            n = attn_metadata.num_actual_tokens
            return self._forward_encoder_attention(
                query[:n], key[:n], value[:n], output[:n], attn_metadata, layer
            )
        if getattr(attn_metadata, "use_cascade", False):
            raise NotImplementedError("TQ4 does not yet support cascade attention")
        if not self._cg_buffers_ready:
            self._init_cg_buffers(kv_cache, compute_dtype=query.dtype)

        n = attn_metadata.num_actual_tokens
        uniform_decode = attn_metadata.max_query_len == 1 and n <= attn_metadata.seq_lens.shape[0]
        if not self._needs_fallback():
            if uniform_decode:
                return self._fused_decode_path(query, key, value, kv_cache, attn_metadata, output)
            return self._int8_prefill_path(query, key, value, kv_cache, attn_metadata, output)
        return self._flash_fallback(layer, query, key, value, kv_cache, attn_metadata, output,
                                    decode=uniform_decode and n == 1)

    def _flash_fallback(self, layer, query, key, value, kv_cache, attn_metadata, output, *, decode):
        """Decompress the referenced blocks and run FlashAttention in rotated space
        (the reference's default path, tq4_backend.py:1040-1095)."""
        from vllm.v1.attention.backends.fa_utils import flash_attn_varlen_func

        n = attn_metadata.num_actual_tokens
        if decode:
            q_rot, kc, vc, bt = self._tq4_decode(query, key, value, kv_cache, attn_metadata)
        else:
            q_rot, kc, vc, bt = self._tq4_prefill(query, key, value, kv_cache, attn_metadata)
        shape = (attn_metadata.query_start_loc.shape[0] - 1, self.num_kv_heads)
        flash_attn_varlen_func(
            q=q_rot, k=kc, v=vc, out=output[:n],
            cu_seqlens_q=attn_metadata.query_start_loc,
            max_seqlen_q=attn_metadata.max_query_len,
            seqused_k=attn_metadata.seq_lens,
            max_seqlen_k=attn_metadata.max_seq_len,
            softmax_scale=self.scale,
            causal=attn_metadata.causal,
            alibi_slopes=self.alibi_slopes,
            window_size=list(self.sliding_window) if self.sliding_window is not None else None,
            block_table=bt,
            softcap=self.logits_soft_cap,
            scheduler_metadata=attn_metadata.scheduler_metadata,
            fa_version=self.vllm_flash_attn_version,
            q_descale=layer._q_scale.expand(shape),
            k_descale=layer._k_scale.expand(shape),
            v_descale=layer._v_scale.expand(shape),
            num_splits=attn_metadata.max_num_splits,
            s_aux=self.sinks,
        )
        o = output[:n]
        output[:n] = (o.float() @ self._tq4_rotation).to(o.dtype)
        return output


# --------------------------------------------------------------------------------------
# registration (reference: tq4_backend.py:1105-1153)
# --------------------------------------------------------------------------------------
_original_get_kv_cache_spec = None


def register_tq4_backend() -> None:
    """Register TQ4 as vLLM's ``CUSTOM`` attention backend.  Idempotent.

    Also teaches the KV-cache manager about :class:`TQ4FullAttentionSpec` (vLLM looks specs
    up by exact type) and patches ``Attention.get_kv_cache_spec`` so decoder layers report
    uint8 pages of the packed size.
    """
    global _original_get_kv_cache_spec  # noqa: PLW0603

    register_backend(
        AttentionBackendEnum.CUSTOM, "turboquant_vllm.vllm.tq4_backend.TQ4AttentionBackend"
    )
    from vllm.v1.core.single_type_kv_cache_manager import spec_manager_map

    spec_manager_map.setdefault(TQ4FullAttentionSpec, spec_manager_map[FullAttentionSpec])

    from vllm.model_executor.layers.attention.attention import Attention

    if _original_get_kv_cache_spec is None:
        _original_get_kv_cache_spec = Attention.get_kv_cache_spec

    def _tq4_get_kv_cache_spec(self, vllm_config):
        spec = _original_get_kv_cache_spec(self, vllm_config)
        if isinstance(spec, FullAttentionSpec) and not isinstance(spec, TQ4FullAttentionSpec):
            kw = {f.name: getattr(spec, f.name) for f in dc_fields(spec)}
            kw["dtype"] = torch.uint8
            return TQ4FullAttentionSpec(**kw)
        return spec

    Attention.get_kv_cache_spec = _tq4_get_kv_cache_spec
    logger.info("TQ4 attention backend registered as CUSTOM (packed cache)")


__all__ = [
    "TQ4_BITS",
    "TQ4_SEED",
    "TQ4AttentionBackend",
    "TQ4AttentionImpl",
    "TQ4FullAttentionSpec",
    "TQ4MetadataBuilder",
    "register_tq4_backend",
    "tq4_compress",
    "tq4_decompress",
]
