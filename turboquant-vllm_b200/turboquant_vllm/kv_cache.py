"""HuggingFace ``DynamicCache`` wrapper that stores TQ-compressed K/V (GPU only).

Same public surface as the reference's ``CompressedDynamicCache``
(src/turboquant_vllm/kv_cache.py:275-1044): it replaces ``update`` / ``get_seq_length`` of the
wrapped cache, keeps uint8 centroid indices (nibble-packed at 4 bits) plus fp32 norms per layer,
hands the fused attention path the packed tensors through ``get_compressed``, and otherwise
returns incrementally dequantised K/V.  Differences under the surface:

* compress and dequantise are single launches of the sm_100a kernels (norm + rotate + bucketize
  + pack; unpack + LUT + scale), not chains of PyTorch ops;
* storage grows by capacity doubling, so appending a token does not re-copy the whole layer
  (the reference ``torch.cat``s every step);
* in fused mode a 4-bit layer is kept as token rows in the paged kernels' own format
  (:class:`turboquant_vllm.token_rows.TokenRowStore`): an update is one launch of the paged write
  kernel and the fused attention reads the rows in place; ``get_compressed`` then returns strided
  views of that buffer;
* tensors must live on a CUDA device — there is no CPU compute path.
"""

from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Any

import torch

from turboquant_vllm.compressors import CompressedValues, TurboQuantCompressorMSE
from turboquant_vllm.quantizer import nibble_pack, nibble_unpack
from turboquant_vllm.token_rows import TokenRowStore


def _packed_size(bits: int, head_dim: int) -> int:
    """Index bytes per token per head: nibble-packed at 4 bits, one byte per index otherwise."""
    return head_dim // 2 if bits == 4 else head_dim


@dataclass
class _CompressedLayer:
    """Indices (uint8, ``[B, H, S, D]`` or ``[B, H, S, D/2]`` when ``packed``) + fp32 norms ``[B, H, S, 1]``."""

    indices: torch.Tensor
    norms: torch.Tensor
    packed: bool = False


class _GrowBuffer:
    """A ``[B, H, capacity, W]`` tensor that is appended to along dim 2 with amortised O(1) copies."""

    def __init__(self) -> None:
        self.buf: torch.Tensor | None = None
        self.len = 0

    def append(self, x: torch.Tensor) -> torch.Tensor:
        n = x.shape[2]
        if self.buf is None or self.buf.shape[:2] != x.shape[:2] or self.buf.shape[3] != x.shape[3]:
            cap = max(64, 1 << (max(n, 1) - 1).bit_length())
            self.buf = torch.empty(*x.shape[:2], cap, x.shape[3], dtype=x.dtype, device=x.device)
            self.len = 0
        elif self.len + n > self.buf.shape[2]:
            cap = max(2 * self.buf.shape[2], 1 << (self.len + n - 1).bit_length())
            grown = torch.empty(*x.shape[:2], cap, x.shape[3], dtype=x.dtype, device=x.device)
            grown[:, :, : self.len] = self.buf[:, :, : self.len]
            self.buf = grown
        self.buf[:, :, self.len : self.len + n] = x
        self.len += n
        return self.view()

    def view(self) -> torch.Tensor:
        assert self.buf is not None
        return self.buf[:, :, : self.len]


class _RowsField:
    """One of the four reference tensors of a row-format layer, with the ``len`` / ``view()`` face of
    :class:`_GrowBuffer` (0 = K indices, 1 = K norms, 2 = V indices, 3 = V norms)."""

    def __init__(self, store: TokenRowStore, which: int) -> None:
        self.store, self.which = store, which

    @property
    def len(self) -> int:
        return self.store.len

    def view(self) -> torch.Tensor:
        return self.store.views()[self.which]


class CompressedDynamicCache:
    """KV cache wrapper with real memory savings (uint8 indices + fp32 norms).

    Args:
        cache: a HuggingFace ``DynamicCache``.
        head_dim: primary head dimension; even when any component uses 4 bits.
        bits: shorthand for ``k_bits = v_bits = bits``.
        k_bits, v_bits: per-component bit widths (2-4).
        seed: rotation seed.
        model_config: optional model config; when its ``layer_types`` mixes sliding and full
            attention, FULL-attention layers bypass compression (they are the only retrieval path
            for tokens beyond the window) and sliding layers are compressed.

    Raises:
        ValueError: no bit width given, or a 4-bit component with odd ``head_dim``.
    """

    def __init__(
        self,
        cache: Any,
        head_dim: int,
        bits: int | None = 3,
        *,
        k_bits: int | None = None,
        v_bits: int | None = None,
        seed: int = 42,
        model_config: Any = None,
    ) -> None:
        kb = k_bits if k_bits is not None else bits
        vb = v_bits if v_bits is not None else bits
        if kb is None or vb is None:
            raise ValueError(
                "No bit-width specified. Provide `bits` as shorthand, or `k_bits` and `v_bits` individually."
            )
        for name, b in (("k_bits", kb), ("v_bits", vb)):
            if b == 4 and head_dim % 2:
                raise ValueError(f"{name}=4 requires even head_dim for nibble packing, got {head_dim}")
        self.cache = cache
        self.head_dim = head_dim
        self.bits = kb  # kept for callers that read a single width
        self.k_bits, self.v_bits = kb, vb
        self._k_nibble_packed, self._v_nibble_packed = kb == 4, vb == 4
        self._seed = seed
        self.enabled = True
        self.fused_mode = False
        self._original_dtype: torch.dtype = torch.bfloat16
        self._key_compressors: dict[int, TurboQuantCompressorMSE] = {
            head_dim: TurboQuantCompressorMSE(head_dim, kb, seed=seed)
        }
        self._value_compressors: dict[int, TurboQuantCompressorMSE] = {
            head_dim: TurboQuantCompressorMSE(head_dim, vb, seed=seed)
        }
        # per layer: growable storage; None = layer not compressed (bypassed)
        self._k_store: list[tuple[_GrowBuffer, _GrowBuffer] | None] = []
        self._v_store: list[tuple[_GrowBuffer, _GrowBuffer] | None] = []
        self._dec_k: list[_GrowBuffer | None] = []
        self._dec_v: list[_GrowBuffer | None] = []
        # per layer: token-row storage while the layer is in fused mode (then _k_store/_v_store
        # hold _RowsField views of it)
        self._rows: list[TokenRowStore | None] = []

        if hasattr(cache.update, "__self__") and isinstance(cache.update.__self__, CompressedDynamicCache):
            warnings.warn(
                "Cache is already wrapped by TurboQuant. Call restore() on the existing wrapper first.",
                UserWarning, stacklevel=2,
            )
        layer_types = getattr(model_config, "layer_types", None)
        mixed = bool(layer_types) and any("sliding" in t for t in layer_types)
        self._full_attn_bypass: set[int] = (
            {i for i, t in enumerate(layer_types) if "full" in t} if mixed else set()
        )
        if model_config is not None and mixed and not any(
            getattr(layer, "is_sliding", False) for layer in cache.layers
        ):
            warnings.warn(
                "Cache appears to lack sliding window layer metadata. Create cache with "
                "`DynamicCache(config=model.config)` for correct Gemma support.",
                UserWarning, stacklevel=2,
            )
        self._original_update = cache.update
        self._original_get_seq_length = cache.get_seq_length
        cache.update = self._compressed_update
        cache.get_seq_length = self._compressed_get_seq_length

    # ----- compressors ------------------------------------------------------------------------
    def _get_compressors(self, dim: int):
        """Compressors for ``dim`` (created on first use: heterogeneous head dims)."""
        if dim not in self._key_compressors:
            for name, packed in (("k_bits", self._k_nibble_packed), ("v_bits", self._v_nibble_packed)):
                if packed and dim % 2:
                    raise ValueError(
                        f"{name}=4 requires even head_dim for nibble packing, got layer head_dim={dim}"
                    )
            self._key_compressors[dim] = TurboQuantCompressorMSE(dim, self.k_bits, seed=self._seed)
            self._value_compressors[dim] = TurboQuantCompressorMSE(dim, self.v_bits, seed=self._seed)
        return self._key_compressors[dim], self._value_compressors[dim]

    @property
    def key_compressor(self) -> TurboQuantCompressorMSE:
        return self._key_compressors[self.head_dim]

    @property
    def value_compressor(self) -> TurboQuantCompressorMSE:
        return self._value_compressors[self.head_dim]

    @property
    def rotation(self) -> torch.Tensor:
        """Shared rotation ``[head_dim, head_dim]`` fp32 (K and V use the same seed)."""
        return self.key_compressor.quantizer.rotation

    @property
    def centroids(self) -> torch.Tensor:
        """Key codebook ``[2^k_bits]`` fp32."""
        return self.key_compressor.quantizer.codebook.centroids

    _nibble_pack = staticmethod(nibble_pack)
    _nibble_unpack = staticmethod(nibble_unpack)

    # ----- compress / dequantise one tensor ------------------------------------------------------
    def _compress_tensor(self, compressor: TurboQuantCompressorMSE, tensor: torch.Tensor, *,
                         nibble_packed: bool) -> _CompressedLayer:
        """``[B, H, S, D]`` -> indices + fp32 norms; one fused kernel launch."""
        packed, norms = compressor.quantizer.quantize_packed(tensor)
        if nibble_packed:
            return _CompressedLayer(packed, norms, True)
        return _CompressedLayer(nibble_unpack(packed).to(torch.uint8), norms, False)

    def _dequantize_layer(self, compressor: TurboQuantCompressorMSE, layer: _CompressedLayer) -> torch.Tensor:
        """Indices + norms -> reconstructed tensor in the dtype of the last update."""
        packed = layer.indices if layer.packed else nibble_pack(layer.indices)
        return compressor.quantizer.dequantize_packed(packed, layer.norms, self._original_dtype)

    @staticmethod
    def _cat_layers(existing: _CompressedLayer, new: _CompressedLayer) -> _CompressedLayer:
        return _CompressedLayer(
            torch.cat([existing.indices, new.indices], dim=-2),
            torch.cat([existing.norms, new.norms], dim=-2),
            existing.packed,
        )

    def _ensure_layer_initialized(self, layer: Any, key_states, value_states) -> None:
        if not layer.is_initialized:
            try:
                layer.lazy_initialization(key_states, value_states)
            except TypeError:  # transformers 4.x signature
                layer.lazy_initialization(key_states)

    def _pad_to(self, layer_idx: int) -> None:
        while len(self._k_store) <= layer_idx:
            self._k_store.append(None)
            self._v_store.append(None)
            self._dec_k.append(None)
            self._dec_v.append(None)
            self._rows.append(None)

    # ----- the patched cache methods ----------------------------------------------------------------
    def _compressed_update(self, key_states, value_states, layer_idx: int, cache_kwargs=None):
        """Compress the new tokens, append, return K/V for attention (or placeholders in fused mode)."""
        if not self.enabled:
            return self._original_update(key_states, value_states, layer_idx, cache_kwargs)
        if layer_idx in self._full_attn_bypass:
            self._pad_to(layer_idx)
            return self._original_update(key_states, value_states, layer_idx, cache_kwargs)
        self._original_dtype = key_states.dtype
        if self.cache.layer_class_to_replicate is not None:
            while len(self.cache.layers) <= layer_idx:
                self.cache.layers.append(self.cache.layer_class_to_replicate())
        dim = key_states.shape[-1]
        if self.fused_mode and dim != self.head_dim:
            raise RuntimeError(
                f"Fused TQ4 mode only supports the primary head_dim={self.head_dim}, but layer "
                f"{layer_idx} has head_dim={dim}. Disable fused mode for heterogeneous architectures."
            )
        k_comp, v_comp = self._get_compressors(dim)
        self._pad_to(layer_idx)
        if self.fused_mode and self._k_nibble_packed and self._v_nibble_packed:
            self._append_rows(layer_idx, key_states, value_states, k_comp, v_comp)
            layer = self.cache.layers[layer_idx]
            self._ensure_layer_initialized(layer, key_states, value_states)
            layer.keys, layer.values = key_states, value_states  # placeholders; attention reads the rows
            return key_states, value_states
        if self._rows[layer_idx] is not None:
            self._rows_to_buffers(layer_idx, k_comp, v_comp)
        new_k = self._compress_tensor(k_comp, key_states, nibble_packed=self._k_nibble_packed)
        new_v = self._compress_tensor(v_comp, value_states, nibble_packed=self._v_nibble_packed)
        self._pad_to(layer_idx)
        if self._k_store[layer_idx] is None:
            self._k_store[layer_idx] = (_GrowBuffer(), _GrowBuffer())
            self._v_store[layer_idx] = (_GrowBuffer(), _GrowBuffer())
        ks, vs = self._k_store[layer_idx], self._v_store[layer_idx]
        ks[0].append(new_k.indices)
        ks[1].append(new_k.norms)
        vs[0].append(new_v.indices)
        vs[1].append(new_v.norms)

        layer = self.cache.layers[layer_idx]
        self._ensure_layer_initialized(layer, key_states, value_states)
        if self.fused_mode:  # the fused kernel reads get_compressed(); K/V here are placeholders
            layer.keys, layer.values = key_states, value_states
            return key_states, value_states
        if self._dec_k[layer_idx] is None:
            self._dec_k[layer_idx], self._dec_v[layer_idx] = _GrowBuffer(), _GrowBuffer()
        dk = self._dec_k[layer_idx].append(self._dequantize_layer(k_comp, new_k))
        dv = self._dec_v[layer_idx].append(self._dequantize_layer(v_comp, new_v))
        layer.keys, layer.values = dk, dv
        return dk, dv

    # ----- token-row storage (fused mode) -------------------------------------------------------------
    def _append_rows(self, layer_idx: int, key_states, value_states, k_comp, v_comp) -> None:
        """Fused-mode update: compress and store the new tokens as token rows, one kernel launch."""
        b, h, _, d = key_states.shape
        store = self._rows[layer_idx]
        if store is None or not store.matches(b, h, d, key_states.device):
            held = self._k_store[layer_idx]
            if store is None and held is not None and held[0].len and held[0].view().shape[:2] == (b, h):
                # tokens stored before fused mode was switched on: carry them over
                ks, vs = held, self._v_store[layer_idx]
                store = TokenRowStore.from_tensors(ks[0].view(), ks[1].view(), vs[0].view(), vs[1].view())
            else:
                store = TokenRowStore(b, h, d, key_states.device)
            self._rows[layer_idx] = store
            self._k_store[layer_idx] = (_RowsField(store, 0), _RowsField(store, 1))
            self._v_store[layer_idx] = (_RowsField(store, 2), _RowsField(store, 3))
            self._dec_k[layer_idx] = self._dec_v[layer_idx] = None
        store.append(key_states, value_states, k_comp.quantizer, v_comp.quantizer)

    def _rows_to_buffers(self, layer_idx: int, k_comp, v_comp) -> None:
        """Leave fused mode for one layer: four growable tensors again, plus the dequantised K/V of
        the tokens held so far (what the non-fused ``update`` returns)."""
        store = self._rows[layer_idx]
        assert store is not None
        k_idx, k_n, v_idx, v_n = (x.contiguous() for x in store.views())
        self._rows[layer_idx] = None
        for slot, idx, norm, comp, dec in ((self._k_store, k_idx, k_n, k_comp, self._dec_k),
                                           (self._v_store, v_idx, v_n, v_comp, self._dec_v)):
            pair = (_GrowBuffer(), _GrowBuffer())
            pair[0].append(idx)
            pair[1].append(norm)
            slot[layer_idx] = pair
            dec[layer_idx] = _GrowBuffer()
            dec[layer_idx].append(self._dequantize_layer(comp, _CompressedLayer(idx, norm, True)))

    def get_token_rows(self, layer_idx: int) -> TokenRowStore | None:
        """The layer's token-row storage, or ``None`` when the layer is not held in that format
        (not in fused mode, a bit width other than 4, bypassed, or never updated)."""
        return self._rows[layer_idx] if layer_idx < len(self._rows) else None

    def _compressed_get_seq_length(self, layer_idx: int = 0) -> int:
        if not self.enabled or layer_idx in self._full_attn_bypass:
            return self._original_get_seq_length(layer_idx)
        if layer_idx >= len(self._k_store):
            return 0
        entry = self._k_store[layer_idx]
        if entry is None:
            return self._original_get_seq_length(layer_idx)
        return int(entry[0].len)

    # ----- views used by callers / tests of the reference ----------------------------------------------
    @property
    def _compressed_keys(self) -> list[_CompressedLayer | None]:
        return [None if e is None else _CompressedLayer(e[0].view(), e[1].view(), self._k_nibble_packed)
                for e in self._k_store]

    @property
    def _compressed_values(self) -> list[_CompressedLayer | None]:
        return [None if e is None else _CompressedLayer(e[0].view(), e[1].view(), self._v_nibble_packed)
                for e in self._v_store]

    def get_compressed(self, layer_idx: int):
        """``(k_indices, k_norms, v_indices, v_norms)`` of a layer, no dequantisation.

        Raises:
            ValueError: the layer has no compressed data (never updated, or bypassed).
        """
        if layer_idx >= len(self._k_store):
            raise ValueError(f"Layer {layer_idx} has no compressed data (not yet updated)")
        if self._k_store[layer_idx] is None:
            raise ValueError(f"Layer {layer_idx} has no compressed data (SWA-bypassed layer)")
        ks, vs = self._k_store[layer_idx], self._v_store[layer_idx]
        return ks[0].view(), ks[1].view(), vs[0].view(), vs[1].view()

    # ----- lifecycle --------------------------------------------------------------------------------------
    def disable(self) -> None:
        self.enabled = False

    def enable(self) -> None:
        self.enabled = True

    def restore(self) -> None:
        """Put the wrapped cache's original ``update`` / ``get_seq_length`` back."""
        self.cache.update = self._original_update
        self.cache.get_seq_length = self._original_get_seq_length

    def __enter__(self) -> "CompressedDynamicCache":
        return self

    def __exit__(self, *exc: object) -> bool:
        self.restore()
        return False

    # ----- statistics (keys as in the reference, kv_cache.py:953-1044) -----------------------------------------
    def vram_bytes(self) -> int:
        """Bytes of compressed storage in use (keys + values, bypassed layers excluded)."""
        total = 0
        for store in (self._k_store, self._v_store):
            for e in store:
                if e is not None:
                    for gb in e:
                        v = gb.view()
                        total += v.numel() * v.element_size()
        return total

    def baseline_vram_bytes(self) -> int:
        """Bytes the same tokens would take as fp16 tensors."""
        total = 0
        for store, packed in ((self._k_store, self._k_nibble_packed), (self._v_store, self._v_nibble_packed)):
            for e in store:
                if e is not None:
                    b, h, s, d = e[0].view().shape
                    total += b * h * s * (2 * d if packed else d) * 2
        return total

    def compression_stats(self) -> dict[str, Any]:
        layers = [e for e in self._k_store if e is not None]
        if not layers:
            return {}
        comp, base = self.vram_bytes(), self.baseline_vram_bytes()
        b, h, s, _ = layers[0][0].view().shape
        per_token = len(layers) * h * (
            _packed_size(self.k_bits, self.head_dim) + 4 + _packed_size(self.v_bits, self.head_dim) + 4
        )
        return {
            "num_layers": len(layers), "seq_len": s, "batch_size": b, "num_heads": h,
            "head_dim": self.head_dim, "bits": self.bits, "k_bits": self.k_bits, "v_bits": self.v_bits,
            "k_nibble_packed": self._k_nibble_packed, "v_nibble_packed": self._v_nibble_packed,
            "compressed_mib": comp / 2**20, "baseline_mib": base / 2**20,
            "compression_ratio": round(base / comp, 2) if comp else 0.0,
            "savings_mib": (base - comp) / 2**20,
            "vram_estimate": {n: round(per_token * n / 2**20, 2) for n in (4096, 16384, 32768)},
        }


__all__ = ["CompressedDynamicCache", "CompressedValues"]
