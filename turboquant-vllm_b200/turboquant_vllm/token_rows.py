"""Contiguous (HuggingFace-side) TQ4 storage in the paged kernels' own row format.

The reference keeps a layer's compressed K/V as four tensors ``[B, H, S, D/2]`` u8 /
``[B, H, S, 1]`` f32 and reads them with a second, contiguous-layout attention kernel
(src/turboquant_vllm/triton/flash_attention_tq4_kv.py:76-355).  Here a layer is ONE buffer of
token rows ``[B, capacity, H*(D+8)]`` -- ``[K_idx | K_norm | V_idx | V_norm]`` per token, exactly the
row the paged cache holds -- so that

* an update is a single launch of the paged write kernel (norm, rotate, bucketize, pack, scatter),
* attention is the paged kernel itself over 256-token pages with an identity block table
  (batch ``b`` owns pages ``b*P .. b*P+P-1``), with no re-packing and no second kernel family,
* the four reference tensors are zero-copy strided views of the buffer.

Capacity doubles when it runs out, so appending a token never re-copies a layer
(the reference ``torch.cat``s every step, src/turboquant_vllm/kv_cache.py:640-672).
"""

from __future__ import annotations

import math

import torch

PAGE_TOKENS = 256  # tokens per page of the identity-mapped row buffer (the kernels' largest page)
_TABLE_ENTRIES = 1 << 22  # largest batch * capacity for which the per-step index rows are kept (48 MB)


_index_row_cache: dict = {}  # (device, batch, capacity) -> (len_rows, slot_rows); shared by all layers


def _index_rows(device: torch.device, batch: int, cap: int):
    """``len_rows [cap+1, B]`` int32 (row n = n repeated) and ``slot_rows [cap, B]`` int64
    (row n = b*cap + n), or ``(None, None)`` when they would be too large."""
    if batch * (cap + 1) > _TABLE_ENTRIES:
        return None, None
    key = (device, batch, cap)
    hit = _index_row_cache.get(key)
    if hit is None:
        if len(_index_row_cache) >= 4:  # layers of a model share one entry; keep the dict small
            _index_row_cache.pop(next(iter(_index_row_cache)))
        steps = torch.arange(cap + 1, device=device)
        base = torch.arange(batch, dtype=torch.int64, device=device) * cap
        hit = (steps.to(torch.int32)[:, None].expand(cap + 1, batch).contiguous(),
               (steps[:cap, None] + base[None, :]).contiguous())
        _index_row_cache[key] = hit
    return hit


class TokenRowStore:
    """K and V of one layer for ``batch`` sequences of equal length, as packed token rows.

    Attributes:
        rows: uint8 ``[batch, capacity, heads*(dim+8)]``; ``capacity`` is a multiple of 256.
        len: tokens stored per sequence.
    """

    def __init__(self, batch: int, heads: int, dim: int, device: torch.device, min_tokens: int = 0) -> None:
        if dim % 2:
            raise ValueError(f"nibble-packed rows need an even head_dim, got {dim}")
        if (heads * (dim // 2)) % 4:
            raise ValueError(f"token rows need heads*head_dim/2 to be a multiple of 4 (fp32 norms), "
                             f"got heads={heads}, head_dim={dim}")
        self.batch, self.heads, self.dim = batch, heads, dim
        self.device = torch.device(device)
        self.half = heads * (dim // 2 + 4)  # bytes of the K (or V) half of a row
        self.row_bytes = 2 * self.half
        self.len = 0
        self.rows: torch.Tensor = torch.empty(0, dtype=torch.uint8, device=self.device)
        self._capacity = 0
        self._reserve(max(min_tokens, 1))

    # ----- storage ------------------------------------------------------------------------------
    @property
    def capacity(self) -> int:
        return self._capacity

    def _reserve(self, tokens: int) -> None:
        if tokens <= self._capacity:
            return
        cap = max(2 * self._capacity, PAGE_TOKENS * math.ceil(tokens / PAGE_TOKENS))
        grown = torch.empty(self.batch, cap, self.row_bytes, dtype=torch.uint8, device=self.device)
        if self.len:
            grown[:, : self.len] = self.rows[:, : self.len]
        self.rows, self._capacity = grown, cap
        pages = cap // PAGE_TOKENS
        self._block_table = torch.arange(self.batch * pages, dtype=torch.int32, device=self.device).view(
            self.batch, pages)
        self._slot_base = torch.arange(self.batch, dtype=torch.int64, device=self.device) * cap
        # decode steps index ready-made rows instead of launching small kernels: row n of
        # _len_rows is [n]*B (sequence lengths), row n of _slot_rows the slots of token n
        self._len_rows, self._slot_rows = _index_rows(self.device, self.batch, cap)

    def matches(self, batch: int, heads: int, dim: int, device: torch.device) -> bool:
        return (batch, heads, dim) == (self.batch, self.heads, self.dim) and torch.device(device) == self.device

    # ----- write -------------------------------------------------------------------------------------
    def append(self, key_states: torch.Tensor, value_states: torch.Tensor, k_quantizer, v_quantizer) -> None:
        """Compress ``[B, H, S_new, D]`` K and V and store them behind the tokens already held.

        One launch: the paged write kernel scatters the packed rows to slots
        ``b*capacity + len + s``.
        """
        from turboquant_vllm.kernels.ops import tq4_write_paged

        b, h, s, d = key_states.shape
        assert (b, h, d) == (self.batch, self.heads, self.dim) and value_states.shape == key_states.shape
        if s == 0:
            return
        self._reserve(self.len + s)
        _, even, odd, _, k_bounds = k_quantizer.device_primitives(self.device)
        v_bounds = v_quantizer.device_primitives(self.device)[4]  # K and V share the rotation (one seed)
        key = key_states.transpose(1, 2).reshape(b * s, h, d)
        value = value_states.transpose(1, 2).reshape(b * s, h, d)
        if s == 1:
            slots = self._slot_rows[self.len] if self._slot_rows is not None else self._slot_base + self.len
        else:
            slots = (self._slot_base[:, None] + torch.arange(self.len, self.len + s, device=self.device)).reshape(-1)
        tq4_write_paged(key, value, self.paged_cache(), slots, even, odd, k_bounds, v_bounds)
        self.len += s

    @classmethod
    def from_tensors(cls, k_packed: torch.Tensor, k_norms: torch.Tensor, v_packed: torch.Tensor,
                     v_norms: torch.Tensor) -> "TokenRowStore":
        """Rows assembled from the reference's four tensors (``[B, H, S, D/2]`` u8, ``[B, H, S(,1)]`` f32)."""
        b, h, s, half_d = k_packed.shape
        assert v_packed.shape == k_packed.shape and k_packed.dtype == v_packed.dtype == torch.uint8
        assert k_norms.dtype == v_norms.dtype == torch.float32
        store = cls(b, h, 2 * half_d, k_packed.device, min_tokens=s)
        store.len = s
        k_idx, k_n, v_idx, v_n = store.views()
        k_idx.copy_(k_packed)
        v_idx.copy_(v_packed)
        k_n.copy_(k_norms.reshape(b, h, s, 1))
        v_n.copy_(v_norms.reshape(b, h, s, 1))
        return store

    # ----- read --------------------------------------------------------------------------------------
    def views(self):
        """``(k_idx [B,H,S,D/2] u8, k_norm [B,H,S,1] f32, v_idx, v_norm)``: strided views, no copy."""
        b, h, s, hd = self.batch, self.heads, self.len, self.dim // 2
        rows = self.rows[:, :s]
        out = []
        for base in (0, self.half):
            idx = rows[:, :, base : base + h * hd].unflatten(2, (h, hd)).permute(0, 2, 1, 3)
            norm = rows[:, :, base + h * hd : base + self.half].view(torch.float32).permute(0, 2, 1).unsqueeze(-1)
            out += [idx, norm]
        return tuple(out)

    def paged_cache(self) -> torch.Tensor:
        """The buffer as pages ``[B*capacity/256, 256, row_bytes]``."""
        return self.rows.view(-1, PAGE_TOKENS, self.row_bytes)

    def block_table(self) -> torch.Tensor:
        """Identity block table ``[B, capacity/256]`` int32."""
        return self._block_table

    def attention(self, q: torch.Tensor, k_centroids: torch.Tensor, v_centroids: torch.Tensor,
                  rotation: torch.Tensor, sm_scale: float | None = None, is_causal: bool = False,
                  out_dtype: torch.dtype | None = None) -> torch.Tensor:
        """Attention of ``q [B, Hq, Sq, D]`` over the stored rows -> ``[B, Sq, Hq, D]`` (q's dtype
        unless ``out_dtype`` is given).

        Masking follows the reference kernel
        (src/turboquant_vllm/triton/flash_attention_tq4_kv.py:163-199, 301-302): ``is_causal`` lets
        query ``i`` see keys ``0..i``; a single query row is never masked.
        """
        from turboquant_vllm.kernels.ops import paged_tq4_attention

        b, hq, sq, d = q.shape
        assert b == self.batch and d == self.dim and hq % self.heads == 0
        dev = self.device
        q_rows = q.transpose(1, 2).reshape(b * sq, hq, d)
        table = self._block_table
        causal = bool(is_causal) and sq > 1
        if causal and sq != self.len:
            # top-left aligned mask: row (b, i) is a one-token sequence of length min(i + 1, S)
            lens = torch.arange(1, sq + 1, dtype=torch.int32, device=dev).clamp_(max=self.len).repeat(b)
            table = table.repeat_interleave(sq, dim=0)
            qsl = None
        else:
            lens = (self._len_rows[self.len] if self._len_rows is not None
                    else torch.full((b,), self.len, dtype=torch.int32, device=dev))
            qsl = None if sq == 1 else torch.arange(0, (b + 1) * sq, sq, dtype=torch.int32, device=dev)
        out = paged_tq4_attention(
            q_rows, self.paged_cache(), table, lens, k_centroids, v_centroids, rotation, self.heads,
            PAGE_TOKENS, sm_scale, query_start_loc=qsl, causal=causal, out_dtype=out_dtype)
        return out.view(b, sq, hq, d)


__all__ = ["PAGE_TOKENS", "TokenRowStore"]
