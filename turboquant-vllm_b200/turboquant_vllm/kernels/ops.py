"""Python entry points of the sm_100a TQ4 kernels.

The four public functions keep the names, argument order and ``out=`` behaviour of the
reference's Triton wrappers so existing callers and tests keep working:

* ``tq4_compress``            (reference: src/turboquant_vllm/triton/tq4_compress.py:173-245)
* ``tq4_decompress``          (reference: src/turboquant_vllm/triton/tq4_decompress.py:126-184)
* ``fused_paged_tq4_decode``  (reference: src/turboquant_vllm/triton/fused_paged_tq4_attention.py:255-370)
* ``fused_paged_tq4_int8_prefill`` (reference: src/turboquant_vllm/triton/fused_paged_tq4_int8_prefill.py:291-417)

plus the fused cache write ``tq4_write_paged`` and the general ``paged_tq4_attention``.
Everything runs through the C ABI in ``include/tq4.h``; CPU tensors are rejected.
"""

from __future__ import annotations

import math
import os

import torch

from turboquant_vllm import _native as nv

# --------------------------------------------------------------------------------------
# per-device scratch: attention workspace (grown on demand, reused) and the error flag
# --------------------------------------------------------------------------------------
_workspaces: dict[int, torch.Tensor] = {}
_err_flags: dict[int, torch.Tensor] = {}


def attention_workspace_bytes(max_query_rows: int, num_q_heads: int, num_kv_heads: int, head_dim: int) -> int:
    """Bytes of scratch ``paged_tq4_attention`` needs for up to ``max_query_rows`` rows."""
    n = nv.lib().tq4_attention_workspace_bytes(max_query_rows, num_q_heads, num_kv_heads, head_dim)
    if n == 0:
        raise ValueError(
            f"unsupported attention shape: Hq={num_q_heads}, Hkv={num_kv_heads}, D={head_dim}"
        )
    return int(n)


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _workspaces[idx] = ws
    return ws


def error_flag(device: torch.device) -> torch.Tensor:
    """Device int32 that kernels OR with TQ4_DEV_* bits (bad slot / bad block id)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    f = _err_flags.get(idx)
    if f is None:
        f = torch.zeros(1, dtype=torch.int32, device=device)
        _err_flags[idx] = f
    return f


def read_and_clear_errors(device: torch.device) -> int:
    """Synchronising read of the device error flag; clears it."""
    f = error_flag(device)
    v = int(f.item())
    if v:
        f.zero_()
    return v


def error_checks_enabled() -> bool:
    """``TQ4_CHECK_ERRORS`` (``1/true/yes``): the host layers (vLLM impl, HF cache, split-KV decode)
    read the device error flag after each call and raise.  Off by default: the read synchronises
    the stream, and it cannot happen while a CUDA graph is being captured."""
    return os.environ.get("TQ4_CHECK_ERRORS", "").lower() in ("1", "true", "yes")


def raise_on_device_errors(device: torch.device, where: str, *, flag: int | None = None) -> None:
    """Raise ``RuntimeError`` if a kernel reported an out-of-range slot or block id, or a device-side
    wait that gave up (the offending work was skipped, so outputs are incomplete).

    Reads and clears the device flag (synchronising); ``flag`` substitutes an already known value.
    Skipped while the current stream is capturing a CUDA graph.
    """
    if flag is None:
        if torch.cuda.is_current_stream_capturing():
            return
        flag = read_and_clear_errors(device)
    if flag:
        raise RuntimeError(f"{where}: TQ4 kernel reported {nv.describe_device_errors(flag)} "
                           f"(flag {flag:#x}); the affected rows were skipped")


def maybe_raise_on_device_errors(device: torch.device, where: str) -> None:
    """:func:`raise_on_device_errors` when ``TQ4_CHECK_ERRORS`` is set."""
    if error_checks_enabled():
        raise_on_device_errors(device, where)


def _inner_contiguous(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


# --------------------------------------------------------------------------------------
# compress / decompress
# --------------------------------------------------------------------------------------
def tq4_compress(
    x: torch.Tensor,
    rotation_T_even: torch.Tensor,
    rotation_T_odd: torch.Tensor,
    boundaries: torch.Tensor,
    out: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """``x [N, H, D]`` fp16/bf16/fp32 -> ``(packed u8 [N, H, D/2], norms f32 [N, H, 1])``.

    With ``out=(packed, norms)`` the results are written into those buffers and the same
    objects are returned.
    """
    n, h, d = x.shape
    assert d % 2 == 0, f"HEAD_DIM must be even, got {d}"
    nv.require_cuda(x, rotation_T_even, rotation_T_odd, boundaries)
    x = _inner_contiguous(x)
    if out is not None:
        packed, norms = out
        nv.require_cuda(packed, norms)
        assert packed.is_contiguous() and norms.is_contiguous()
        assert packed.numel() >= n * h * (d // 2) and norms.numel() >= n * h
    else:
        packed = torch.empty(n, h, d // 2, dtype=torch.uint8, device=x.device)
        norms = torch.empty(n, h, 1, dtype=torch.float32, device=x.device)
    st = nv.call(x.device, "tq4_compress_rows",
        x.data_ptr(), nv.dtype_code(x.dtype), n, h, d, x.stride(0), x.stride(1),
        rotation_T_even.data_ptr(), rotation_T_odd.data_ptr(),
        boundaries.data_ptr(), boundaries.numel(),
        packed.data_ptr(), norms.data_ptr(), nv.stream_ptr(x.device),
    )
    nv.check(st, "tq4_compress")
    return packed, norms


def tq4_pack_rotated(rotated: torch.Tensor, boundaries: torch.Tensor) -> torch.Tensor:
    """Bucketize + nibble-pack rows that are already rotated: fp32 ``[M, D]`` -> u8 ``[M, D/2]``."""
    nv.require_cuda(rotated, boundaries)
    assert rotated.dtype == torch.float32 and rotated.dim() == 2
    rotated = rotated.contiguous()
    m, d = rotated.shape
    packed = torch.empty(m, d // 2, dtype=torch.uint8, device=rotated.device)
    st = nv.call(rotated.device, "tq4_pack_rotated_rows",
        rotated.data_ptr(), m, d, boundaries.data_ptr(), boundaries.numel(),
        packed.data_ptr(), nv.stream_ptr(rotated.device),
    )
    nv.check(st, "tq4_pack_rotated")
    return packed


def tq4_decompress(
    packed: torch.Tensor,
    norms: torch.Tensor,
    centroids: torch.Tensor,
    dtype: torch.dtype = torch.float16,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """``packed [N, H, D/2]`` + ``norms [N, H, 1]`` -> ``[N, H, D]`` in ``dtype`` (rotated space)."""
    n, h, half = packed.shape
    d = half * 2
    nv.require_cuda(packed, norms, centroids)
    packed = packed.contiguous()
    norms = norms.contiguous()
    caller_out = out
    if out is None:
        out = torch.empty(n, h, d, dtype=dtype, device=packed.device)
    else:
        nv.require_cuda(out)
        assert out.is_contiguous() and out.numel() >= n * h * d
    st = nv.call(packed.device, "tq4_decompress_rows",
        packed.data_ptr(), norms.data_ptr(), centroids.data_ptr(), centroids.numel(),
        n * h, d, out.data_ptr(), nv.dtype_code(out.dtype), nv.stream_ptr(packed.device),
    )
    nv.check(st, "tq4_decompress")
    return caller_out if caller_out is not None else out


def tq4_decompress_cache(
    kv_cache: torch.Tensor,
    num_kv_heads: int,
    head_dim: int,
    k_centroids: torch.Tensor,
    v_centroids: torch.Tensor,
    dtype: torch.dtype,
    out_k: torch.Tensor | None = None,
    out_v: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Every token row of a ``(NB, BS, bytes)`` cache -> K, V ``[NB*BS, H, D]`` (rotated space)."""
    nv.require_cuda(kv_cache, k_centroids, v_centroids)
    assert kv_cache.dtype == torch.uint8 and kv_cache.is_contiguous()
    nb, bs, width = kv_cache.shape
    n = nb * bs
    if out_k is None:
        out_k = torch.empty(n, num_kv_heads, head_dim, dtype=dtype, device=kv_cache.device)
    if out_v is None:
        out_v = torch.empty(n, num_kv_heads, head_dim, dtype=dtype, device=kv_cache.device)
    assert out_k.dtype == out_v.dtype and out_k.is_contiguous() and out_v.is_contiguous()
    assert out_k.numel() >= n * num_kv_heads * head_dim and out_v.numel() >= n * num_kv_heads * head_dim
    st = nv.call(kv_cache.device, "tq4_decompress_cache",
        kv_cache.data_ptr(), width, n, num_kv_heads, head_dim,
        k_centroids.data_ptr(), k_centroids.numel(), v_centroids.data_ptr(), v_centroids.numel(),
        out_k.data_ptr(), out_v.data_ptr(), nv.dtype_code(out_k.dtype), nv.stream_ptr(kv_cache.device),
    )
    nv.check(st, "tq4_decompress_cache")
    return out_k, out_v


# --------------------------------------------------------------------------------------
# fused cache write
# --------------------------------------------------------------------------------------
def tq4_write_paged(
    key: torch.Tensor,
    value: torch.Tensor,
    kv_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    rotation_T_even: torch.Tensor,
    rotation_T_odd: torch.Tensor,
    k_boundaries: torch.Tensor,
    v_boundaries: torch.Tensor,
) -> None:
    """Compress ``key``/``value`` ``[N, H, D]`` and scatter the packed rows into ``kv_cache``
    ``(NB, BS, >= H*(D+8))`` at ``slot_mapping`` in one launch (negative slots are skipped)."""
    nv.require_cuda(key, value, kv_cache, slot_mapping, rotation_T_even, rotation_T_odd,
                    k_boundaries, v_boundaries)
    assert kv_cache.dtype == torch.uint8 and kv_cache.is_contiguous()
    assert key.shape == value.shape and key.dtype == value.dtype
    n, h, d = key.shape
    key = _inner_contiguous(key)
    value = _inner_contiguous(value)
    if slot_mapping.dtype != torch.int64:
        slot_mapping = slot_mapping.to(torch.int64)
    slot_mapping = slot_mapping.contiguous()
    nb, bs, width = kv_cache.shape
    st = nv.call(key.device, "tq4_write_paged",
        key.data_ptr(), value.data_ptr(), nv.dtype_code(key.dtype), n, h, d,
        key.stride(0), key.stride(1), value.stride(0), value.stride(1),
        slot_mapping.data_ptr(), slot_mapping.numel(),
        rotation_T_even.data_ptr(), rotation_T_odd.data_ptr(),
        k_boundaries.data_ptr(), k_boundaries.numel(),
        v_boundaries.data_ptr(), v_boundaries.numel(),
        kv_cache.data_ptr(), width, nb * bs,
        error_flag(key.device).data_ptr(), nv.stream_ptr(key.device),
    )
    nv.check(st, "tq4_write_paged")


# --------------------------------------------------------------------------------------
# fused paged attention
# --------------------------------------------------------------------------------------
def paged_tq4_attention(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    k_centroids: torch.Tensor,
    v_centroids: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    block_size: int,
    sm_scale: float | None = None,
    *,
    query_start_loc: torch.Tensor | None = None,
    causal: bool = True,
    sliding_window: int | None = None,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    lse_out: torch.Tensor | None = None,
    out_rotated: bool = False,
    workspace: torch.Tensor | None = None,
    mode: int = 0,
    write: tuple | None = None,
) -> torch.Tensor:
    """Attention of ``q [T, Hq, D]`` over the packed paged cache.

    ``write = (key, value, slot_mapping, rotation_T_even, rotation_T_odd, k_boundaries,
    v_boundaries)``: first store these new tokens into the cache (as :func:`tq4_write_paged`),
    folded into the attention's first kernel -- see :func:`tq4_write_and_attention`.

    ``query_start_loc=None``: decode, row i is the one new token of sequence i.  Otherwise
    int32 ``[num_seqs + 1]`` offsets of each sequence's query chunk (bottom-right aligned
    causal mask).  ``mode``: 0 auto, 1 fp32 CUDA-core kernel, 2 streaming tensor-core LUT kernel,
    3 chunked-prefill tcgen05 kernel (head_dim 128 only), 4 the same with single fp16 terms for
    queries and probabilities (faster, about 1e-3 absolute error; never picked automatically).
    """
    nv.require_cuda(q, kv_cache, block_table, seq_lens, k_centroids, v_centroids, rotation)
    t, hq, d = q.shape
    assert hq % num_kv_heads == 0
    assert kv_cache.dtype == torch.uint8 and kv_cache.stride(2) == 1
    assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
    assert seq_lens.dtype == torch.int32 and seq_lens.is_contiguous()
    assert rotation.dtype == torch.float32
    if not rotation.is_contiguous():  # e.g. the column-major Q factor of torch.linalg.qr
        rotation = rotation.contiguous()
    if query_start_loc is not None:
        assert query_start_loc.dtype == torch.int32 and query_start_loc.is_contiguous()
        nv.require_cuda(query_start_loc)
    q = _inner_contiguous(q)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    if out is None:
        out = torch.empty(t, hq, d, dtype=out_dtype or q.dtype, device=q.device)
    else:
        nv.require_cuda(out)
        assert out.shape == (t, hq, d) and out.stride(2) == 1
    if lse_out is not None:
        assert lse_out.dtype == torch.float32 and lse_out.is_contiguous() and lse_out.numel() >= t * hq
    need = attention_workspace_bytes(max(t, 1), hq, num_kv_heads, d)
    ws = workspace if workspace is not None else _workspace(q.device, need)
    if ws.numel() * ws.element_size() < need:
        raise ValueError(f"workspace has {ws.numel() * ws.element_size()} bytes, {need} needed")
    wargs: tuple = ()
    if write is not None:
        key, value, slot_mapping, rot_even, rot_odd, k_bounds, v_bounds = write
        nv.require_cuda(key, value, slot_mapping, rot_even, rot_odd, k_bounds, v_bounds)
        assert kv_cache.is_contiguous(), "the fused write addresses flat slots: block-major contiguous cache"
        assert key.shape == value.shape and key.dtype == value.dtype and key.shape[1:] == (num_kv_heads, d)
        key = _inner_contiguous(key)
        value = _inner_contiguous(value)
        if slot_mapping.dtype != torch.int64:
            slot_mapping = slot_mapping.to(torch.int64)
        slot_mapping = slot_mapping.contiguous()
        wargs = (key.data_ptr(), value.data_ptr(), nv.dtype_code(key.dtype), key.shape[0],
                 key.stride(0), key.stride(1), value.stride(0), value.stride(1),
                 slot_mapping.data_ptr(), slot_mapping.numel(), rot_even.data_ptr(), rot_odd.data_ptr(),
                 k_bounds.data_ptr(), k_bounds.numel(), v_bounds.data_ptr(), v_bounds.numel())
    st = nv.call(
        q.device, "tq4_write_and_attention" if write is not None else "tq4_paged_attention",
        *wargs,
        q.data_ptr(), nv.dtype_code(q.dtype), t, seq_lens.numel(), hq, num_kv_heads, d,
        q.stride(0), q.stride(1),
        kv_cache.data_ptr(), kv_cache.stride(0), kv_cache.stride(1), kv_cache.shape[0], block_size,
        block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(), nv.ptr(query_start_loc),
        k_centroids.data_ptr(), k_centroids.numel(), v_centroids.data_ptr(), v_centroids.numel(),
        rotation.data_ptr(), float(sm_scale), int(bool(causal)), int(sliding_window or 0),
        out.data_ptr(), nv.dtype_code(out.dtype), out.stride(0), out.stride(1),
        nv.ptr(lse_out), int(bool(out_rotated)),
        ws.data_ptr(), ws.numel() * ws.element_size(), mode,
        error_flag(q.device).data_ptr(), nv.stream_ptr(q.device),
    )
    nv.check(st, "paged_tq4_attention")
    return out


def tq4_write_and_attention(
    key: torch.Tensor,
    value: torch.Tensor,
    slot_mapping: torch.Tensor,
    rotation_T_even: torch.Tensor,
    rotation_T_odd: torch.Tensor,
    k_boundaries: torch.Tensor,
    v_boundaries: torch.Tensor,
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    k_centroids: torch.Tensor,
    v_centroids: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    block_size: int,
    sm_scale: float | None = None,
    **kwargs,
) -> torch.Tensor:
    """One decode step of a layer: :func:`tq4_write_paged` of the new tokens, then
    :func:`paged_tq4_attention`, in three launches (the cache write rides in the kernel that rotates
    the queries and plans the tiles) or, for decode calls with more than 512 (row, KV head) pairs, in
    two (that work happens inside the attention kernel; token i must then be the newest token of
    sequence i).  In the three-launch form the results equal the two calls in sequence bit for bit; in
    the two-launch form the norms do and the indices agree within the write path's 1e-4 bound."""
    return paged_tq4_attention(
        q, kv_cache, block_table, seq_lens, k_centroids, v_centroids, rotation, num_kv_heads,
        block_size, sm_scale,
        write=(key, value, slot_mapping, rotation_T_even, rotation_T_odd, k_boundaries, v_boundaries),
        **kwargs)


def fused_paged_tq4_decode(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    centroids: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    head_dim: int,
    block_size: int,
    sm_scale: float | None = None,
    out: torch.Tensor | None = None,
    *,
    v_centroids: torch.Tensor | None = None,
    sliding_window: int | None = None,
    workspace: torch.Tensor | None = None,
    mode: int = 0,
) -> torch.Tensor:
    """Fused paged TQ4 decode: one query token per sequence, ``q [num_seqs, Hq, D]``.

    Same positional signature as the reference.  Keyword extras: a separate value codebook
    (asymmetric K4/V3), a sliding window, a pre-allocated workspace (CUDA graphs).
    """
    num_seqs, hq, d = q.shape
    assert d == head_dim
    assert hq % num_kv_heads == 0
    assert kv_cache.dtype == torch.uint8
    assert block_table.dtype == torch.int32
    assert seq_lens.dtype == torch.int32
    return paged_tq4_attention(
        q, kv_cache, block_table, seq_lens, centroids,
        centroids if v_centroids is None else v_centroids, rotation, num_kv_heads, block_size,
        sm_scale, sliding_window=sliding_window, out=out, workspace=workspace, mode=mode,
    )


def fused_paged_tq4_prefill(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    query_start_loc: torch.Tensor,
    centroids: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    head_dim: int,
    block_size: int,
    sm_scale: float | None = None,
    out: torch.Tensor | None = None,
    *,
    v_centroids: torch.Tensor | None = None,
    causal: bool = True,
    sliding_window: int | None = None,
    workspace: torch.Tensor | None = None,
    mode: int = 0,
) -> torch.Tensor:
    """Multi-sequence, prefix-aware chunked prefill over the packed cache."""
    assert q.shape[2] == head_dim
    return paged_tq4_attention(
        q, kv_cache, block_table, seq_lens, centroids,
        centroids if v_centroids is None else v_centroids, rotation, num_kv_heads, block_size,
        sm_scale, query_start_loc=query_start_loc, causal=causal, sliding_window=sliding_window,
        out=out, workspace=workspace, mode=mode,
    )


def fused_paged_tq4_int8_prefill(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    centroids: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    head_dim: int,
    block_size: int,
    sm_scale: float | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Single-sequence causal prefill with the reference's name and signature.

    The reference kernel quantises Q and K to INT8 per tile; this one keeps fp32
    accumulation (the name is kept for drop-in compatibility).  As in the reference, exactly
    one sequence is accepted and query row i sits at absolute position
    ``seq_len - num_tokens + i`` (= i when the whole sequence is new).
    """
    num_tokens, hq, d = q.shape
    assert d == head_dim
    assert hq % num_kv_heads == 0
    assert kv_cache.dtype == torch.uint8
    assert block_table.dtype == torch.int32
    assert seq_lens.dtype == torch.int32
    if seq_lens.numel() != 1:
        raise ValueError(
            "fused_paged_tq4_int8_prefill supports only a single sequence, "
            f"but got seq_lens.numel() == {seq_lens.numel()}."
        )
    if block_table.shape[0] != 1:
        raise ValueError(
            "fused_paged_tq4_int8_prefill supports only a single sequence "
            f"(block_table.shape[0] must be 1), but got {block_table.shape[0]}."
        )
    qsl = torch.tensor([0, num_tokens], dtype=torch.int32, device=q.device)
    return paged_tq4_attention(
        q, kv_cache, block_table, seq_lens, centroids, centroids, rotation, num_kv_heads,
        block_size, sm_scale, query_start_loc=qsl, causal=True, out=out,
    )


def combine_partials(
    parts_o: torch.Tensor,
    parts_lse: torch.Tensor,
    rotation: torch.Tensor,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """Log-sum-exp merge of per-shard partials ``[W, T, Hq, D]`` / ``[W, T, Hq]`` + un-rotation."""
    nv.require_cuda(parts_o, parts_lse, rotation)
    assert parts_o.dtype == torch.float32 and parts_lse.dtype == torch.float32
    parts_o = parts_o.contiguous()
    parts_lse = parts_lse.contiguous()
    rotation = rotation.contiguous()
    w, t, hq, d = parts_o.shape
    if out is None:
        out = torch.empty(t, hq, d, dtype=out_dtype, device=parts_o.device)
    st = nv.call(parts_o.device, "tq4_combine_partials",
        parts_o.data_ptr(), parts_lse.data_ptr(), w, t, hq, d, rotation.data_ptr(),
        out.data_ptr(), nv.dtype_code(out.dtype), out.stride(0), out.stride(1),
        nv.stream_ptr(parts_o.device),
    )
    nv.check(st, "combine_partials")
    return out


def paged_tq4_attention_static(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    k_centroids: torch.Tensor,
    v_centroids: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    block_size: int,
    out: torch.Tensor,
    sm_scale: float | None = None,
    *,
    query_start_loc: torch.Tensor | None = None,
    causal: bool = True,
    sliding_window: int | None = None,
    mode: int = 0,
) -> torch.Tensor:
    """``paged_tq4_attention`` for callers that must not allocate device memory.

    Nothing is allocated here or in the library: ``out`` must be supplied, every tensor must
    already be in the layout the kernel wants (no hidden ``.contiguous()`` copies), and the
    scratch is a fixed area built into the library (``STATIC_SCRATCH_BYTES`` per GPU).  A request
    that needs more scratch than that raises ``ValueError``.  Calls on one device share the area,
    so they must not overlap on the GPU; make the first call on a device outside stream capture.
    """
    nv.require_cuda(q, kv_cache, block_table, seq_lens, k_centroids, v_centroids, rotation, out)
    t, hq, d = q.shape
    assert q.stride(2) == 1 and out.shape == (t, hq, d) and out.stride(2) == 1
    assert kv_cache.dtype == torch.uint8 and kv_cache.stride(2) == 1
    assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
    assert seq_lens.dtype == torch.int32 and seq_lens.is_contiguous()
    assert rotation.dtype == torch.float32 and rotation.is_contiguous()
    if query_start_loc is not None:
        assert query_start_loc.dtype == torch.int32 and query_start_loc.is_contiguous()
    st = nv.call(q.device, "tq4_paged_attention_static",
        q.data_ptr(), nv.dtype_code(q.dtype), t, seq_lens.numel(), hq, num_kv_heads, d,
        q.stride(0), q.stride(1),
        kv_cache.data_ptr(), kv_cache.stride(0), kv_cache.stride(1), kv_cache.shape[0], block_size,
        block_table.data_ptr(), block_table.stride(0), seq_lens.data_ptr(), nv.ptr(query_start_loc),
        k_centroids.data_ptr(), k_centroids.numel(), v_centroids.data_ptr(), v_centroids.numel(),
        rotation.data_ptr(), float(1.0 / math.sqrt(d) if sm_scale is None else sm_scale),
        int(bool(causal)), int(sliding_window or 0),
        out.data_ptr(), nv.dtype_code(out.dtype), out.stride(0), out.stride(1),
        mode, error_flag(q.device).data_ptr(), nv.stream_ptr(q.device),
    )
    nv.check(st, "paged_tq4_attention_static")
    return out
