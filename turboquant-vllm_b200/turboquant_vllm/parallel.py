"""Multi-GPU layouts of the TQ4 hot path (one process per GPU, ``torch.distributed``).

The reference has no multi-GPU code; under vLLM tensor parallelism its backend simply receives
per-rank head counts (src/turboquant_vllm/vllm/tq4_backend.py:362-368).  Two layouts are
supported here:

* **head sharding** (tensor parallel): rank r owns KV heads ``[r*Hkv/W, (r+1)*Hkv/W)`` and the
  matching query heads, with its own packed cache.  Attention needs no collective.
* **sequence split** (long context): every rank holds a contiguous slice of every sequence's
  tokens.  Each rank runs the fused kernel on its slice and emits, per (query row, head), the
  normalised output in rotated space and the log-sum-exp of its scores; ONE all-gather of those
  partials (``rows * Hq * (D + 1)`` floats per rank) is followed by a local log-sum-exp merge +
  un-rotation kernel.
"""

from __future__ import annotations

from typing import Callable

import torch


def shard_heads(rank: int, world: int, num_q_heads: int, num_kv_heads: int) -> tuple[range, range]:
    """Query-head and KV-head ranges owned by ``rank`` under head sharding."""
    if num_kv_heads % world or num_q_heads % num_kv_heads:
        raise ValueError(
            f"cannot shard {num_kv_heads} KV heads / {num_q_heads} query heads over {world} ranks"
        )
    kv_per = num_kv_heads // world
    group = num_q_heads // num_kv_heads
    return (range(rank * kv_per * group, (rank + 1) * kv_per * group),
            range(rank * kv_per, (rank + 1) * kv_per))


def split_sequence(seq_len: int, world: int, block_size: int) -> list[tuple[int, int]]:
    """Token ranges ``[start, end)`` of one sequence per rank: contiguous, block aligned, the
    tail (where new tokens are appended) on the last rank that holds anything."""
    blocks = (seq_len + block_size - 1) // block_size
    per = (blocks + world - 1) // world
    out = []
    for r in range(world):
        s = min(seq_len, r * per * block_size)
        e = min(seq_len, (r + 1) * per * block_size)
        out.append((s, e))
    return out


def gather_partials(o_local: torch.Tensor, lse_local: torch.Tensor, group=None):
    """All-gather per-rank partials: ``o [T, Hq, D]`` fp32, ``lse [T, Hq]`` fp32 ->
    ``([W, T, Hq, D], [W, T, Hq])``.  One collective: output and LSE travel in one buffer."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    t, hq, d = o_local.shape
    packed = torch.cat([o_local.reshape(t, hq, d), lse_local.reshape(t, hq, 1)], dim=-1).contiguous()
    gathered = torch.empty(world, t, hq, d + 1, dtype=packed.dtype, device=packed.device)
    if packed.is_cuda:
        dist.all_gather_into_tensor(gathered, packed, group=group)
    else:  # gloo (CPU ranks in tests) has no tensor-form all-gather
        dist.all_gather(list(gathered.unbind(0)), packed, group=group)
    return gathered[..., :d].contiguous(), gathered[..., d].contiguous()


def split_kv_decode(
    q: torch.Tensor,
    kv_cache_local: torch.Tensor,
    block_table_local: torch.Tensor,
    seq_lens_local: torch.Tensor,
    k_centroids: torch.Tensor,
    v_centroids: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    block_size: int,
    sm_scale: float | None = None,
    *,
    group=None,
    out_dtype: torch.dtype | None = None,
    attend: Callable | None = None,
    combine: Callable | None = None,
    exchange_events: list | None = None,
) -> torch.Tensor:
    """Decode attention when each rank holds a token slice of every sequence.

    ``seq_lens_local[i]`` is the number of tokens of sequence i stored on THIS rank (0 allowed),
    ``block_table_local`` addresses this rank's cache.  Returns the full attention output
    ``[num_seqs, Hq, D]`` on every rank.  ``attend`` / ``combine`` default to the CUDA kernels
    (injectable so that the wiring can be exercised without a GPU).  ``exchange_events``: a list
    that receives one ``(start, end)`` pair of CUDA events recorded on the current stream around the
    exchange (packing, all-gather, unpacking), for callers that want its share of the step.
    """
    from turboquant_vllm.kernels import ops

    t, hq, d = q.shape
    if attend is None:
        def attend(q_, lse_):
            return ops.paged_tq4_attention(
                q_, kv_cache_local, block_table_local, seq_lens_local, k_centroids, v_centroids,
                rotation, num_kv_heads, block_size, sm_scale, out_dtype=torch.float32,
                lse_out=lse_, out_rotated=True)
    if combine is None:
        def combine(po, pl):
            return ops.combine_partials(po, pl, rotation, out_dtype=out_dtype or q.dtype)
    lse = torch.empty(t, hq, dtype=torch.float32, device=q.device)
    o_rot = attend(q, lse)
    if exchange_events is not None and q.is_cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        parts_o, parts_lse = gather_partials(o_rot, lse, group)
        e1.record()
        exchange_events.append((e0, e1))
    else:
        parts_o, parts_lse = gather_partials(o_rot, lse, group)
    out = combine(parts_o, parts_lse)
    if q.is_cuda:
        ops.maybe_raise_on_device_errors(q.device, "split_kv_decode")
    return out
