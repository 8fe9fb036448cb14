"""GPU parity of the vLLM plugin hooks themselves: ``TQ4AttentionImpl.forward`` and the methods it
dispatches to, ``_init_cg_buffers``, ``_decompress_cache`` / ``_decompress_cache_paged`` and the
decompress + FlashAttention fallback, each against the fp32 oracle on an oracle-written cache.

The impl is built the way the reference's own tests build it (``object.__new__`` plus the
attributes ``__init__`` would set: reference tests/helpers/vllm_impl.py:26-76), the metadata is a
``SimpleNamespace`` with the ``FlashAttentionMetadata`` fields ``forward`` consumes.
"""

from __future__ import annotations

import logging
from types import SimpleNamespace

import numpy as np
import pytest
import torch

pytest.importorskip("vllm", reason="vLLM not installed")

from oracle import tq4_oracle as O  # noqa: E402
from tests.helpers import Prims, build_paged_case, cosine, index_mismatch  # noqa: E402

pytestmark = pytest.mark.gpu

MIN_COS, MAX_ABS = 0.9999, 2e-3  # fp32 output vs the fp32 oracle on the same packed cache
H_Q, H_KV, D, BS = 32, 8, 128, 16


@pytest.fixture(scope="module")
def backend(cuda_lib):
    from turboquant_vllm.vllm import tq4_backend

    return tq4_backend


def make_impl(backend, *, k_bits=4, v_bits=4, h_q=H_Q, h_kv=H_KV, d=D, sliding_window=None, fused=True,
              max_prefill_len=2048, max_model_len=6144):
    from vllm.v1.attention.backend import AttentionType

    impl = object.__new__(backend.TQ4AttentionImpl)
    impl.num_heads, impl.num_kv_heads, impl.head_size = h_q, h_kv, d
    impl.scale = 1.0 / d**0.5
    impl.alibi_slopes = None
    impl.logits_soft_cap = 0
    impl.sinks = None
    impl.sliding_window = None if sliding_window is None else (sliding_window - 1, 0)
    impl.attn_type = AttentionType.DECODER
    impl.kv_cache_dtype = "auto"
    impl.vllm_flash_attn_version = 2
    impl._setup_tq4(k_bits, v_bits, torch.device("cuda"), max_prefill_len=max_prefill_len,
                    max_model_len=max_model_len)
    impl._fused_paged_available = fused
    impl._int8_prefill_available = fused
    return impl


def metadata(case, q_lens, dev="cuda", *, slot_mapping=None, causal=True):
    """FlashAttentionMetadata stand-in for a batch whose sequence i has q_lens[i] new tokens."""
    qsl = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    n = int(qsl[-1])
    if slot_mapping is None:  # slots of the last q_len tokens of every sequence
        sm, off = [], 0
        for s, ql in zip(case["seq_lens"].tolist(), q_lens):
            sm += case["slot_mapping"][off + s - ql: off + s].tolist()
            off += s
        slot_mapping = torch.tensor(sm, dtype=torch.int64)
    return SimpleNamespace(
        num_actual_tokens=n, slot_mapping=slot_mapping.to(dev), block_table=case["block_table"].to(dev),
        seq_lens=case["seq_lens"].to(dev), query_start_loc=qsl.to(dev), max_query_len=max(q_lens),
        max_seq_len=int(case["seq_lens"].max()), causal=causal, use_cascade=False,
        scheduler_metadata=None, max_num_splits=0,
    )


def new_tokens(case, q_lens):
    """K/V rows of the last q_len tokens of every sequence (the step's new tokens)."""
    ks, vs, off = [], [], 0
    for s, ql in zip(case["seq_lens"].tolist(), q_lens):
        ks.append(case["key"][off + s - ql: off + s])
        vs.append(case["value"][off + s - ql: off + s])
        off += s
    return torch.cat(ks), torch.cat(vs)


def cache_without_new_tokens(case, q_lens):
    """The oracle-written cache with the rows of the step's new tokens zeroed (what vLLM hands to
    ``forward`` before the step's cache update)."""
    cache = case["cache"].clone()
    flat = cache.view(-1, cache.shape[-1])
    off = 0
    for s, ql in zip(case["seq_lens"].tolist(), q_lens):
        flat[case["slot_mapping"][off + s - ql: off + s]] = 0
        off += s
    return cache


def check(out, ref):
    out = out.float().cpu()
    assert torch.isfinite(out).all()
    c, err = cosine(out, ref), (out - ref).abs().max().item()
    assert c >= MIN_COS and err <= MAX_ABS, (c, err)


def data_bytes(cache, h_kv=H_KV, d=D):
    return cache[..., : h_kv * (d + 8)].cpu()


# ---------------------------------------------------------------------------------------------
# forward: fused paths
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("k_bits,v_bits", [(4, 4), (4, 3)])
def test_forward_uniform_decode(backend, k_bits, v_bits):
    """Decode batch through ``forward``: cache update of the new tokens + attention, vs the oracle."""
    pr = Prims(D, k_bits, v_bits)
    seq_lens = [300, 17, 64, 1, 129]
    q_lens = [1] * len(seq_lens)
    case = build_paged_case(seq_lens, H_KV, D, BS, pr, seed=3, padded=True)
    impl = make_impl(backend, k_bits=k_bits, v_bits=v_bits)
    q = torch.randn(len(seq_lens), H_Q, D, generator=torch.Generator().manual_seed(1)).bfloat16()
    ref = O.paged_decode_fp32(q, case["cache"], case["block_table"], seq_lens, pr.kc, pr.vc, pr.rot, H_KV)
    key, value = new_tokens(case, q_lens)
    cache = cache_without_new_tokens(case, q_lens).cuda()
    out = torch.full((len(seq_lens), H_Q, D), 7.0, dtype=torch.float32, device="cuda")
    r = impl.forward(None, q.cuda(), key.cuda(), value.cuda(), cache, metadata(case, q_lens), output=out)
    assert r is out and impl._cg_buffers_ready
    check(out, ref)
    # the cache update wrote the same rows the oracle wrote (padding untouched)
    assert index_mismatch(data_bytes(cache)[..., : H_KV * D // 2], data_bytes(case["cache"])[..., : H_KV * D // 2]) <= 1e-4
    assert torch.equal(cache[..., H_KV * (D + 8):].cpu(), case["cache"][..., H_KV * (D + 8):])
    # 16-bit output, as vLLM passes it: the rounded fp32 result
    cache2 = cache_without_new_tokens(case, q_lens).cuda()
    out16 = torch.empty(len(seq_lens), H_Q, D, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, q.cuda(), key.cuda(), value.cuda(), cache2, metadata(case, q_lens), output=out16)
    assert torch.equal(out16, out.bfloat16())
    from turboquant_vllm.kernels import ops

    assert ops.read_and_clear_errors(out.device) == 0


def test_forward_mixed_batch_with_prefix(backend):
    """Decode rows and prefill chunks (with packed prefixes) in one step -> `_int8_prefill_path`."""
    pr = Prims(D)
    seq_lens, q_lens = [200, 150, 33, 64, 90], [1, 40, 33, 1, 17]
    case = build_paged_case(seq_lens, H_KV, D, BS, pr, seed=5, padded=True)
    impl = make_impl(backend)
    n = sum(q_lens)
    q = torch.randn(n, H_Q, D, generator=torch.Generator().manual_seed(2)).bfloat16()
    qsl = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    ref = O.paged_attention_fp32(q, case["cache"], case["block_table"], seq_lens, qsl, pr.kc, pr.vc,
                                 pr.rot, H_KV, None, True, None)
    key, value = new_tokens(case, q_lens)
    cache = cache_without_new_tokens(case, q_lens).cuda()
    # vLLM pads the token dimension: query/key/value/output longer than num_actual_tokens
    pad = 5
    qp = torch.cat([q, torch.zeros(pad, H_Q, D, dtype=q.dtype)]).cuda()
    kp = torch.cat([key, torch.zeros(pad, H_KV, D, dtype=key.dtype)]).cuda()
    vp = torch.cat([value, torch.zeros(pad, H_KV, D, dtype=value.dtype)]).cuda()
    out = torch.full((n + pad, H_Q, D), 7.0, dtype=torch.float32, device="cuda")
    impl.forward(None, qp, kp, vp, cache, metadata(case, q_lens), output=out)
    check(out[:n], ref)
    assert (out[n:] == 7.0).all()  # rows past num_actual_tokens are not touched
    assert index_mismatch(data_bytes(cache)[..., : H_KV * D // 2], data_bytes(case["cache"])[..., : H_KV * D // 2]) <= 1e-4


def test_forward_sliding_window(backend):
    pr = Prims(D)
    seq_lens, q_lens, window = [300, 90, 20], [1, 30, 20], 48
    case = build_paged_case(seq_lens, H_KV, D, BS, pr, seed=7, padded=True)
    impl = make_impl(backend, sliding_window=window)
    q = torch.randn(sum(q_lens), H_Q, D, generator=torch.Generator().manual_seed(4)).bfloat16()
    qsl = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    ref = O.paged_attention_fp32(q, case["cache"], case["block_table"], seq_lens, qsl, pr.kc, pr.vc,
                                 pr.rot, H_KV, None, True, window)
    key, value = new_tokens(case, q_lens)
    out = torch.empty(sum(q_lens), H_Q, D, dtype=torch.float32, device="cuda")
    impl.forward(None, q.cuda(), key.cuda(), value.cuda(), cache_without_new_tokens(case, q_lens).cuda(),
                 metadata(case, q_lens), output=out)
    check(out, ref)


def test_forward_padded_decode_batch(backend):
    """CUDA-graph style padding: more sequence rows than live requests; padded rows have slot -1 and
    sequence length 0, write nothing and produce zeros."""
    pr = Prims(D)
    live = [70, 33]
    case = build_paged_case(live, H_KV, D, BS, pr, seed=9, padded=True)
    impl = make_impl(backend)
    rows = 4
    q = torch.randn(rows, H_Q, D, generator=torch.Generator().manual_seed(6)).bfloat16()
    ref = O.paged_decode_fp32(q[:2], case["cache"], case["block_table"], live, pr.kc, pr.vc, pr.rot, H_KV)
    key, value = new_tokens(case, [1, 1])
    key = torch.cat([key, torch.randn(2, H_KV, D).to(key.dtype)])
    value = torch.cat([value, torch.randn(2, H_KV, D).to(value.dtype)])
    md = metadata(case, [1, 1])
    md.num_actual_tokens = rows
    md.slot_mapping = torch.cat([md.slot_mapping, torch.full((2,), -1, dtype=torch.int64, device="cuda")])
    md.seq_lens = torch.cat([md.seq_lens, torch.zeros(2, dtype=torch.int32, device="cuda")])
    md.block_table = torch.cat([md.block_table, torch.zeros(2, md.block_table.shape[1], dtype=torch.int32, device="cuda")])
    md.query_start_loc = torch.arange(rows + 1, dtype=torch.int32, device="cuda")
    cache = cache_without_new_tokens(case, [1, 1]).cuda()
    out = torch.full((rows, H_Q, D), 7.0, dtype=torch.float32, device="cuda")
    impl.forward(None, q.cuda(), key.cuda(), value.cuda(), cache, md, output=out)
    check(out[:2], ref)
    assert not out[2:].any()
    assert index_mismatch(data_bytes(cache)[..., : H_KV * D // 2], data_bytes(case["cache"])[..., : H_KV * D // 2]) <= 1e-4


def test_forward_without_metadata_or_cache_zero_fills(backend):
    impl = make_impl(backend)
    q = torch.randn(3, H_Q, D, device="cuda", dtype=torch.bfloat16)
    kv = torch.randn(3, H_KV, D, device="cuda", dtype=torch.bfloat16)
    out = torch.full((3, H_Q, D), 7.0, dtype=torch.bfloat16, device="cuda")
    assert impl.forward(None, q, kv, kv, None, None, output=out) is out
    assert not out.any()
    out.fill_(7.0)
    md = SimpleNamespace(num_actual_tokens=3)
    impl.forward(None, q, kv, kv, None, md, output=out)
    assert not out.any()
    with pytest.raises(NotImplementedError):
        impl.forward(None, q, kv, kv, None, md, output=out, output_scale=torch.ones(1))


def test_forward_decode_cuda_graph_replay_equals_eager(backend):
    """Uniform decode captured into a CUDA graph (after one eager warm-up step that allocates the
    scratch) and replayed: bit-equal to the eager result, including the cache update."""
    pr = Prims(D)
    seq_lens = [257, 40, 64, 1000]
    q_lens = [1] * 4
    case = build_paged_case(seq_lens, H_KV, D, BS, pr, seed=11, padded=True)
    impl = make_impl(backend)
    q = torch.randn(4, H_Q, D, generator=torch.Generator().manual_seed(8)).bfloat16().cuda()
    key, value = (x.cuda() for x in new_tokens(case, q_lens))
    md = metadata(case, q_lens)
    cache_e = cache_without_new_tokens(case, q_lens).cuda()
    out_e = torch.empty(4, H_Q, D, dtype=torch.bfloat16, device="cuda")
    impl.forward(None, q, key, value, cache_e, md, output=out_e)  # eager; allocates the scratch
    cache_g = cache_without_new_tokens(case, q_lens).cuda()
    out_g = torch.zeros_like(out_e)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        impl.forward(None, q, key, value, cache_g, md, output=out_g)  # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    cache_g.copy_(cache_without_new_tokens(case, q_lens))
    out_g.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        impl.forward(None, q, key, value, cache_g, md, output=out_g)
    out_g.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out_g, out_e)
    assert torch.equal(cache_g, cache_e)
    graph.replay()  # a second replay over the already written cache gives the same answer
    torch.cuda.synchronize()
    assert torch.equal(out_g, out_e)


def test_forward_consumes_inputs_produced_on_the_stream_just_before(backend):
    """q, key and value come out of kernels enqueued on the same stream immediately before the
    call (as a QKV projection + RoPE would): the first kernel of the step must not read them early."""
    pr = Prims(D)
    seq_lens = [513, 77, 4096, 30] * 4
    q_lens = [1] * len(seq_lens)
    case = build_paged_case(seq_lens, H_KV, D, BS, pr, seed=13, padded=True)
    impl = make_impl(backend)
    n = len(seq_lens)
    q = torch.randn(n, H_Q, D, generator=torch.Generator().manual_seed(9)).bfloat16()
    ref = O.paged_decode_fp32(q, case["cache"], case["block_table"], seq_lens, pr.kc, pr.vc, pr.rot, H_KV)
    key, value = new_tokens(case, q_lens)
    md = metadata(case, q_lens)
    big = torch.randn(4096, 4096, device="cuda")
    q_src, k_src, v_src = (q.cuda().float() / 3, key.cuda().float() / 3, value.cuda().float() / 3)
    for _ in range(3):
        cache = cache_without_new_tokens(case, q_lens).cuda()
        out = torch.empty(n, H_Q, D, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        _ = big @ big  # keep the GPU busy so the producers below are still queued at the call
        qd = (q_src * 3).bfloat16()
        kd = (k_src * 3).to(key.dtype)
        vd = (v_src * 3).to(value.dtype)
        impl.forward(None, qd, kd, vd, cache, md, output=out)
        check(out, ref)
        assert index_mismatch(data_bytes(cache)[..., : H_KV * D // 2], data_bytes(case["cache"])[..., : H_KV * D // 2]) <= 1e-4


def test_forward_surfaces_device_errors_when_asked(backend, monkeypatch):
    """TQ4_CHECK_ERRORS=1: a block id outside the cache raises instead of silently skipping rows."""
    from turboquant_vllm.kernels import ops

    pr = Prims(D)
    case = build_paged_case([40, 17], H_KV, D, BS, pr, seed=15, padded=True)
    impl = make_impl(backend)
    q = torch.randn(2, H_Q, D).bfloat16().cuda()
    md = metadata(case, [1, 1])
    md.block_table = md.block_table.clone()
    md.block_table[0, 1] = 10_000
    out = torch.empty(2, H_Q, D, dtype=torch.float32, device="cuda")
    ops.read_and_clear_errors(out.device)
    impl.forward(None, q, None, None, case["cache"].cuda(), md, output=out)  # default: no check, no raise
    assert ops.read_and_clear_errors(out.device) & 2
    monkeypatch.setenv("TQ4_CHECK_ERRORS", "1")
    with pytest.raises(RuntimeError, match="TQ4_DEV_BAD_BLOCK"):
        impl.forward(None, q, None, None, case["cache"].cuda(), md, output=out)
    assert ops.read_and_clear_errors(out.device) == 0  # the raise cleared the flag


# ---------------------------------------------------------------------------------------------
# forward: decompress + FlashAttention fallback (TQ4_USE_FUSED_PAGED=0 / unsupported features)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("q_lens", [[1, 1, 1], [1, 24, 33]])
def test_forward_flash_fallback(backend, q_lens):
    """The reference's default path: rotate Q, decompress the referenced blocks to 16-bit, vLLM's
    FlashAttention in rotated space, un-rotate.  K, V, P are rounded to 16 bits on this path, so
    the gate is the reference's own (cosine > 0.999), not the fused kernels' fp32 gate."""
    pr = Prims(D)
    seq_lens = [120, 64, 33]
    case = build_paged_case(seq_lens, H_KV, D, BS, pr, seed=17, padded=True)
    impl = make_impl(backend, fused=False)
    assert impl._needs_fallback()
    n = sum(q_lens)
    q = torch.randn(n, H_Q, D, generator=torch.Generator().manual_seed(10)).half()
    qsl = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    ref = O.paged_attention_fp32(q, case["cache"], case["block_table"], seq_lens, qsl, pr.kc, pr.vc,
                                 pr.rot, H_KV, None, True, None)
    key, value = new_tokens(case, q_lens)
    cache = cache_without_new_tokens(case, q_lens).cuda()
    layer = SimpleNamespace(_q_scale=torch.ones(1, device="cuda"), _k_scale=torch.ones(1, device="cuda"),
                            _v_scale=torch.ones(1, device="cuda"))
    out = torch.empty(n, H_Q, D, dtype=torch.float16, device="cuda")
    impl.forward(layer, q.cuda(), key.half().cuda(), value.half().cuda(), cache, metadata(case, q_lens), output=out)
    o = out.float().cpu()
    assert torch.isfinite(o).all()
    assert cosine(o, ref) > 0.999 and (o - ref).abs().max().item() < 2e-2
    assert impl._fallback_buffers_ready and impl._cg_prefill_k.dtype == torch.float16


# ---------------------------------------------------------------------------------------------
# _init_cg_buffers / _decompress_cache / _decompress_cache_paged
# (reference: tests/test_vllm_cache_cudagraph.py:56-156, 263-389, tests/test_vllm_paged_decompress.py:31-318)
# ---------------------------------------------------------------------------------------------
def empty_cache(num_blocks, padded=True):
    width = H_KV * (O.padded_slot_bytes(D) if padded else D + 8)
    return torch.zeros(num_blocks, BS, width, dtype=torch.uint8, device="cuda")


@pytest.mark.parametrize("fused", [False, True])
def test_init_cg_buffers_shapes(backend, fused):
    impl = make_impl(backend, fused=fused)
    cache = empty_cache(4)
    assert not impl._cg_buffers_ready
    impl._init_cg_buffers(cache, compute_dtype=torch.float16)
    assert impl._cg_buffers_ready
    max_tokens = 4 * BS
    # the reference-named decompress targets exist whatever the path (lazily on the fused path)
    assert impl._cg_decompress_k.shape == (max_tokens, H_KV, D) and impl._cg_decompress_k.dtype == torch.float16
    assert impl._cg_decompress_v.shape == (max_tokens, H_KV, D)
    assert impl._cg_prefill_k.shape == (min(impl._max_prefill_len, max_tokens), H_KV, D)
    assert impl._cg_prefill_v.shape == impl._cg_prefill_k.shape
    assert impl._max_prefill_blocks == min(impl._max_prefill_len, max_tokens) // BS
    assert impl._cg_compress_packed.shape == (1, H_KV, D // 2) and impl._cg_compress_packed.dtype == torch.uint8
    assert impl._cg_compress_norms.shape == (1, H_KV, 1) and impl._cg_compress_norms.dtype == torch.float32
    assert impl._cg_q_rot.shape == (1, H_Q, D) and impl._cg_q_rot.dtype == torch.float32
    assert impl._cg_q_rot_cast.shape == (1, H_Q, D) and impl._cg_q_rot_cast.dtype == torch.float16
    assert impl._cg_compress_row.shape == (1, impl._total_bytes) and impl._cg_compress_row.dtype == torch.uint8
    from turboquant_vllm.kernels import ops

    assert impl._cg_workspace.numel() >= ops.attention_workspace_bytes(max_tokens, H_Q, H_KV, D)


def test_cg_buffers_bounded_by_scheduler_limits(backend):
    impl = make_impl(backend, fused=False, max_prefill_len=2048, max_model_len=6144)
    impl._init_cg_buffers(empty_cache(500, padded=False), compute_dtype=torch.bfloat16)
    assert impl._cg_decompress_k.shape == (min(6144, 500 * BS), H_KV, D)
    assert impl._cg_decompress_k.dtype == torch.bfloat16
    assert impl._cg_prefill_k.shape == (2048, H_KV, D)
    assert impl._max_prefill_blocks == 2048 // BS


def test_lazy_buffers_do_not_exist_before_init(backend):
    impl = make_impl(backend)
    with pytest.raises(AttributeError):
        impl._cg_decompress_k  # noqa: B018
    with pytest.raises(AttributeError):
        impl._no_such_attribute  # noqa: B018


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_preallocated_decompress_matches_dynamic_and_ignores_stale_data(backend, dtype):
    pr = Prims(D)
    impl = make_impl(backend, fused=False)
    cache = empty_cache(4, padded=False)
    key = torch.randn(3, H_KV, D, device="cuda", dtype=dtype)
    value = torch.randn(3, H_KV, D, device="cuda", dtype=dtype)
    slots = torch.tensor([0, 5, 33], device="cuda")
    impl._compress_and_store(key, value, cache, slots)
    k_dyn, v_dyn = impl._decompress_cache(cache, dtype, apply_rotation=False)
    assert k_dyn.shape == (4, BS, H_KV, D) and k_dyn.dtype == dtype
    impl._init_cg_buffers(cache, compute_dtype=dtype)
    impl._cg_decompress_k.fill_(99.0)
    impl._cg_decompress_v.fill_(99.0)
    k_pre, v_pre = impl._decompress_cache(cache, dtype, apply_rotation=False,
                                          out_k=impl._cg_decompress_k, out_v=impl._cg_decompress_v)
    assert torch.equal(k_dyn, k_pre) and torch.equal(v_dyn, v_pre)
    assert k_pre.data_ptr() == impl._cg_decompress_k.data_ptr()
    # against the oracle: rows of the written slots, rotated space, rounded to the 16-bit dtype
    kp, kn, vp, vn = O.split_rows(cache.cpu().view(-1, cache.shape[-1])[slots.cpu()], H_KV, D)
    want_k = O.decompress_rows(kp, kn, pr.kc).to(dtype)
    assert torch.equal(k_pre.view(-1, H_KV, D)[slots].cpu(), want_k.view(3, H_KV, D))
    # with apply_rotation the rows come back near the original vectors
    k_rot, _ = impl._decompress_cache(cache, dtype)
    cos = torch.nn.functional.cosine_similarity(k_rot.view(-1, H_KV, D)[slots].float(), key.float(), dim=-1)
    assert cos.min() > 0.95


def test_paged_decompress_dedup_remap_and_overflow(backend, caplog):
    pr = Prims(D)
    impl = make_impl(backend, fused=False, max_prefill_len=64)  # room for 4 blocks
    seq_lens = [40, 17, 64]
    case = build_paged_case(seq_lens, H_KV, D, BS, pr, seed=19, padded=True, extra_blocks=20)
    cache = case["cache"].cuda()
    impl._init_cg_buffers(cache, compute_dtype=torch.float16)
    assert impl._max_prefill_blocks == 4
    k_full, v_full = impl._decompress_cache(cache, torch.float16, apply_rotation=False)

    # (a) two sequences sharing a prefix block: the block is decompressed once
    bt = case["block_table"].clone()
    bt[1, 0] = bt[0, 0]
    sl = torch.tensor([40, 17], dtype=torch.int32)
    kp, vp, remap = impl._decompress_cache_paged(cache, bt[:2].cuda(), sl.cuda(), torch.float16,
                                                  out_k=impl._cg_prefill_k, out_v=impl._cg_prefill_v)
    used = sorted({int(bt[0, 0]), int(bt[0, 1]), int(bt[0, 2]), int(bt[1, 0]), int(bt[1, 1])})
    assert len(used) == 4  # five referenced entries, one block shared
    assert kp.shape == (len(used), BS, H_KV, D) and remap.dtype == torch.int32
    assert kp.data_ptr() == impl._cg_prefill_k.data_ptr()  # the pre-allocated buffer was used
    for i, s in enumerate(sl.tolist()):
        for j in range((s + BS - 1) // BS):
            assert torch.equal(kp[int(remap[i, j])], k_full[int(bt[i, j])])
            assert torch.equal(vp[int(remap[i, j])], v_full[int(bt[i, j])])
    # compact indices follow the sorted unique block ids
    assert [int(remap[0, j]) for j in range(3)] == [used.index(int(bt[0, j])) for j in range(3)]

    # (b) more unique blocks than the pre-allocated capacity: dynamic buffers + a warning
    sl3 = torch.tensor(seq_lens, dtype=torch.int32)
    with caplog.at_level(logging.WARNING, logger="turboquant_vllm.vllm.tq4_backend"):
        kp, vp, remap = impl._decompress_cache_paged(cache, case["block_table"].cuda(), sl3.cuda(), torch.float16,
                                                      out_k=impl._cg_prefill_k, out_v=impl._cg_prefill_v)
    assert any("exceed pre-allocated capacity" in r.message for r in caplog.records)
    assert kp.shape[0] == 3 + 2 + 4 and kp.data_ptr() != impl._cg_prefill_k.data_ptr()
    for i, s in enumerate(seq_lens):
        for j in range((s + BS - 1) // BS):
            assert torch.equal(kp[int(remap[i, j])], k_full[int(case["block_table"][i, j])])
