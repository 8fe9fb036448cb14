"""Pin the CPU oracle against golden vectors produced by the reference implementation."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import tq4_oracle as O


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


@pytest.mark.parametrize("d", [64, 96, 128, 256])
@pytest.mark.parametrize("bits", [2, 3, 4])
def test_codebook_bit_exact(golden, d, bits):
    g = golden("codebooks.npz")
    c, b = O.solve_lloyd_max(d, bits)
    assert np.array_equal(c.numpy(), g[f"c_{d}_{bits}"])
    assert np.array_equal(b.numpy(), g[f"b_{d}_{bits}"])


def test_codebook_known_answers():
    c, b = O.solve_lloyd_max(128, 4)
    ref = [0.010850, 0.032771, 0.055385, 0.079279, 0.105281, 0.134743, 0.170284, 0.218535]
    assert np.allclose(c[8:].numpy(), ref, atol=5e-7)
    assert np.allclose(c[:8].numpy(), [-x for x in reversed(ref)], atol=5e-7)
    assert b[7].item() == 0.0


@pytest.mark.parametrize("d", [64, 96, 128, 256])
@pytest.mark.parametrize("seed", [42, 7])
def test_rotation_matches_reference(golden, d, seed):
    g = golden("rotations.npz")
    r = O.rotation_matrix(d, seed)
    assert np.allclose(r[0].numpy(), g[f"row0_{d}_{seed}"], atol=1e-6)
    assert np.allclose(torch.diag(r).numpy(), g[f"diag_{d}_{seed}"], atol=1e-6)
    assert np.allclose(r.double().sum(0).numpy(), g[f"colsum_{d}_{seed}"], atol=1e-5)
    assert torch.allclose(r @ r.T, torch.eye(d), atol=1e-5)
    if (d, seed) == (64, 42):
        assert np.allclose(r.numpy(), g["full_64_42"], atol=1e-6)


@pytest.mark.parametrize("d", [64, 96, 128, 256])
def test_pack_bit_exact_given_rotated(golden, d):
    """Bit-exact bytes from the reference's own rotated rows (the tie at 0.0 included)."""
    g = golden("compress.npz")
    _, b = O.solve_lloyd_max(d, 4)
    packed = O.pack_from_rotated(t(g[f"rotated_{d}"]), b)
    assert np.array_equal(packed.numpy(), g[f"packed_{d}"].reshape(-1, d // 2))


@pytest.mark.parametrize("d", [64, 96, 128, 256])
def test_compress_end_to_end(golden, d):
    g = golden("compress.npz")
    _, b = O.solve_lloyd_max(d, 4)
    rot = O.rotation_matrix(d, 42)
    packed, norms = O.compress_rows(t(g[f"x_{d}"]), rot, b)
    ref = t(g[f"packed_{d}"])
    mism = (O.nibble_unpack(packed) != O.nibble_unpack(ref)).float().mean().item()
    assert mism <= 1e-4, mism
    assert torch.equal(O.nibble_unpack(packed), t(g[f"idx_{d}"]).long().reshape(packed.shape[0], packed.shape[1], d)) or mism <= 1e-4
    assert np.array_equal(norms.numpy(), g[f"norms_{d}"])


@pytest.mark.parametrize("d", [64, 96, 128, 256])
def test_decompress_and_dequantize(golden, d):
    g = golden("compress.npz")
    c, _ = O.solve_lloyd_max(d, 4)
    rot = O.rotation_matrix(d, 42)
    dec = O.decompress_rows(t(g[f"packed_{d}"]), t(g[f"norms_{d}"]), c)
    assert np.array_equal(dec.numpy(), g[f"dec_{d}"])
    deq = O.dequantize(t(g[f"idx_{d}"]), t(g[f"norms_{d}"]), c, rot)
    assert np.allclose(deq.numpy(), g[f"deq_{d}"], rtol=1e-5, atol=1e-5)


def test_compress_fp32_input_3bit(golden):
    g = golden("compress.npz")
    _, b = O.solve_lloyd_max(128, 3)
    rot = O.rotation_matrix(128, 42)
    packed, norms = O.compress_rows(t(g["x_f32_128"]), rot, b)
    ref = t(g["packed_f32_128_b3"])
    mism = (O.nibble_unpack(packed) != O.nibble_unpack(ref)).float().mean().item()
    assert mism <= 1e-4
    assert O.nibble_unpack(packed).max() <= 7
    assert np.array_equal(norms.numpy(), g["norms_f32_128_b3"])


def test_zero_vector_tie_rule():
    """All-zero vector -> rotated == 0.0 exactly -> index 7 (count of boundaries < 0)."""
    _, b = O.solve_lloyd_max(128, 4)
    rot = O.rotation_matrix(128, 42)
    packed, norms = O.compress_rows(torch.zeros(1, 1, 128), rot, b)
    assert norms.item() == 0.0
    assert torch.all(packed == 0x77)


PAGED_TAGS = ["k4v4", "k4v3", "d96", "d64g7", "k4v4h4"]


def _paged(golden, tag):
    g = golden("paged.npz")
    d, h_kv, h_q, kb, vb, bs = [int(x) for x in g[f"{tag}_meta"]]
    kc, kbd = O.solve_lloyd_max(d, kb)
    vc, vbd = O.solve_lloyd_max(d, vb)
    rot = O.rotation_matrix(d, 42)
    return g, d, h_kv, h_q, bs, kc, kbd, vc, vbd, rot


@pytest.mark.parametrize("tag", PAGED_TAGS)
def test_paged_write_matches_reference(golden, tag):
    g, d, h_kv, h_q, bs, kc, kbd, vc, vbd, rot = _paged(golden, tag)
    ref = t(g[f"{tag}_cache"])
    cache = torch.zeros_like(ref)
    O.write_paged(t(g[f"{tag}_key"]), t(g[f"{tag}_value"]), cache, t(g[f"{tag}_slot_mapping"]),
                  rot, kbd, vbd)
    assert torch.equal(cache, ref)


@pytest.mark.parametrize("tag", PAGED_TAGS)
def test_paged_decode_matches_reference(golden, tag):
    g, d, h_kv, h_q, bs, kc, kbd, vc, vbd, rot = _paged(golden, tag)
    out = O.paged_decode_fp32(t(g[f"{tag}_q_dec"]), t(g[f"{tag}_cache"]), t(g[f"{tag}_block_table"]),
                              g[f"{tag}_seq_lens"], kc, vc, rot, h_kv)
    assert np.allclose(out.numpy(), g[f"{tag}_dec_out"], rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("tag", PAGED_TAGS)
@pytest.mark.parametrize("window", [None, 9])
def test_paged_prefill_matches_reference(golden, tag, window):
    g, d, h_kv, h_q, bs, kc, kbd, vc, vbd, rot = _paged(golden, tag)
    qsl = np.concatenate([[0], np.cumsum(g[f"{tag}_q_lens"])])
    out = O.paged_attention_fp32(t(g[f"{tag}_q_pre"]), t(g[f"{tag}_cache"]), t(g[f"{tag}_block_table"]),
                                 g[f"{tag}_seq_lens"], qsl, kc, vc, rot, h_kv, None, True, window)
    ref = g[f"{tag}_pre_out"] if window is None else g[f"{tag}_pre_out_w9"]
    assert np.allclose(out.numpy(), ref, rtol=1e-4, atol=2e-5)


def test_byte_size_known_answers(golden):
    g = golden("sizes.npz")
    assert int(g["bytes_per_token_128_4"]) == 68
    assert int(g["bytes_per_token_64_4"]) == 36
    assert int(g["bytes_per_token_128_3"]) == 132
    assert int(g["bytes_per_token_kv_128"]) == 136
    assert int(g["bytes_per_token_kv_64"]) == 72
    for d in (64, 96, 128, 256):
        assert O.padded_slot_bytes(d) == int(g[f"padded_slot_{d}"])
    assert tuple(g["cache_shape_100_16_8_128"]) == (100, 16, 8 * O.padded_slot_bytes(128))
    assert O.row_layout(8, 128) == (512, 544, 1056, 1088)


def test_config1_roundtrip_and_decode(golden):
    """CPU reference configuration: K,V fp32 [1,8,1024,128] seed 0 with outlier channels."""
    g = golden("config1.npz")
    d, h_kv, h_q, n = 128, 8, 32, 1024
    c, b = O.solve_lloyd_max(d, 4)
    rot = O.rotation_matrix(d, 42)
    k, v = O.synthetic_kv(n, h_kv, d, seed=0)
    kp, kn = O.compress_rows(k, rot, b)
    vp, vn = O.compress_rows(v, rot, b)
    assert (O.nibble_unpack(kp) != O.nibble_unpack(t(g["k_packed"]))).float().mean() <= 1e-4
    assert (O.nibble_unpack(vp) != O.nibble_unpack(t(g["v_packed"]))).float().mean() <= 1e-4
    assert np.array_equal(kn.numpy(), g["k_norms"])
    # decode through the paged oracle on a contiguous block table
    bs = 16
    cache = torch.zeros(n // bs, bs, O.row_layout(h_kv, d)[3], dtype=torch.uint8)
    O.write_paged(k, v, cache, torch.arange(n), rot, b, b)
    bt = torch.arange(n // bs, dtype=torch.int32).unsqueeze(0)
    out = O.paged_decode_fp32(t(g["q"]).unsqueeze(0), cache, bt, [n], c, c, rot, h_kv)[0]
    assert np.allclose(out.numpy(), g["out_compressed"], rtol=1e-4, atol=2e-5)
    cos = torch.nn.functional.cosine_similarity(out.flatten(), t(g["out_uncompressed"]).flatten(), dim=0)
    assert cos > 0.9


def test_lse_combine_equals_full_attention(golden):
    """Splitting the keys of every sequence over two shards and merging the shard partials
    (normalised output + log-sum-exp, rotated space) reproduces full attention."""
    g, d, h_kv, h_q, bs, kc, kbd, vc, vbd, rot = _paged(golden, "k4v4")
    q, cache, bt = t(g["k4v4_q_dec"]), t(g["k4v4_cache"]), t(g["k4v4_block_table"])
    sl = g["k4v4_seq_lens"]
    full = O.paged_decode_fp32(q, cache, bt, sl, kc, vc, rot, h_kv)
    eye = torch.eye(d)  # identity "rotation": feed pre-rotated queries, keep rotated outputs
    q_rot = q.float() @ rot.T
    qsl = torch.arange(q.shape[0] + 1)
    first = [min(int(s), 16) for s in sl]  # shard 0: keys [0, 16)
    o0, l0 = O.paged_attention_fp32(q_rot, cache, bt, first, qsl, kc, vc, eye, h_kv, None, False, None, True)
    o1 = torch.zeros_like(o0)  # shard 1: keys [16, len) = a window of len-16 at the last position
    l1 = torch.full_like(l0, float("-inf"))
    for i, s in enumerate(sl):
        if s > 16:
            oo, ll = O.paged_attention_fp32(q_rot[i:i + 1], cache, bt[i:i + 1], [int(s)], [0, 1], kc, vc,
                                            eye, h_kv, None, True, int(s) - 16, True)
            o1[i], l1[i] = oo[0], ll[0]
    merged = O.lse_combine(torch.stack([o0, o1]), torch.stack([l0, l1])) @ rot
    assert torch.allclose(merged, full, rtol=1e-4, atol=1e-5)
