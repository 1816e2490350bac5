"""Oracle pins for TurboQuant packing, int4 group-32, KV caches, GDN, greedy and the fp16 refs.
Known-answer cases cite the reference test they mirror."""
import numpy as np
import pytest

import oracle_lib as O


# ---- crates/quant/src/lib.rs ---------------------------------------------------------------------

def test_turbo4_pack_matches_golden_pattern():  # lib.rs:552-564
    idx = np.arange(32) % 16
    expected = [0x10, 0x32, 0x54, 0x76, 0x98, 0xba, 0xdc, 0xfe] * 2
    assert O.pack_turbo4(idx).tolist() == expected
    assert O.unpack_turbo4(expected).tolist() == idx.tolist()


def test_turbo3_pack_matches_golden_pattern():  # lib.rs:538-549
    idx = np.arange(32) % 8
    expected = [0x88, 0xc6, 0xfa] * 4
    assert O.pack_turbo3(idx).tolist() == expected
    assert O.unpack_turbo3(expected).tolist() == idx.tolist()


def test_pack_rejects_out_of_range_index():  # lib.rs:567-590
    bad = np.zeros(32, np.uint8); bad[5] = 8
    with pytest.raises(ValueError):
        O.pack_turbo3(bad)
    bad[5] = 16
    with pytest.raises(ValueError):
        O.pack_turbo4(bad)


def test_int4_nibble_order_is_the_turbo4_order():
    codes = ((np.arange(64) % 16) - 8).astype(np.int8).reshape(2, 32)
    packed = O.int4_pack(codes)
    for r in range(2):
        t4 = O.pack_turbo4((codes[r].astype(np.int16) & 0xF).astype(np.uint8))
        assert packed[r].tolist() == t4.tolist()
    assert (O.int4_unpack(packed) == codes).all()
    with pytest.raises(ValueError):
        O.int4_pack(np.full((1, 32), 8, np.int8))


def test_int4_gemv_equals_linear_t_on_dequantised_weight():
    rng = np.random.default_rng(3)
    n, k, b = 48, 256, 5
    codes = rng.integers(-8, 8, (n, k)).astype(np.int8)
    scales = np.abs(rng.standard_normal((n, k // 32)) * 0.02).astype(np.float16)
    packed = O.int4_pack(codes)
    w = O.int4_dequant(packed, scales.view(np.uint16))
    assert (w == codes.astype(np.float32) * np.repeat(scales.astype(np.float32), 32, 1)).all()
    x = rng.standard_normal((b, k)).astype(np.float32)
    y = O.int4_gemv(packed, scales.view(np.uint16), x)
    ref = O.linear_t(x, w, None, b, n, k).reshape(b, n)
    assert np.abs(y - ref).max() < 1e-5


def test_int4_quantize_roundtrip_error_bound():
    rng = np.random.default_rng(4)
    w = (rng.standard_normal((16, 128)) * 0.02).astype(np.float32)
    packed, scales = O.int4_quantize(w)
    d = O.int4_dequant(packed, scales)
    s = np.repeat(scales.view(np.float16).astype(np.float32), 32, 1)
    assert (np.abs(d - w) <= 0.5 * s + 1e-9).all()
    codes = O.int4_unpack(packed)
    assert codes.min() >= -8 and codes.max() <= 7


# ---- crates/cache/src/flat.rs ---------------------------------------------------------------------

def test_flat_cache_roundtrip_and_errors():  # flat_tests.rs:30-260
    c = O.FlatKvCache(2, 24, 8)  # F32 x 2 heads x 3 head_dim, max_seq 8
    k = np.arange(12, dtype=np.float32).reshape(2, 6); v = -k
    c.put(0, k, v)
    assert c.len_of(0) == 2 and c.len_of(1) == 0 and c.len_of(2) is None
    c.put(0, k[:1] + 100, v[:1])
    gk, gv = c.get(0, 3)
    assert (gk.view(np.float32).reshape(3, 6) == np.vstack([k, k[:1] + 100])).all()
    assert (gv.view(np.float32).reshape(3, 6) == np.vstack([v, v[:1]])).all()
    assert c.get(0, 0)[0].shape[0] == 0
    with pytest.raises(ValueError, match="ReadBeyondWritten"):
        c.get(0, 4)
    with pytest.raises(ValueError, match="LayerOutOfRange"):
        c.put(2, k, v)
    with pytest.raises(ValueError, match="LenOverflow"):
        c.put(1, np.zeros((9, 6), np.float32), np.zeros((9, 6), np.float32))
    c.reset()
    assert c.len_of(0) == 0


def test_little_endian_row_encoding_pins():  # flat_tests.rs:376-404
    assert np.array([1.0], np.float32).view(np.uint8).tolist() == [0x00, 0x00, 0x80, 0x3F]
    assert np.array([0x01020304], np.int32).view(np.uint8).tolist() == [0x04, 0x03, 0x02, 0x01]
    assert np.array([1.0], np.float16).view(np.uint8).tolist() == [0x00, 0x3C]
    assert O.to_bf16_bits(np.array([1.0], np.float32)).view(np.uint8).tolist() == [0x80, 0x3F]


def test_bf16_conversion_is_round_to_nearest_even():
    import torch
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    x[:4] = [1.00390625, 1.01171875, -0.0, 3.3895314e38]
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert (O.to_bf16_bits(x) == want).all()


def test_paged_cache_equals_flat_cache_for_the_same_puts():
    rng = np.random.default_rng(8)
    bs, row, n_blocks = 16, 512, 12
    kp = np.zeros((n_blocks, bs, row), np.uint8); vp = np.zeros_like(kp)
    table = rng.permutation(n_blocks)[:5].astype(np.int32)
    flat = O.FlatKvCache(1, row, 80)
    for t in range(70):
        kr = rng.integers(0, 256, row, dtype=np.uint8); vr = rng.integers(0, 256, row, dtype=np.uint8)
        flat.put(0, kr[None], vr[None])
        O.paged_append(kp, vp, bs, table, t, kr, vr)
    for n in (0, 1, 16, 17, 70):
        fk, fv = flat.get(0, n)
        pk, pv = O.paged_gather(kp, vp, bs, table, n)
        assert (fk == pk).all() and (fv == pv).all()
    with pytest.raises(ValueError):
        O.paged_append(kp, vp, bs, table, 5 * bs, kp[0, 0], kp[0, 0])  # beyond the table
    with pytest.raises(ValueError):
        O.paged_gather(kp, vp, bs, np.array([99], np.int32), 1)  # bad block id


def test_decode_attention_is_last_row_of_causal_attention():
    rng = np.random.default_rng(9)
    hidden, nh, nkv, d, S = 64, 4, 2, 16, 19
    w = {n: (rng.standard_normal(s) * 0.3).astype(np.float32) for n, s in
         dict(wq=(hidden, hidden), bq=(hidden,), wk=(nkv * d, hidden), bk=(nkv * d,),
              wv=(nkv * d, hidden), bv=(nkv * d,)).items()}
    w["wo"] = np.eye(hidden, dtype=np.float32)  # identity o_proj exposes the merged heads
    x = rng.standard_normal((S, hidden)).astype(np.float32)
    cos, sin = O.build_rope_table_f32(32, d, 1e4)
    full = O.attention_forward(w, hidden, nh, nkv, d, x, np.ones(S, np.uint8), cos, sin, 32, causal=True)
    q = O.linear_t(x, w["wq"], w["bq"], S, hidden, hidden)
    k = O.linear_t(x, w["wk"], w["bk"], S, nkv * d, hidden)
    v = O.linear_t(x, w["wv"], w["bv"], S, nkv * d, hidden).reshape(S, nkv * d)
    cq, sq = O.rope_gather(cos, sin, 32, d, np.repeat(np.arange(S), nh))
    ck, sk = O.rope_gather(cos, sin, 32, d, np.repeat(np.arange(S), nkv))
    O.rope_halves_in_place(q, cq, sq, S * nh, d); O.rope_halves_in_place(k, ck, sk, S * nkv, d)
    out = O.decode_attention(q.reshape(S, hidden)[-1], k.reshape(S, nkv * d), v, nh, nkv, d)
    assert np.abs(out - full[-1]).max() < 1e-5


def test_build_packing_equals_per_sequence_indices():
    rng = np.random.default_rng(10)
    bs, n_pool = 16, 64
    cached = np.array([0, 37, 16, 255], np.int32); new = np.array([20, 1, 1, 3], np.int32)
    perm = rng.permutation(n_pool).astype(np.int32)
    tables = -np.ones((4, 17), np.int32); o = 0
    for i in range(4):
        nb = -(-(cached[i] + new[i]) // bs)
        tables[i, :nb] = perm[o:o + nb]; o += nb
    cu, pos, slots, sid = O.build_packing(cached, new, tables, bs, n_pool)
    assert cu.tolist() == [0, 20, 21, 22, 25]
    for i in range(4):
        p = np.arange(cached[i], cached[i] + new[i])
        assert pos[cu[i]:cu[i + 1]].tolist() == p.tolist()
        assert slots[cu[i]:cu[i + 1]].tolist() == (tables[i, p // bs].astype(np.int64) * bs + p % bs).tolist()
        assert (sid[cu[i]:cu[i + 1]] == i).all()
    assert len(set(slots.tolist())) == slots.size
    tables[3, 15] = -1
    with pytest.raises(ValueError):
        O.build_packing(cached, new, tables, bs, n_pool)


# ---- crates/kernels/src/gated_delta_rule/cpu.rs ---------------------------------------------------

def test_l2_norm_rows():  # cpu.rs:264-286
    x = np.array([1, 0, 0, 1], np.float32); O.l2_norm_rows(x, 2)
    assert np.abs(x - [1, 0, 0, 1]).max() < 1e-6
    x = np.array([3, 4], np.float32); O.l2_norm_rows(x, 2)
    assert np.abs(x - [0.6, 0.8]).max() < 1e-6
    x = np.zeros(4, np.float32); O.l2_norm_rows(x, 2)
    assert np.isfinite(x).all()


def test_cumsum_basic():  # cpu.rs:289-293
    assert O.cumsum([1, 2, 3]).tolist() == [1, 3, 6]


def test_recurrent_zero_beta_preserves_state():  # cpu.rs:296-313
    t, kd, vd = 3, 2, 2
    o, s = O.gdn_recurrent_fwd(np.ones(t * kd), np.ones(t * kd), np.ones(t * vd), np.zeros(t), np.zeros(t), 1.0,
                               np.full(kd * vd, 2.0), kd, vd)
    assert np.abs(s - 2.0).max() < 1e-6


def test_recurrent_hand_computed_single_step():  # cpu.rs:316-332 (values derived by hand)
    o, s = O.gdn_recurrent_fwd(np.zeros(2), np.ones(2), np.ones(2), [1.0], [0.0], 1.0, np.zeros(4), 2, 2)
    assert np.isfinite(o).all() and s.tolist() == [1, 1, 1, 1] and o.tolist() == [0, 0]
    # with a query: o[v] = sum_k h[k,v] q[k] * scale
    o, s = O.gdn_recurrent_fwd([1.0, 2.0], np.ones(2), [1.0, 3.0], [0.5], [np.log(0.5)], 0.5, np.full(4, 2.0), 2, 2)
    # decay -> h = 1; h^T k = [2,2]; vd = 0.5*([1,3]-[2,2]) = [-0.5,0.5]; h = [[0.5,1.5],[0.5,1.5]]
    assert np.abs(s - [0.5, 1.5, 0.5, 1.5]).max() < 1e-6
    assert np.abs(o - [0.75, 2.25]).max() < 1e-6


def test_chunk_fwd_matches_recurrent():  # cpu.rs:352-402
    rng = np.random.default_rng(11)
    t, kd, vd = 37, 8, 6
    q, k = rng.standard_normal((2, t * kd)).astype(np.float32) * 0.3
    v = rng.standard_normal(t * vd).astype(np.float32)
    beta = rng.uniform(0, 1, t).astype(np.float32); g = -rng.uniform(0, 0.2, t).astype(np.float32)
    s0 = rng.standard_normal(kd * vd).astype(np.float32)
    o1, s1 = O.gdn_recurrent_fwd(q, k, v, beta, g, 0.35, s0, kd, vd)
    o2, st = O.gdn_chunk_fwd(q, k, v, beta, g, 0.35, s0, kd, vd, 8)
    assert st.shape[0] == 5 and np.abs(o1 - o2).max() < 1e-5 and np.abs(st[-1] - s1).max() < 1e-5
    o3, st3 = O.gdn_chunk_fwd(q, k, v, beta, g, 0.35, s0, kd, vd, t)
    assert np.abs(o1 - o3).max() < 1e-5 and st3.shape[0] == 1


def test_gdn_gates():
    a = np.array([[0.0, 30.0]], np.float32); b = np.array([[0.0, 2.0]], np.float32)
    g, beta = O.gdn_gates(a, b, np.array([0.0, np.log(2.0)], np.float32), np.array([0.0, 0.0], np.float32))
    assert abs(g[0, 0] + np.log(2.0)) < 1e-6 and abs(g[0, 1] + 60.0) < 1e-4
    assert abs(beta[0, 0] - 0.5) < 1e-7 and abs(beta[0, 1] - 1 / (1 + np.exp(-2.0))) < 1e-6


# ---- crates/decode/src/lib.rs ---------------------------------------------------------------------

def test_greedy_returns_first_max_index():  # lib.rs:90-92
    assert O.greedy([0.0, 2.0, 2.0]) == 1
    assert O.greedy([np.nan, 1.0, np.nan]) == 1
    assert O.greedy([-np.inf, -np.inf]) == 0


# ---- fp16 references ------------------------------------------------------------------------------

def test_fp16_refs():
    rng = np.random.default_rng(12)
    eye = np.eye(4, dtype=np.float16); a = rng.uniform(-1, 1, (4, 4)).astype(np.float16)
    assert (O.matmul_fp16_ref(a, eye, 4, 4, 4) == a).all()  # matmul/cpu.rs identity_matmul
    y = O.rms_norm_fp16_ref(np.array([1, 2, 3, 4], np.float16), np.ones(4, np.float16), 1, 4, 1e-6)
    assert np.abs(y.astype(np.float32) - np.array([1, 2, 3, 4]) / np.sqrt(7.5)).max() < 5e-3  # rms_norm/cpu.rs
    x = (np.arange(10) / 3.0).astype(np.float16)
    sm = O.softmax_fp16_ref(x, 2, 5)
    assert np.abs(sm.astype(np.float32).sum(1) - 1).max() < 1e-2  # softmax/cpu.rs row_sums_to_one
    with pytest.raises(ValueError):
        O.softmax_fp16_ref(np.ones(9, np.float16), 2, 5)
    assert np.abs(O.softmax_fp16_ref(np.full(4, -np.inf, np.float16), 1, 4).astype(np.float32) - 0.25).max() < 1e-3
    t = O.build_cos_sin_table(1, 4, 10_000.0)
    assert np.abs(t - [1, 0, 1, 0]).max() < 1e-6  # rope/cpu.rs zero_positions_are_identity
    qk = np.array([1, 2, 3, 4], np.float16)
    O.rope_apply_fp16_ref(qk, t, 1, 1, 1, 4)
    assert qk.tolist() == [1, 2, 3, 4]
    with pytest.raises(ValueError):
        O.rope_apply_fp16_ref(np.ones(7, np.float16), t, 1, 1, 1, 4)


def test_turbo3_head_codec_reference_properties():
    """crates/quant/src/lib.rs:658-697: the transform is an involution and preserves the norm; the
    reference's round-trip vector stays under its MSE bound; block layout: the fp16 norm, little-endian,
    repeated in each of the four 14-byte blocks."""
    i = np.arange(128, dtype=np.float32)
    d = (np.sin(i) * 0.5).astype(np.float32)
    assert np.abs(O.fwht_128(O.fwht_128(d)) - d).max() < 1e-5
    c = (np.cos(i) * 0.3).astype(np.float32)
    assert abs(np.linalg.norm(O.fwht_128(c)) - np.linalg.norm(c)) < 1e-5
    src = (np.sin(i * 0.1) * 0.1 + np.cos(i * 0.03) * 0.1).astype(np.float32)
    blocks = O.turbo3_encode(src)
    assert blocks.shape == (56,)
    dec = O.turbo3_decode(blocks)
    assert np.mean((src - dec) ** 2) < 0.05
    norm_bits = np.float16(np.sqrt(np.sum(src.astype(np.float32) ** 2, dtype=np.float32))).view(np.uint16)
    for b in range(4):
        assert blocks[14 * b] == norm_bits & 0xff and blocks[14 * b + 1] == norm_bits >> 8
    # indices come back through the pinned 3-bit packing
    idx = np.concatenate([O.unpack_turbo3(blocks[14 * b + 2:14 * b + 14]) for b in range(4)])
    assert idx.max() <= 7 and idx.shape == (128,)
    # an all-zero chunk: norm 0, the transform of zeros picks the centroid nearest to 0, decode gives zeros
    z = O.turbo3_decode(O.turbo3_encode(np.zeros(128, np.float32)))
    assert (z == 0).all()
