"""Oracle pins for attention / MLP / Stella composition.

Known-answer cases mirror crates/transformers/src/attention.rs tests (:430-520) and
crates/transformers/src/rope.rs tests (:104-125); the end-to-end pin is the committed golden
fixture produced with the reference's own golden method (HF Qwen2Model fp32 with a padding-only
mask, phases/03-stella/golden/generate.py), gated as the reference gates its Rust path
(crates/logismos/tests/phase_3_stella_parity.rs:132: max abs <= 1e-3 and cos > 0.999).
"""
import os

import numpy as np
import pytest

import oracle_lib as O
from stella_weights import TINY, make_weights

GOLD = os.path.join(os.path.dirname(__file__), "golden", "stella_tiny_hf.npz")


def test_transpose_roundtrips():  # attention.rs:430-438
    x = np.arange(12, dtype=np.float32)
    t = O.transpose_seq_heads(x, 3, 2, 2)
    assert O.merge_heads(t, 2, 3, 2).tolist() == x.tolist()
    assert t.tolist() == [0, 1, 4, 5, 8, 9, 2, 3, 6, 7, 10, 11]


def test_repeat_kv_basic():  # attention.rs:441-455
    rep = O.repeat_kv(np.array([1, 2, 10, 20], np.float32), 2, 3, 1, 2)
    assert rep.tolist() == [1, 2, 1, 2, 1, 2, 10, 20, 10, 20, 10, 20]


def test_rope_gather_rejects_out_of_range_position():  # rope.rs:104-125
    cos, sin = O.build_rope_table_f32(4, 8, 1e6)
    c, s = O.rope_gather(cos, sin, 4, 8, [3, 0])
    assert c[:4].tolist() == cos[12:16].tolist() and s[4:].tolist() == sin[0:4].tolist()
    with pytest.raises(ValueError):
        O.rope_gather(cos, sin, 4, 8, [4])


def test_forward_with_fully_masked_row_returns_finite_output():  # attention.rs:487-520
    w = dict(wq=np.full(16, 0.1), bq=np.zeros(4), wk=np.full(8, 0.1), bk=np.zeros(2),
             wv=np.full(8, 0.1), bv=np.zeros(2), wo=np.full(16, 0.1))
    cos, sin = O.build_rope_table_f32(1, 2, 1e6)
    out = O.attention_forward(w, 4, 2, 1, 2, np.array([1, 2, 3, 4], np.float32), [0], cos, sin, 1)
    assert np.isfinite(out).all()


def test_forward_rejects_seq_beyond_rope_table():  # attention.rs:151-159
    w = dict(wq=np.zeros(16), bq=np.zeros(4), wk=np.zeros(8), bk=np.zeros(2), wv=np.zeros(8),
             bv=np.zeros(2), wo=np.zeros(16))
    cos, sin = O.build_rope_table_f32(1, 2, 1e6)
    with pytest.raises(ValueError):
        O.attention_forward(w, 4, 2, 1, 2, np.zeros(8, np.float32), [1, 1], cos, sin, 1)


def _naive_attention(w, hidden, nh, nkv, d, x, mask, theta, causal):
    """Independent float64 numpy restatement (HF convention) to cross-check the C++ oracle."""
    x = x.astype(np.float64); S = x.shape[0]
    q = x @ w["wq"].astype(np.float64).T + w["bq"]
    k = x @ w["wk"].astype(np.float64).T + w["bk"]
    v = x @ w["wv"].astype(np.float64).T + w["bv"]
    q = q.reshape(S, nh, d); k = k.reshape(S, nkv, d); v = v.reshape(S, nkv, d)
    inv = theta ** (-(2.0 * np.arange(d // 2)) / d)
    ang = np.arange(S)[:, None] * inv[None]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]

    def rope(t):
        a, b = t[..., : d // 2], t[..., d // 2:]
        return np.concatenate([a * c - b * s, a * s + b * c], -1)

    q, k = rope(q), rope(k)
    out = np.zeros((S, nh, d))
    for h in range(nh):
        kh = h // (nh // nkv)
        sc = q[:, h] @ k[:, kh].T / np.sqrt(d)
        allow = np.broadcast_to(np.asarray(mask, bool)[None, :], (S, S)).copy()
        if causal:
            allow &= np.tril(np.ones((S, S), bool))
        sc = np.where(allow, sc, -np.inf)
        sc = sc - sc.max(1, keepdims=True)
        p = np.exp(sc); p /= p.sum(1, keepdims=True)
        out[:, h] = p @ v[:, kh]
    return out.reshape(S, hidden) @ w["wo"].astype(np.float64).T


@pytest.mark.parametrize("causal", [False, True])
def test_attention_matches_independent_float64(causal):
    rng = np.random.default_rng(5)
    hidden, nh, nkv, d, S = 96, 6, 2, 16, 23
    w = {n: (rng.standard_normal(s) * 0.2).astype(np.float32) for n, s in
         dict(wq=(hidden, hidden), bq=(hidden,), wk=(nkv * d, hidden), bk=(nkv * d,),
              wv=(nkv * d, hidden), bv=(nkv * d,), wo=(hidden, hidden)).items()}
    x = rng.standard_normal((S, hidden)).astype(np.float32)
    mask = np.ones(S, np.uint8); mask[[3, 17]] = 0
    cos, sin = O.build_rope_table_f32(64, d, 1e4)
    got = O.attention_forward(w, hidden, nh, nkv, d, x, mask, cos, sin, 64, causal=causal)
    want = _naive_attention(w, hidden, nh, nkv, d, x, mask, 1e4, causal)
    assert np.abs(got - want).max() < 2e-5 * max(1, np.abs(want).max())


def test_swiglu_matches_float64():
    rng = np.random.default_rng(6)
    h, inter, S = 48, 112, 9
    wg, wu, wd = (rng.standard_normal(s).astype(np.float32) * 0.2 for s in ((inter, h), (inter, h), (h, inter)))
    x = rng.standard_normal((S, h)).astype(np.float32)
    g = x.astype(np.float64) @ wg.T.astype(np.float64); u = x.astype(np.float64) @ wu.T.astype(np.float64)
    want = (g / (1 + np.exp(-g)) * u) @ wd.T.astype(np.float64)
    assert np.abs(O.swiglu_forward(wg, wu, wd, h, inter, x) - want).max() < 1e-5


def test_stella_oracle_matches_hf_golden_fixture():
    g = np.load(GOLD)
    w = make_weights(TINY, int(g["seed_w"]))
    m = O.OracleStella(TINY, w)
    ids, cu = g["ids"], g["cu_seqlens"]
    for i in range(len(cu) - 1):
        s = ids[cu[i]:cu[i + 1]]
        emb = m.encode_raw(s)
        want = g["embeddings"][i]
        assert np.abs(emb - want).max() <= 1e-3
        assert float(emb @ want) / (np.linalg.norm(emb) * np.linalg.norm(want)) > 0.999
        # far tighter than the reference's own gate in practice
        assert np.abs(emb - want).max() <= 2e-5
        hs = m.forward(s)
        assert np.abs(hs[-1] - g["last_token_hidden"][i]).max() <= 1e-3
    batch = m.encode_batch(ids, cu, n_threads=3)
    assert np.abs(batch - g["embeddings"]).max() <= 2e-5


def test_stella_forward_rejects_bad_inputs():  # encoders/src/stella.rs:279-295
    w = make_weights(TINY, 1)
    m = O.OracleStella(TINY, w)
    with pytest.raises(ValueError):
        m.forward(np.zeros(4, np.uint32), np.ones(3, np.uint8))
    with pytest.raises(ValueError):
        m.forward(np.zeros(TINY["max_pos"] + 1, np.uint32))


def test_out_of_range_token_id_embeds_as_zero_row():  # cpu_f32/mod.rs:96-104
    w = make_weights(TINY, 1)
    m = O.OracleStella(TINY, w)
    a = m.forward(np.array([5, TINY["vocab"] + 7, 9], np.uint32))
    assert np.isfinite(a).all()


def test_count_physical_cores_rule():  # embed/src/stella.rs:470-500
    two_sockets = "".join(f"processor\t: {i}\nphysical id\t: {i // 4}\ncore id\t: {i % 2}\n\n" for i in range(8))
    assert O.count_physical_cores_text(two_sockets) == 4
    no_socket = "".join(f"processor\t: {i}\ncore id\t: {i // 2}\n\n" for i in range(8))
    assert O.count_physical_cores_text(no_socket) == 4
    assert O.count_physical_cores_text("processor\t: 0\n\n") == 0
    assert O.count_physical_cores_text("processor\t: 0\nphysical id\t: 0\ncore id\t: 3") == 1
    assert O.physical_cores() >= 1
