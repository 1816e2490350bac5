"""The hybrid decoder oracle (no reference model exists; parity unpinned) against properties that
its pinned building blocks imply: causality of the whole stack, and the linear-attention mixer
written out in numpy on top of the pinned recurrence."""
import numpy as np

import oracle_lib as O
from hybrid_weights import TINY_HYBRID, TINY_HYBRID_128, make_hybrid


def test_stack_is_causal_and_deterministic():
    for cfg in (TINY_HYBRID, TINY_HYBRID_128):
        _, deq = make_hybrid(cfg, 11)
        m = O.OracleHybrid(cfg, deq)
        ids = np.random.default_rng(0).integers(0, cfg["vocab"], 24).astype(np.uint32)
        full, lg = m.forward(ids)
        part, _ = m.forward(ids[:13])
        np.testing.assert_allclose(full[:13], part, rtol=2e-5, atol=2e-5)
        again, lg2 = m.forward(ids)
        assert np.array_equal(full, again) and np.array_equal(lg, lg2)
        np.testing.assert_allclose(lg, deq["lm_head"] @ full[-1], rtol=1e-4, atol=1e-4)
        assert np.isfinite(full).all() and np.abs(full).max() < 1e3


def test_linear_attention_layer_matches_numpy_composition():
    cfg = dict(TINY_HYBRID, n_layers=1)
    _, deq = make_hybrid(cfg, 5)
    lw = deq["layers"][0]
    assert lw["kind"] == 1
    H, GH, I = cfg["hidden"], cfg["gdn_heads"], cfg["intermediate"]
    GW = GH * 128
    ids = np.random.default_rng(2).integers(0, cfg["vocab"], 9).astype(np.uint32)
    got, _ = O.OracleHybrid(cfg, deq).forward(ids, logits=False)

    def rms(x, w):
        return (x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + cfg["rms_eps"])).astype(np.float32) * w

    x = deq["tok_embed"][ids]
    h = rms(x, lw["norm1"])
    p = h @ lw["w_mix_in"].T
    ab = h @ lw["w_ab"].T
    a, b = ab[:, :GH], ab[:, GH:]
    sp = np.where(a + lw["dt_bias"] > 20, a + lw["dt_bias"], np.log1p(np.exp(np.minimum(a + lw["dt_bias"], 20))))
    g = -np.exp(lw["A_log"]) * sp
    beta = 1 / (1 + np.exp(-b))
    o = np.zeros((ids.size, GW), np.float32)
    for j in range(GH):
        q = p[:, j * 128:(j + 1) * 128].copy()
        k = p[:, GW + j * 128:GW + (j + 1) * 128].copy()
        v = p[:, 2 * GW + j * 128:2 * GW + (j + 1) * 128]
        z = p[:, 3 * GW + j * 128:3 * GW + (j + 1) * 128]
        q /= np.maximum(np.linalg.norm(q, axis=-1, keepdims=True), 1e-12)
        k /= np.maximum(np.linalg.norm(k, axis=-1, keepdims=True), 1e-12)
        S = np.zeros((128, 128), np.float64)
        for t in range(ids.size):
            S *= np.exp(g[t, j])
            S += np.outer(k[t], beta[t, j] * (v[t] - k[t] @ S))
            o[t, j * 128:(j + 1) * 128] = (q[t] @ S) / np.sqrt(128.0) * (z[t] / (1 + np.exp(-z[t])))
    x = x + o @ lw["w_mix_out"].T
    h = rms(x, lw["norm2"])
    gate, up = h @ lw["w_gate"].T, h @ lw["w_up"].T
    x = x + ((gate / (1 + np.exp(-gate))) * up) @ lw["w_down"].T
    want = rms(x, deq["final_norm"])
    np.testing.assert_allclose(got, want, rtol=2e-3, atol=2e-3)
