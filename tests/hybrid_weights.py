"""Seeded random weights for the hybrid decoder stack (gated-delta-rule linear-attention layers and
gated full-attention layers), int4 group-32 quantised, in the two layouts the tests need: the
(codes, scales) pairs the GPU executor uploads and the dequantised fp32 matrices the CPU oracle runs."""
import numpy as np

import oracle_lib as O

# three linear-attention layers then one full-attention layer, head_dim 256 as in the serving config
TINY_HYBRID = dict(vocab=1000, hidden=512, n_layers=4, n_heads=4, n_kv_heads=2, attn_head_dim=256, gdn_heads=8,
                   intermediate=1024, max_pos=512, full_attn_interval=4, rms_eps=1e-6, rope_theta=1e6)
# alternating layers, head_dim 128, grouped-query ratio 4
TINY_HYBRID_128 = dict(vocab=1000, hidden=512, n_layers=2, n_heads=8, n_kv_heads=2, attn_head_dim=128, gdn_heads=8,
                       intermediate=512, max_pos=512, full_attn_interval=2, rms_eps=1e-6, rope_theta=1e4)
from logismos_b200.hybrid import HYBRID_SERVING  # noqa: E402,F401  (the serving-sweep architecture)


def make_hybrid(cfg, seed):
    """Returns (qw, deq): executor weights and oracle weights holding the same values."""
    rng = np.random.Generator(np.random.PCG64(seed))
    H, I, V = cfg["hidden"], cfg["intermediate"], cfg["vocab"]
    QW, KW, GW, GH = cfg["n_heads"] * cfg["attn_head_dim"], cfg["n_kv_heads"] * cfg["attn_head_dim"], cfg["gdn_heads"] * 128, cfg["gdn_heads"]

    def mat(n, k, gain=1.0):
        return rng.standard_normal((n, k), dtype=np.float32) * np.float32(gain / np.sqrt(k))

    def quant(m):
        c, s = O.int4_quantize(m)
        return (c, s), O.int4_dequant(c, s)

    def norm():
        return (1.0 + 0.1 * rng.standard_normal(H, dtype=np.float32)).astype(np.float32)

    tok = rng.standard_normal((V, H), dtype=np.float32) * np.float32(0.5)
    qw = {"tok_embed": tok, "final_norm": norm(), "layers": []}
    deq = {"tok_embed": O.bf16_round(tok), "final_norm": qw["final_norm"], "layers": []}
    qw["lm_head"], deq["lm_head"] = quant(mat(V, H))
    for l in range(cfg["n_layers"]):
        full = (l + 1) % cfg["full_attn_interval"] == 0
        ql = {"norm1": norm(), "norm2": norm()}
        dl = {"kind": 0 if full else 1, "norm1": ql["norm1"], "norm2": ql["norm2"]}
        d = {}
        if full:
            for n, rows, k in (("wq", QW, H), ("wgate", QW, H), ("wk", KW, H), ("wv", KW, H), ("wo", H, QW)):
                ql[n], d[n] = quant(mat(rows, k))
            dl["w_mix_in"] = np.ascontiguousarray(np.concatenate([d["wq"], d["wgate"], d["wk"], d["wv"]]))
        else:
            for n, rows, k in (("wq", GW, H), ("wk", GW, H), ("wv", GW, H), ("wgate", GW, H), ("wo", H, GW), ("wa", GH, H), ("wb", GH, H)):
                ql[n], d[n] = quant(mat(rows, k, 2.0 if n in ("wa", "wb") else 1.0))
            dl["w_mix_in"] = np.ascontiguousarray(np.concatenate([d["wq"], d["wk"], d["wv"], d["wgate"]]))
            dl["w_ab"] = np.ascontiguousarray(np.concatenate([d["wa"], d["wb"]]))
            ql["A_log"] = np.log(rng.uniform(0.5, 4.0, GH)).astype(np.float32)
            ql["dt_bias"] = rng.uniform(-3.0, 0.0, GH).astype(np.float32)
            dl["A_log"], dl["dt_bias"] = ql["A_log"], ql["dt_bias"]
        dl["w_mix_out"] = d["wo"]
        for n, rows, k in (("w_gate", I, H), ("w_up", I, H), ("w_down", H, I)):
            ql[n], dl[n] = quant(mat(rows, k))
        qw["layers"].append(ql)
        deq["layers"].append(dl)
    return qw, deq
