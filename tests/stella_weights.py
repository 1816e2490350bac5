"""Seeded synthetic Stella-architecture weights and ragged id batches (test/bench helper).

Weights follow the benchmark configuration: every matrix and bias N(0, 0.02) from one
numpy PCG64 stream, norm gains 1. The same fp32 draw feeds the CPU oracle (fp32) and the GPU
path (cast to bf16).
"""
import numpy as np

STELLA_1_5B = dict(vocab=151646, hidden=1536, n_layers=28, n_heads=12, n_kv_heads=2,
                   intermediate=8960, max_pos=32768, head_out_dim=1024, rms_eps=1e-6,
                   rope_theta=1e6)

# Stella structure at small dims; head_dim stays 128 (what the GPU kernels support), GQA 2:1
TINY = dict(vocab=1000, hidden=512, n_layers=2, n_heads=4, n_kv_heads=2, intermediate=1024,
            max_pos=512, head_out_dim=128, rms_eps=1e-6, rope_theta=1e6)


def make_weights(cfg, seed, std=0.02):
    rng = np.random.Generator(np.random.PCG64(seed))
    h, inter = cfg["hidden"], cfg["intermediate"]
    kvw = cfg["n_kv_heads"] * (h // cfg["n_heads"])

    def mat(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std))

    w = {"tok_embed": mat(cfg["vocab"], h), "final_norm": np.ones(h, np.float32), "layers": []}
    for _ in range(cfg["n_layers"]):
        w["layers"].append({
            "norm1": np.ones(h, np.float32), "norm2": np.ones(h, np.float32),
            "wq": mat(h, h), "bq": mat(h), "wk": mat(kvw, h), "bk": mat(kvw),
            "wv": mat(kvw, h), "bv": mat(kvw), "wo": mat(h, h),
            "w_gate": mat(inter, h), "w_up": mat(inter, h), "w_down": mat(h, inter)})
    w["head_w"] = mat(cfg["head_out_dim"], h)
    w["head_b"] = mat(cfg["head_out_dim"])
    return w


def make_batch(cfg, seed, n_seq=8, lo=32, hi=512):
    """Token ids uniform over the vocabulary, lengths uniform in [lo, hi]; returns (ids, cu_seqlens)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    lens = rng.integers(lo, hi + 1, size=n_seq)
    cu = np.zeros(n_seq + 1, np.int32)
    cu[1:] = np.cumsum(lens)
    ids = rng.integers(0, cfg["vocab"], size=int(cu[-1]), dtype=np.uint32)
    return ids, cu


def quantize_weights(cfg, w, seed_lm=5):
    """int4 group-32 version of a Stella-architecture weight dict, for the decoder executor.

    Returns (qw, deq): ``qw`` in the layout logismos_b200.decoder.DecoderModel takes, and ``deq``, the
    fp32 weight dict holding exactly the dequantised values (what the CPU oracle runs on), plus
    ``deq['lm_head']`` fp32 [vocab, hidden]."""
    import oracle_lib as O
    rng = np.random.Generator(np.random.PCG64(seed_lm))
    lm = rng.standard_normal((cfg["vocab"], cfg["hidden"]), dtype=np.float32) * np.float32(0.02)
    qw = {"tok_embed": w["tok_embed"], "final_norm": w["final_norm"], "layers": []}
    deq = {"tok_embed": O.bf16_round(w["tok_embed"]), "final_norm": w["final_norm"], "layers": [],
           "head_w": w["head_w"], "head_b": w["head_b"]}
    c, s = O.int4_quantize(lm)
    qw["lm_head"] = (c, s)
    deq["lm_head"] = O.int4_dequant(c, s)
    for lw in w["layers"]:
        ql = {n: lw[n] for n in ("norm1", "norm2", "bq", "bk", "bv")}
        dl = dict(ql)
        for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down"):
            c, s = O.int4_quantize(lw[n])
            ql[n] = (c, s)
            dl[n] = O.int4_dequant(c, s)
        qw["layers"].append(ql)
        deq["layers"].append(dl)
    return qw, deq
