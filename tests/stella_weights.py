"""Seeded synthetic Stella-architecture weights for the tests: the generators of
``logismos_b200.synthetic`` (shared with the benchmark) plus the int4 quantisation of a weight set
through the CPU oracle."""
import numpy as np

from logismos_b200.synthetic import STELLA_1_5B, TINY, make_batch, make_weights  # noqa: F401


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
