"""Seeded synthetic weights and inputs of the benchmark configurations (no checkpoint or dataset is
needed anywhere on this path): the Stella-architecture encoder weights and ragged id batches, and
random int4 group-32 weights for the Qwen2-style decoder stack. The hybrid decoder's generator lives
beside its model (``hybrid.random_int4_weights``), the serving load in ``serving.synthetic_load``.

Stella weights follow the benchmark configuration: every matrix and bias N(0, 0.02) from one numpy
PCG64 stream, norm gains 1. The same fp32 draw feeds a CPU reference (fp32) and the GPU path (cast
to bf16).
"""
from __future__ import annotations

import numpy as np

# StellaConfig::stella_1_5b (crates/encoders/src/stella.rs:67-80) plus the 1024-wide dense head
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


def random_int4_decoder_weights(cfg, seed):
    """Random int4 group-32 weights of the Qwen2-style decoder stack in the layout
    ``decoder.DecoderModel`` takes: uniform codes, |N(0, 0.02)| fp16 scales (the quantized-GEMV
    benchmark's distribution), zero biases, unit norm gains. The layers share their host arrays; every
    layer still gets its own copy on the device."""
    rng = np.random.Generator(np.random.PCG64(seed))
    h, inter = cfg["hidden"], cfg["intermediate"]
    kv = cfg["n_kv_heads"] * (h // cfg["n_heads"])

    def qmat(n, k):
        return (rng.integers(0, 256, (n, k // 2), dtype=np.uint8),
                np.abs(rng.standard_normal((n, k // 32), dtype=np.float32) * 0.02).astype(np.float16))

    layer = {"norm1": np.ones(h, np.float32), "norm2": np.ones(h, np.float32), "bq": np.zeros(h, np.float32),
             "bk": np.zeros(kv, np.float32), "bv": np.zeros(kv, np.float32), "wq": qmat(h, h), "wk": qmat(kv, h), "wv": qmat(kv, h),
             "wo": qmat(h, h), "w_gate": qmat(inter, h), "w_up": qmat(inter, h), "w_down": qmat(h, inter)}
    return {"tok_embed": rng.standard_normal((cfg["vocab"], h), dtype=np.float32) * np.float32(0.02), "final_norm": np.ones(h, np.float32),
            "layers": [layer] * cfg["n_layers"], "lm_head": qmat(cfg["vocab"], h)}
