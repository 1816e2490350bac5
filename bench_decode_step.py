"""Decode-step benchmark of the hybrid decoder executor on one GPU: S sequences with `ctx` cached
tokens each decode one token; the step's device work is replayed and timed with CUDA events, and
the host-buffer entry point is timed around it. Used for launch lists and per-step rooflines.

  python bench_decode_step.py [--seqs S --ctx C --layers L --iters I --prefill-chunk P --profiler-range]
  python bench_decode_step.py --prefill-step TOKENS --ctx C [--seqs S]     (one prefill step of TOKENS / C prompts)

Prints one JSON line: device ms per step, host-entry ms per step, launches per step, and the
algorithmic HBM bytes of the step (int4 weights once, recurrent states read + written, KV rows of
the contexts read).
"""
from __future__ import annotations

import argparse
import json
import time

import numpy as np
import torch

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from logismos_b200.decoder import BlockAllocator  # noqa: E402
from logismos_b200.hybrid import HYBRID_SERVING, HybridModel, random_int4_weights  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser(prog="bench_decode_step.py")
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--prefill-chunk", type=int, default=8, help="sequences prefilled per step while building the contexts")
    ap.add_argument("--profiler-range", action="store_true", help="bracket one extra untimed step with cudaProfilerStart/Stop")
    ap.add_argument("--prefill-step", type=int, default=0, metavar="TOKENS",
                    help="time one prefill step instead: TOKENS prompt tokens as sequences of --ctx tokens each, from empty caches")
    a = ap.parse_args(argv)
    cfg = dict(HYBRID_SERVING, n_layers=a.layers)
    w = random_int4_weights(cfg, 17)
    S, ctx = a.seqs, a.ctx
    max_blocks = (ctx + 64 + 15) // 16
    n_pool = S * max_blocks + 8
    model = HybridModel(cfg, w, n_pool_blocks=n_pool, max_blocks_per_seq=max_blocks, max_step_tokens=max(a.prefill_chunk * ctx, S, a.prefill_step),
                        max_step_seqs=S, n_state_slots=S)
    alloc = BlockAllocator(n_pool, max_blocks, seed=1)
    rng = np.random.Generator(np.random.PCG64(3))
    if a.prefill_step:
        n = max(1, min(S, a.prefill_step // ctx))
        tabs = np.stack([alloc.ensure(i, ctx) for i in range(n)])
        ids = rng.integers(0, cfg["vocab"], n * ctx, dtype=np.uint32)
        model.step(ids, [0] * n, [ctx] * n, tabs, list(range(n)))
        stream = torch.cuda.current_stream()
        for _ in range(3):
            model.replay_device(stream.cuda_stream)
        torch.cuda.synchronize()
        if a.profiler_range:
            torch.cuda.profiler.start()
            model.replay_device(stream.cuda_stream)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(a.iters):
            model.replay_device(stream.cuda_stream)
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.iters
        H, I = cfg["hidden"], cfg["intermediate"]
        n_full = sum((l + 1) % cfg["full_attn_interval"] == 0 for l in range(a.layers))
        QW, KW, GW, GH = cfg["n_heads"] * cfg["attn_head_dim"], cfg["n_kv_heads"] * cfg["attn_head_dim"], cfg["gdn_heads"] * 128, cfg["gdn_heads"]
        params = n_full * ((2 * QW + 2 * KW) * H + H * QW) + (a.layers - n_full) * (4 * GW * H + 2 * GH * H + H * GW) + a.layers * 3 * H * I
        print(json.dumps({"bench": "hybrid_prefill_step", "seqs": n, "tokens": n * ctx, "layers": a.layers, "device_ms_per_step": ms,
                          "tokens_per_s_device": n * ctx / ms * 1e3, "linear_tflops": 2.0 * n * ctx * params / ms / 1e9,
                          "launches_per_step": model.launches_last_step(), "device_status": model.device_status()}))
        model.close()
        return
    nxt = np.zeros(S, np.uint32)
    t_pre = time.perf_counter()
    for s0 in range(0, S, a.prefill_chunk):
        sids = list(range(s0, min(S, s0 + a.prefill_chunk)))
        tabs = np.stack([alloc.ensure(i, ctx) for i in sids])
        ids = rng.integers(0, cfg["vocab"], len(sids) * ctx, dtype=np.uint32)
        nxt[sids] = model.step(ids, [0] * len(sids), [ctx] * len(sids), tabs, sids)
    t_pre = time.perf_counter() - t_pre
    tabs = np.stack([alloc.ensure(i, ctx + 1) for i in range(S)])
    cached, new, slots = np.full(S, ctx, np.int32), np.ones(S, np.int32), np.arange(S, dtype=np.int32)
    model.step(nxt, cached, new, tabs, slots)
    stream = torch.cuda.current_stream()
    for _ in range(3):
        model.replay_device(stream.cuda_stream)
    torch.cuda.synchronize()
    if a.profiler_range:
        torch.cuda.profiler.start()
        model.replay_device(stream.cuda_stream)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(a.iters):
        model.replay_device(stream.cuda_stream)
    e1.record(stream)
    torch.cuda.synchronize()
    dev_ms = e0.elapsed_time(e1) / a.iters
    t0 = time.perf_counter()
    for _ in range(a.iters):
        model.step(nxt, cached, new, tabs, slots)
    host_ms = 1e3 * (time.perf_counter() - t0) / a.iters
    H, I = cfg["hidden"], cfg["intermediate"]
    n_full = sum((l + 1) % cfg["full_attn_interval"] == 0 for l in range(a.layers))
    n_lin = a.layers - n_full
    QW, KW, GW, GH = cfg["n_heads"] * cfg["attn_head_dim"], cfg["n_kv_heads"] * cfg["attn_head_dim"], cfg["gdn_heads"] * 128, cfg["gdn_heads"]
    w_full = (2 * QW + 2 * KW) * H + H * QW
    w_lin = 4 * GW * H + 2 * GH * H + H * GW
    w_mlp = 3 * H * I
    weight_bytes = 0.5625 * (n_full * w_full + n_lin * w_lin + a.layers * w_mlp + cfg["vocab"] * H)
    state_bytes = 2.0 * S * n_lin * GH * 128 * 128 * 4
    kv_bytes = 2.0 * S * (ctx + 1) * KW * 2 * n_full
    total = weight_bytes + state_bytes + kv_bytes
    print(json.dumps({"bench": "hybrid_decode_step", "seqs": S, "ctx": ctx, "layers": a.layers, "device_ms_per_step": dev_ms,
                      "host_entry_ms_per_step": host_ms, "tokens_per_s_device": S / dev_ms * 1e3, "launches_per_step": model.launches_last_step(),
                      "algorithmic_gb": {"int4_weights": weight_bytes / 1e9, "recurrent_state_rw": state_bytes / 1e9, "kv_read": kv_bytes / 1e9},
                      "hbm_gbs_algorithmic": total / 1e9 / (dev_ms * 1e-3), "prefill_tokens_per_s": S * ctx / t_pre,
                      "device_status": model.device_status()}))
    model.close()


if __name__ == "__main__":
    main()
