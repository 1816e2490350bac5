#!/usr/bin/env python
"""Benchmark of the Stella-1.5B-architecture ragged-batch embedding forward on B200.

Workload (the configuration the headline metric "Stella-1.5B embeddings/s" is quoted on): a
Qwen2-style encoder with 28 layers, hidden 1536, 12 query / 2 KV heads of 128, SwiGLU 8960, vocab
151646, mean pooling -> 1536->1024 dense -> L2; seeded random weights N(0, 0.02); a batch of 8
sequences with lengths uniform in [32, 512] and uniform token ids. One step = one forward of the
batch. Weak scaling over GPUs: every rank holds a full replica and its own batch (request
sharding, no collective on the data path).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]
  python bench.py --workload ragged_step                    (continuous-batching step of the int4 decoder)
  python bench.py --workload serving_sweep [--requests R --max-seqs S --arrival-rate L --tp T]
                                                            (hybrid decoder under the host scheduler)

`value`  embeddings/s with ids already resident on the device (CUDA events on the launch stream)
`e2e`    the same through lg_stella_encode_ids_batch with host buffers (H2D + D2H inside)
`roofline`      the dominant kernel (gate/up tcgen05 GEMM) against the measured bf16 peak
`extra_rooflines` the HBM-bound decode kernels (int4 GEMV, paged attention, fused-dequant linear) against HBM peak
`cpu_baseline`  the CPU oracle (a port of the reference's fp32 path) on the host cores
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from stella_weights import STELLA_1_5B, make_batch, make_weights  # noqa: E402

SEED_W, SEED_B = 2024, 7


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tf_burst=d["bf16_tflops"], tf_sust=d.get("bf16_tflops_sustained", d["bf16_tflops"]), src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sust=1400.0, src="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


def flops_per_forward(cfg, lens, n_layers):
    h, i, kv = cfg["hidden"], cfg["intermediate"], cfg["n_kv_heads"] * (cfg["hidden"] // cfg["n_heads"])
    per_tok = 2 * (h * h + 2 * kv * h + h * h + 3 * h * i) * n_layers
    attn = sum(4 * cfg["n_heads"] * (cfg["hidden"] // cfg["n_heads"]) * L * L for L in lens) * n_layers
    return per_tok * int(sum(lens)) + attn


# ------------------------------------------------------------------------------------ CPU arm

def cpu_baseline(cfg, w, ids, cu, budget_s=20.0):
    """The oracle's encode_batch (one worker per sequence on the physical cores, single-threaded
    GEMM inside each, as crates/embed/src/stella.rs:264-294) on a bounded sample: all sequences
    of the batch through the first L' layers, the time scaled by n_layers / L'."""
    import oracle_lib as O
    cores = O.physical_cores()
    n_seq = len(cu) - 1
    threads = min(cores, n_seq)
    probe = dict(cfg, n_layers=1)
    m1 = O.OracleStella(probe, dict(w, layers=w["layers"][:1]))
    t0 = time.perf_counter(); m1.encode_batch(ids, cu, threads); t1 = time.perf_counter() - t0
    layers = int(max(1, min(cfg["n_layers"], budget_s / max(t1, 1e-3))))
    if layers > 1:
        mL = O.OracleStella(dict(cfg, n_layers=layers), dict(w, layers=w["layers"][:layers]))
        t0 = time.perf_counter(); mL.encode_batch(ids, cu, threads); tL = time.perf_counter() - t0
    else:
        tL = t1
    full = tL * cfg["n_layers"] / layers
    return {"value": n_seq / full, "unit": "embeddings/s", "cores": threads, "kind": "port",
            "sample": f"{n_seq} sequences x {layers} of {cfg['n_layers']} layers, {tL:.1f} s measured, scaled by {cfg['n_layers']}/{layers}; "
                      f"oracle C++ port of the reference fp32 path (blocked SGEMM standing in for matrixmultiply), "
                      f"{cores} physical cores detected"}, full


def run_reference(args, cfg, rank, world):
    if rank != 0:
        return
    w = make_weights(cfg, SEED_W)
    ids, cu = make_batch(cfg, SEED_B, n_seq=8, lo=32, hi=512)
    vals = []
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_baseline(cfg, w, ids, cu, budget_s=3.0)
    t_all = 0.0
    for _ in range(args.steps):
        cb, full = cpu_baseline(cfg, w, ids, cu, budget_s=max(3.0, 60.0 / max(args.steps, 1)))
        vals.append(cb["value"]); t_all += full
    v = float(np.mean(vals))
    cb["value"] = v
    print(json.dumps({"impl": "reference", "metric": "stella_1.5b_embeddings_per_s", "value": v, "unit": "embeddings/s",
                      "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_all / args.steps,
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": workload_config(cfg, cu), "cpu_baseline": cb,
                      "e2e": {"value": v, "unit": "embeddings/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def workload_config(cfg, cu):
    return {"workload": "stella-1.5b-arch embedding forward, 8 sequences x U[32,512] tokens, 28 layers, seeded random weights",
            "tokens_per_step": int(cu[-1]), "n_layers": cfg["n_layers"], "l2": "weights (2.6 GB bf16) exceed L2 (126 MB); no explicit flush",
            "parallelism": "request sharding, one replica per GPU"}


# ------------------------------------------------------------------------------------ GPU arm

def time_kernel(fn, iters, stream):
    """Seconds per launch: the launches are captured into one CUDA graph and the replay is timed with
    CUDA events on the launch stream, so that host launch cost (ctypes, descriptor encoding, ~10 us per
    call) is not charged to kernels of a few tens of microseconds."""
    from logismos_b200.microbench import timeit
    return timeit(fn, iters)


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/ (same kernels; where the capture ran a smaller case the traffic is scaled by the units
# processed, as the summaries state). bytes per unit: gate/up GEMM at M=2176 (read 61.97 + write 7.44 MB,
# the bf16 output lands in L2 first); GEMV lm_head (131.30 + 5.89 MB); paged decode 1027 B per context
# token + 7.09 MB of partials per 328868 tokens.
NCU_TRAFFIC = {"gemm_m2176": 69.41e6, "gemv_lm_head": 135.47e6, "paged_per_context_token": (337.73e6 + 4.56e6) / 328868}


def micro_rooflines(peaks, T, cfg):
    """Per-launch rooflines of the dominant GEMM and the two HBM-bound decode kernels, timed with
    CUDA events on the launch stream, operands rotated so that each launch reads from HBM."""
    import torch
    from logismos_b200 import ops
    dev = "cuda"
    st = torch.cuda.current_stream()
    out = {}
    # gate/up GEMM with fused SwiGLU at the benchmark's token count
    h, i2 = cfg["hidden"], 2 * cfg["intermediate"]
    a = torch.randn((T, h), device=dev).to(torch.bfloat16)
    ws = [(torch.randn((i2, h), device=dev) * 0.02).to(torch.bfloat16) for _ in range(4)]
    t = time_kernel(lambda i: ops.linear_t(a, ws[i % 4], swiglu=True, sync=False), 20, st)
    fl = 2.0 * T * i2 * h
    out["gemm"] = {"kernel": "linear_t_tcgen05 (gate/up + SwiGLU epilogue)", "bound": "tensor", "achieved": fl / t / 1e12,
                   "peak": peaks["tf_burst"], "unit": "TFLOP/s", "frac": fl / t / 1e12 / peaks["tf_burst"],
                   "traffic": NCU_TRAFFIC["gemm_m2176"] * T / 2176.0, "traffic_note": "ncu capture at M=2176 scaled by tokens (A and output grow with M; W 55 MB does not, so this over-states slightly above 2176)",
                   "flops_per_launch": fl, "us_per_launch": t * 1e6, "peak_source": peaks["src"] + " burst"}
    del ws
    # int4 GEMV, lm_head shape, batch 1
    n, k = 151936, 1536
    codes = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev) for _ in range(3)]
    scales = [(torch.rand((n, k // 32), device=dev) * 0.02).to(torch.float16) for _ in range(3)]
    x = torch.randn((1, k), device=dev).to(torch.bfloat16)
    y = torch.empty((1, n), dtype=torch.bfloat16, device=dev)
    t = time_kernel(lambda i: ops.gemv_int4(codes[i % 3], scales[i % 3], x, out=y, sync=False), 30, st)
    by = n * k / 2 + n * (k // 32) * 2 + k * 2 + n * 2
    out["gemv"] = {"kernel": "gemv_int4_g32 (151936 x 1536, batch 1)", "bound": "hbm", "achieved": by / t / 1e9, "peak": peaks["hbm"],
                   "unit": "GB/s", "frac": by / t / 1e9 / peaks["hbm"], "traffic": NCU_TRAFFIC["gemv_lm_head"], "bytes_per_launch": by, "us_per_launch": t * 1e6,
                   "peak_source": peaks["src"]}
    # the same stream through the fused-dequant tensor-core linear (decode of 64 tokens, hybrid lm_head shape)
    k2 = 2048
    codes2 = [torch.randint(0, 256, (n, k2 // 2), dtype=torch.uint8, device=dev) for _ in range(2)]
    scales2 = [(torch.rand((n, k2 // 32), device=dev) * 0.02).to(torch.float16) for _ in range(2)]
    x2 = torch.randn((64, k2), device=dev).to(torch.bfloat16)
    acc = torch.zeros((64, n), dtype=torch.float32, device=dev)
    stw = torch.zeros(1, dtype=torch.int32, device=dev)
    t = time_kernel(lambda i: ops.check(ops.lib.logismos_launch_qlinear_int4_g32_acc_f32(
        x2.data_ptr(), codes2[i % 2].data_ptr(), scales2[i % 2].data_ptr(), acc.data_ptr(), 64, n, k2, k2, n, stw.data_ptr(),
        torch.cuda.current_stream().cuda_stream), "qlinear"), 20, st)  # the stream is looked up per call: graph capture switches it
    by2 = n * k2 / 2 + n * (k2 // 32) * 2 + 64 * k2 * 2 + 64 * n * 4
    out["qlinear"] = {"kernel": "qlinear_int4_tcgen05 (151936 x 2048, 64 tokens, fp32 accumulate)", "bound": "hbm", "achieved": by2 / t / 1e9,
                      "peak": peaks["hbm"], "unit": "GB/s", "frac": by2 / t / 1e9 / peaks["hbm"], "traffic": None, "bytes_per_launch": by2,
                      "us_per_launch": t * 1e6, "tflops": 2.0 * 64 * n * k2 / t / 1e12, "device_status": int(stw.item()), "peak_source": peaks["src"]}
    del codes, scales, codes2, scales2, acc
    # paged-attention decode: 256 sequences, contexts log-uniform in [128, 32768], block 16, fused append
    rng = np.random.default_rng(3)
    ctx = np.exp(rng.uniform(np.log(128), np.log(32768), 256)).round().astype(np.int64)
    nb = (ctx + 15) // 16
    n_pool = int(nb.sum())
    perm = rng.permutation(n_pool).astype(np.int32)
    tables = np.zeros((256, int(nb.max())), np.int32); o = 0
    for s_ in range(256):
        tables[s_, :nb[s_]] = perm[o:o + nb[s_]]; o += nb[s_]
    kp = torch.randn((n_pool, 16, 256), device=dev).to(torch.bfloat16); vp = torch.randn((n_pool, 16, 256), device=dev).to(torch.bfloat16)
    q = torch.randn((256, 2048), device=dev).to(torch.bfloat16)
    nk = torch.randn((256, 256), device=dev).to(torch.bfloat16); nv = torch.randn((256, 256), device=dev).to(torch.bfloat16)
    chunk = ops.pick_decode_chunk(ctx.astype(np.int32), 2, 128)  # the choice the executors make for a step
    off, total = ops.build_decode_chunks(ctx.astype(np.int32), chunk)
    d_tab, d_ctx, d_off = torch.from_numpy(tables).to(dev), torch.from_numpy(ctx.astype(np.int32)).to(dev), off.to(dev)
    scratch = torch.empty(int(ops.lib.logismos_paged_decode_scratch_bytes(total, 16, 128)), dtype=torch.uint8, device=dev)
    t = time_kernel(lambda i: ops.paged_attention_decode(q, kp, vp, nk, nv, d_tab, d_ctx, d_off, total, chunk, 16, 2, 128, scratch=scratch,
                                                         sync=False), 10, st)
    by = float(ctx.sum()) * 1024 + 256 * (2048 * 2 * 2 + 512 * 2) + tables.size * 4
    out["paged"] = {"kernel": "paged_attention_decode (256 seqs, ctx log-U[128,32768], GQA 16/2, fused append) incl. merge kernel",
                    "bound": "hbm", "achieved": by / t / 1e9, "peak": peaks["hbm"], "unit": "GB/s", "frac": by / t / 1e9 / peaks["hbm"],
                    "traffic": NCU_TRAFFIC["paged_per_context_token"] * float(ctx.sum()), "traffic_note": "ncu capture of 64 sequences (2048-token chunks) scaled by context tokens",
                    "bytes_per_launch": by, "us_per_launch": t * 1e6, "context_tokens": int(ctx.sum()), "chunk_tokens": chunk,
                    "peak_source": peaks["src"]}
    return out


def run_ours(args, cfg, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from logismos_b200.embed import StellaModel
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = measured_peaks()
    w = make_weights(cfg, SEED_W)
    ids, cu = make_batch(cfg, SEED_B + rank, n_seq=8, lo=32, hi=512)
    lens = (cu[1:] - cu[:-1]).tolist()
    T, n_seq = int(cu[-1]), len(lens)
    model = StellaModel(cfg, w, device=local_rank, max_batch_tokens=4608, max_batch_seqs=16)
    pos = np.concatenate([np.arange(L) for L in lens]).astype(np.int32)
    d_ids = torch.from_numpy(ids.view(np.int32)).cuda(); d_cu = torch.from_numpy(cu).cuda(); d_pos = torch.from_numpy(pos).cuda()
    d_out = torch.empty((n_seq, cfg["head_out_dim"]), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream()

    def step():
        model.forward_device(d_ids.data_ptr(), d_cu.data_ptr(), d_pos.data_ptr(), T, n_seq, max(lens), d_out.data_ptr(), stream.cuda_stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    if rank == 0:  # nvidia-smi needs a moment to start: keep the GPU busy until the first sample arrives
        t_wait = time.perf_counter()
        while not sampler.rows and time.perf_counter() - t_wait < 5.0:
            step(); torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    dt = e0.elapsed_time(e1) * 1e-3
    # end to end through the public entry point, host buffers in, host embeddings out
    for _ in range(2):
        emb = model.encode_ids_batch(ids, cu)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        emb = model.encode_ids_batch(ids, cu)
    dt_e2e = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        tt = torch.tensor([dt, dt_e2e], device="cuda", dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt, dt_e2e = float(tt[0]), float(tt[1])
    status = model.device_status()
    if rank == 0:
        total_emb = world * n_seq * args.steps
        fl = flops_per_forward(cfg, lens, cfg["n_layers"])
        line = {"metric": "stella_1.5b_embeddings_per_s", "value": total_emb / dt, "unit": "embeddings/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(cfg, cu),
                "e2e": {"value": total_emb / dt_e2e, "unit": "embeddings/s", "h2d_bytes_per_step": int(T * 8 + (n_seq + 1) * 4),
                        "d2h_bytes_per_step": int(n_seq * cfg["head_out_dim"] * 4)},
                "gpu_launches": model.launches_per_forward() * args.steps, "clocks": clocks, "device_status": status,
                "model_tflops": fl * args.steps / dt / 1e12, "model_frac_of_sustained_peak": fl * args.steps / dt / 1e12 / peaks["tf_sust"],
                "embedding_norm_check": float(np.abs(np.linalg.norm(emb, axis=1) - 1).max())}
        if world == 1 and not args.no_micro:
            mr = micro_rooflines(peaks, T, cfg)
            line["roofline"] = mr["gemm"]
            line["extra_rooflines"] = [mr["gemv"], mr["paged"], mr["qlinear"]]
        else:
            line["roofline"] = {"bound": "tensor", "achieved": fl * args.steps / dt / 1e12 / 1.0, "peak": peaks["tf_sust"], "unit": "TFLOP/s",
                                "frac": fl * args.steps / dt / 1e12 / peaks["tf_sust"], "traffic": None,
                                "note": "whole-forward FLOPs over whole-forward time (per-kernel rooflines are reported at N=1)"}
        if world == 1 and not args.no_cpu:
            del model
            line["cpu_baseline"], _ = cpu_baseline(cfg, w, ids, cu, budget_s=args.cpu_budget)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_ragged_step(args, rank, world, local_rank):
    """Continuous-batching step of the benchmark's third configuration: a 28-layer Stella-dim causal
    stack with int4 group-32 weights, 64 decode sequences (contexts uniform in [256, 8192]) plus 4
    prefill chunks of 512 tokens, paged KV cache with 16-token blocks. Weights are random int4 codes
    with |N(0, 0.02)| scales; the cache rows of the claimed contexts hold zeros (only their traffic
    matters for timing). One step = 2112 tokens."""
    import torch
    from logismos_b200.decoder import BlockAllocator, DecoderModel
    torch.cuda.set_device(local_rank)
    cfg = dict(STELLA_1_5B, vocab=151936)
    if args.layers:
        cfg["n_layers"] = args.layers
    rng = np.random.Generator(np.random.PCG64(11 + rank))
    h, inter, kv = cfg["hidden"], cfg["intermediate"], 256

    def qmat(n, k):
        return (rng.integers(0, 256, (n, k // 2), dtype=np.uint8), np.abs(rng.standard_normal((n, k // 32), dtype=np.float32) * 0.02).astype(np.float16))

    layer = {"norm1": np.ones(h, np.float32), "norm2": np.ones(h, np.float32), "bq": np.zeros(h, np.float32),
             "bk": np.zeros(kv, np.float32), "bv": np.zeros(kv, np.float32), "wq": qmat(h, h), "wk": qmat(kv, h), "wv": qmat(kv, h),
             "wo": qmat(h, h), "w_gate": qmat(inter, h), "w_up": qmat(inter, h), "w_down": qmat(h, inter)}
    w = {"tok_embed": (rng.standard_normal((cfg["vocab"], h), dtype=np.float32) * np.float32(0.02)), "final_norm": np.ones(h, np.float32),
         "layers": [layer] * cfg["n_layers"], "lm_head": qmat(cfg["vocab"], h)}
    ctx = rng.integers(256, 8193, 64)
    cached = np.concatenate([ctx, np.zeros(4, np.int64)]).astype(np.int32)
    new = np.concatenate([np.ones(64, np.int64), np.full(4, 512)]).astype(np.int32)
    max_blocks = 520
    n_pool = int(((cached + new + 15) // 16).sum()) + 8
    alloc = BlockAllocator(n_pool, max_blocks, seed=1)
    tables = np.stack([alloc.ensure(i, int(cached[i] + new[i])) for i in range(68)])
    ids = rng.integers(0, cfg["vocab"], int(new.sum()), dtype=np.uint32)
    model = DecoderModel(cfg, w, n_pool_blocks=n_pool, max_blocks_per_seq=max_blocks, max_step_tokens=2112, max_step_seqs=68, device=local_rank)
    toks = model.step(ids, cached, new, tables)
    stream = torch.cuda.current_stream()
    for _ in range(max(args.warmup, 3)):
        model.replay_device(stream.cuda_stream)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        model.replay_device(stream.cuda_stream)
    e1.record(stream)
    torch.cuda.synchronize()
    dt = e0.elapsed_time(e1) * 1e-3
    t0 = time.perf_counter()
    for _ in range(args.steps):
        toks = model.step(ids, cached, new, tables)
    dt_e2e = time.perf_counter() - t0
    T = int(new.sum())
    kv_bytes = float(ctx.sum() + 64) * 1024 * cfg["n_layers"]
    w_bytes = (h * h * 2 + 2 * kv * h + 3 * h * inter) * 0.5625 * cfg["n_layers"]
    if rank == 0:
        print(json.dumps({"metric": "ragged_step_tokens_per_s", "value": T * args.steps / dt, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                          "warmup": max(args.warmup, 3), "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "bf16 activations, int4-g32 weights", "data": "synthetic",
                          "config": {"workload": "ragged continuous-batching step: 64 decode seqs (ctx U[256,8192]) + 4 x 512-token prefill chunks, 28 layers, int4-g32 weights, paged KV block 16",
                                     "tokens_per_step": T, "decode_context_tokens": int(ctx.sum()), "n_layers": cfg["n_layers"]},
                          "e2e": {"value": T * args.steps / dt_e2e, "unit": "tokens/s", "h2d_bytes_per_step": int(T * 16 + 68 * (max_blocks + 4) * 4), "d2h_bytes_per_step": 68 * 4},
                          "gpu_launches": model.launches_last_step() * args.steps, "device_status": model.device_status(),
                          "algorithmic": {"linear_tflop_per_step": 2.0 * T * (h * h * 2 + 2 * kv * h + 3 * h * inter) * cfg["n_layers"] / 1e12,
                                          "decode_kv_gb_per_step": kv_bytes / 1e9, "int4_weight_gb_per_step": w_bytes / 1e9},
                          "next_tokens_sample": [int(t) for t in toks[:4]]}))


def run_serving_sweep(args, rank, world, local_rank):
    """Serving sweep of the hybrid decoder (the benchmark's last configuration): 48 layers, three
    gated-delta-rule linear-attention layers (16 heads of 128, fp32 state) per gated full-attention
    layer (16 query / 2 KV heads of 256, paged KV cache), hidden 2048, SwiGLU 6144, vocab 151936, int4
    group-32 random weights. Requests: prompt lengths lognormal (median 1024, sigma 1, capped at
    16384), output lengths uniform in [64, 1024], seeded Poisson arrivals; request-sharded round-robin
    over the ranks (every rank holds a full replica; no data-path collective). --requests is the
    number of requests PER GPU (the full configuration has 4096 in total; the default is a bounded
    sample of the same distributions so the run ends within minutes). One step = one scheduler
    step (every running sequence decodes one token, admitted prompts are prefilled whole); the value
    is generated tokens per second over the timed steps through the host-buffer entry point (each
    step copies its ids and index arrays to the device and its tokens back)."""
    import torch
    import torch.distributed as dist
    from logismos_b200.hybrid import HYBRID_SERVING, HybridModel, random_int4_weights
    from logismos_b200.serving import Scheduler, shard_requests, synthetic_load
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    cfg = dict(HYBRID_SERVING)
    if args.layers:
        cfg["n_layers"] = args.layers
    w = random_int4_weights(cfg, 17)
    tp = args.tp
    if tp > 1:
        # tensor parallel: the ranks form ONE replica; every rank sees every request and must plan the
        # same steps, so arrivals are not clocked (everything has arrived at time 0)
        if world != tp:
            raise SystemExit("--tp %d needs exactly %d ranks" % (tp, tp))
        from logismos_b200.tp import nccl_allreduce_hook, slice_hybrid_weights
        cfg_local, w = slice_hybrid_weights(cfg, w, tp, rank)
    else:
        cfg_local = cfg
    n_req = args.requests
    if tp > 1:
        reqs = synthetic_load(n_req, 4096, cfg["vocab"], rate_per_s=0.0)
    else:
        reqs = shard_requests(synthetic_load(n_req * world, 4096, cfg["vocab"], rate_per_s=args.arrival_rate * world), world, rank)
    max_seqs = min(args.max_seqs, n_req)
    max_blocks = (16384 + 1024 + 15) // 16
    lifetime = sorted((-(-(len(r.prompt) + r.max_new) // 16) for r in reqs), reverse=True)
    n_pool = int(sum(lifetime[:max_seqs])) + 8
    step_tokens = 16384 + max_seqs
    model = HybridModel(cfg_local, w, n_pool_blocks=n_pool, max_blocks_per_seq=max_blocks, max_step_tokens=step_tokens, max_step_seqs=max_seqs,
                        n_state_slots=max_seqs, device=local_rank)
    if tp > 1:
        model.set_allreduce(nccl_allreduce_hook())
    sched = Scheduler(n_pool, max_blocks, max_seqs, step_tokens, max_seqs, prefill_token_budget=args.prefill_budget)
    for r in reqs:
        sched.add(r)
    launches = h2d = 0
    steps = dec_tokens = pre_tokens = gen = 0
    warm = max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_start = time.perf_counter()
    t_timed = None
    step_ms = []
    while not sched.idle() and (args.steps <= 0 or steps < warm + args.steps):
        if steps == warm:
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t_timed = time.perf_counter()
            gen = dec_tokens = pre_tokens = launches = h2d = 0
        now = time.perf_counter() - t_start
        plan = sched.plan(now)
        if plan is None:
            continue
        t0 = time.perf_counter()
        toks = model.step(plan.ids, plan.cached, plan.new, plan.tables, plan.slots)
        step_ms.append((1e3 * (time.perf_counter() - t0), plan.n_decode, plan.n_prefill_tokens))
        sched.commit(plan, toks, time.perf_counter() - t_start)
        steps += 1
        gen += len(plan.rids); dec_tokens += plan.n_decode; pre_tokens += plan.n_prefill_tokens
        launches += model.launches_last_step()
        h2d += int(plan.ids.size * 16 + len(plan.rids) * (max_blocks + 6) * 4)
    torch.cuda.synchronize()
    dt = time.perf_counter() - (t_timed if t_timed is not None else t_start)
    timed_steps = max(steps - warm, 0) if t_timed is not None else steps
    clocks = sampler.stop() if rank == 0 else None
    status = model.device_status()
    tt = torch.tensor([dt, float(gen), float(pre_tokens), float(timed_steps), float(launches)], device="cuda", dtype=torch.float64)
    if world > 1:
        mx = tt.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(tt, op=dist.ReduceOp.SUM)
        dt = float(mx[0])
    gen_all, pre_all, steps_all, launches_all = float(tt[1]), float(tt[2]), float(tt[3]), float(tt[4])
    if tp > 1:  # one replica: its tokens count once
        gen_all, pre_all = gen_all / tp, pre_all / tp
    if rank == 0:
        dec_only = [m for m, nd, npre in step_ms[warm:] if npre == 0]
        line = {"metric": "hybrid_decoder_generated_tokens_per_s", "value": gen_all / dt, "unit": "tokens/s", "n_gpus": world,
                "steps": int(steps_all / world), "warmup": warm, "ms_per_step": 1e3 * dt / max(timed_steps, 1), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations, int4-g32 weights, fp32 recurrent state", "data": "synthetic",
                "config": {"workload": "hybrid decoder serving sweep, %d requests per GPU (prompts lognormal median 1024 cap 16384, outputs U[64,1024], Poisson %.0f req/s per GPU), %d layers 3:1 linear:full attention" % (n_req, args.arrival_rate, cfg["n_layers"]),
                           "parallelism": ("tp%d (all-reduce of the output projections over NCCL)" % tp) if tp > 1 else ("request-sharded x%d" % world),
                           "max_concurrent_per_gpu": max_seqs, "kv_pool_blocks": n_pool, "inputs": "every step's working set (int4 weights, KV pool, recurrent states) exceeds L2"},
                "e2e": {"value": gen_all / dt, "unit": "tokens/s", "h2d_bytes_per_step": int(h2d / max(timed_steps, 1)), "d2h_bytes_per_step": int(4 * gen / max(timed_steps, 1))},
                "gpu_launches": int(launches_all), "clocks": clocks, "device_status": status,
                "prefill_tokens_per_s": pre_all / dt, "total_tokens_per_s": (pre_all + gen_all) / dt,
                "decode_only_step_ms_median": float(np.median(dec_only)) if dec_only else None,
                "decode_only_steps": len(dec_only), "decode_only_ms_total": float(np.sum(dec_only)) if dec_only else 0.0,
                "prefill_steps": len(step_ms[warm:]) - len(dec_only),
                "prefill_steps_ms_total": float(sum(m for m, nd, npre in step_ms[warm:] if npre > 0)),
                "longest_step_ms": float(max(m for m, nd, npre in step_ms[warm:])) if step_ms[warm:] else None,
                "requests_finished_rank0": len(sched.done), "sweep_complete": sched.idle()}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default 20; serving_sweep: 0 = the whole sweep)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override depth (development only; the reported config is 28)")
    ap.add_argument("--no-micro", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-budget", type=float, default=20.0)
    ap.add_argument("--workload", default="stella", choices=["stella", "ragged_step", "serving_sweep"])
    ap.add_argument("--requests", type=int, default=96, help="serving_sweep: requests per GPU")
    ap.add_argument("--max-seqs", type=int, default=256, help="serving_sweep: concurrent sequences per GPU")
    ap.add_argument("--arrival-rate", type=float, default=64.0, help="serving_sweep: Poisson arrivals per second per GPU")
    ap.add_argument("--tp", type=int, default=1, help="serving_sweep: tensor-parallel degree (ranks form one replica)")
    ap.add_argument("--prefill-budget", type=int, default=16384, help="serving_sweep: prompt tokens admitted per step (larger = better prefill throughput, longer steps)")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = 0 if args.workload == "serving_sweep" else 20
    cfg = dict(STELLA_1_5B)
    if args.layers:
        cfg["n_layers"] = args.layers
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "serving_sweep":
        run_serving_sweep(args, rank, world, local)
    elif args.workload == "ragged_step":
        run_ragged_step(args, rank, world, local)
    elif args.impl == "reference":
        run_reference(args, cfg, rank, world)
    else:
        run_ours(args, cfg, rank, world, local)


if __name__ == "__main__":
    main()
