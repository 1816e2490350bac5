#!/usr/bin/env python
"""Benchmark of the Stella-1.5B-architecture ragged-batch embedding forward on B200, with the decode
workloads of the same metric reported beside it.

Headline workload (the configuration "Stella-1.5B embeddings/s" is quoted on): a Qwen2-style encoder
with 28 layers, hidden 1536, 12 query / 2 KV heads of 128, SwiGLU 8960, vocab 151646, mean pooling ->
1536->1024 dense -> L2; seeded random weights N(0, 0.02); a batch of 8 sequences with lengths uniform
in [32, 512] and uniform token ids. One step = one forward of the batch. Weak scaling over GPUs:
every rank holds a full replica and its own batch (request sharding, no collective on the data path).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]
  python bench.py --workload ragged_step                    (continuous-batching step of the int4 decoder)
  python bench.py --workload serving_sweep [--requests R --max-seqs S --arrival-rate L --tp T]
                                                            (hybrid decoder under the host scheduler)

`value`  embeddings/s with ids already resident on the device (CUDA events on the launch stream)
`e2e`    the same through lg_stella_encode_ids_batch with host buffers (H2D + D2H inside)
`roofline`        the dominant kernel (gate/up tcgen05 GEMM) against the measured bf16 peak
`extra_rooflines` the HBM-bound decode kernels against the measured HBM peak: the int4 GEMV over the
                  whole grid of the quantized-GEMV configuration (4 shapes x batch 1/4/16/64, weights
                  rotated through HBM and L2-resident), the fused projections the executors launch,
                  the paged-attention decode, the fused-dequant tensor-core linear
`extra_workloads` decode tokens/s: one ragged continuous-batching step (64 decode sequences + 4
                  prefill chunks of 512 tokens, 28-layer int4 decoder) and a bounded sample of the
                  hybrid-decoder serving sweep, request-sharded over the ranks at every N
`cpu_baseline`    the CPU oracle (a port of the reference's fp32 path) on the host cores
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

from logismos_b200.synthetic import STELLA_1_5B, make_batch, make_weights, random_int4_decoder_weights  # noqa: E402

SEED_W, SEED_B = 2024, 7


def oracle_lib():
    """The CPU oracle's ctypes wrapper (test infrastructure; used only by the CPU legs)."""
    p = os.path.join(ROOT, "tests")
    if p not in sys.path:
        sys.path.insert(0, p)
    import oracle_lib as O
    return O


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


class Ranks:
    """Rank plumbing: barrier and reductions over the NCCL group (no-ops on one rank)."""

    def __init__(self, rank, world, local_rank):
        self.rank, self.world, self.local = rank, world, local_rank

    def barrier(self):
        import torch
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def reduce(self, values, op="max"):
        import torch
        if self.world == 1:
            return [float(v) for v in values]
        import torch.distributed as dist
        t = torch.tensor([float(v) for v in values], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
        return t.tolist()


# ------------------------------------------------------------------------------------ CPU arm

def cpu_full_batch(cfg, w, ids, cu):
    """One full-depth batch through the oracle's encode_batch, parallelised as the reference is (one
    worker per sequence on the physical cores, single-threaded GEMM inside each worker,
    crates/embed/src/stella.rs:264-294). Returns (seconds, threads, physical cores)."""
    O = oracle_lib()
    cores = O.physical_cores()
    n_seq = len(cu) - 1
    threads = min(cores, n_seq)
    model = O.OracleStella(cfg, w)
    t0 = time.perf_counter()
    emb = model.encode_batch(ids, cu, threads)
    dt = time.perf_counter() - t0
    assert np.isfinite(emb).all()
    return dt, threads, cores


CPU_KIND_NOTE = ("oracle C++ port of the reference fp32 path (blocked SGEMM standing in for matrixmultiply, built -O3 -march=x86-64-v3; "
                 "the reference is Rust and cannot be built here)")


def cpu_baseline(cfg, w, ids, cu):
    dt, threads, cores = cpu_full_batch(cfg, w, ids, cu)
    n_seq = len(cu) - 1
    return {"value": n_seq / dt, "unit": "embeddings/s", "cores": threads, "kind": "port",
            "sample": f"one full batch: {n_seq} sequences ({int(cu[-1])} tokens) x {cfg['n_layers']} layers, {dt:.1f} s measured, nothing extrapolated; "
                      f"{CPU_KIND_NOTE}; {cores} physical cores detected, one worker per sequence"}


def run_reference(args, cfg, rank, world):
    """The reference arm: the CPU implementation of the same path on the host cores. Every timed step is
    one full-depth batch of the workload (about 15 s on 8 workers), so the number of steps is bounded by
    a time budget and the line says how many were actually timed."""
    if rank != 0:
        return
    w = make_weights(cfg, SEED_W)
    ids, cu = make_batch(cfg, SEED_B, n_seq=8, lo=32, hi=512)
    n_seq = len(cu) - 1
    warm = 1 if args.warmup > 0 else 0
    t_warm = 0.0
    for _ in range(warm):
        t_warm, _, _ = cpu_full_batch(cfg, w, ids, cu)
    budget = args.ref_budget
    steps = max(1, min(args.steps, int(budget / max(t_warm, 1.0)) if t_warm > 0 else 4))
    times = []
    threads = cores = 0
    for _ in range(steps):
        dt, threads, cores = cpu_full_batch(cfg, w, ids, cu)
        times.append(dt)
    total = float(sum(times))
    v = n_seq * steps / total
    cb = {"value": v, "unit": "embeddings/s", "cores": threads, "kind": "port",
          "sample": f"{steps} timed steps, each one full batch of {n_seq} sequences ({int(cu[-1])} tokens) x {cfg['n_layers']} layers "
                    f"({total:.1f} s in all, {warm} warm-up batch); --steps {args.steps} was capped to fit {budget:.0f} s; {CPU_KIND_NOTE}; "
                    f"{cores} physical cores detected, one worker per sequence"}
    print(json.dumps({"impl": "reference", "metric": "stella_1.5b_embeddings_per_s", "value": v, "unit": "embeddings/s",
                      "n_gpus": args.gpus, "steps": steps, "steps_requested": args.steps, "warmup": warm, "ms_per_step": 1e3 * total / steps,
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": workload_config(cfg, cu), "cpu_baseline": cb,
                      "e2e": {"value": v, "unit": "embeddings/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def workload_config(cfg, cu):
    return {"workload": "stella-1.5b-arch embedding forward, 8 sequences x U[32,512] tokens, 28 layers, seeded random weights",
            "tokens_per_step": int(cu[-1]), "n_layers": cfg["n_layers"], "l2": "weights (2.6 GB bf16) exceed L2 (126 MB); no explicit flush",
            "parallelism": "request sharding, one replica per GPU"}


# ------------------------------------------------------------------------------------ GPU arm: kernels

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/ (same kernels; where the capture ran a smaller case the traffic is scaled by the units
# processed, as the summaries state). bytes per unit: gate/up GEMM at M=2176 (read 61.97 + write 7.44 MB,
# the bf16 output lands in L2 first); GEMV lm_head (131.30 + 5.89 MB); paged decode 1027 B per context
# token + 7.09 MB of partials per 328868 tokens.
NCU_TRAFFIC = {"gemm_m2176": 69.41e6, "gemm_m2929": 77.52e6, "gemv_lm_head": 135.47e6, "paged_per_context_token": (337.73e6 + 4.56e6) / 328868}

PROFILER_RANGE = False


def profiler_range(fn):
    """With --profiler-range: run fn once between cudaProfilerStart and cudaProfilerStop (a profiler started
    with its collection off captures exactly that step); otherwise nothing."""
    if not PROFILER_RANGE:
        return
    import torch
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    fn()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


GEMV_SHAPES = [(1536, 1536), (8960, 1536), (1536, 8960), (151936, 1536)]
# what the decoder executors launch per layer at these dims: q|k|v and gate|up as one matrix each
GEMV_FUSED_SHAPES = [("q|k|v", 2048, 1536), ("gate|up", 17920, 1536)]
GEMV_BATCHES = [1, 4, 16, 64]


def gemv_grid(peaks, shapes):
    """int4 group-32 GEMV / skinny GEMM over (name, N, K) x batch: time per launch with the weights
    rotated through more distinct bytes than the L2 holds (every launch reads HBM), and with one copy
    re-read (L2-resident). Bytes per launch: N K / 2 + 2 N K / 32 + 2 B K + 2 B N."""
    import torch
    from logismos_b200 import ops
    from logismos_b200.timing import timeit
    dev, out = "cuda", []
    for name, n, k in shapes:
        wbytes = n * k // 2 + n * (k // 32) * 2
        copies = max(3, min(320, int(320e6 // wbytes) + 1))
        codes = torch.randint(0, 256, (copies, n, k // 2), dtype=torch.uint8, device=dev)
        scales = (torch.rand((copies, n, k // 32), device=dev) * 0.02).to(torch.float16)
        ws = torch.zeros(64 * n, dtype=torch.float32, device=dev)  # fp32 workspace of the route above 16 rows (kept zero by it)
        stw = torch.zeros(1, dtype=torch.int32, device=dev)
        for b in GEMV_BATCHES:
            x = torch.randn((b, k), device=dev).to(torch.bfloat16)
            y = torch.empty((b, n), dtype=torch.bfloat16, device=dev)
            iters = copies if copies > 6 else 2 * copies
            t_hbm = timeit(lambda i: ops.skinny_int4(codes[i % copies], scales[i % copies], x, ws, out=y, status=stw, sync=False), iters, reps=2)
            t_l2 = timeit(lambda i: ops.skinny_int4(codes[0], scales[0], x, ws, out=y, status=stw, sync=False), 20) if wbytes < 100e6 else None
            by = wbytes + b * k * 2 + b * n * 2
            out.append({"kernel": "qlinear_int4_tcgen05 + finish (skinny route)" if ops.lib.logismos_skinny_int4_route(b, n, k) else "gemv_int4_g32", "shape": name, "n": n, "k": k, "batch": b, "bound": "hbm", "bytes_per_launch": by,
                        "us_per_launch": t_hbm * 1e6, "achieved": by / t_hbm / 1e9, "peak": peaks["hbm"], "unit": "GB/s",
                        "frac": by / t_hbm / 1e9 / peaks["hbm"], "weight_copies_rotated": copies,
                        "us_per_launch_l2_resident": t_l2 * 1e6 if t_l2 else None, "achieved_l2_resident": by / t_l2 / 1e9 if t_l2 else None,
                        "traffic": NCU_TRAFFIC["gemv_lm_head"] if (n, k, b) == (151936, 1536, 1) else None, "peak_source": peaks["src"]})
        assert int(stw.item()) == 0
        del codes, scales, ws
    return out


def micro_rooflines(peaks, T, cfg):
    """Per-launch rooflines of the dominant GEMM and the HBM-bound decode kernels, timed with CUDA
    events on the launch stream, operands rotated so that each launch reads from HBM."""
    import torch
    from logismos_b200 import ops
    from logismos_b200.timing import timeit
    dev = "cuda"
    out = {}
    # gate/up GEMM with fused SwiGLU at the benchmark's token count
    h, i2 = cfg["hidden"], 2 * cfg["intermediate"]
    a = torch.randn((T, h), device=dev).to(torch.bfloat16)
    ws = [(torch.randn((i2, h), device=dev) * 0.02).to(torch.bfloat16) for _ in range(4)]
    t = timeit(lambda i: ops.linear_t(a, ws[i % 4], swiglu=True, sync=False), 20)
    fl = 2.0 * T * i2 * h
    out["gemm"] = {"kernel": "linear_t_tcgen05 (gate/up + SwiGLU epilogue)", "bound": "tensor", "achieved": fl / t / 1e12,
                   "peak": peaks["tf_burst"], "unit": "TFLOP/s", "frac": fl / t / 1e12 / peaks["tf_burst"],
                   "traffic": NCU_TRAFFIC["gemm_m2929"] if T == 2929 else NCU_TRAFFIC["gemm_m2176"] * T / 2176.0,
                   "traffic_note": "ncu capture at M=2929 (dram read + write of one launch)" if T == 2929 else
                                   "ncu capture at M=2176 scaled by tokens (A and output grow with M; W 55 MB does not, so this over-states slightly above 2176)",
                   "flops_per_launch": fl, "us_per_launch": t * 1e6, "peak_source": peaks["src"] + " burst"}
    del ws
    out["gemv_grid"] = gemv_grid(peaks, [("%dx%d" % s, s[0], s[1]) for s in GEMV_SHAPES])
    out["gemv_fused"] = gemv_grid(peaks, GEMV_FUSED_SHAPES)
    # the same stream through the fused-dequant tensor-core linear (decode of 64 tokens, hybrid lm_head shape)
    n, k2 = 151936, 2048
    codes2 = [torch.randint(0, 256, (n, k2 // 2), dtype=torch.uint8, device=dev) for _ in range(2)]
    scales2 = [(torch.rand((n, k2 // 32), device=dev) * 0.02).to(torch.float16) for _ in range(2)]
    x2 = torch.randn((64, k2), device=dev).to(torch.bfloat16)
    acc = torch.zeros((64, n), dtype=torch.float32, device=dev)
    stw = torch.zeros(1, dtype=torch.int32, device=dev)
    t = timeit(lambda i: ops.check(ops.lib.logismos_launch_qlinear_int4_g32_acc_f32(
        x2.data_ptr(), codes2[i % 2].data_ptr(), scales2[i % 2].data_ptr(), acc.data_ptr(), 64, n, k2, k2, n, stw.data_ptr(),
        torch.cuda.current_stream().cuda_stream), "qlinear"), 20)  # the stream is looked up per call: graph capture switches it
    by2 = n * k2 / 2 + n * (k2 // 32) * 2 + 64 * k2 * 2 + 64 * n * 4
    out["qlinear"] = {"kernel": "qlinear_int4_tcgen05 (151936 x 2048, 64 tokens, fp32 accumulate)", "bound": "hbm", "achieved": by2 / t / 1e9,
                      "peak": peaks["hbm"], "unit": "GB/s", "frac": by2 / t / 1e9 / peaks["hbm"], "traffic": None, "bytes_per_launch": by2,
                      "us_per_launch": t * 1e6, "tflops": 2.0 * 64 * n * k2 / t / 1e12, "device_status": int(stw.item()), "peak_source": peaks["src"]}
    del codes2, scales2, acc
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
    t = timeit(lambda i: ops.paged_attention_decode(q, kp, vp, nk, nv, d_tab, d_ctx, d_off, total, chunk, 16, 2, 128, scratch=scratch,
                                                    sync=False), 10)
    by = float(ctx.sum()) * 1024 + 256 * (2048 * 2 * 2 + 512 * 2) + tables.size * 4
    out["paged"] = {"kernel": "paged_attention_decode (256 seqs, ctx log-U[128,32768], GQA 16/2, fused append) incl. merge kernel",
                    "bound": "hbm", "achieved": by / t / 1e9, "peak": peaks["hbm"], "unit": "GB/s", "frac": by / t / 1e9 / peaks["hbm"],
                    "traffic": NCU_TRAFFIC["paged_per_context_token"] * float(ctx.sum()), "traffic_note": "ncu capture of 64 sequences (2048-token chunks) scaled by context tokens",
                    "bytes_per_launch": by, "us_per_launch": t * 1e6, "context_tokens": int(ctx.sum()), "chunk_tokens": chunk,
                    "peak_source": peaks["src"]}
    return out


# ------------------------------------------------------------------------------------ GPU arm: decode workloads

def ragged_step_measure(R: Ranks, steps, warmup, layers=0):
    """Continuous-batching step of the benchmark's third configuration on this rank: a 28-layer
    Stella-dim causal stack with int4 group-32 weights (random codes, |N(0, 0.02)| scales), 64 decode
    sequences (contexts uniform in [256, 8192]) plus 4 prefill chunks of 512 tokens (chunks of longer
    prompts: they continue cached prefixes of 0, 512, 1024 and 2048 tokens), paged KV cache with
    16-token blocks. The cache is filled by real steps first: every context is prefilled in chunks
    through the same executor. One step = 2112 tokens. Returns this rank's figures."""
    import torch
    from logismos_b200.decoder import BlockAllocator, DecoderModel
    cfg = dict(STELLA_1_5B, vocab=151936)
    if layers:
        cfg["n_layers"] = layers
    w = random_int4_decoder_weights(cfg, 11)
    rng = np.random.Generator(np.random.PCG64(12 + R.rank))
    h, inter, kv = cfg["hidden"], cfg["intermediate"], 256
    ctx = rng.integers(256, 8193, 64)
    cached = np.concatenate([ctx, [0, 512, 1024, 2048]]).astype(np.int32)
    new = np.concatenate([np.ones(64, np.int64), np.full(4, 512)]).astype(np.int32)
    n_seq, step_tokens, max_blocks = 68, 2112, 520
    n_pool = int(((cached + new + 15) // 16).sum()) + 8
    alloc = BlockAllocator(n_pool, max_blocks, seed=1)
    tables = np.stack([alloc.ensure(i, int(cached[i] + new[i])) for i in range(n_seq)])
    hist = [rng.integers(0, cfg["vocab"], int(cached[i] + new[i]), dtype=np.uint32) for i in range(n_seq)]
    model = DecoderModel(cfg, w, n_pool_blocks=n_pool, max_blocks_per_seq=max_blocks, max_step_tokens=step_tokens, max_step_seqs=n_seq, device=R.local)
    # fill the cache: every sequence's first cached[i] tokens, chunked into steps of at most 2112 tokens
    done = np.zeros(n_seq, np.int64)
    fill_steps, t_fill = 0, time.perf_counter()
    while (done < cached).any():
        ids, c_, n_, tb = [], [], [], []
        room = step_tokens
        for i in range(n_seq):
            if room <= 0:
                break
            take = int(min(cached[i] - done[i], room))
            if take <= 0:
                continue
            ids.append(hist[i][done[i]:done[i] + take]); c_.append(done[i]); n_.append(take); tb.append(tables[i])
            done[i] += take; room -= take
        model.step(np.concatenate(ids), c_, n_, np.stack(tb))
        fill_steps += 1
    t_fill = time.perf_counter() - t_fill
    ids = np.concatenate([hist[i][cached[i]:cached[i] + new[i]] for i in range(n_seq)])
    toks = model.step(ids, cached, new, tables)
    logits = model.last_logits()
    assert model.device_status() == 0 and np.isfinite(logits).all() and (toks < cfg["vocab"]).all()
    assert (toks == logits.argmax(axis=1)).all()
    del logits
    stream = torch.cuda.current_stream()
    for _ in range(max(warmup, 3)):
        model.replay_device(stream.cuda_stream)
    profiler_range(lambda: model.replay_device(stream.cuda_stream))
    R.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        model.replay_device(stream.cuda_stream)
    e1.record(stream)
    R.barrier()
    dt = e0.elapsed_time(e1) * 1e-3
    t0 = time.perf_counter()
    for _ in range(steps):
        toks = model.step(ids, cached, new, tables)
    dt_e2e = time.perf_counter() - t0
    status, launches = model.device_status(), model.launches_last_step()
    model.close()
    dt, dt_e2e = R.reduce([dt, dt_e2e], "max")
    T = int(new.sum())
    w_bytes = (h * h * 2 + 2 * kv * h + 3 * h * inter) * 0.5625 * cfg["n_layers"]
    return {"metric": "ragged_step_tokens_per_s", "value": R.world * T * steps / dt, "unit": "tokens/s", "n_gpus": R.world, "steps": steps,
            "ms_per_step": 1e3 * dt / steps, "scaling": "weak", "dtype": "bf16 activations, int4-g32 weights",
            "config": {"workload": "ragged continuous-batching step per GPU: 64 decode seqs (ctx U[256,8192]) + 4 x 512-token prefill chunks "
                                   "(cached prefixes 0/512/1024/2048), %d layers, int4-g32 weights, paged KV block 16; cache filled by %d real chunked-prefill steps (%.1f s)"
                                   % (cfg["n_layers"], fill_steps, t_fill),
                       "tokens_per_step": T, "decode_context_tokens": int(ctx.sum()), "n_layers": cfg["n_layers"]},
            "e2e": {"value": R.world * T * steps / dt_e2e, "unit": "tokens/s", "h2d_bytes_per_step": int(T * 16 + n_seq * (max_blocks + 4) * 4), "d2h_bytes_per_step": n_seq * 4},
            "gpu_launches": launches * steps, "device_status": status,
            "algorithmic": {"linear_tflop_per_step": 2.0 * T * (h * h * 2 + 2 * kv * h + 3 * h * inter) * cfg["n_layers"] / 1e12,
                            "decode_kv_gb_per_step": float(ctx.sum() + 64) * 1024 * cfg["n_layers"] / 1e9, "int4_weight_gb_per_step": w_bytes / 1e9},
            "next_tokens_sample": [int(t) for t in toks[:4]]}


def serving_measure(R: Ranks, n_req, max_seqs, arrival_rate, prefill_budget, chunked, tp=1, layers=0, steps_cap=0, warmup=3, sample_clocks=False):
    """Serving sweep of the hybrid decoder (the benchmark's last configuration): 48 layers, three
    gated-delta-rule linear-attention layers (16 heads of 128, fp32 state) per gated full-attention
    layer (16 query / 2 KV heads of 256, paged KV cache), hidden 2048, SwiGLU 6144, vocab 151936, int4
    group-32 random weights. Requests: prompt lengths lognormal (median 1024, sigma 1, capped at
    16384), output lengths uniform in [64, 1024], seeded Poisson arrivals; request-sharded round-robin
    over the ranks (every rank holds a full replica; no data-path collective), or with tp > 1 the ranks
    form one tensor-parallel replica. n_req is the number of requests PER GPU. One step = one scheduler
    step (every running sequence decodes one token; prompts are fed whole, or in chunks of the step's
    prefill budget against their cached prefix); the value is generated tokens per second over the
    timed steps through the host-buffer entry point (each step copies its ids and index arrays to the
    device and its tokens back)."""
    import torch
    from logismos_b200.hybrid import HYBRID_SERVING, HybridModel, random_int4_weights
    from logismos_b200.serving import Scheduler, shard_requests, synthetic_load
    rank, world = R.rank, R.world
    cfg = dict(HYBRID_SERVING)
    if layers:
        cfg["n_layers"] = layers
    w = random_int4_weights(cfg, 17)
    if tp > 1:
        # tensor parallel: the ranks form ONE replica; every rank sees every request and must plan the
        # same steps, so arrivals are not clocked (everything has arrived at time 0)
        if world != tp:
            raise SystemExit("--tp %d needs exactly %d ranks" % (tp, tp))
        from logismos_b200.tp import slice_hybrid_weights
        cfg_local, w = slice_hybrid_weights(cfg, w, tp, rank)
        reqs = synthetic_load(n_req, 4096, cfg["vocab"], rate_per_s=0.0)
    else:
        cfg_local = cfg
        reqs = shard_requests(synthetic_load(n_req * world, 4096, cfg["vocab"], rate_per_s=arrival_rate * world), world, rank)
    max_seqs = min(max_seqs, n_req)
    max_blocks = (16384 + 1024 + 15) // 16
    lifetime = sorted((-(-(len(r.prompt) + r.max_new) // 16) for r in reqs), reverse=True)
    n_pool = int(sum(lifetime[:max_seqs])) + 8
    step_tokens = (prefill_budget if chunked else 16384) + max_seqs
    model = HybridModel(cfg_local, w, n_pool_blocks=n_pool, max_blocks_per_seq=max_blocks, max_step_tokens=step_tokens, max_step_seqs=max_seqs,
                        n_state_slots=max_seqs, device=R.local)
    comm = None
    if tp > 1:
        from logismos_b200.tp import install_allreduce
        comm = install_allreduce(model, rank, tp)
    sched = Scheduler(n_pool, max_blocks, max_seqs, step_tokens, max_seqs, prefill_token_budget=prefill_budget, chunked_prefill=chunked)
    for r in reqs:
        sched.add(r)
    launches = h2d = 0
    steps = dec_tokens = pre_tokens = gen = 0
    sampler = ClockSampler(R.local)
    if rank == 0 and sample_clocks:
        sampler.start()
    t_start = time.perf_counter()
    t_timed = None
    step_ms = []
    while not sched.idle() and (steps_cap <= 0 or steps < warmup + steps_cap):
        if steps == warmup:
            R.barrier()
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
        gen += int(plan.emits.sum()); dec_tokens += plan.n_decode; pre_tokens += plan.n_prefill_tokens
        launches += model.launches_last_step()
        h2d += int(plan.ids.size * 16 + len(plan.rids) * (max_blocks + 6) * 4)
    torch.cuda.synchronize()
    dt = time.perf_counter() - (t_timed if t_timed is not None else t_start)
    timed_steps = max(steps - warmup, 0) if t_timed is not None else steps
    clocks = sampler.stop() if (rank == 0 and sample_clocks) else None
    status = model.device_status()
    finished, idle = len(sched.done), sched.idle()
    model.close()
    del comm
    dt_max, = R.reduce([dt], "max")
    gen_all, pre_all, steps_all, launches_all = R.reduce([gen, pre_tokens, timed_steps, launches], "sum")
    if tp > 1:  # one replica: its tokens count once
        gen_all, pre_all = gen_all / tp, pre_all / tp
    timed = step_ms[warmup:] if t_timed is not None else step_ms
    dec_only = [m for m, nd, npre in timed if npre == 0]
    return {"metric": "hybrid_decoder_generated_tokens_per_s", "value": gen_all / dt_max, "unit": "tokens/s", "n_gpus": world,
            "steps": int(steps_all / world), "warmup": warmup, "ms_per_step": 1e3 * dt_max / max(timed_steps, 1), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16 activations, int4-g32 weights, fp32 recurrent state", "data": "synthetic",
            "config": {"workload": "hybrid decoder serving sweep, %d requests per GPU (prompts lognormal median 1024 cap 16384, outputs U[64,1024], Poisson %.0f req/s per GPU), %d layers 3:1 linear:full attention"
                                   % (n_req, arrival_rate, cfg["n_layers"]),
                       "parallelism": ("tp%d (all-reduce of the output projections over NVLink)" % tp) if tp > 1 else ("request-sharded x%d" % world),
                       "prefill": ("chunked, %d prompt tokens per step" % prefill_budget) if chunked else ("whole prompts, up to %d prompt tokens per step" % prefill_budget),
                       "max_concurrent_per_gpu": max_seqs, "kv_pool_blocks": n_pool, "inputs": "every step's working set (int4 weights, KV pool, recurrent states) exceeds L2"},
            "e2e": {"value": gen_all / dt_max, "unit": "tokens/s", "h2d_bytes_per_step": int(h2d / max(timed_steps, 1)), "d2h_bytes_per_step": int(4 * gen / max(timed_steps, 1))},
            "gpu_launches": int(launches_all), "clocks": clocks, "device_status": status,
            "prefill_tokens_per_s": pre_all / dt_max, "total_tokens_per_s": (pre_all + gen_all) / dt_max,
            "decode_only_step_ms_median": float(np.median(dec_only)) if dec_only else None,
            "decode_only_steps": len(dec_only), "decode_only_ms_total": float(np.sum(dec_only)) if dec_only else 0.0,
            "prefill_steps": len(timed) - len(dec_only), "prefill_steps_ms_total": float(sum(m for m, nd, npre in timed if npre > 0)),
            "longest_step_ms": float(max(m for m, nd, npre in timed)) if timed else None,
            "requests_finished_rank0": finished, "sweep_complete": idle}


# ------------------------------------------------------------------------------------ GPU arm: headline

def run_ours(args, cfg, R: Ranks):
    import torch
    from logismos_b200.embed import StellaModel
    rank, world = R.rank, R.world
    peaks = measured_peaks()
    w = make_weights(cfg, SEED_W)
    ids, cu = make_batch(cfg, SEED_B + rank, n_seq=8, lo=32, hi=512)
    lens = (cu[1:] - cu[:-1]).tolist()
    T, n_seq = int(cu[-1]), len(lens)
    model = StellaModel(cfg, w, device=R.local, max_batch_tokens=4608, max_batch_seqs=16)
    pos = np.concatenate([np.arange(L) for L in lens]).astype(np.int32)
    d_ids = torch.from_numpy(ids.view(np.int32)).cuda(); d_cu = torch.from_numpy(cu).cuda(); d_pos = torch.from_numpy(pos).cuda()
    d_out = torch.empty((n_seq, cfg["head_out_dim"]), dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream()

    def step():
        model.forward_device(d_ids.data_ptr(), d_cu.data_ptr(), d_pos.data_ptr(), T, n_seq, max(lens), d_out.data_ptr(), stream.cuda_stream)

    sampler = ClockSampler(R.local)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    if rank == 0:  # nvidia-smi needs a moment to start: keep the GPU busy until the first sample arrives
        t_wait = time.perf_counter()
        while not sampler.rows and time.perf_counter() - t_wait < 5.0:
            step(); torch.cuda.synchronize()
    profiler_range(step)
    R.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    R.barrier()
    dt = e0.elapsed_time(e1) * 1e-3
    # end to end through the public entry point, host buffers in, host embeddings out. On several GPUs
    # the call a user makes is the request dispatcher: ONE ragged batch of 8 sequences per GPU, split by
    # sequence over the ranks (token-balanced), each shard encoded on its replica, the embeddings
    # gathered back in request order on every rank.
    if world > 1:
        from logismos_b200.sharding import all_gather_embeddings, shard_batch
        g_ids, g_cu = make_batch(cfg, SEED_B + 1000, n_seq=n_seq * world, lo=32, hi=512)
        my_ids, my_cu, mine = shard_batch(g_ids, g_cu, world, rank)
        e2e_in = int(my_ids.size * 8 + (len(mine) + 1) * 4)

        def e2e_step():
            local = model.encode_ids_batch(my_ids, my_cu)
            return all_gather_embeddings(local, mine, n_seq * world, cfg["head_out_dim"])
    else:
        e2e_in = int(T * 8 + (n_seq + 1) * 4)

        def e2e_step():
            return model.encode_ids_batch(ids, cu)
    for _ in range(2):
        emb = e2e_step()
    R.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        emb = e2e_step()
    dt_e2e = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    dt, dt_e2e = R.reduce([dt, dt_e2e], "max")
    status = model.device_status()
    launches = model.launches_per_forward()
    total_emb = world * n_seq * args.steps
    fl = flops_per_forward(cfg, lens, cfg["n_layers"])
    line = {"metric": "stella_1.5b_embeddings_per_s", "value": total_emb / dt, "unit": "embeddings/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(cfg, cu),
            "e2e": {"value": total_emb / dt_e2e, "unit": "embeddings/s", "h2d_bytes_per_step": e2e_in,
                    "d2h_bytes_per_step": int(n_seq * cfg["head_out_dim"] * 4),
                    "path": "request dispatcher: shard_batch -> lg_stella_encode_ids_batch per rank -> all_gather_embeddings" if world > 1 else "lg_stella_encode_ids_batch"},
            "gpu_launches": launches * args.steps, "clocks": clocks, "device_status": status,
            "model_tflops": fl * args.steps / dt / 1e12, "model_frac_of_sustained_peak": fl * args.steps / dt / 1e12 / peaks["tf_sust"],
            "embedding_norm_check": float(np.abs(np.linalg.norm(emb, axis=1) - 1).max())}
    if world == 1 and not args.no_micro:
        mr = micro_rooflines(peaks, T, cfg)
        line["roofline"] = mr["gemm"]
        lm = [c for c in mr["gemv_grid"] if (c["n"], c["batch"]) == (151936, 1)][0]
        line["extra_rooflines"] = [lm, mr["paged"], mr["qlinear"]]
        line["gemv_grid"] = mr["gemv_grid"]
        line["gemv_fused_projections"] = mr["gemv_fused"]
    else:
        line["roofline"] = {"bound": "tensor", "achieved": fl * args.steps / dt / 1e12 / 1.0, "peak": peaks["tf_sust"], "unit": "TFLOP/s",
                            "frac": fl * args.steps / dt / 1e12 / peaks["tf_sust"], "traffic": None,
                            "note": "whole-forward FLOPs over whole-forward time (per-kernel rooflines are reported at N=1)"}
    model.close()
    del model, d_ids, d_cu, d_pos, d_out
    torch.cuda.empty_cache()
    if not args.no_extra:
        # decode tokens/s of the same metric, at every N: each rank runs the ragged step on its own batch
        # and serves its round-robin share of the request load
        extra = [ragged_step_measure(R, steps=max(5, min(args.steps, 20)), warmup=3, layers=args.layers),
                 serving_measure(R, n_req=args.extra_requests, max_seqs=args.extra_requests, arrival_rate=args.arrival_rate,
                                 prefill_budget=args.prefill_budget, chunked=not args.whole_prompts, layers=args.layers)]
        if world == 2:
            extra.append(serving_measure(R, n_req=32, max_seqs=32, arrival_rate=0.0, prefill_budget=args.prefill_budget,
                                         chunked=not args.whole_prompts, tp=2, layers=args.layers))
        line["extra_workloads"] = extra
    if rank == 0:
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(cfg, w, ids, cu)
        print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default 20; serving_sweep: 0 = the whole sweep)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override depth (development only; the reported configs are 28 / 48)")
    ap.add_argument("--profiler-range", action="store_true", help="bracket one extra untimed step with cudaProfilerStart/Stop")
    ap.add_argument("--no-micro", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the decode workloads of the default line")
    ap.add_argument("--ref-budget", type=float, default=150.0, help="--impl reference: seconds of timed CPU work (each step is a full batch)")
    ap.add_argument("--workload", default="stella", choices=["stella", "ragged_step", "serving_sweep"])
    ap.add_argument("--requests", type=int, default=96, help="serving_sweep: requests per GPU")
    ap.add_argument("--extra-requests", type=int, default=64, help="requests per GPU of the serving sample inside the default line")
    ap.add_argument("--max-seqs", type=int, default=256, help="serving_sweep: concurrent sequences per GPU")
    ap.add_argument("--arrival-rate", type=float, default=64.0, help="serving_sweep: Poisson arrivals per second per GPU")
    ap.add_argument("--tp", type=int, default=1, help="serving_sweep: tensor-parallel degree (ranks form one replica)")
    ap.add_argument("--prefill-budget", type=int, default=4096, help="serving_sweep: prompt tokens fed per step")
    ap.add_argument("--whole-prompts", action="store_true", help="serving_sweep: prefill every prompt whole in one step instead of in chunks")
    args = ap.parse_args()
    global PROFILER_RANGE
    PROFILER_RANGE = args.profiler_range
    if args.steps is None:
        args.steps = 0 if args.workload == "serving_sweep" else 20
    cfg = dict(STELLA_1_5B)
    if args.layers:
        cfg["n_layers"] = args.layers
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.workload != "stella":
            raise SystemExit("--impl reference measures the headline workload only")
        run_reference(args, cfg, rank, world)
        return
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    R = Ranks(rank, world, local)
    if args.workload == "serving_sweep":
        budget = args.prefill_budget if not args.whole_prompts else max(args.prefill_budget, 16384)
        line = serving_measure(R, n_req=args.requests, max_seqs=args.max_seqs, arrival_rate=args.arrival_rate, prefill_budget=budget,
                               chunked=not args.whole_prompts, tp=args.tp, layers=args.layers, steps_cap=args.steps,
                               warmup=max(args.warmup, 3), sample_clocks=True)
        if rank == 0:
            print(json.dumps(line))
    elif args.workload == "ragged_step":
        line = ragged_step_measure(R, steps=args.steps, warmup=args.warmup, layers=args.layers)
        if rank == 0:
            line.update({"warmup": max(args.warmup, 3), "higher_is_better": True, "vs_baseline": None, "data": "synthetic"})
            print(json.dumps(line))
    else:
        run_ours(args, cfg, R)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
