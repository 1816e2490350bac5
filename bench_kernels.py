"""Per-kernel microbenchmarks on one GPU (the quantized GEMV and paged-decode benchmark
configurations, and the model's GEMM shapes), each launch timed with CUDA events on the launch
stream, operands rotated over several copies so that every launch reads from HBM.

  python bench_kernels.py gemv  [--n N --k K --batch B --iters I]
  python bench_kernels.py gemm  [--m M --n N --k K --epi bf16|resid|swiglu --iters I]
  python bench_kernels.py qlinear [--m M --n N --k K --iters I]   (m <= 256, fused int4 dequant)
  python bench_kernels.py qdense  [--m M --n N --k K --iters I]   (bf16 expansion + dense GEMM)
  python bench_kernels.py gdn     [--seqs S --len L]                 (token-serial vs chunk-parallel)
  python bench_kernels.py paged [--seqs S --min-ctx A --max-ctx B --chunk C --iters I]
  python bench_kernels.py attn  [--seqs S --len L --iters I]
  python bench_kernels.py prefix [--seqs S --len CHUNK --prefix P --turbo3]   (prefill chunks over a cached, paged prefix)
  python bench_kernels.py sampling [--seqs ROWS --n VOCAB]           (sampling chain over fp32 logits)
  python bench_kernels.py sweep          (every benchmark shape, one JSON line each)

Prints one JSON line per case: achieved GB/s or TFLOP/s, the measured peak it is compared with
(MEASURED_PEAKS.json next to the package, else the documented fallback) and the fraction.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from logismos_b200 import ops  # noqa: E402
from logismos_b200._lib import lib  # noqa: E402
from logismos_b200 import timing  # noqa: E402
from logismos_b200.timing import timeit  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm": d["hbm_gbs"], "tf": d["bf16_tflops"], "src": "measured"}
    return {"hbm": 6650.0, "tf": 1590.0, "src": "fallback"}


def bench_gemv(n, k, batch, iters, copies=None, pk=None):
    pk = pk or peaks()
    wbytes = n * k // 2 + n * (k // 32) * 2
    copies = copies or max(2, min(16, int(300e6 // wbytes) + 1))  # > 256 MB of distinct weights in rotation
    codes = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda") for _ in range(copies)]
    scales = [(torch.rand((n, k // 32), device="cuda") * 0.02).to(torch.float16) for _ in range(copies)]
    x = torch.randn((batch, k), device="cuda").to(torch.bfloat16)
    y = torch.empty((batch, n), dtype=torch.bfloat16, device="cuda")
    t = timeit(lambda i: ops.gemv_int4(codes[i % copies], scales[i % copies], x, out=y, sync=False), iters)
    t_l2 = timeit(lambda i: ops.gemv_int4(codes[0], scales[0], x, out=y, sync=False), iters)
    by = wbytes + batch * k * 2 + batch * n * 2
    return {"kernel": "gemv_int4_g32", "n": n, "k": k, "batch": batch, "bytes": by, "us": t * 1e6, "GBps": by / t / 1e9,
            "frac_hbm": by / t / 1e9 / pk["hbm"], "us_l2_resident": t_l2 * 1e6, "GBps_l2_resident": by / t_l2 / 1e9,
            "TFLOPs": 2.0 * batch * n * k / t / 1e12, "peak": pk["hbm"], "peak_src": pk["src"], "weight_copies": copies}


def bench_qlinear(m, n, k, iters, copies=None, pk=None):
    """Fused-dequant tensor-core linear for m <= 256 tokens, accumulating into fp32."""
    pk = pk or peaks()
    wbytes = n * k // 2 + n * (k // 32) * 2
    copies = copies or max(2, min(16, int(300e6 // wbytes) + 1))
    codes = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda") for _ in range(copies)]
    scales = [(torch.rand((n, k // 32), device="cuda") * 0.02).to(torch.float16) for _ in range(copies)]
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    acc = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def run(i):
        ops.check(lib.logismos_launch_qlinear_int4_g32_acc_f32(x.data_ptr(), codes[i % copies].data_ptr(), scales[i % copies].data_ptr(),
                                                               acc.data_ptr(), m, n, k, k, n, status.data_ptr(),
                                                               torch.cuda.current_stream().cuda_stream), "qlinear")
    t = timeit(run, iters)
    by = wbytes + m * k * 2 + m * n * 4
    fl = 2.0 * m * n * k
    return {"kernel": "qlinear_int4_tcgen05", "m": m, "n": n, "k": k, "bytes": by, "us": t * 1e6, "GBps": by / t / 1e9,
            "frac_hbm": by / t / 1e9 / pk["hbm"], "TFLOPs": fl / t / 1e12, "frac_tensor": fl / t / 1e12 / pk["tf"],
            "device_status": int(status.item()), "peak_src": pk["src"], "weight_copies": copies}


def bench_qdense(m, n, k, iters, copies=None, pk=None):
    """The dense route for more rows: expand the int4 matrix to bf16, then the tcgen05 GEMM (fp32 accumulate epilogue)."""
    pk = pk or peaks()
    wbytes = n * k // 2 + n * (k // 32) * 2
    copies = copies or max(2, min(16, int(300e6 // wbytes) + 1))
    codes = [torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device="cuda") for _ in range(copies)]
    scales = [(torch.rand((n, k // 32), device="cuda") * 0.02).to(torch.float16) for _ in range(copies)]
    x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    acc = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    w = torch.empty((n, k), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def run(i):
        s = torch.cuda.current_stream().cuda_stream
        ops.check(lib.logismos_launch_dequant_int4_g32_bf16(codes[i % copies].data_ptr(), scales[i % copies].data_ptr(), w.data_ptr(), n, k, s), "dequant")
        ops.check(lib.logismos_launch_linear_t_bf16(x.data_ptr(), w.data_ptr(), None, acc.data_ptr(), m, n, k, k, n, 1, status.data_ptr(), s), "linear_t")
    t = timeit(run, iters)
    fl = 2.0 * m * n * k
    return {"kernel": "dequant_int4 + linear_t_tcgen05", "m": m, "n": n, "k": k, "us": t * 1e6, "TFLOPs": fl / t / 1e12,
            "GBps": (wbytes + m * k * 2 + m * n * 4) / t / 1e9, "frac_hbm": 0.0, "device_status": int(status.item())}


def bench_gdn(n_seq, length, iters, heads=16, pk=None):
    """Gated delta rule over n_seq sequences of `length` tokens (16 heads of 128 x 128 fp32 state): the
    token-serial kernel and the chunk-parallel kernel on the same inputs."""
    pk = pk or peaks()
    D, T = 128, n_seq * length
    mk = lambda: torch.randn((T, heads, D), device="cuda").to(torch.bfloat16)
    q, k, v, z = mk(), mk(), mk(), mk()
    q = torch.nn.functional.normalize(q.float(), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(k.float(), dim=-1).to(torch.bfloat16)
    g = -torch.rand((T, heads), device="cuda") * 0.1
    beta = torch.rand((T, heads), device="cuda")
    cu = torch.arange(0, T + 1, length, dtype=torch.int32, device="cuda")
    st = torch.zeros((n_seq, heads, D, D), device="cuda")
    t_serial = timeit(lambda i: ops.gdn_prefill_(st, q, k, v, g, beta, cu, D ** -0.5, gate_z=z, sync=False), iters)
    out = {"kernel": "gated_delta_rule", "seqs": n_seq, "len": length, "heads": heads, "us_token_serial": t_serial * 1e6,
           "state_GBps_token_serial": 2.0 * n_seq * heads * D * D * 4 / t_serial / 1e9, "peak": pk["hbm"], "peak_src": pk["src"]}
    if length > 1:
        scratch = torch.empty(int(lib.logismos_gdn_chunked_scratch_bytes(T, n_seq, heads)), dtype=torch.uint8, device="cuda")
        t_chunk = timeit(lambda i: ops.gdn_chunked_(st, q, k, v, g, beta, cu, D ** -0.5, gate_z=z, sync=False, scratch=scratch), iters)
        t_one = timeit(lambda i: ops.gdn_chunked_(st, q, k, v, g, beta, cu, D ** -0.5, gate_z=z, sync=False, split=False), iters)
        out.update({"us_chunk_parallel": t_chunk * 1e6, "us_chunk_parallel_one_launch": t_one * 1e6, "us_per_token_chunk_parallel": t_chunk * 1e6 / length,
                    "us_per_token_serial": t_serial * 1e6 / length, "speedup": t_serial / t_chunk})
    else:
        out["frac_hbm_token_serial"] = out["state_GBps_token_serial"] / pk["hbm"]
    return out


def bench_gemm(m, n, k, epi, iters, pk=None):
    pk = pk or peaks()
    a = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    copies = 4
    ws = [(torch.randn((n, k), device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
    res = torch.zeros((m, n), dtype=torch.float32, device="cuda") if epi == "resid" else None

    def run(i):
        if epi == "resid":
            ops.linear_t(a, ws[i % copies], residual=res, sync=False)
        else:
            ops.linear_t(a, ws[i % copies], swiglu=(epi == "swiglu"), sync=False)
    t = timeit(run, iters)
    fl = 2.0 * m * n * k
    return {"kernel": "linear_t_tcgen05", "m": m, "n": n, "k": k, "epilogue": epi, "flops": fl, "us": t * 1e6, "TFLOPs": fl / t / 1e12,
            "frac_tensor": fl / t / 1e12 / pk["tf"], "peak": pk["tf"], "peak_src": pk["src"] + " burst"}


def paged_case(seqs, min_ctx, max_ctx, seed=3):
    rng = np.random.default_rng(seed)
    ctx = np.exp(rng.uniform(np.log(min_ctx), np.log(max_ctx), seqs)).round().astype(np.int64)
    nb = (ctx + 15) // 16
    n_pool = int(nb.sum())
    perm = rng.permutation(n_pool).astype(np.int32)
    tables = np.zeros((seqs, int(nb.max())), np.int32)
    o = 0
    for s in range(seqs):
        tables[s, :nb[s]] = perm[o:o + nb[s]]
        o += nb[s]
    return ctx, tables, n_pool


def bench_paged(seqs, min_ctx, max_ctx, chunk, iters, n_heads=16, n_kv=2, pk=None, d=128):
    pk = pk or peaks()
    ctx, tables, n_pool = paged_case(seqs, min_ctx, max_ctx)
    row = n_kv * d
    kp = torch.randn((n_pool, 16, row), device="cuda").to(torch.bfloat16)
    vp = torch.randn((n_pool, 16, row), device="cuda").to(torch.bfloat16)
    q = torch.randn((seqs, n_heads * d), device="cuda").to(torch.bfloat16)
    nk = torch.randn((seqs, row), device="cuda").to(torch.bfloat16)
    nv = torch.randn((seqs, row), device="cuda").to(torch.bfloat16)
    if chunk <= 0:
        chunk = ops.pick_decode_chunk(ctx.astype(np.int32), n_kv, d)
    off, total = ops.build_decode_chunks(ctx.astype(np.int32), chunk)
    d_tab, d_ctx, d_off = torch.from_numpy(tables).cuda(), torch.from_numpy(ctx.astype(np.int32)).cuda(), off.cuda()
    scratch = torch.empty(int(lib.logismos_paged_decode_scratch_bytes(total, n_heads, d)), dtype=torch.uint8, device="cuda")
    t = timeit(lambda i: ops.paged_attention_decode(q, kp, vp, nk, nv, d_tab, d_ctx, d_off, total, chunk, n_heads, n_kv, d,
                                                    scratch=scratch, sync=False), iters)
    by = float(ctx.sum()) * row * 2 * 2 + seqs * (n_heads * d * 2 * 2 + row * 2 * 2) + tables.size * 4
    return {"kernel": "paged_attention_decode+merge", "seqs": seqs, "context_tokens": int(ctx.sum()), "pool_blocks": n_pool,
            "head_dim": d, "chunk_tokens": chunk, "total_chunks": total, "bytes": by, "us": t * 1e6, "GBps": by / t / 1e9,
            "frac_hbm": by / t / 1e9 / pk["hbm"], "scratch_bytes": scratch.numel(), "peak": pk["hbm"], "peak_src": pk["src"]}


def bench_attn(seqs, length, iters, n_heads=12, n_kv=2):
    d = 128
    T = seqs * length
    qkv = torch.randn((T, (n_heads + 2 * n_kv) * d), device="cuda").to(torch.bfloat16)
    cu = torch.arange(0, T + 1, length, dtype=torch.int32, device="cuda")
    t = timeit(lambda i: ops.varlen_attention(qkv, cu, n_heads, n_kv, d, max_seqlen=length, sync=False), iters)
    scratch = torch.empty(int(lib.logismos_varlen_attention_tc_scratch_bytes(T, seqs, n_kv, d)), dtype=torch.uint8, device="cuda")
    t_tc = timeit(lambda i: ops.varlen_attention_tc(qkv, cu, n_heads, n_kv, max_seqlen=length, sync=False, scratch=scratch), iters)
    fl = 4.0 * n_heads * d * length * length * seqs
    return {"kernel": "varlen_attention", "seqs": seqs, "len": length, "flops": fl, "us_mma_sync": t * 1e6, "TFLOPs_mma_sync": fl / t / 1e12,
            "us_tcgen05": t_tc * 1e6, "TFLOPs_tcgen05": fl / t_tc / 1e12}


def bench_prefix(seqs, chunk, prefix, iters, n_heads=12, n_kv=2, d=128, turbo3=False):
    """Causal attention of `seqs` prefill chunks of `chunk` tokens, each continuing a cached prefix of `prefix`
    tokens read through block tables (gather launch + attention launch), bf16 or TurboQuant 3-bit pool rows."""
    kv_len = prefix + chunk
    nb = (kv_len + 15) // 16
    T = seqs * chunk
    row = n_kv * d
    g = torch.Generator(device="cpu").manual_seed(5)
    tables = torch.randperm(seqs * nb, generator=g).to(torch.int32).reshape(seqs, nb).cuda()
    if turbo3:
        rb = int(lib.logismos_turbo3_row_bytes(row))
        kp = torch.randint(0, 256, (seqs * nb, 16, rb), dtype=torch.uint8, device="cuda")
        vp = torch.randint(0, 256, (seqs * nb, 16, rb), dtype=torch.uint8, device="cuda")
        kp[..., 0::14] = 0; kp[..., 1::14] = 0x3c; vp[..., 0::14] = 0; vp[..., 1::14] = 0x3c   # fp16 norm 1.0 in every block header
    else:
        kp = torch.randn((seqs * nb, 16, row), device="cuda").to(torch.bfloat16)
        vp = torch.randn((seqs * nb, 16, row), device="cuda").to(torch.bfloat16)
    q = torch.randn((T, n_heads * d), device="cuda").to(torch.bfloat16)
    cu = torch.arange(0, T + 1, chunk, dtype=torch.int32, device="cuda")
    kv = torch.full((seqs,), kv_len, dtype=torch.int32, device="cuda")
    out = torch.empty((T, n_heads * d), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(int(lib.logismos_paged_prefix_attention_scratch_bytes(seqs * kv_len, seqs, n_kv, d)), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = lib.logismos_launch_paged_prefix_attention_turbo3_bf16 if turbo3 else lib.logismos_launch_paged_prefix_attention_tc_bf16

    def run(i):
        ops.check(fn(q.data_ptr(), q.shape[1], cu.data_ptr(), kv.data_ptr(), kp.data_ptr(), vp.data_ptr(), tables.data_ptr(), nb, seqs * nb,
                     out.data_ptr(), scratch.data_ptr(), T, seqs * kv_len, seqs, chunk, kv_len, n_heads, n_kv, d, status.data_ptr(),
                     torch.cuda.current_stream().cuda_stream), "paged_prefix_attention")
    t = timeit(run, iters)
    fl = 4.0 * n_heads * d * seqs * (chunk * prefix + chunk * (chunk + 1) / 2.0)
    return {"kernel": "paged_prefix_attention" + ("_turbo3" if turbo3 else ""), "seqs": seqs, "chunk": chunk, "prefix": prefix, "us": t * 1e6,
            "TFLOPs": fl / t / 1e12, "gathered_bytes": 2 * seqs * kv_len * row * 2, "device_status": int(status.item())}


def bench_sampling(rows, vocab, iters):
    """The device sampling chain over fp32 logits [rows, vocab]: time per launch of each processor and of the sampler."""
    from logismos_b200 import sampling as S
    base = torch.randn((rows, vocab), device="cuda") * 3.0
    work = base.clone()
    uni = torch.rand((rows,), device="cuda")
    tok = torch.empty((rows,), dtype=torch.int32, device="cuda")
    st = lambda: torch.cuda.current_stream().cuda_stream
    out = {"kernel": "sampling", "rows": rows, "vocab": vocab, "logit_bytes": rows * vocab * 4}

    def timed(name, fn):
        def run(i):
            work.copy_(base)
            fn()
        def ref(i):
            work.copy_(base)
        out["us_" + name] = (timeit(run, iters) - timeit(ref, iters)) * 1e6
    timed("temperature", lambda: ops.check(lib.logismos_launch_temperature_f32(work.data_ptr(), rows, vocab, 0.8, st()), "temperature"))
    timed("top_k_50", lambda: ops.check(lib.logismos_launch_top_k_f32(work.data_ptr(), rows, vocab, 50, st()), "top_k"))
    timed("top_p_0.95", lambda: ops.check(lib.logismos_launch_top_p_f32(work.data_ptr(), rows, vocab, 0.95, st()), "top_p"))
    timed("min_p_0.05", lambda: ops.check(lib.logismos_launch_min_p_f32(work.data_ptr(), rows, vocab, 0.05, st()), "min_p"))
    timed("multinomial", lambda: ops.check(lib.logismos_launch_multinomial_f32(work.data_ptr(), rows, vocab, uni.data_ptr(), tok.data_ptr(), st()), "multinomial"))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(prog="bench_kernels.py")
    ap.add_argument("what", choices=["gemv", "gemm", "qlinear", "qdense", "gdn", "paged", "attn", "prefix", "sampling", "sweep"])
    ap.add_argument("--m", type=int, default=2176)
    ap.add_argument("--n", type=int, default=151936)
    ap.add_argument("--k", type=int, default=1536)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--epi", default="bf16", choices=["bf16", "resid", "swiglu"])
    ap.add_argument("--seqs", type=int, default=256)
    ap.add_argument("--len", type=int, default=512)
    ap.add_argument("--min-ctx", type=int, default=128)
    ap.add_argument("--max-ctx", type=int, default=32768)
    ap.add_argument("--chunk", type=int, default=0, help="paged: tokens per chunk; 0 = the library's choice for the contexts")
    ap.add_argument("--head-dim", type=int, default=128, help="paged: 128 or 256")
    ap.add_argument("--prefix", type=int, default=2048, help="prefix: cached tokens in front of every chunk of --len tokens")
    ap.add_argument("--turbo3", action="store_true", help="prefix: TurboQuant 3-bit pool rows")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-graph", action="store_true", help="time back-to-back launches from Python instead of a CUDA graph")
    a = ap.parse_args(argv)
    timing.USE_GRAPH = not a.no_graph
    if a.what == "gemv":
        print(json.dumps(bench_gemv(a.n, a.k, a.batch, a.iters)))
    elif a.what == "gemm":
        print(json.dumps(bench_gemm(a.m, a.n, a.k, a.epi, a.iters)))
    elif a.what == "gdn":
        print(json.dumps(bench_gdn(a.seqs, a.len, min(a.iters, 5))))
    elif a.what == "qdense":
        print(json.dumps(bench_qdense(a.m, a.n, a.k, a.iters)))
    elif a.what == "qlinear":
        print(json.dumps(bench_qlinear(a.m, a.n, a.k, a.iters)))
    elif a.what == "paged":
        print(json.dumps(bench_paged(a.seqs, a.min_ctx, a.max_ctx, a.chunk, a.iters, d=a.head_dim)))
    elif a.what == "attn":
        print(json.dumps(bench_attn(a.seqs, a.len, a.iters)))
    elif a.what == "prefix":
        print(json.dumps(bench_prefix(a.seqs, a.len, a.prefix, a.iters, turbo3=a.turbo3)))
    elif a.what == "sampling":
        print(json.dumps(bench_sampling(a.seqs, a.n, a.iters)))
    else:
        pk = peaks()
        for (n, k) in [(1536, 1536), (8960, 1536), (1536, 8960), (151936, 1536)]:
            for b in (1, 4, 16, 64):
                print(json.dumps(bench_gemv(n, k, b, a.iters, pk=pk)), flush=True)
        for (n, k) in [(8192, 2048), (2048, 2048), (12288, 2048), (2048, 6144), (151936, 2048)]:
            for m in (16, 64, 128, 256):
                print(json.dumps(bench_qlinear(m, n, k, a.iters, pk=pk)), flush=True)
        print(json.dumps(bench_paged(256, 128, 32768, 512, 10, pk=pk)), flush=True)
        for (n, k, epi) in [(2048, 1536, "bf16"), (1536, 1536, "resid"), (17920, 1536, "swiglu"), (1536, 8960, "resid")]:
            print(json.dumps(bench_gemm(a.m, n, k, epi, a.iters, pk=pk)), flush=True)
        print(json.dumps(bench_attn(8, 512, a.iters)), flush=True)


if __name__ == "__main__":
    main()
