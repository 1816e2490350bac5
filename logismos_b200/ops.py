"""Tensor-level ops over the CUDA launchers: the mirror of the reference's op layer
(crates/praxis/src/{matmul,norm,softmax,rope}.rs) plus the ops this build adds in the same style.

Rules kept from the reference (crates/praxis/src/matmul.rs:31-82, :154-166):
  * inputs are immutable, the output is freshly allocated;
  * dtype, rank and contiguity are checked and reported as ``InvalidOp``;
  * there is no silent transfer: a CPU operand is an ``InvalidOp`` (the GPU build has no CPU arm);
  * an op synchronises its stream before returning (crates/praxis/src/stream_pool.rs:11-21) unless
    ``sync=False`` is passed by a caller that times kernels itself.
torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import check, lib


class InvalidOp(ValueError):
    """praxis::Error::Invalid"""


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(0) if t is None else C.c_void_p(t.data_ptr())


def _req(t, name, dtype, rank=None, contiguous=True):
    if not isinstance(t, torch.Tensor):
        raise InvalidOp(f"{name}: not a tensor")
    if t.device.type != "cuda":
        raise InvalidOp(f"{name}: operands must all be on the same CUDA device (no CPU arm, no implicit transfer)")
    if t.dtype != dtype:
        raise InvalidOp(f"{name}: expected {dtype}, got {t.dtype}")
    if rank is not None and t.dim() != rank:
        raise InvalidOp(f"{name}: expected rank {rank}, got {t.dim()}")
    if contiguous and not t.is_contiguous():
        raise InvalidOp(f"{name}: must be contiguous")


def _same_device(*ts):
    devs = {t.device for t in ts if t is not None}
    if len(devs) > 1:
        raise InvalidOp("operands must be on the same CUDA device")


def _done(sync):
    if sync:
        torch.cuda.current_stream().synchronize()


# ---- the reference's four ops (fp16) ---------------------------------------------------------

def matmul(a, b, sync=True):
    """praxis::matmul (matmul.rs:30-168): D = A @ B, fp16 rank-2; tensor-core variant when every
    dim is a multiple of 16, else the naive kernel (:113-117)."""
    _req(a, "a", torch.float16, 2); _req(b, "b", torch.float16, 2); _same_device(a, b)
    m, k = a.shape
    k2, n = b.shape
    if k != k2:
        raise InvalidOp(f"matmul: inner dims differ ({k} vs {k2})")
    d = torch.zeros((m, n), dtype=torch.float16, device=a.device)
    with torch.cuda.device(a.device):
        fn = lib.logismos_launch_matmul_wmma_fp16 if (m % 16 == 0 and n % 16 == 0 and k % 16 == 0) \
            else lib.logismos_launch_matmul_naive_fp16
        check(fn(_p(a), _p(b), _p(d), m, n, k, _stream()), "matmul_fp16")
        _done(sync)
    return d


def rms_norm(x, w, eps, sync=True):
    """praxis::rms_norm (norm.rs:28-122)."""
    _req(x, "x", torch.float16, 2); _req(w, "w", torch.float16, 1); _same_device(x, w)
    if w.shape[0] != x.shape[1]:
        raise InvalidOp("rms_norm: weight length != row length")
    y = torch.zeros_like(x)
    with torch.cuda.device(x.device):
        check(lib.logismos_launch_rms_norm_fp16(_p(x), _p(w), _p(y), x.shape[0], x.shape[1], float(eps), _stream()), "rms_norm_fp16")
        _done(sync)
    return y


def softmax(x, sync=True):
    """praxis::softmax (softmax.rs:25-86): row softmax over the last dim of a rank-2 tensor."""
    _req(x, "x", torch.float16, 2)
    y = torch.zeros_like(x)
    with torch.cuda.device(x.device):
        check(lib.logismos_launch_softmax_fp16(_p(x), _p(y), x.shape[0], x.shape[1], _stream()), "softmax_fp16")
        _done(sync)
    return y


def rope_apply(x, cos_sin, sync=True):
    """praxis::rope_apply (rope.rs:102-208): interleaved-pair RoPE on (B,S,H,D) fp16 with an fp32
    (S,D) table; returns a rotated copy (the input is left untouched)."""
    _req(x, "x", torch.float16, 4); _req(cos_sin, "cos_sin", torch.float32, 2); _same_device(x, cos_sin)
    b, s, h, d = x.shape
    if tuple(cos_sin.shape) != (s, d):
        raise InvalidOp("rope_apply: table must be (seq, head_dim)")
    y = x.clone()
    with torch.cuda.device(x.device):
        check(lib.logismos_launch_rope_fp16(_p(y), _p(cos_sin), b, s, h, d, _stream()), "rope_fp16")
        _done(sync)
    return y


# ---- encoder path ----------------------------------------------------------------------------

EPI_BF16, EPI_RESID_F32, EPI_SWIGLU = 0, 1, 2
EPI_STATIC_W = 0x100       # or-ed into the epilogue: nothing in flight writes the weights
GDN_STATIC_STATE = 0x100   # or-ed into the gdn_prefill mode: nothing in flight writes the states


def embed_lookup(table, ids, sync=True):
    _req(table, "table", torch.bfloat16, 2); _req(ids, "ids", torch.int32, 1)
    out = torch.empty((ids.shape[0], table.shape[1]), dtype=torch.float32, device=table.device)
    with torch.cuda.device(table.device):
        check(lib.logismos_launch_embed_lookup_bf16(_p(table), _p(ids), _p(out), ids.shape[0], table.shape[1], table.shape[0], _stream()), "embed_lookup")
        _done(sync)
    return out


def rms_norm_f32(x, w, eps, out_f32=False, sync=True):
    _req(x, "x", torch.float32, 2); _req(w, "w", torch.float32, 1)
    y = torch.empty(x.shape, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.logismos_launch_rms_norm_f32(_p(x), _p(w), _p(y), x.shape[0], x.shape[1], float(eps), int(out_f32), _stream()), "rms_norm_f32")
        _done(sync)
    return y


def linear_t(a, w, bias=None, residual=None, swiglu=False, naive=False, sync=True, static_w=False):
    """C = A W^T (+bias). residual: fp32 tensor updated in place (returns it). swiglu: W holds gate/up
    rows interleaved in blocks of 32; returns silu(gate)*up. static_w: the caller's promise that nothing
    still in flight writes w (the kernel may then fetch weights before the preceding kernel has finished)."""
    _req(a, "a", torch.bfloat16, 2); _req(w, "w", torch.bfloat16, 2)
    if bias is not None:
        _req(bias, "bias", torch.float32, 1)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise InvalidOp("linear_t: inner dims differ")
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    if residual is not None:
        _req(residual, "residual", torch.float32, 2)
        out, epi, ldc = residual, EPI_RESID_F32, n
    elif swiglu:
        out, epi, ldc = torch.empty((m, n // 2), dtype=torch.bfloat16, device=a.device), EPI_SWIGLU, n // 2
    else:
        out, epi, ldc = torch.empty((m, n), dtype=torch.bfloat16, device=a.device), EPI_BF16, n
    with torch.cuda.device(a.device):
        if naive:
            check(lib.logismos_launch_linear_t_naive_bf16(_p(a), _p(w), _p(bias), _p(out), m, n, k, k, ldc, epi, _stream()), "linear_t_naive")
        else:
            check(lib.logismos_launch_linear_t_bf16(_p(a), _p(w), _p(bias), _p(out), m, n, k, k, ldc, epi | (EPI_STATIC_W if static_w else 0),
                                                    _p(status), _stream()), "linear_t")
        _done(sync)
        if sync and not naive and int(status.item()) != 0:
            raise InvalidOp(f"linear_t: device status {int(status.item())} (a bounded wait expired)")
    return out


def rope_halves_(qk, cos, sin, positions, n_rot_heads, head_dim, sync=True):
    """In-place halves-RoPE on the first n_rot_heads heads of each row of qk [tokens, row_stride]."""
    _req(qk, "qk", torch.bfloat16, 2); _req(cos, "cos", torch.float32, 2); _req(sin, "sin", torch.float32, 2)
    _req(positions, "positions", torch.int32, 1)
    status = torch.zeros(1, dtype=torch.int32, device=qk.device)
    with torch.cuda.device(qk.device):
        check(lib.logismos_launch_rope_halves_bf16(_p(qk), _p(cos), _p(sin), _p(positions), qk.shape[0], n_rot_heads, head_dim,
                                                   qk.shape[1], cos.shape[0], _p(status), _stream()), "rope_halves")
        _done(sync)
        if sync and int(status.item()) != 0:
            raise InvalidOp("RopeTable::gather: position >= max_seq")
    return qk


def swiglu(gu, sync=True):
    _req(gu, "gu", torch.bfloat16, 2)
    inter = gu.shape[1] // 2
    out = torch.empty((gu.shape[0], inter), dtype=torch.bfloat16, device=gu.device)
    with torch.cuda.device(gu.device):
        check(lib.logismos_launch_swiglu_bf16(_p(gu), _p(out), gu.shape[0], inter, _stream()), "swiglu")
        _done(sync)
    return out


def varlen_attention_tc(qkv, cu_seqlens, n_heads, n_kv_heads, causal=False, max_seqlen=None, sync=True, scratch=None, status=None,
                        head_dim=128):
    """Ragged-batch attention at head_dim 128 or 256 on the tcgen05 tensor cores (same layout contract as
    varlen_attention). Returns out bf16 [n_tokens, n_heads * head_dim]."""
    _req(qkv, "qkv", torch.bfloat16, 2); _req(cu_seqlens, "cu_seqlens", torch.int32, 1)
    n_seqs, T, D = cu_seqlens.shape[0] - 1, qkv.shape[0], head_dim
    if max_seqlen is None:
        max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item()) if n_seqs > 0 else 0
    out = torch.empty((T, n_heads * D), dtype=torch.bfloat16, device=qkv.device)
    if scratch is None:
        scratch = torch.empty(max(256, int(lib.logismos_varlen_attention_tc_scratch_bytes(T, n_seqs, n_kv_heads, D))), dtype=torch.uint8, device=qkv.device)
    with torch.cuda.device(qkv.device):
        check(lib.logismos_launch_varlen_attention_tc_bf16(_p(qkv), _p(cu_seqlens), _p(out), _p(scratch), T, n_seqs, max_seqlen, n_heads,
                                                           n_kv_heads, D, qkv.shape[1], n_heads * D, (n_heads + n_kv_heads) * D,
                                                           int(causal), _p(status) if status is not None else None, _stream()), "varlen_attention_tc")
        _done(sync)
    return out


def paged_prefix_attention(q, cu_seqlens_q, kv_lens, k_pool, v_pool, block_tables, n_heads, n_kv_heads, head_dim, sync=True,
                           status=None, turbo3=False):
    """Causal attention of prefill chunks that continue cached sequences: the queries of sequence s are
    rows cu_seqlens_q[s]..cu_seqlens_q[s+1] of q (q heads at column 0), its kv_lens[s] keys and values
    (cached prefix + the chunk itself, already stored) are read from the paged pools through
    block_tables. Returns out bf16 [n_q_tokens, n_heads * head_dim]."""
    _req(q, "q", torch.bfloat16, 2); _req(cu_seqlens_q, "cu_seqlens_q", torch.int32, 1); _req(kv_lens, "kv_lens", torch.int32, 1)
    pool_dt = torch.uint8 if turbo3 else torch.bfloat16   # turbo3: TurboQuant 3-bit rows (paged_kv_store_turbo3)
    _req(k_pool, "k_pool", pool_dt, 3); _req(v_pool, "v_pool", pool_dt, 3); _req(block_tables, "block_tables", torch.int32, 2)
    n_seqs, T, D = kv_lens.shape[0], q.shape[0], head_dim
    cu = cu_seqlens_q.cpu(); kv = kv_lens.cpu()
    max_q = int((cu[1:] - cu[:-1]).max().item()) if n_seqs > 0 else 0
    total_kv, max_kv = (int(kv.sum().item()), int(kv.max().item())) if n_seqs > 0 else (0, 0)
    out = torch.empty((T, n_heads * D), dtype=torch.bfloat16, device=q.device)
    scratch = torch.empty(max(256, int(lib.logismos_paged_prefix_attention_scratch_bytes(total_kv, n_seqs, n_kv_heads, D))),
                          dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        fn = lib.logismos_launch_paged_prefix_attention_turbo3_bf16 if turbo3 else lib.logismos_launch_paged_prefix_attention_tc_bf16
        check(fn(_p(q), q.shape[1], _p(cu_seqlens_q), _p(kv_lens), _p(k_pool), _p(v_pool),
                                                                 _p(block_tables), block_tables.shape[1], k_pool.shape[0], _p(out),
                                                                 _p(scratch), T, total_kv, n_seqs, max_q, max_kv, n_heads, n_kv_heads, D,
                                                                 _p(status) if status is not None else None, _stream()),
              "paged_prefix_attention")
        _done(sync)
    return out


def rope_varlen_attention_tc_(qkv, cos, sin, positions, cu_seqlens, n_heads, n_kv_heads, causal=False, max_seqlen=None, sync=True,
                             scratch=None, status=None, head_dim=128):
    """halves-RoPE of the q and k heads of qkv (in place) fused into the first launch of varlen_attention_tc."""
    _req(qkv, "qkv", torch.bfloat16, 2); _req(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _req(cos, "cos", torch.float32, 2); _req(sin, "sin", torch.float32, 2); _req(positions, "positions", torch.int32, 1)
    n_seqs, T, D = cu_seqlens.shape[0] - 1, qkv.shape[0], head_dim
    if max_seqlen is None:
        max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item()) if n_seqs > 0 else 0
    out = torch.empty((T, n_heads * D), dtype=torch.bfloat16, device=qkv.device)
    if scratch is None:
        scratch = torch.empty(max(256, int(lib.logismos_varlen_attention_tc_scratch_bytes(T, n_seqs, n_kv_heads, D))), dtype=torch.uint8, device=qkv.device)
    with torch.cuda.device(qkv.device):
        check(lib.logismos_launch_rope_varlen_attention_tc_bf16(_p(qkv), _p(cos), _p(sin), _p(positions), n_heads + n_kv_heads, cos.shape[0],
                                                                _p(cu_seqlens), _p(out), _p(scratch), T, n_seqs, max_seqlen, n_heads, n_kv_heads, D,
                                                                qkv.shape[1], n_heads * D, (n_heads + n_kv_heads) * D, int(causal),
                                                                _p(status) if status is not None else None, _stream()), "rope_varlen_attention_tc")
        _done(sync)
    return out


def varlen_attention(qkv, cu_seqlens, n_heads, n_kv_heads, head_dim, causal=False, max_seqlen=None, sync=True):
    _req(qkv, "qkv", torch.bfloat16, 2); _req(cu_seqlens, "cu_seqlens", torch.int32, 1)
    n_seqs = cu_seqlens.shape[0] - 1
    if max_seqlen is None:
        max_seqlen = int((cu_seqlens[1:] - cu_seqlens[:-1]).max().item()) if n_seqs > 0 else 0
    out = torch.empty((qkv.shape[0], n_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    with torch.cuda.device(qkv.device):
        check(lib.logismos_launch_varlen_attention_bf16(_p(qkv), _p(cu_seqlens), _p(out), n_seqs, max_seqlen, n_heads, n_kv_heads,
                                                        head_dim, qkv.shape[1], n_heads * head_dim,
                                                        (n_heads + n_kv_heads) * head_dim, int(causal), _stream()), "varlen_attention")
        _done(sync)
    return out


def pool_head(hidden, cu_seqlens, head_w, head_b, sync=True):
    _req(hidden, "hidden", torch.float32, 2); _req(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _req(head_w, "head_w", torch.bfloat16, 2); _req(head_b, "head_b", torch.float32, 1)
    n_seqs = cu_seqlens.shape[0] - 1
    out = torch.empty((n_seqs, head_w.shape[0]), dtype=torch.float32, device=hidden.device)
    scratch = torch.empty((n_seqs, hidden.shape[1]), dtype=torch.float32, device=hidden.device)
    with torch.cuda.device(hidden.device):
        check(lib.logismos_launch_pool_head_f32(_p(hidden), _p(cu_seqlens), _p(head_w), _p(head_b), _p(out), _p(scratch), n_seqs, hidden.shape[1],
                                                head_w.shape[0], _stream()), "pool_head")
        _done(sync)
    return out


# ---- decode path -----------------------------------------------------------------------------

def gemv_int4(codes, scales, x, out=None, sync=True, out_f32=False):
    """y = x @ dequant(codes, scales)^T. codes u8 [n, k/2], scales f16 [n, k/32], x bf16 [b, k]; y bf16, or
    the unrounded fp32 accumulators with ``out_f32`` (what the lm_head hands to the argmax)."""
    _req(codes, "codes", torch.uint8, 2); _req(scales, "scales", torch.float16, 2); _req(x, "x", torch.bfloat16, 2)
    n, k = codes.shape[0], codes.shape[1] * 2
    if x.shape[1] != k or tuple(scales.shape) != (n, k // 32):
        raise InvalidOp("gemv_int4: shape mismatch")
    y = out if out is not None else torch.empty((x.shape[0], n), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    if y.dtype != (torch.float32 if out_f32 else torch.bfloat16):
        raise InvalidOp("gemv_int4: out has the wrong dtype")
    fn = lib.logismos_launch_gemv_int4_g32_f32 if out_f32 else lib.logismos_launch_gemv_int4_g32_bf16
    with torch.cuda.device(x.device):
        check(fn(_p(codes), _p(scales), _p(x), _p(y), x.shape[0], n, k, _stream()), "gemv_int4_g32")
        _done(sync)
    return y


def skinny_int4(codes, scales, x, workspace, out=None, status=None, sync=True):
    """y = x @ dequant(codes, scales)^T for 1..64 rows with the kernel chosen by shape and row count
    (``lib.logismos_skinny_int4_route``: streaming GEMV, or the fused-dequant tensor-core linear above 16
    rows, for k >= 3 n, and from 8 rows up to n = 16384). ``workspace``: fp32 CUDA tensor of at least
    batch * n elements, all zero on entry; it is left all zero."""
    _req(codes, "codes", torch.uint8, 2); _req(scales, "scales", torch.float16, 2); _req(x, "x", torch.bfloat16, 2)
    _req(workspace, "workspace", torch.float32, None)
    n, k = codes.shape[0], codes.shape[1] * 2
    if x.shape[1] != k or tuple(scales.shape) != (n, k // 32) or workspace.numel() < x.shape[0] * n:
        raise InvalidOp("skinny_int4: shape mismatch")
    y = out if out is not None else torch.empty((x.shape[0], n), dtype=torch.bfloat16, device=x.device)
    st = status if status is not None else torch.zeros(1, dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.logismos_launch_skinny_int4_g32_bf16(_p(codes), _p(scales), _p(x), _p(y), x.shape[0], n, k, _p(workspace), _p(st), _stream()),
              "skinny_int4_g32")
        _done(sync)
    return y


def dequant_int4(codes, scales, sync=True):
    """codes u8 [n, k/2], scales f16 [n, k/32] -> bf16 [n, k] = bf16(scale * code)."""
    _req(codes, "codes", torch.uint8, 2); _req(scales, "scales", torch.float16, 2)
    n, k = codes.shape[0], codes.shape[1] * 2
    out = torch.empty((n, k), dtype=torch.bfloat16, device=codes.device)
    with torch.cuda.device(codes.device):
        check(lib.logismos_launch_dequant_int4_g32_bf16(_p(codes), _p(scales), _p(out), n, k, _stream()), "dequant_int4_g32")
        _done(sync)
    return out


def qlinear_int4_acc_(acc, a, codes, scales, sync=True, static_w=False):
    """acc f32 [m, n] += a bf16 [m, k] @ dequant(codes, scales)[n, k]^T for m <= 256 (fused dequant on
    the tensor cores). Rows of a and acc may be strided. Returns the device status word's tensor.
    static_w: the caller's promise that nothing still in flight writes codes or scales."""
    _req(a, "a", torch.bfloat16, 2, contiguous=False); _req(acc, "acc", torch.float32, 2, contiguous=False)
    _req(codes, "codes", torch.uint8, 2); _req(scales, "scales", torch.float16, 2)
    m, k = a.shape
    n = codes.shape[0]
    if codes.shape[1] * 2 != k or scales.shape != (n, k // 32) or acc.shape != (m, n) or a.stride(1) != 1 or acc.stride(1) != 1:
        raise InvalidOp("qlinear_int4_acc_: shape mismatch")
    if not (1 <= m <= 256) or k % 256:
        raise InvalidOp("qlinear_int4_acc_: needs 1 <= m <= 256 and k % 256 == 0")
    status = torch.zeros(1, dtype=torch.int32, device=a.device)
    with torch.cuda.device(a.device):
        fn = lib.logismos_launch_qlinear_int4_g32_acc_f32_static if static_w else lib.logismos_launch_qlinear_int4_g32_acc_f32
        check(fn(_p(a), _p(codes), _p(scales), _p(acc), m, n, k, a.stride(0), acc.stride(0), _p(status), _stream()), "qlinear_int4_g32")
        _done(sync)
    return status


def qlinear_finish(acc, bias=None, swiglu=False, sync=True):
    """bf16 [m, n] = acc (+ bias), or SwiGLU over the 32-interleaved gate/up columns -> [m, n/2]; zeroes acc."""
    _req(acc, "acc", torch.float32, 2)
    m, n = acc.shape
    out = torch.empty((m, n // 2 if swiglu else n), dtype=torch.bfloat16, device=acc.device)
    with torch.cuda.device(acc.device):
        check(lib.logismos_launch_qlinear_finish_bf16(_p(acc), _p(bias) if bias is not None else None, _p(out), m, n, n, out.shape[1],
                                                      int(swiglu), _stream()), "qlinear_finish")
        _done(sync)
    return out


def pick_decode_chunk(context_lens_host, n_kv_heads, head_dim) -> int:
    """Host helper: tokens per decode chunk for one step's contexts (512, 1024 or 2048)."""
    cl = torch.as_tensor(context_lens_host, dtype=torch.int32).contiguous()
    return int(lib.logismos_pick_decode_chunk(C.c_void_p(cl.data_ptr()), cl.numel(), n_kv_heads, head_dim))


def build_decode_chunks(context_lens_host, chunk_tokens):
    """Host helper: (chunk_offsets int32 CPU tensor [n+1], total_chunks)."""
    cl = torch.as_tensor(context_lens_host, dtype=torch.int32).contiguous()
    off = torch.empty(cl.numel() + 1, dtype=torch.int32)
    total = lib.logismos_build_decode_chunks(C.c_void_p(cl.data_ptr()), cl.numel(), chunk_tokens, C.c_void_p(off.data_ptr()))
    if total < 0:
        raise InvalidOp("build_decode_chunks: bad arguments")
    return off, int(total)


def paged_attention_decode(q, k_pool, v_pool, new_k, new_v, block_tables, context_lens, chunk_offsets, total_chunks,
                           chunk_tokens, n_heads, n_kv_heads, head_dim, scratch=None, sync=True):
    _req(q, "q", torch.bfloat16, 2); _req(k_pool, "k_pool", torch.bfloat16, 3); _req(v_pool, "v_pool", torch.bfloat16, 3)
    _req(block_tables, "block_tables", torch.int32, 2); _req(context_lens, "context_lens", torch.int32, 1)
    _req(chunk_offsets, "chunk_offsets", torch.int32, 1)
    n_seqs = q.shape[0]
    need = lib.logismos_paged_decode_scratch_bytes(total_chunks, n_heads, head_dim)
    if scratch is None:
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    elif scratch.numel() * scratch.element_size() < need:
        raise InvalidOp("paged_attention_decode: scratch too small")
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=q.device)
    with torch.cuda.device(q.device):
        check(lib.logismos_launch_paged_attention_decode_bf16(
            _p(q), _p(k_pool), _p(v_pool), _p(new_k), _p(new_v), _p(block_tables), _p(context_lens), _p(chunk_offsets),
            _p(out), _p(scratch), _p(status), n_seqs, total_chunks, chunk_tokens, block_tables.shape[1], k_pool.shape[0],
            n_heads, n_kv_heads, head_dim, _stream()), "paged_attention_decode")
        _done(sync)
        if sync and int(status.item()) != 0:
            raise InvalidOp("paged_attention_decode: a block id fell outside the pool")
    return out


def paged_kv_store(k, v, k_pool, v_pool, slot_mapping, sync=True):
    _req(k, "k", torch.bfloat16, 2); _req(v, "v", torch.bfloat16, 2); _req(slot_mapping, "slot_mapping", torch.int64, 1)
    status = torch.zeros(1, dtype=torch.int32, device=k.device)
    row = k_pool.shape[-1]
    with torch.cuda.device(k.device):
        check(lib.logismos_launch_paged_kv_store_bf16(_p(k), _p(v), k.shape[1], _p(k_pool), _p(v_pool), _p(slot_mapping), k.shape[0], row,
                                                      k_pool.shape[0] * k_pool.shape[1], _p(status), _stream()), "paged_kv_store")
        _done(sync)
        if sync and int(status.item()) != 0:
            raise InvalidOp("paged_kv_store: slot outside the pool")


def paged_kv_store_turbo3(k, v, k_pool, v_pool, slot_mapping, sync=True):
    """KvCache::put into TurboQuant 3-bit pools (uint8 [n_blocks, 16, row_elems / 128 * 56])."""
    _req(k, "k", torch.bfloat16, 2); _req(v, "v", torch.bfloat16, 2); _req(slot_mapping, "slot_mapping", torch.int64, 1)
    _req(k_pool, "k_pool", torch.uint8, 3); _req(v_pool, "v_pool", torch.uint8, 3)
    status = torch.zeros(1, dtype=torch.int32, device=k.device)
    row = k.shape[1]
    if k_pool.shape[-1] != lib.logismos_turbo3_row_bytes(row):
        raise InvalidOp("paged_kv_store_turbo3: pool rows must hold row_elems / 128 chunks of 56 bytes")
    with torch.cuda.device(k.device):
        check(lib.logismos_launch_paged_kv_store_turbo3(_p(k), _p(v), k.stride(0), _p(k_pool), _p(v_pool), _p(slot_mapping), k.shape[0], row,
                                                        k_pool.shape[0] * k_pool.shape[1], _p(status), _stream()), "paged_kv_store_turbo3")
        _done(sync)
        if sync and int(status.item()) != 0:
            raise InvalidOp("paged_kv_store_turbo3: slot outside the pool")


def paged_kv_gather_turbo3(k_pool, v_pool, block_table, length, row_elems, sync=True):
    """KvCache::get from TurboQuant 3-bit pools: decoded bf16 [length, row_elems] K and V."""
    _req(block_table, "block_table", torch.int32, 1); _req(k_pool, "k_pool", torch.uint8, 3)
    ko = torch.empty((length, row_elems), dtype=torch.bfloat16, device=k_pool.device)
    vo = torch.empty_like(ko)
    status = torch.zeros(1, dtype=torch.int32, device=k_pool.device)
    with torch.cuda.device(k_pool.device):
        check(lib.logismos_launch_paged_kv_gather_turbo3(_p(k_pool), _p(v_pool), _p(block_table), block_table.shape[0], length, row_elems,
                                                         k_pool.shape[0], _p(ko), _p(vo), _p(status), _stream()), "paged_kv_gather_turbo3")
        _done(sync)
        if sync and int(status.item()) != 0:
            raise InvalidOp("paged_kv_gather_turbo3: block id outside the pool")
    return ko, vo


def paged_kv_gather(k_pool, v_pool, block_table, length, sync=True):
    _req(block_table, "block_table", torch.int32, 1)
    row = k_pool.shape[-1]
    ko = torch.empty((length, row), dtype=torch.bfloat16, device=k_pool.device)
    vo = torch.empty_like(ko)
    status = torch.zeros(1, dtype=torch.int32, device=k_pool.device)
    with torch.cuda.device(k_pool.device):
        check(lib.logismos_launch_paged_kv_gather_bf16(_p(k_pool), _p(v_pool), _p(block_table), block_table.shape[0], length, row,
                                                       k_pool.shape[0], _p(ko), _p(vo), _p(status), _stream()), "paged_kv_gather")
        _done(sync)
        if sync and int(status.item()) != 0:
            raise InvalidOp("paged_kv_gather: block table entry missing or outside the pool")
    return ko, vo


def gdn_decode_step_(state, q, k, v, g, beta, scale, sync=True):
    """One gated-delta-rule decode step; state f32 [n_seqs, heads, 128, 128] is updated in place."""
    _req(state, "state", torch.float32, 4); _req(q, "q", torch.bfloat16, 3); _req(k, "k", torch.bfloat16, 3)
    _req(v, "v", torch.bfloat16, 3); _req(g, "g", torch.float32, 2); _req(beta, "beta", torch.float32, 2)
    if tuple(state.shape[2:]) != (128, 128):
        raise InvalidOp("gdn: head_dim must be 128")
    o = torch.empty_like(v)
    with torch.cuda.device(state.device):
        check(lib.logismos_launch_gdn_decode_step(_p(state), _p(q), _p(k), _p(v), _p(g), _p(beta), _p(o), state.shape[0], state.shape[1],
                                                  float(scale), _stream()), "gdn_decode_step")
        _done(sync)
    return o


def gdn_prefill_(state, q, k, v, g, beta, cu_seqlens, scale, gate_z=None, mode=0, sync=True, static_state=False):
    """Gated delta rule over a ragged batch; q, k, v bf16 [T, heads, 128]; state updated in place.
    gate_z bf16 [T, heads, 128] (optional) multiplies the output by silu(z) in the same pass.
    static_state: the caller's promise that nothing still in flight writes state or cu_seqlens."""
    _req(state, "state", torch.float32, 4); _req(q, "q", torch.bfloat16, 3); _req(k, "k", torch.bfloat16, 3)
    _req(v, "v", torch.bfloat16, 3); _req(g, "g", torch.float32, 2); _req(beta, "beta", torch.float32, 2)
    _req(cu_seqlens, "cu_seqlens", torch.int32, 1)
    if tuple(state.shape[2:]) != (128, 128) or state.shape[0] != cu_seqlens.shape[0] - 1:
        raise InvalidOp("gdn_prefill: state must be [n_seqs, heads, 128, 128]")
    o = torch.empty_like(v)
    with torch.cuda.device(state.device):
        check(lib.logismos_launch_gdn_prefill(_p(state), _p(q), _p(k), _p(v), _p(g), _p(beta), _p(o), _p(gate_z) if gate_z is not None else None, _p(cu_seqlens), _p(None), _p(None),
                                              state.shape[0], state.shape[1], q.shape[1] * q.shape[2], float(scale),
                                              int(mode) | (GDN_STATIC_STATE if static_state else 0), _stream()), "gdn_prefill")
        _done(sync)
    return o


def gdn_chunked_(state, q, k, v, g, beta, cu_seqlens, scale, gate_z=None, sync=True, scratch=None, split=True):
    """Chunk-parallel gated delta rule over a ragged batch (same arguments and results as gdn_prefill_,
    to tensor-core precision); state updated in place. split: the two-launch form (state-independent part
    of all chunks at once, then the chains) through ``scratch`` (uint8 CUDA tensor, allocated here when
    None); split=False: the one-launch form."""
    _req(state, "state", torch.float32, 4); _req(q, "q", torch.bfloat16, 3); _req(k, "k", torch.bfloat16, 3)
    _req(v, "v", torch.bfloat16, 3); _req(g, "g", torch.float32, 2); _req(beta, "beta", torch.float32, 2)
    _req(cu_seqlens, "cu_seqlens", torch.int32, 1)
    if tuple(state.shape[2:]) != (128, 128) or state.shape[0] != cu_seqlens.shape[0] - 1:
        raise InvalidOp("gdn_chunked: state must be [n_seqs, heads, 128, 128]")
    o = torch.empty_like(v)
    n_tokens = q.shape[0]
    if split and scratch is None:
        scratch = torch.empty(max(128, int(lib.logismos_gdn_chunked_scratch_bytes(n_tokens, state.shape[0], state.shape[1]))),
                              dtype=torch.uint8, device=state.device)
    with torch.cuda.device(state.device):
        check(lib.logismos_launch_gdn_chunked(_p(state), _p(q), _p(k), _p(v), _p(g), _p(beta), _p(o), _p(gate_z) if gate_z is not None else None,
                                              _p(cu_seqlens), _p(None), _p(None), state.shape[0], state.shape[1], q.shape[1] * q.shape[2],
                                              float(scale), _p(scratch) if split else None, n_tokens, _stream()), "gdn_chunked")
        _done(sync)
    return o


def gdn_prepare_(q, k, a, b, A_log, dt_bias, sync=True):
    """L2-normalises q, k head rows in place and returns (g, beta) fp32 [T, heads]."""
    _req(q, "q", torch.bfloat16, 3); _req(k, "k", torch.bfloat16, 3); _req(a, "a", torch.float32, 2); _req(b, "b", torch.float32, 2)
    _req(A_log, "A_log", torch.float32, 1); _req(dt_bias, "dt_bias", torch.float32, 1)
    g = torch.empty_like(a); beta = torch.empty_like(a)
    with torch.cuda.device(q.device):
        check(lib.logismos_launch_gdn_prepare(_p(q), _p(k), _p(a), _p(b), _p(A_log), _p(dt_bias), _p(g), _p(beta), q.shape[0], q.shape[1],
                                              q.shape[1] * q.shape[2], a.shape[1], _stream()), "gdn_prepare")
        _done(sync)
    return g, beta


def greedy(logits, sync=True):
    """decode::greedy per row: first maximum wins, NaN never selected."""
    if logits.dtype not in (torch.float32, torch.bfloat16):
        raise InvalidOp("greedy: logits must be f32 or bf16")
    _req(logits, "logits", logits.dtype, 2)
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    with torch.cuda.device(logits.device):
        check(lib.logismos_launch_greedy_argmax(_p(logits), int(logits.dtype == torch.float32), _p(out), logits.shape[0], logits.shape[1], _stream()), "greedy_argmax")
        _done(sync)
    return out
