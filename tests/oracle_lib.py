"""ctypes access to the CPU oracle (test infrastructure; never imported by the package).

The oracle is the shared library built from ``oracle/*.cpp``. It restates the reference's
CPU arithmetic; every wrapper below names the reference function it stands for.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(_ROOT, "oracle", "liblogismos_oracle.so")

c_sz = C.c_size_t
f32p = C.POINTER(C.c_float)
u8p = C.POINTER(C.c_uint8)
u16p = C.POINTER(C.c_uint16)
u32p = C.POINTER(C.c_uint32)
i32p = C.POINTER(C.c_int32)
i64p = C.POINTER(C.c_int64)
i8p = C.POINTER(C.c_int8)


def _load():
    if not os.path.exists(_SO):
        subprocess.check_call(["make", "-C", os.path.join(_ROOT, "oracle")])
    lib = C.CDLL(_SO)
    lib.orc_stella_create.restype = C.c_void_p
    lib.orc_flatkv_create.restype = C.c_void_p
    lib.orc_flatkv_len_of.restype = C.c_long
    lib.orc_build_packing.restype = C.c_long
    lib.orc_physical_cores.restype = c_sz
    lib.orc_count_physical_cores_text.restype = c_sz
    lib.orc_greedy.restype = C.c_uint32
    return lib


lib = _load()


def P(a, t=f32p):
    """Pointer to a C-contiguous numpy array (or NULL for None)."""
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle wants C-contiguous arrays"
    return a.ctypes.data_as(t)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- cpu_f32 -----------------------------------------------------------------------------

def embed_lookup(weight, hidden, vocab, ids):
    weight, ids = f32(weight), np.ascontiguousarray(ids, dtype=np.uint32)
    out = np.empty(ids.size * hidden, np.float32)
    lib.orc_embed_lookup(P(weight), c_sz(hidden), c_sz(vocab), P(ids, u32p), c_sz(ids.size), P(out))
    return out


def rms_norm(x, w, rows, n, eps):
    x, w = f32(x), f32(w)
    y = np.empty(rows * n, np.float32)
    lib.orc_rms_norm(P(x), P(w), c_sz(rows), c_sz(n), C.c_float(eps), P(y))
    return y


class OraclePanic(Exception):
    """The reference would panic here (assert on shapes)."""


def _lin(fn, a, b, bias, m, n, k):
    a, b = f32(a).ravel(), f32(b).ravel()
    bias = None if bias is None else f32(bias).ravel()
    mn = m * n if m * n < (1 << 40) else 0
    c = np.empty(mn, np.float32)
    rc = fn(P(a), c_sz(a.size), P(b), c_sz(b.size), P(bias), c_sz(0 if bias is None else bias.size),
            c_sz(m), c_sz(n), c_sz(k), P(c))
    if rc:
        raise OraclePanic(rc)
    return c


def linear(a, b, bias, m, n, k):
    return _lin(lib.orc_linear, a, b, bias, m, n, k)


def linear_t(a, b, bias, m, n, k):
    return _lin(lib.orc_linear_t, a, b, bias, m, n, k)


def silu(x):
    x = f32(x)
    y = np.empty_like(x)
    lib.orc_silu(P(x), c_sz(x.size), P(y))
    return y


def hadamard(a, b):
    a, b = f32(a), f32(b)
    c = np.empty(max(a.size, b.size), np.float32)
    if lib.orc_hadamard(P(a), c_sz(a.size), P(b), c_sz(b.size), P(c)):
        raise OraclePanic("hadamard: mismatched operand lengths")
    return c[: a.size]


def softmax_last_dim(x, rows, n):
    x = f32(x)
    y = np.empty(rows * n, np.float32)
    lib.orc_softmax_last_dim(P(x), c_sz(rows), c_sz(n), P(y))
    return y


def mask_additive_in_place(scores, mask, rows, n):
    mask = np.ascontiguousarray(mask, dtype=np.uint8)
    if lib.orc_mask_additive_in_place(P(scores), c_sz(scores.size), P(mask, u8p), c_sz(mask.size), c_sz(rows), c_sz(n)):
        raise OraclePanic("not a multiple of mask_rows")


def rope_halves_in_place(x, cos, sin, rows, head_dim):
    cos, sin = f32(cos), f32(sin)
    lib.orc_rope_halves_in_place(P(x), P(cos), P(sin), c_sz(rows), c_sz(head_dim))


def build_rope_table_f32(seq, head_dim, theta):
    cos = np.empty(seq * head_dim // 2, np.float32)
    sin = np.empty_like(cos)
    lib.orc_build_rope_table_f32(c_sz(seq), c_sz(head_dim), C.c_double(theta), P(cos), P(sin))
    return cos, sin


def mean_pool_masked(h, mask, seq, hidden):
    h, mask = f32(h), np.ascontiguousarray(mask, dtype=np.uint8)
    out = np.empty(hidden, np.float32)
    lib.orc_mean_pool_masked(P(h), P(mask, u8p), c_sz(seq), c_sz(hidden), P(out))
    return out


def l2_normalize_in_place(v):
    lib.orc_l2_normalize_in_place(P(v), c_sz(v.size))


# ---- transformers ----------------------------------------------------------------------------

class AttnT(C.Structure):
    _fields_ = [("hidden", c_sz), ("n_heads", c_sz), ("n_kv_heads", c_sz), ("head_dim", c_sz)] + [
        (n, f32p) for n in ("wq", "bq", "wk", "bk", "wv", "bv", "wo")]


def attention_forward(w, hidden, n_heads, n_kv, head_dim, x, mask, cos_tab, sin_tab, max_seq, causal=False):
    """w: dict with wq,bq,wk,bk,wv,bv,wo (fp32 arrays). x [seq, hidden]."""
    x = f32(x)
    seq = x.size // hidden
    mask = np.ascontiguousarray(mask, dtype=np.uint8)
    keep = {k: f32(v) for k, v in w.items()}
    a = AttnT(hidden, n_heads, n_kv, head_dim, *[P(keep[n]) for n in ("wq", "bq", "wk", "bk", "wv", "bv", "wo")])
    out = np.empty(seq * hidden, np.float32)
    rc = lib.orc_attention_forward(C.byref(a), P(x), P(mask, u8p), c_sz(seq), P(cos_tab), P(sin_tab),
                                   c_sz(max_seq), C.c_int(int(causal)), P(out))
    if rc:
        raise ValueError(f"attention.forward shape error {rc}")
    return out.reshape(seq, hidden)


def sdpa(q, k, v, n_heads, n_kv, d, mask=None, causal=False):
    """attention.rs:217-299 on projected + rotated q [S, n_heads*d], k, v [S, n_kv*d] -> [S, n_heads*d]."""
    q, k, v = f32(q), f32(k), f32(v)
    seq = q.size // (n_heads * d)
    mask = np.ones(seq, np.uint8) if mask is None else np.ascontiguousarray(mask, dtype=np.uint8)
    out = np.empty((seq, n_heads * d), np.float32)
    if lib.orc_sdpa(P(q), P(k), P(v), P(mask, u8p), c_sz(seq), c_sz(n_heads), c_sz(n_kv), c_sz(d), C.c_int(int(causal)), P(out)):
        raise ValueError("sdpa shape error")
    return out


def transpose_seq_heads(x, seq, heads, d):
    x = f32(x); out = np.empty_like(x)
    lib.orc_transpose_seq_heads(P(x), c_sz(seq), c_sz(heads), c_sz(d), P(out))
    return out


def merge_heads(x, heads, seq, d):
    x = f32(x); out = np.empty_like(x)
    lib.orc_merge_heads(P(x), c_sz(heads), c_sz(seq), c_sz(d), P(out))
    return out


def repeat_kv(kv, n_kv, groups, seq, d):
    kv = f32(kv); out = np.empty(kv.size * groups, np.float32)
    lib.orc_repeat_kv(P(kv), c_sz(n_kv), c_sz(groups), c_sz(seq), c_sz(d), P(out))
    return out


def rope_gather(cos_tab, sin_tab, max_seq, head_dim, positions):
    pos = np.ascontiguousarray(positions, dtype=np.uint64)
    half = head_dim // 2
    c = np.empty(pos.size * half, np.float32); s = np.empty_like(c)
    if lib.orc_rope_gather(P(cos_tab), P(sin_tab), c_sz(max_seq), c_sz(head_dim),
                           pos.ctypes.data_as(C.POINTER(c_sz)), c_sz(pos.size), P(c), P(s)):
        raise ValueError("RopeTable::gather: position >= max_seq")
    return c, s


def swiglu_forward(w_gate, w_up, w_down, hidden, inter, x):
    x = f32(x); seq = x.size // hidden
    w_gate, w_up, w_down = f32(w_gate), f32(w_up), f32(w_down)
    out = np.empty(seq * hidden, np.float32)
    lib.orc_swiglu_forward(P(w_gate), P(w_up), P(w_down), c_sz(hidden), c_sz(inter), P(x), c_sz(seq), P(out))
    return out.reshape(seq, hidden)


# ---- Stella ------------------------------------------------------------------------------------

class LayerW(C.Structure):
    _fields_ = [(n, f32p) for n in ("norm1", "norm2", "wq", "bq", "wk", "bk", "wv", "bv", "wo",
                                    "w_gate", "w_up", "w_down")]


class StellaT(C.Structure):
    _fields_ = [(n, c_sz) for n in ("vocab", "hidden", "n_layers", "n_heads", "n_kv_heads",
                                    "intermediate", "max_pos", "head_out_dim")] + [
        ("rms_eps", C.c_float), ("rope_theta", C.c_double), ("tok_embed", f32p), ("final_norm", f32p),
        ("layers", C.POINTER(LayerW)), ("head_w", f32p), ("head_b", f32p)]


class OracleStella:
    """StellaEncoder + the embedding head of StellaModel::encode_raw, fp32 on the CPU.

    ``weights``: dict with tok_embed, final_norm, head_w, head_b and ``layers`` (list of dicts
    with the 12 per-layer tensors). Arrays must stay alive as long as the object does.
    """

    def __init__(self, cfg, weights):
        self.cfg = cfg
        self._keep = weights
        L = (LayerW * cfg["n_layers"])()
        for i, lw in enumerate(weights["layers"]):
            for n, _ in LayerW._fields_:
                assert lw[n].dtype == np.float32 and lw[n].flags["C_CONTIGUOUS"]
                setattr(L[i], n, P(lw[n]))
        self._layers = L
        d = StellaT(cfg["vocab"], cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"],
                    cfg["intermediate"], cfg["max_pos"], cfg["head_out_dim"], cfg["rms_eps"],
                    cfg["rope_theta"], P(weights["tok_embed"]), P(weights["final_norm"]), L,
                    P(weights["head_w"]), P(weights["head_b"]))
        self._h = C.c_void_p(lib.orc_stella_create(C.byref(d)))

    def __del__(self):
        if getattr(self, "_h", None):
            lib.orc_stella_destroy(self._h)
            self._h = None

    def forward(self, ids, mask=None, causal=False):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        mask = np.ones(ids.size, np.uint8) if mask is None else np.ascontiguousarray(mask, dtype=np.uint8)
        if mask.size != ids.size:
            raise ValueError("forward: ids.len() != mask.len()")
        out = np.empty((ids.size, self.cfg["hidden"]), np.float32)
        rc = lib.orc_stella_forward(self._h, P(ids, u32p), P(mask, u8p), c_sz(ids.size), C.c_int(int(causal)), P(out))
        if rc:
            raise ValueError(f"forward: shape error {rc}")
        return out

    def encode_raw(self, ids, mask=None):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        mask = np.ones(ids.size, np.uint8) if mask is None else np.ascontiguousarray(mask, dtype=np.uint8)
        out = np.empty(self.cfg["head_out_dim"], np.float32)
        rc = lib.orc_stella_encode_raw(self._h, P(ids, u32p), P(mask, u8p), c_sz(ids.size), P(out))
        if rc:
            raise ValueError(f"encode_raw: shape error {rc}")
        return out

    def encode_batch(self, ids, cu_seqlens, n_threads):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        cu = np.ascontiguousarray(cu_seqlens, dtype=np.int32)
        n = cu.size - 1
        out = np.empty((n, self.cfg["head_out_dim"]), np.float32)
        rc = lib.orc_stella_encode_batch(self._h, P(ids, u32p), P(cu, i32p), c_sz(n), c_sz(n_threads), P(out))
        if rc:
            raise ValueError(f"encode_batch: shape error {rc}")
        return out


def physical_cores():
    return int(lib.orc_physical_cores())


def count_physical_cores_text(text):
    return int(lib.orc_count_physical_cores_text(text.encode()))


# ---- gated delta rule ------------------------------------------------------------------------

def l2_norm_rows(x, k):
    lib.orc_l2_norm_rows(P(x), c_sz(x.size), c_sz(k))


def cumsum(g):
    g = f32(g); out = np.empty_like(g)
    lib.orc_cumsum(P(g), c_sz(g.size), P(out))
    return out


def gdn_recurrent_fwd(q, k, v, beta, g, scale, state_in, k_dim, v_dim):
    q, k, v, beta, g, state_in = map(f32, (q, k, v, beta, g, state_in))
    t = beta.size
    o = np.empty(t * v_dim, np.float32); s = np.empty(k_dim * v_dim, np.float32)
    lib.orc_gdn_recurrent_fwd(P(q), P(k), P(v), P(beta), P(g), c_sz(t), C.c_float(scale), P(state_in),
                              c_sz(k_dim), c_sz(v_dim), P(o), P(s))
    return o, s


def gdn_chunk_fwd(q, k, v, beta, g, scale, state_in, k_dim, v_dim, bt):
    q, k, v, beta, g, state_in = map(f32, (q, k, v, beta, g, state_in))
    t = beta.size
    nch = (t + bt - 1) // bt
    o = np.empty(t * v_dim, np.float32); s = np.empty((nch, k_dim * v_dim), np.float32)
    lib.orc_gdn_chunk_fwd(P(q), P(k), P(v), P(beta), P(g), c_sz(t), C.c_float(scale), P(state_in),
                          c_sz(k_dim), c_sz(v_dim), c_sz(bt), P(o), P(s))
    return o, s


def gdn_gates(a, b, A_log, dt_bias):
    a, b, A_log, dt_bias = map(f32, (a, b, A_log, dt_bias))
    t, heads = a.shape
    g = np.empty_like(a); beta = np.empty_like(a)
    lib.orc_gdn_gates(P(a), P(b), P(A_log), P(dt_bias), c_sz(t), c_sz(heads), P(g), P(beta))
    return g, beta


# ---- quant -------------------------------------------------------------------------------------

def pack_turbo4(idx):
    idx = np.ascontiguousarray(idx, dtype=np.uint8); out = np.empty(16, np.uint8)
    if lib.orc_pack_turbo4(P(idx, u8p), P(out, u8p)):
        raise ValueError("IndexOutOfRange")
    return out


def unpack_turbo4(packed):
    packed = np.ascontiguousarray(packed, dtype=np.uint8); out = np.empty(32, np.uint8)
    lib.orc_unpack_turbo4(P(packed, u8p), P(out, u8p))
    return out


def pack_turbo3(idx):
    idx = np.ascontiguousarray(idx, dtype=np.uint8); out = np.empty(12, np.uint8)
    if lib.orc_pack_turbo3(P(idx, u8p), P(out, u8p)):
        raise ValueError("IndexOutOfRange")
    return out


def unpack_turbo3(packed):
    packed = np.ascontiguousarray(packed, dtype=np.uint8); out = np.empty(32, np.uint8)
    lib.orc_unpack_turbo3(P(packed, u8p), P(out, u8p))
    return out


def int4_pack(codes):
    codes = np.ascontiguousarray(codes, dtype=np.int8)
    n, k = codes.shape
    out = np.empty((n, k // 2), np.uint8)
    if lib.orc_int4_pack(P(codes, i8p), c_sz(n), c_sz(k), P(out, u8p)):
        raise ValueError("int4 code out of [-8, 7]")
    return out


def int4_unpack(packed):
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    n, k2 = packed.shape
    out = np.empty((n, k2 * 2), np.int8)
    lib.orc_int4_unpack(P(packed, u8p), c_sz(n), c_sz(k2 * 2), P(out, i8p))
    return out


def int4_quantize(w):
    w = f32(w); n, k = w.shape
    packed = np.empty((n, k // 2), np.uint8); scales = np.empty((n, k // 32), np.uint16)
    lib.orc_int4_quantize(P(w), c_sz(n), c_sz(k), P(packed, u8p), P(scales, u16p))
    return packed, scales


def int4_dequant(packed, scales):
    n, k2 = packed.shape
    w = np.empty((n, k2 * 2), np.float32)
    lib.orc_int4_dequant(P(packed, u8p), P(scales, u16p), c_sz(n), c_sz(k2 * 2), P(w))
    return w


def int4_gemv(packed, scales, x):
    x = f32(x); batch, k = x.shape
    n = packed.shape[0]
    y = np.empty((batch, n), np.float32)
    lib.orc_int4_gemv(P(packed, u8p), P(scales, u16p), c_sz(n), c_sz(k), P(x), c_sz(batch), P(y))
    return y


# ---- caches --------------------------------------------------------------------------------------

class FlatKvCache:
    """crates/cache/src/flat.rs, at byte level (rows are little-endian element bytes)."""
    ERR = {1: "LayerOutOfRange", 2: "LenOverflow", 3: "ReadBeyondWritten", 4: "ShapeMismatch"}

    def __init__(self, num_layers, row_bytes, max_seq_len):
        self.row_bytes = row_bytes
        self._h = C.c_void_p(lib.orc_flatkv_create(c_sz(num_layers), c_sz(row_bytes), c_sz(max_seq_len)))

    def __del__(self):
        if getattr(self, "_h", None):
            lib.orc_flatkv_destroy(self._h); self._h = None

    def put(self, layer, k, v):
        k = np.ascontiguousarray(k).view(np.uint8).reshape(-1, self.row_bytes)
        v = np.ascontiguousarray(v).view(np.uint8).reshape(-1, self.row_bytes)
        if k.shape[0] != v.shape[0]:
            raise ValueError("ShapeMismatch")
        rc = lib.orc_flatkv_put(self._h, c_sz(layer), P(k, u8p), P(v, u8p), c_sz(k.shape[0]))
        if rc:
            raise ValueError(self.ERR[rc])

    def get(self, layer, n):
        k = np.empty((n, self.row_bytes), np.uint8); v = np.empty_like(k)
        rc = lib.orc_flatkv_get(self._h, c_sz(layer), c_sz(n), P(k, u8p), P(v, u8p))
        if rc:
            raise ValueError(self.ERR[rc])
        return k, v

    def len_of(self, layer):
        r = lib.orc_flatkv_len_of(self._h, c_sz(layer))
        return None if r < 0 else int(r)

    def reset(self):
        lib.orc_flatkv_reset(self._h)


def paged_append(k_pool, v_pool, block_size, table, pos, k_row, v_row):
    n_blocks = k_pool.shape[0]
    row_bytes = k_pool.strides[1] if k_pool.ndim == 3 else k_pool.shape[-1]
    table = np.ascontiguousarray(table, dtype=np.int32)
    k_row = np.ascontiguousarray(k_row).view(np.uint8); v_row = np.ascontiguousarray(v_row).view(np.uint8)
    rc = lib.orc_paged_append(P(k_pool, u8p), P(v_pool, u8p), c_sz(n_blocks), c_sz(block_size), c_sz(row_bytes),
                              P(table, i32p), c_sz(table.size), c_sz(pos), P(k_row, u8p), P(v_row, u8p))
    if rc:
        raise ValueError(f"paged_append error {rc}")


def paged_gather(k_pool, v_pool, block_size, table, n):
    n_blocks = k_pool.shape[0]
    row_bytes = k_pool.shape[-1]
    table = np.ascontiguousarray(table, dtype=np.int32)
    k = np.empty((n, row_bytes), np.uint8); v = np.empty_like(k)
    rc = lib.orc_paged_gather(P(k_pool, u8p), P(v_pool, u8p), c_sz(n_blocks), c_sz(block_size), c_sz(row_bytes),
                              P(table, i32p), c_sz(table.size), c_sz(n), P(k, u8p), P(v, u8p))
    if rc:
        raise ValueError(f"paged_gather error {rc}")
    return k, v


def decode_attention(q, k, v, n_heads, n_kv, d):
    q, k, v = f32(q), f32(k), f32(v)
    n = k.size // (n_kv * d)
    out = np.empty(n_heads * d, np.float32)
    lib.orc_decode_attention(P(q), P(k), P(v), c_sz(n), c_sz(n_heads), c_sz(n_kv), c_sz(d), P(out))
    return out


def build_packing(cached_lens, new_lens, tables, block_size, n_pool_blocks):
    cached = np.ascontiguousarray(cached_lens, dtype=np.int32)
    new = np.ascontiguousarray(new_lens, dtype=np.int32)
    tables = np.ascontiguousarray(tables, dtype=np.int32)
    n = cached.size
    total = int(new.sum())
    cu = np.empty(n + 1, np.int32); pos = np.empty(total, np.int32)
    slots = np.empty(total, np.int64); sid = np.empty(total, np.int32)
    r = lib.orc_build_packing(P(cached, i32p), P(new, i32p), c_sz(n), P(tables, i32p), c_sz(tables.shape[1]),
                              c_sz(block_size), c_sz(n_pool_blocks), P(cu, i32p), P(pos, i32p), P(slots, i64p),
                              P(sid, i32p))
    if r < 0:
        raise ValueError("build_packing: block table entry missing or out of range")
    return cu, pos, slots, sid


def greedy(logits):
    logits = f32(logits)
    return int(lib.orc_greedy(P(logits), c_sz(logits.size)))


# ---- fp16 references -----------------------------------------------------------------------------

def matmul_fp16_ref(a, b, m, n, k):
    a = np.ascontiguousarray(a, dtype=np.float16); b = np.ascontiguousarray(b, dtype=np.float16)
    d = np.empty((m, n), np.float16)
    lib.orc_matmul_fp16_ref(P(a, u16p), P(b, u16p), c_sz(m), c_sz(n), c_sz(k), P(d, u16p))
    return d


def rms_norm_fp16_ref(x, w, m, n, eps):
    x = np.ascontiguousarray(x, dtype=np.float16); w = np.ascontiguousarray(w, dtype=np.float16)
    y = np.empty((m, n), np.float16)
    lib.orc_rms_norm_fp16_ref(P(x, u16p), P(w, u16p), c_sz(m), c_sz(n), C.c_float(eps), P(y, u16p))
    return y


def softmax_fp16_ref(x, m, n):
    x = np.ascontiguousarray(x, dtype=np.float16)
    y = np.empty(m * n, np.float16)
    if lib.orc_softmax_fp16_ref(P(x, u16p), c_sz(x.size), c_sz(m), c_sz(n), P(y, u16p)):
        raise ValueError("UnsupportedShape: x.len() != m*n")
    return y.reshape(m, n)


def build_cos_sin_table(seq, head_dim, theta):
    t = np.empty(seq * head_dim, np.float32)
    lib.orc_build_cos_sin_table(c_sz(seq), c_sz(head_dim), C.c_float(theta), P(t))
    return t


def rope_apply_fp16_ref(qk, cos_sin, batch, seq, heads, head_dim):
    assert qk.dtype == np.float16
    if lib.orc_rope_apply_fp16_ref(P(qk, u16p), c_sz(qk.size), P(cos_sin), c_sz(cos_sin.size), c_sz(batch),
                                   c_sz(seq), c_sz(heads), c_sz(head_dim)):
        raise ValueError("UnsupportedShape")


def to_bf16_bits(x):
    x = f32(x); y = np.empty(x.shape, np.uint16)
    lib.orc_f32_to_bf16(P(x), c_sz(x.size), P(y, u16p))
    return y


def from_bf16_bits(x):
    x = np.ascontiguousarray(x, dtype=np.uint16); y = np.empty(x.shape, np.float32)
    lib.orc_bf16_to_f32(P(x, u16p), c_sz(x.size), P(y))
    return y


def bf16_round(x):
    """fp32 -> bf16 (round to nearest even) -> fp32."""
    return from_bf16_bits(to_bf16_bits(x))


class HybridLayerW(C.Structure):
    _fields_ = [("kind", C.c_int)] + [(n, f32p) for n in ("norm1", "norm2", "w_mix_in", "w_mix_out", "w_ab", "A_log", "dt_bias",
                                                          "w_gate", "w_up", "w_down")]


class HybridT(C.Structure):
    _fields_ = [(n, c_sz) for n in ("vocab", "hidden", "n_layers", "n_heads", "n_kv_heads", "attn_head_dim", "gdn_heads",
                                    "intermediate", "max_pos")] + [
        ("rms_eps", C.c_float), ("rope_theta", C.c_double), ("tok_embed", f32p), ("final_norm", f32p), ("lm_head", f32p),
        ("layers", C.POINTER(HybridLayerW))]


lib.orc_hybrid_create.restype = C.c_void_p
lib.orc_hybrid_create.argtypes = [C.c_void_p]
lib.orc_hybrid_destroy.argtypes = [C.c_void_p]
lib.orc_hybrid_destroy.restype = None
lib.orc_hybrid_forward.argtypes = [C.c_void_p, u32p, c_sz, f32p, f32p]
lib.orc_hybrid_forward.restype = C.c_int


class OracleHybrid:
    """The hybrid decoder stack on the CPU, one sequence per call, full recomputation.

    ``weights``: tok_embed, final_norm, lm_head (fp32) and ``layers``: dicts with kind (0 full
    attention, 1 linear attention), norm1, norm2, w_mix_in, w_mix_out, w_gate, w_up, w_down and, for
    kind 1, w_ab, A_log, dt_bias (row layouts as in oracle.h)."""

    def __init__(self, cfg, weights):
        self.cfg, self._keep = cfg, weights
        L = (HybridLayerW * cfg["n_layers"])()
        for i, lw in enumerate(weights["layers"]):
            L[i].kind = int(lw["kind"])
            for n, _ in HybridLayerW._fields_[1:]:
                if n in lw:
                    assert lw[n].dtype == np.float32 and lw[n].flags["C_CONTIGUOUS"]
                    setattr(L[i], n, P(lw[n]))
        self._layers = L
        d = HybridT(cfg["vocab"], cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"], cfg["attn_head_dim"],
                    cfg["gdn_heads"], cfg["intermediate"], cfg["max_pos"], cfg["rms_eps"], cfg["rope_theta"],
                    P(weights["tok_embed"]), P(weights["final_norm"]), P(weights["lm_head"]), L)
        self._h = C.c_void_p(lib.orc_hybrid_create(C.byref(d)))

    def __del__(self):
        if getattr(self, "_h", None):
            lib.orc_hybrid_destroy(self._h)
            self._h = None

    def forward(self, ids, logits=True):
        """(hidden [seq, hidden] after the final norm, logits [vocab] of the last token)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        hid = np.empty((ids.size, self.cfg["hidden"]), np.float32)
        lg = np.empty(self.cfg["vocab"], np.float32) if logits else None
        rc = lib.orc_hybrid_forward(self._h, P(ids, u32p), c_sz(ids.size), P(hid), P(lg) if logits else None)
        if rc:
            raise ValueError(f"hybrid forward: error {rc}")
        return hid, lg


# ---- crates/decode: logit processors and samplers --------------------------------------------

lib.orc_multinomial.restype = C.c_uint32
lib.orc_top_k.argtypes = [f32p, c_sz, c_sz]
lib.orc_temperature.argtypes = [f32p, c_sz, C.c_float]
lib.orc_top_p.argtypes = [f32p, c_sz, C.c_float]
lib.orc_min_p.argtypes = [f32p, c_sz, C.c_float]
lib.orc_repetition_penalty.argtypes = [f32p, c_sz, u32p, c_sz, C.c_float]
lib.orc_multinomial.argtypes = [f32p, c_sz, C.c_float]


def temperature(logits, t):
    """TemperatureScale::process (crates/decode/src/processors.rs:18-28) on a copy of one row."""
    x = f32(logits).copy(); lib.orc_temperature(P(x), c_sz(x.size), C.c_float(t)); return x


def top_k(logits, k):
    """TopK::process (processors.rs:50-82)."""
    x = f32(logits).copy(); lib.orc_top_k(P(x), c_sz(x.size), c_sz(k)); return x


def top_p(logits, p):
    """TopP::process (processors.rs:89-122)."""
    x = f32(logits).copy(); lib.orc_top_p(P(x), c_sz(x.size), C.c_float(p)); return x


def min_p(logits, p):
    """MinP::process (processors.rs:130-146)."""
    x = f32(logits).copy(); lib.orc_min_p(P(x), c_sz(x.size), C.c_float(p)); return x


def repetition_penalty(logits, tokens, penalty):
    """RepetitionPenalty::process (processors.rs:160-181)."""
    x = f32(logits).copy()
    t = np.ascontiguousarray(tokens, dtype=np.uint32)
    lib.orc_repetition_penalty(P(x), c_sz(x.size), P(t, u32p), c_sz(t.size), C.c_float(penalty))
    return x


def multinomial(logits, u):
    """MultinomialSampler::sample (crates/decode/src/sampler.rs:31-58) for the uniform draw u."""
    x = f32(logits)
    return int(lib.orc_multinomial(P(x), c_sz(x.size), C.c_float(u)))


# ---- TurboQuant 3-bit head codec (crates/quant/src/lib.rs:90-114, :316-413) ----------------------

def fwht_128(x):
    d = f32(x).copy(); assert d.size == 128
    lib.orc_fwht_128(P(d)); return d


def turbo3_encode(values):
    """[..., 128] fp32 -> [..., 56] uint8 (four 14-byte blocks per 128-value head chunk)."""
    v = f32(values).reshape(-1, 128)
    out = np.empty((v.shape[0], 56), np.uint8)
    for i in range(v.shape[0]):
        lib.orc_turbo3_encode_head(P(v[i]), P(out[i], u8p))
    return out.reshape(np.shape(values)[:-1] + (56,))


def turbo3_decode(blocks):
    b = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1, 56)
    out = np.empty((b.shape[0], 128), np.float32)
    for i in range(b.shape[0]):
        lib.orc_turbo3_decode_head(P(b[i], u8p), P(out[i]))
    return out.reshape(np.shape(blocks)[:-1] + (128,))
