"""Hybrid decoder step (gated-delta-rule linear-attention layers interleaved with gated
full-attention layers, int4 group-32 weights) over the C ABI (``lg_hybrid_*``), with the host-side
slot allocator for the recurrent states.

The reference has no decoder model (crates/decoders is an empty scaffold); the recurrence is
crates/kernels/src/gated_delta_rule/cpu.rs:92-182 and the contract is "a packed step equals running
every sequence alone".
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Sequence

import numpy as np

from ._lib import lib
from .decoder import _Q, _f, _fp, _q
from .embed import ComputeError, InputTooLong


class _Cfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("vocab", "hidden", "n_layers", "n_heads", "n_kv_heads", "attn_head_dim", "gdn_heads",
                                         "intermediate", "max_pos", "full_attn_interval")] + [
        ("rms_eps", C.c_float), ("rope_theta", C.c_double)] + [
        (n, C.c_int32) for n in ("n_pool_blocks", "max_blocks_per_seq", "max_step_tokens", "max_step_seqs", "n_state_slots", "keep_bf16_copy")]


_QNAMES = ("wq", "wk", "wv", "wgate", "wo", "wa", "wb")
_MLP = ("w_gate", "w_up", "w_down")


class _LayerW(C.Structure):
    _fields_ = [("norm1", _fp), ("norm2", _fp)] + [(n, _Q) for n in _QNAMES] + [("A_log", _fp), ("dt_bias", _fp)] + [
        (n, _Q) for n in _MLP]


class _Weights(C.Structure):
    _fields_ = [("tok_embed", _fp), ("final_norm", _fp), ("layers", C.POINTER(_LayerW)), ("lm_head", _Q)]


def is_full_attention(layer: int, interval: int) -> bool:
    return (layer + 1) % interval == 0


class SlotAllocator:
    """Recurrent-state slots: one per live sequence."""

    def __init__(self, n_slots: int):
        self.free: List[int] = list(range(n_slots - 1, -1, -1))
        self.slots: Dict[int, int] = {}

    def get(self, seq_id: int) -> int:
        if seq_id not in self.slots:
            if not self.free:
                raise MemoryError("state slots exhausted")
            self.slots[seq_id] = self.free.pop()
        return self.slots[seq_id]

    def release(self, seq_id: int):
        s = self.slots.pop(seq_id, None)
        if s is not None:
            self.free.append(s)


class HybridModel:
    """weights: tok_embed, final_norm (fp32), lm_head=(codes, scales), ``layers``: list of dicts with
    norm1, norm2 (fp32), wq, wk, wv, wgate, wo and w_gate, w_up, w_down as (codes, scales) pairs, and
    for linear-attention layers wa, wb pairs plus A_log, dt_bias (fp32 [gdn_heads])."""

    def __init__(self, cfg: dict, weights: dict, n_pool_blocks: int, max_blocks_per_seq: int, max_step_tokens: int,
                 max_step_seqs: int, n_state_slots: int, device: int = 0, keep_bf16_copy: bool = True):
        c = _Cfg(cfg["vocab"], cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"], cfg["attn_head_dim"],
                 cfg["gdn_heads"], cfg["intermediate"], cfg["max_pos"], cfg["full_attn_interval"], cfg["rms_eps"],
                 cfg["rope_theta"], n_pool_blocks, max_blocks_per_seq, max_step_tokens, max_step_seqs, n_state_slots, int(keep_bf16_copy))
        L = (_LayerW * max(1, cfg["n_layers"]))()
        for i, lw in enumerate(weights["layers"]):
            L[i].norm1, L[i].norm2 = _f(lw["norm1"]), _f(lw["norm2"])
            for n in _QNAMES + _MLP:
                if n in lw:
                    setattr(L[i], n, _q(lw[n]))
            if "A_log" in lw:
                L[i].A_log, L[i].dt_bias = _f(lw["A_log"]), _f(lw["dt_bias"])
        w = _Weights(_f(weights["tok_embed"]), _f(weights["final_norm"]), L, _q(weights["lm_head"]))
        self._keep = weights
        h = C.c_void_p()
        if lib.lg_hybrid_create(device, C.byref(c), C.byref(w), C.byref(h)):
            raise ComputeError(lib.lg_last_error().decode())
        self._h, self.cfg, self.max_blocks = h, cfg, max_blocks_per_seq
        self.max_step_tokens, self.device = max_step_tokens, device

    def close(self):
        if getattr(self, "_h", None):
            lib.lg_hybrid_destroy(self._h)
            self._h = None

    __del__ = close

    def step(self, ids: Sequence[int], cached_lens, new_lens, block_tables, state_slots) -> np.ndarray:
        """One packed step; returns the greedy next token of every sequence (uint32 [n_seqs])."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        cached = np.ascontiguousarray(cached_lens, dtype=np.int32)
        new = np.ascontiguousarray(new_lens, dtype=np.int32)
        tables = np.ascontiguousarray(block_tables, dtype=np.int32)
        slots = np.ascontiguousarray(state_slots, dtype=np.int32)
        n = cached.size
        assert new.size == n and slots.size == n and tables.shape == (n, self.max_blocks) and ids.size == int(new.sum())
        out = np.empty(n, np.uint32)
        P = lambda a: a.ctypes.data_as(C.c_void_p)
        rc = lib.lg_hybrid_step(self._h, P(ids), P(cached), P(new), n, P(tables), P(slots), P(out))
        if rc:
            raise (InputTooLong if rc == 1 else ComputeError)(lib.lg_last_error().decode())
        self._n = n
        return out

    def set_allreduce(self, fn):
        """Installs (or with None removes) the cross-rank reduction of the output projections' partial
        sums: a ``tp.ALLREDUCE_FN`` callback (kept alive by this object)."""
        self._allreduce = fn
        if lib.lg_hybrid_set_allreduce(self._h, C.cast(fn, C.c_void_p) if fn is not None else None, None):
            raise ComputeError(lib.lg_last_error().decode())

    def set_reduce_add(self, fn_ptr, user_ptr):
        """Installs (or with fn_ptr None removes) a reduction fused with the residual add: a C function of
        type ``lg_reduce_add_f32_fn`` given by address (``tp.PeerComm`` installs the library's own)."""
        if lib.lg_hybrid_set_reduce_add(self._h, fn_ptr, user_ptr):
            raise ComputeError(lib.lg_last_error().decode())

    def replay_device(self, stream_ptr: int):
        if lib.lg_hybrid_replay_device(self._h, C.c_void_p(stream_ptr)):
            raise ComputeError(lib.lg_last_error().decode())

    def last_hidden(self) -> np.ndarray:
        out = np.empty((self._n, self.cfg["hidden"]), np.float32)
        if lib.lg_hybrid_last_hidden(self._h, self._n, out.ctypes.data_as(C.c_void_p)):
            raise ComputeError(lib.lg_last_error().decode())
        return out

    def last_logits(self) -> np.ndarray:
        out = np.empty((self._n, self.cfg["vocab"]), np.float32)
        if lib.lg_hybrid_last_logits(self._h, self._n, out.ctypes.data_as(C.c_void_p)):
            raise ComputeError(lib.lg_last_error().decode())
        return out

    def launches_last_step(self) -> int:
        return int(lib.lg_hybrid_launches_last_step(self._h))

    def device_status(self) -> int:
        return int(lib.lg_hybrid_device_status(self._h))


# the serving-sweep architecture: 48 layers, three linear-attention layers per full-attention layer
HYBRID_SERVING = dict(vocab=151936, hidden=2048, n_layers=48, n_heads=16, n_kv_heads=2, attn_head_dim=256, gdn_heads=16,
                      intermediate=6144, max_pos=32768, full_attn_interval=4, rms_eps=1e-6, rope_theta=1e7)


def random_int4_weights(cfg: dict, seed: int) -> dict:
    """Seeded random int4 group-32 weights of the hybrid architecture for benchmarks (uniform codes,
    half-normal scales of 0.25 / sqrt(k)). Layers of one kind share their host arrays; every layer
    still gets its own copy on the device."""
    rng = np.random.Generator(np.random.PCG64(seed))
    H, I, GH = cfg["hidden"], cfg["intermediate"], cfg["gdn_heads"]
    QW, KW, GW = cfg["n_heads"] * cfg["attn_head_dim"], cfg["n_kv_heads"] * cfg["attn_head_dim"], GH * 128

    def qmat(n, k):
        return (rng.integers(0, 256, (n, k // 2), dtype=np.uint8),
                np.abs(rng.standard_normal((n, k // 32), dtype=np.float32) * (0.25 / np.sqrt(k))).astype(np.float16))

    mlp = {"w_gate": qmat(I, H), "w_up": qmat(I, H), "w_down": qmat(H, I), "norm1": np.ones(H, np.float32), "norm2": np.ones(H, np.float32)}
    full = dict(mlp, wq=qmat(QW, H), wgate=qmat(QW, H), wk=qmat(KW, H), wv=qmat(KW, H), wo=qmat(H, QW))
    lin = dict(mlp, wq=qmat(GW, H), wk=qmat(GW, H), wv=qmat(GW, H), wgate=qmat(GW, H), wo=qmat(H, GW), wa=qmat(GH, H), wb=qmat(GH, H),
               A_log=np.log(rng.uniform(0.5, 4.0, GH)).astype(np.float32), dt_bias=rng.uniform(-3.0, 0.0, GH).astype(np.float32))
    return {"tok_embed": rng.standard_normal((cfg["vocab"], H), dtype=np.float32) * np.float32(0.5), "final_norm": np.ones(H, np.float32),
            "lm_head": qmat(cfg["vocab"], H),
            "layers": [full if is_full_attention(l, cfg["full_attn_interval"]) else lin for l in range(cfg["n_layers"])]}
