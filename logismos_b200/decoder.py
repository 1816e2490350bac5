"""Continuous-batching decoder step (int4 group-32 weights, paged KV cache) over the C ABI
(``lg_decoder_*``), plus the small host-side block allocator a caller needs to drive it.

The reference has no decoder executor and no scheduler (crates/decoders, crates/sched are empty
scaffolds); the semantics are "a packed step equals running every sequence alone".
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Sequence

import numpy as np

from ._lib import lib
from .embed import ComputeError, InputTooLong

_fp = C.POINTER(C.c_float)
_u8 = C.POINTER(C.c_uint8)
_u16 = C.POINTER(C.c_uint16)


class _Cfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("vocab", "hidden", "n_layers", "n_heads", "n_kv_heads", "intermediate", "max_pos")] + [
        ("rms_eps", C.c_float), ("rope_theta", C.c_double)] + [
        (n, C.c_int32) for n in ("n_pool_blocks", "max_blocks_per_seq", "max_step_tokens", "max_step_seqs", "keep_bf16_copy", "kv_turbo3")]


class _Q(C.Structure):
    _fields_ = [("codes", _u8), ("scales", _u16)]


class _LayerW(C.Structure):
    _fields_ = [(n, _fp) for n in ("norm1", "norm2", "bq", "bk", "bv")] + [
        (n, _Q) for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down")]


class _Weights(C.Structure):
    _fields_ = [("tok_embed", _fp), ("final_norm", _fp), ("layers", C.POINTER(_LayerW)), ("lm_head", _Q)]


def _f(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_fp)


def _q(pair):
    codes, scales = pair
    assert codes.dtype == np.uint8 and codes.flags["C_CONTIGUOUS"] and scales.flags["C_CONTIGUOUS"] and scales.itemsize == 2
    return _Q(codes.ctypes.data_as(_u8), scales.ctypes.data_as(_u16))


class BlockAllocator:
    """Hands out KV blocks of 16 tokens from a fixed pool; one table row per sequence."""

    def __init__(self, n_pool_blocks: int, max_blocks_per_seq: int, seed: int = 0):
        rng = np.random.default_rng(seed)
        self.free: List[int] = rng.permutation(n_pool_blocks).tolist()
        self.max_blocks = max_blocks_per_seq
        self.tables: Dict[int, List[int]] = {}

    def ensure(self, seq_id: int, n_tokens: int) -> np.ndarray:
        t = self.tables.setdefault(seq_id, [])
        need = -(-n_tokens // 16)
        if need > self.max_blocks:
            raise ValueError("sequence exceeds max_blocks_per_seq")
        while len(t) < need:
            if not self.free:
                raise MemoryError("KV pool exhausted")
            t.append(self.free.pop())
        row = np.full(self.max_blocks, -1, np.int32)
        row[: len(t)] = t
        return row

    def release(self, seq_id: int):
        self.free.extend(self.tables.pop(seq_id, []))


class DecoderModel:
    """weights: dict with tok_embed, final_norm (fp32), lm_head=(codes, scales) and ``layers``: list of
    dicts with norm1, norm2, bq, bk, bv (fp32) and wq, wk, wv, wo, w_gate, w_up, w_down as
    (codes u8 [n, k/2], scales f16 [n, k/32]) pairs."""

    def __init__(self, cfg: dict, weights: dict, n_pool_blocks: int, max_blocks_per_seq: int, max_step_tokens: int,
                 max_step_seqs: int, device: int = 0, keep_bf16_copy: bool = True, kv_turbo3: bool = False):
        c = _Cfg(cfg["vocab"], cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"], cfg["intermediate"],
                 cfg["max_pos"], cfg["rms_eps"], cfg["rope_theta"], n_pool_blocks, max_blocks_per_seq, max_step_tokens, max_step_seqs,
                 int(keep_bf16_copy), int(kv_turbo3))
        L = (_LayerW * max(1, cfg["n_layers"]))()
        for i, lw in enumerate(weights["layers"]):
            for n in ("norm1", "norm2", "bq", "bk", "bv"):
                setattr(L[i], n, _f(lw[n]))
            for n in ("wq", "wk", "wv", "wo", "w_gate", "w_up", "w_down"):
                setattr(L[i], n, _q(lw[n]))
        w = _Weights(_f(weights["tok_embed"]), _f(weights["final_norm"]), L, _q(weights["lm_head"]))
        self._keep = weights
        h = C.c_void_p()
        if lib.lg_decoder_create(device, C.byref(c), C.byref(w), C.byref(h)):
            raise ComputeError(lib.lg_last_error().decode())
        self._h, self.cfg, self.max_blocks = h, cfg, max_blocks_per_seq

    @classmethod
    def load(cls, path: str, cfg: dict, n_pool_blocks: int, max_blocks_per_seq: int, max_step_tokens: int, max_step_seqs: int,
             device: int = 0, keep_bf16_copy: bool = True, kv_turbo3: bool = False) -> "DecoderModel":
        """The decoder from a Qwen2-style fp32 safetensors file: tensor accounting and int4 group-32
        quantisation on the device by the native loader (``lg_decoder_load``)."""
        c = _Cfg(cfg["vocab"], cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"], cfg["intermediate"], cfg["max_pos"],
                 cfg["rms_eps"], cfg["rope_theta"], n_pool_blocks, max_blocks_per_seq, max_step_tokens, max_step_seqs, int(keep_bf16_copy),
                 int(kv_turbo3))
        h = C.c_void_p()
        rc = lib.lg_decoder_load(device, str(path).encode(), C.byref(c), C.byref(h))
        if rc:
            raise (IOError if rc == 5 else ComputeError)(lib.lg_last_error().decode())
        self = cls.__new__(cls)
        self._h, self.cfg, self.max_blocks = h, cfg, max_blocks_per_seq
        return self

    def close(self):
        if getattr(self, "_h", None):
            lib.lg_decoder_destroy(self._h)
            self._h = None

    __del__ = close

    def step(self, ids: Sequence[int], cached_lens, new_lens, block_tables) -> np.ndarray:
        """One packed step; returns the greedy next token of every sequence (uint32 [n_seqs])."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        cached = np.ascontiguousarray(cached_lens, dtype=np.int32)
        new = np.ascontiguousarray(new_lens, dtype=np.int32)
        tables = np.ascontiguousarray(block_tables, dtype=np.int32)
        n = cached.size
        assert new.size == n and tables.shape == (n, self.max_blocks) and ids.size == int(new.sum())
        out = np.empty(n, np.uint32)
        P = lambda a: a.ctypes.data_as(C.c_void_p)
        rc = lib.lg_decoder_step(self._h, P(ids), P(cached), P(new), n, P(tables), P(out))
        if rc:
            raise (InputTooLong if rc == 1 else ComputeError)(lib.lg_last_error().decode())
        self._n = n
        return out

    def replay_device(self, stream_ptr: int):
        if lib.lg_decoder_replay_device(self._h, C.c_void_p(stream_ptr)):
            raise ComputeError(lib.lg_last_error().decode())

    def last_hidden(self) -> np.ndarray:
        out = np.empty((self._n, self.cfg["hidden"]), np.float32)
        if lib.lg_decoder_last_hidden(self._h, self._n, out.ctypes.data_as(C.c_void_p)):
            raise ComputeError(lib.lg_last_error().decode())
        return out

    def last_logits(self) -> np.ndarray:
        out = np.empty((self._n, self.cfg["vocab"]), np.float32)
        if lib.lg_decoder_last_logits(self._h, self._n, out.ctypes.data_as(C.c_void_p)):
            raise ComputeError(lib.lg_last_error().decode())
        return out

    def launches_last_step(self) -> int:
        return int(lib.lg_decoder_launches_last_step(self._h))

    def device_status(self) -> int:
        return int(lib.lg_decoder_device_status(self._h))
