"""StellaModel on the GPU behind the EmbeddingModel contract.

Mirrors ``embed::StellaModel`` (crates/embed/src/stella.rs:251-326) and ``core::EmbeddingModel``
(crates/core/src/lib.rs:139-163) at token-id level: same method names, same argument meaning, the
same errors. All compute happens in liblogismos_kernels.so (``lg_stella_*``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from ._lib import lib


class EmbeddingError(Exception):
    """core::EmbeddingError (crates/core/src/lib.rs:75-133)"""


class InputTooLong(EmbeddingError):
    pass


class UnsupportedDim(EmbeddingError):
    pass


class ComputeError(EmbeddingError):
    pass


class TokenizeError(EmbeddingError):
    pass


class IoError(EmbeddingError):
    pass


class UnsupportedPrompt(EmbeddingError):
    pass


_ERR = {1: InputTooLong, 2: UnsupportedDim, 3: TokenizeError, 4: ComputeError, 5: IoError, 6: UnsupportedPrompt}


@dataclass
class EncodeOpts:
    """core::EncodeOpts (crates/core/src/lib.rs:59-69). ``prompt`` (a ``text.Prompt``) is applied by the
    text front end (``text.StellaTextModel``); the id-level entry points ignore it."""
    dim: Optional[int] = None
    max_tokens: Optional[int] = None
    prompt: Optional[object] = None


class _Cfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("vocab", "hidden", "n_layers", "n_heads", "n_kv_heads", "intermediate", "max_pos")] + [
        ("rms_eps", C.c_float), ("rope_theta", C.c_double), ("max_tokens", C.c_int32), ("n_dims", C.c_int32),
        ("dims", C.c_int32 * 8), ("max_batch_tokens", C.c_int32), ("max_batch_seqs", C.c_int32), ("fuse_swiglu", C.c_int32)]


_fp = C.POINTER(C.c_float)


class _LayerW(C.Structure):
    _fields_ = [(n, _fp) for n in ("norm1", "norm2", "wq", "bq", "wk", "bk", "wv", "bv", "wo", "w_gate", "w_up", "w_down")]


class _Weights(C.Structure):
    _fields_ = [("tok_embed", _fp), ("final_norm", _fp), ("layers", C.POINTER(_LayerW)), ("head_w", _fp * 8), ("head_b", _fp * 8)]


def _ptr(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_fp)


class StellaModel:
    """``StellaModel::load`` for in-memory fp32 weights (dict layout of logismos_b200.synthetic.make_weights:
    tok_embed, final_norm, layers[12 tensors], head_w, head_b; ``heads`` maps dim -> (w, b) for
    several dense heads)."""

    def __init__(self, cfg: dict, weights: dict, device: int = 0, max_batch_tokens: int = 8192,
                 max_batch_seqs: int = 256, fuse_swiglu: bool = True, heads: Optional[dict] = None):
        heads = heads or {cfg["head_out_dim"]: (weights["head_w"], weights["head_b"])}
        dims = list(heads.keys())
        c = _Cfg(cfg["vocab"], cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"], cfg["intermediate"],
                 cfg["max_pos"], cfg["rms_eps"], cfg["rope_theta"], cfg.get("max_tokens", 512), len(dims),
                 (C.c_int32 * 8)(*dims), max_batch_tokens, max_batch_seqs, int(fuse_swiglu))
        L = (_LayerW * max(1, cfg["n_layers"]))()
        for i, lw in enumerate(weights["layers"]):
            for n, _ in _LayerW._fields_:
                setattr(L[i], n, _ptr(lw[n]))
        w = _Weights(_ptr(weights["tok_embed"]), _ptr(weights["final_norm"]), L)
        for i, d in enumerate(dims):
            w.head_w[i] = _ptr(heads[d][0])
            w.head_b[i] = _ptr(heads[d][1])
        h = C.c_void_p()
        rc = lib.lg_stella_create(device, C.byref(c), C.byref(w), C.byref(h))
        if rc:
            raise ComputeError(lib.lg_last_error().decode())
        self._h = h
        self.cfg = cfg
        self.device = device

    @classmethod
    def load(cls, root: str, dims: Sequence[int] = (1024,), cfg: Optional[dict] = None, device: int = 0, max_batch_tokens: int = 8192,
             max_batch_seqs: int = 256, fuse_swiglu: bool = True) -> "StellaModel":
        """``StellaModel::load(root, dims)`` (crates/embed/src/stella.rs:138-201) from a checkpoint directory:
        ``root/model.safetensors`` and one ``root/2_Dense_<dim>/model.safetensors`` per requested dim,
        read, validated and uploaded by the native loader (``lg_stella_load``). ``cfg`` defaults to the
        Stella-1.5B configuration the reference hard-codes."""
        if cfg is None:
            from .synthetic import STELLA_1_5B
            cfg = STELLA_1_5B
        dims = list(dims)
        c = _Cfg(cfg["vocab"], cfg["hidden"], cfg["n_layers"], cfg["n_heads"], cfg["n_kv_heads"], cfg["intermediate"],
                 cfg["max_pos"], cfg["rms_eps"], cfg["rope_theta"], cfg.get("max_tokens", 512), len(dims),
                 (C.c_int32 * 8)(*dims), max_batch_tokens, max_batch_seqs, int(fuse_swiglu))
        h = C.c_void_p()
        rc = lib.lg_stella_load(device, str(root).encode(), C.byref(c), C.byref(h))
        if rc:
            raise _ERR.get(rc, ComputeError)(lib.lg_last_error().decode())
        self = cls.__new__(cls)
        self._h, self.cfg, self.device = h, cfg, device
        return self

    def close(self):
        if getattr(self, "_h", None):
            lib.lg_stella_destroy(self._h)
            self._h = None

    __del__ = close

    # ---- EmbeddingModel ----
    def default_dim(self) -> int:
        return int(lib.lg_stella_default_dim(self._h))

    def supported_dims(self):
        out = (C.c_int32 * 8)()
        n = lib.lg_stella_supported_dims(self._h, out, 8)
        return [int(out[i]) for i in range(n)]

    def max_tokens(self) -> int:
        return int(lib.lg_stella_max_tokens(self._h))

    def encode_ids(self, ids: Sequence[int], opts: EncodeOpts = EncodeOpts()) -> np.ndarray:
        """``encode`` at id level: one sequence -> unit-norm fp32 vector."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        return self.encode_ids_batch(ids, np.array([0, ids.size], np.int32), opts)[0]

    def encode_ids_batch(self, ids, cu_seqlens, opts: EncodeOpts = EncodeOpts()) -> np.ndarray:
        """``encode_batch`` at id level: ragged batch (ids, cu_seqlens) -> [n_seqs, dim] fp32."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        cu = np.ascontiguousarray(cu_seqlens, dtype=np.int32)
        n = cu.size - 1
        dim = opts.dim or self.default_dim()
        out = np.empty((n, dim), np.float32)
        rc = lib.lg_stella_encode_ids_batch(self._h, ids.ctypes.data_as(C.c_void_p), cu.ctypes.data_as(C.c_void_p), n,
                                            opts.dim or 0, opts.max_tokens or 0, out.ctypes.data_as(C.c_void_p))
        if rc:
            raise _ERR.get(rc, ComputeError)(lib.lg_last_error().decode())
        return out

    # ---- device-resident forward (kernel-only timing, diagnostics) ----
    def forward_device(self, dev_ids, dev_cu, dev_pos, n_tokens, n_seqs, max_seqlen, dev_out, stream_ptr, dim=0, causal=False):
        rc = lib.lg_stella_forward_device(self._h, C.c_void_p(dev_ids), C.c_void_p(dev_cu), C.c_void_p(dev_pos), n_tokens, n_seqs,
                                          max_seqlen, dim, int(causal), C.c_void_p(dev_out), C.c_void_p(stream_ptr))
        if rc:
            raise _ERR.get(rc, ComputeError)(lib.lg_last_error().decode())

    def last_hidden(self, n_tokens: int) -> np.ndarray:
        out = np.empty((n_tokens, self.cfg["hidden"]), np.float32)
        rc = lib.lg_stella_last_hidden(self._h, n_tokens, out.ctypes.data_as(C.c_void_p))
        if rc:
            raise ComputeError(lib.lg_last_error().decode())
        return out

    def launches_per_forward(self) -> int:
        return int(lib.lg_stella_launches_per_forward(self._h))

    def device_status(self) -> int:
        return int(lib.lg_stella_device_status(self._h))
