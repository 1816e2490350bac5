"""Tensor parallelism for the hybrid decoder: weight slicing and the all-reduce that joins the partial
sums of the output projections. The reference has no tensor parallelism; this is the TP=2 variant of
the serving configuration, whose only collective is this all-reduce.

Rank r of tp holds heads [r * n/tp, (r+1) * n/tp) of every kind (query, KV, linear-attention) and the
matching slice of the MLP: input projections are sliced by output rows, output projections by
input columns (whole groups of 32, so codes and scales slice cleanly); embeddings, norms and the
lm_head are replicated.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Callable, Tuple

import numpy as np

ALLREDUCE_FN = C.CFUNCTYPE(C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p)


def _rows(q, lo, hi):
    codes, scales = q
    return np.ascontiguousarray(codes[lo:hi]), np.ascontiguousarray(scales[lo:hi])


def _cols(q, lo, hi):
    codes, scales = q
    assert lo % 32 == 0 and hi % 32 == 0
    return np.ascontiguousarray(codes[:, lo // 2:hi // 2]), np.ascontiguousarray(scales[:, lo // 32:hi // 32])


def slice_hybrid_weights(cfg: dict, weights: dict, tp: int, rank: int) -> Tuple[dict, dict]:
    """(cfg, weights) of one rank, in the layout HybridModel takes."""
    for n in ("n_heads", "n_kv_heads", "gdn_heads", "intermediate"):
        if cfg[n] % tp:
            raise ValueError(f"{n} = {cfg[n]} is not divisible by tp = {tp}")
    c = dict(cfg, n_heads=cfg["n_heads"] // tp, n_kv_heads=cfg["n_kv_heads"] // tp, gdn_heads=cfg["gdn_heads"] // tp,
             intermediate=cfg["intermediate"] // tp)
    d = cfg["attn_head_dim"]
    qw, kw, gw, gh, inter = c["n_heads"] * d, c["n_kv_heads"] * d, c["gdn_heads"] * 128, c["gdn_heads"], c["intermediate"]
    if inter % 128 or gh % 8:
        raise ValueError("the slice must keep intermediate a multiple of 128 and gdn_heads a multiple of 8")
    out = {"tok_embed": weights["tok_embed"], "final_norm": weights["final_norm"], "lm_head": weights["lm_head"], "layers": []}
    for l, lw in enumerate(weights["layers"]):
        full = (l + 1) % cfg["full_attn_interval"] == 0
        nl = {"norm1": lw["norm1"], "norm2": lw["norm2"]}
        if full:
            nl["wq"], nl["wgate"] = _rows(lw["wq"], rank * qw, (rank + 1) * qw), _rows(lw["wgate"], rank * qw, (rank + 1) * qw)
            nl["wk"], nl["wv"] = _rows(lw["wk"], rank * kw, (rank + 1) * kw), _rows(lw["wv"], rank * kw, (rank + 1) * kw)
            nl["wo"] = _cols(lw["wo"], rank * qw, (rank + 1) * qw)
        else:
            for n in ("wq", "wk", "wv", "wgate"):
                nl[n] = _rows(lw[n], rank * gw, (rank + 1) * gw)
            nl["wa"], nl["wb"] = _rows(lw["wa"], rank * gh, (rank + 1) * gh), _rows(lw["wb"], rank * gh, (rank + 1) * gh)
            nl["A_log"] = np.ascontiguousarray(lw["A_log"][rank * gh:(rank + 1) * gh])
            nl["dt_bias"] = np.ascontiguousarray(lw["dt_bias"][rank * gh:(rank + 1) * gh])
            nl["wo"] = _cols(lw["wo"], rank * gw, (rank + 1) * gw)
        nl["w_gate"], nl["w_up"] = _rows(lw["w_gate"], rank * inter, (rank + 1) * inter), _rows(lw["w_up"], rank * inter, (rank + 1) * inter)
        nl["w_down"] = _cols(lw["w_down"], rank * inter, (rank + 1) * inter)
        out["layers"].append(nl)
    return c, out


class _DevF32:
    """A device fp32 buffer known by address, exposed to torch without copying."""

    def __init__(self, ptr: int, count: int):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 3, "strides": None}


def as_f32_tensor(ptr: int, count: int):
    import torch
    return torch.as_tensor(_DevF32(ptr, count), device="cuda")


def nccl_allreduce_hook(group=None) -> Callable:
    """The reduction for ranks that are processes on different GPUs: torch.distributed's NCCL
    all-reduce, enqueued behind the work already on the executor's stream."""
    import torch
    import torch.distributed as dist

    def fn(_user, ptr, count, stream):
        try:
            with torch.cuda.stream(torch.cuda.ExternalStream(stream)):
                dist.all_reduce(as_f32_tensor(ptr, count), op=dist.ReduceOp.SUM, group=group)
            return 0
        except Exception:  # the C caller only understands a status
            return 1
    return ALLREDUCE_FN(fn)


class ThreadAllReduce:
    """The reduction for ranks that are threads of one process on ONE GPU (tests): every rank
    synchronises its stream, meets the others at a barrier, rank 0 sums the buffers, and every rank
    copies the sum back. Kernels of different ranks never wait on one another on the device."""

    def __init__(self, tp: int):
        self.tp = tp
        self.barrier = threading.Barrier(tp)
        self.bufs = [None] * tp
        self.total = None

    def hook(self, rank: int) -> Callable:
        import torch

        def fn(_user, ptr, count, stream):
            try:
                st = torch.cuda.ExternalStream(stream)
                st.synchronize()
                self.bufs[rank] = as_f32_tensor(ptr, count)
                self.barrier.wait(timeout=60)
                if rank == 0:
                    self.total = torch.stack(self.bufs).sum(0)
                    torch.cuda.synchronize()
                self.barrier.wait(timeout=60)
                self.bufs[rank].copy_(self.total)
                torch.cuda.synchronize()
                self.barrier.wait(timeout=60)
                return 0
            except Exception:
                self.barrier.abort()
                return 1
        return ALLREDUCE_FN(fn)
