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


class PeerComm:
    """The reduction for ranks that are processes on different GPUs of one node: the library's own
    exchange over NVLink peer memory (``lg_tp_reduce_add_f32``: peer stores, flags, one kernel per rank,
    fused with the residual add). The 64-byte cudaIpc handles of the ranks' regions are exchanged over the
    torch.distributed process group (``group``), which must hold exactly the tp ranks in rank order."""

    def __init__(self, rank: int, tp: int, max_elems: int, device: int, group=None):
        import torch
        import torch.distributed as dist
        from ._lib import lib
        self._lib, self._comm = lib, None
        max_elems = (int(max_elems) + 3) & ~3
        region, handle = C.c_void_p(), (C.c_uint8 * 64)()
        rc = lib.lg_tp_comm_alloc(device, tp, max_elems, C.byref(region), handle)
        if rc:
            raise RuntimeError(f"lg_tp_comm_alloc failed with CUDA status {rc}")
        mine = torch.tensor(list(handle), dtype=torch.uint8, device=torch.device("cuda", device) if dist.get_backend(group) == "nccl" else "cpu")
        parts = [torch.zeros_like(mine) for _ in range(tp)]
        dist.all_gather(parts, mine, group=group)
        allh = (C.c_uint8 * (64 * tp))(*[int(v) for p_ in parts for v in p_.cpu().tolist()])
        comm = C.c_void_p()
        rc = lib.lg_tp_comm_open(device, region, rank, tp, max_elems, allh, C.byref(comm))
        if rc:
            raise RuntimeError(f"lg_tp_comm_open failed with CUDA status {rc} (peer access between the GPUs is required)")
        self._comm = comm
        dist.barrier(group=group)  # every rank has mapped every region before the first exchange

    def install(self, model):
        model.set_reduce_add(C.cast(self._lib.lg_tp_reduce_add_f32, C.c_void_p), self._comm)

    def close(self):
        if self._comm:
            self._lib.lg_tp_comm_destroy(self._comm, 1)
            self._comm = None


def install_allreduce(model, rank: int, tp: int, kind: str = "peer", group=None):
    """Joins a rank's HybridModel to its tensor-parallel group. kind "peer": the library's NVLink
    peer-memory exchange (default); "nccl": torch.distributed's NCCL all-reduce through a Python
    callback (the slower, library-only route, kept for comparison). Returns the object to keep alive
    for as long as the model runs."""
    if kind == "nccl":
        hook = nccl_allreduce_hook(group)
        model.set_allreduce(hook)
        return hook
    cfg = model.cfg
    comm = PeerComm(rank, tp, model.max_step_tokens * cfg["hidden"], model.device, group)
    comm.install(model)
    return comm


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
