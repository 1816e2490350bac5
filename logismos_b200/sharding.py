"""Request sharding across GPUs: the multi-GPU form of the reference's only parallelism, one worker
per sentence (``texts.par_iter()`` in StellaModel::encode_batch, crates/embed/src/stella.rs:290-293).

Sequences are independent (crates/transformers/src/attention.rs:13-14), so a ragged batch is split
by sequence, every rank runs its shard on a full replica, and the results are put back in request
order. There is no collective on the data path; ``all_gather_embeddings`` is the only exchange and
it moves results, not activations.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def assign_sequences(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Longest-processing-time greedy: sequences sorted by length (ties by index) go to the rank with
    the fewest tokens so far. Deterministic; returns, per rank, the sequence indices in request order."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        out[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(x) for x in out]


def shard_batch(ids: np.ndarray, cu_seqlens: np.ndarray, world: int, rank: int) -> Tuple[np.ndarray, np.ndarray, List[int]]:
    """The (ids, cu_seqlens) of this rank's shard and the request indices it holds."""
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    lens = cu[1:] - cu[:-1]
    mine = assign_sequences(lens.tolist(), world)[rank]
    parts = [np.asarray(ids[cu[i]:cu[i + 1]]) for i in mine]
    my_ids = np.concatenate(parts).astype(np.uint32) if parts else np.zeros(0, np.uint32)
    my_cu = np.zeros(len(mine) + 1, np.int32)
    if mine:
        my_cu[1:] = np.cumsum([lens[i] for i in mine])
    return my_ids, my_cu, mine


def all_gather_embeddings(local: np.ndarray, mine: List[int], n_total: int, dim: int):
    """Every rank ends with the full [n_total, dim] matrix in request order (torch.distributed must be
    initialised; works with gloo on CPU and nccl on GPUs)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size()
    backend = dist.get_backend()
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    counts = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
    dist.all_gather(counts, torch.tensor([len(mine)], dtype=torch.int64, device=dev))
    cap = int(max(int(c.item()) for c in counts))
    pad_e = torch.zeros((cap, dim), dtype=torch.float32, device=dev)
    pad_i = torch.full((cap,), -1, dtype=torch.int64, device=dev)
    if len(mine):
        pad_e[: len(mine)] = torch.from_numpy(np.ascontiguousarray(local, dtype=np.float32)).to(dev)
        pad_i[: len(mine)] = torch.tensor(mine, dtype=torch.int64, device=dev)
    es = [torch.zeros_like(pad_e) for _ in range(world)]
    ix = [torch.zeros_like(pad_i) for _ in range(world)]
    dist.all_gather(es, pad_e)
    dist.all_gather(ix, pad_i)
    out = np.zeros((n_total, dim), np.float32)
    for e, i in zip(es, ix):
        i = i.cpu().numpy(); e = e.cpu().numpy()
        keep = i >= 0
        out[i[keep]] = e[keep]
    return out
