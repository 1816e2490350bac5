"""Request sharding (the multi-GPU path) on CPU: assignment properties, and a world_size-2 gloo run
in which each rank encodes its shard (with the CPU oracle standing in for the GPU replica) and the
gathered result equals the single-process result in request order."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from logismos_b200.sharding import all_gather_embeddings, assign_sequences, shard_batch
from stella_weights import TINY, make_batch, make_weights


def test_assignment_is_a_balanced_partition():
    rng = np.random.default_rng(0)
    lens = rng.integers(32, 513, 37).tolist()
    for world in (1, 2, 4, 8):
        parts = assign_sequences(lens, world)
        flat = sorted(i for p in parts for i in p)
        assert flat == list(range(37))                       # a partition
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)          # LPT bound
        assert all(p == sorted(p) for p in parts)            # request order inside a shard
    assert assign_sequences([], 4) == [[], [], [], []]
    assert assign_sequences([5], 2) == [[0], []]


def test_shard_batch_slices_ids_by_sequence():
    ids, cu = make_batch(TINY, 3, n_seq=7, lo=3, hi=30)
    seen = {}
    for r in range(3):
        my_ids, my_cu, mine = shard_batch(ids, cu, 3, r)
        assert my_cu[-1] == my_ids.size
        for j, i in enumerate(mine):
            assert (my_ids[my_cu[j]:my_cu[j + 1]] == ids[cu[i]:cu[i + 1]]).all()
            seen[i] = r
    assert sorted(seen) == list(range(7))


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import oracle_lib as O
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = make_weights(TINY, 4)
        model = O.OracleStella(TINY, w)
        ids, cu = make_batch(TINY, 21, n_seq=5, lo=4, hi=24)
        my_ids, my_cu, mine = shard_batch(ids, cu, world, rank)
        local = model.encode_batch(my_ids, my_cu, 1) if mine else np.zeros((0, TINY["head_out_dim"]), np.float32)
        full = all_gather_embeddings(local, mine, 5, TINY["head_out_dim"])
        if rank == 0:
            ref = model.encode_batch(ids, cu, 1)
            ret["err"] = float(np.abs(full - ref).max())
        # a rank that holds nothing still takes part in the exchange
        my_ids, my_cu, mine = shard_batch(ids[:cu[1]], cu[:2], world, rank)
        local = model.encode_batch(my_ids, my_cu, 1) if mine else np.zeros((0, TINY["head_out_dim"]), np.float32)
        one = all_gather_embeddings(local, mine, 1, TINY["head_out_dim"])
        if rank == 1:
            ret["err1"] = float(np.abs(one - model.encode_batch(ids[:cu[1]], cu[:2], 1)).max())
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo_reproduce_the_single_process_result():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = 29500 + (os.getpid() % 1000)
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
            assert p.exitcode == 0
        assert ret["err"] == 0.0 and ret["err1"] == 0.0
