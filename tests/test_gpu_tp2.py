"""Tensor-parallel hybrid decoder across TWO GPUs (ranks = processes): each rank holds half of the
heads and of the MLP and the partial sums of the output projections meet in the library's own
exchange over NVLink peer memory (lg_tp_reduce_add_f32: peer stores + flags + fused residual add).
Both ranks must emit the same tokens and reproduce the unsplit model (the CPU oracle). Skipped on a
machine with one GPU; the single-GPU test of the slicing and of the hook slot is test_gpu_tp.py."""
import os
import traceback

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _rank_main(rank, world, port, q):
    try:
        import torch
        import torch.distributed as dist
        import oracle_lib as O
        from gpu_util import TOL, max_rel
        from hybrid_weights import TINY_HYBRID, make_hybrid
        from logismos_b200.decoder import BlockAllocator
        from logismos_b200.hybrid import HybridModel
        from logismos_b200.tp import install_allreduce, slice_hybrid_weights
        os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", rank=rank, world_size=world)  # host-side exchange of the ipc handles only
        cfg = dict(TINY_HYBRID, gdn_heads=16)
        qw, deq = make_hybrid(cfg, 31)
        c, w = slice_hybrid_weights(cfg, qw, world, rank)
        m = HybridModel(c, w, n_pool_blocks=32, max_blocks_per_seq=8, max_step_tokens=256, max_step_seqs=4, n_state_slots=4, device=rank)
        comm = install_allreduce(m, rank, world, kind="peer")
        rng = np.random.default_rng(5)
        blocks = BlockAllocator(32, 8, seed=1)
        hist = {0: [], 1: []}
        oracle = O.OracleHybrid(cfg, deq) if rank == 0 else None

        def step(entries):
            ids, cached, new, tabs, slots = [], [], [], [], []
            for sid, toks in entries:
                cached.append(len(hist[sid])); new.append(len(toks)); ids.extend(toks)
                hist[sid].extend(int(t) for t in toks)
                tabs.append(blocks.ensure(sid, len(hist[sid]))); slots.append(sid)
            out = m.step(ids, cached, new, np.stack(tabs), slots)
            assert m.device_status() == 0
            both = [None, None]
            dist.all_gather_object(both, (out.tolist(), m.last_hidden().tobytes()))
            assert both[0] == both[1], "the ranks disagree on the reduced sums"
            if rank == 0:
                for row, (sid, _) in enumerate(entries):
                    h_ref, l_ref = oracle.forward(np.asarray(hist[sid], np.uint32))
                    assert max_rel(m.last_hidden()[row], h_ref[-1]) <= TOL
                    assert max_rel(m.last_logits()[row], l_ref) <= TOL
            return {sid: int(t) for (sid, _), t in zip(entries, out)}

        nxt = step([(0, rng.integers(0, 1000, 37)), (1, rng.integers(0, 1000, 9))])
        for _ in range(4):
            nxt = step([(1, [nxt[1]]), (0, [nxt[0]])])
        step([(0, rng.integers(0, 1000, 70))])  # a chunk continuing a cached prefix, 70 rows through the dense route
        dist.barrier()
        m.close()
        comm.close()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:
        q.put((rank, traceback.format_exc()))


def test_two_gpus_reproduce_the_unsplit_model_over_peer_memory():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    results = [q.get(timeout=600) for _ in range(2)]
    [p.join(timeout=60) for p in procs]
    assert sorted(results) == [(0, "ok"), (1, "ok")], results
