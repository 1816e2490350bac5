"""Tensor-parallel form of the hybrid decoder (TP=2): two rank models, each holding half of the heads
and of the MLP, joined by an all-reduce after every output projection, must reproduce the unsplit
model. The two ranks run as threads of this process on one GPU with a host-side reduction (their
kernels never wait on one another on the device); between processes on two GPUs the same hook slot
takes an NCCL all-reduce."""
import threading

import numpy as np
import pytest

import oracle_lib as O
from gpu_util import TOL, max_rel
from hybrid_weights import TINY_HYBRID, make_hybrid
from logismos_b200.decoder import BlockAllocator
from logismos_b200.hybrid import HybridModel
from logismos_b200.tp import ThreadAllReduce, slice_hybrid_weights

pytestmark = pytest.mark.gpu

CFG = dict(TINY_HYBRID, gdn_heads=16)


def test_two_ranks_reproduce_the_unsplit_model():
    qw, deq = make_hybrid(CFG, 31)
    oracle = O.OracleHybrid(CFG, deq)
    red = ThreadAllReduce(2)
    models = []
    for r in range(2):
        c, w = slice_hybrid_weights(CFG, qw, 2, r)
        m = HybridModel(c, w, n_pool_blocks=32, max_blocks_per_seq=8, max_step_tokens=256, max_step_seqs=4, n_state_slots=4)
        m.set_allreduce(red.hook(r))
        models.append(m)
    rng = np.random.default_rng(5)
    blocks = BlockAllocator(32, 8, seed=1)
    hist = {0: [], 1: []}

    def step(entries):
        ids, cached, new, tabs, slots = [], [], [], [], []
        for sid, toks in entries:
            cached.append(len(hist[sid])); new.append(len(toks)); ids.extend(toks)
            hist[sid].extend(int(t) for t in toks)
            tabs.append(blocks.ensure(sid, len(hist[sid]))); slots.append(sid)
        out, err = [None, None], [None, None]

        def run(r):
            try:
                out[r] = models[r].step(ids, cached, new, np.stack(tabs), slots)
            except Exception as e:  # surfaces in the main thread below
                err[r] = e
                red.barrier.abort()
        ts = [threading.Thread(target=run, args=(r,)) for r in range(2)]
        [t.start() for t in ts]
        [t.join(timeout=300) for t in ts]
        assert err == [None, None], err
        assert np.array_equal(out[0], out[1])       # both ranks see the same reduced sums
        h0, h1 = models[0].last_hidden(), models[1].last_hidden()
        assert np.array_equal(h0, h1)
        for row, (sid, _) in enumerate(entries):
            h_ref, l_ref = oracle.forward(np.asarray(hist[sid], np.uint32))
            assert max_rel(h0[row], h_ref[-1]) <= TOL
            assert max_rel(models[0].last_logits()[row], l_ref) <= TOL
        return {sid: int(t) for (sid, _), t in zip(entries, out[0])}

    nxt = step([(0, rng.integers(0, 1000, 37)), (1, rng.integers(0, 1000, 9))])
    for _ in range(3):
        nxt = step([(1, [nxt[1]]), (0, [nxt[0]])])
    for m in models:
        m.set_allreduce(None)
        m.close()
