"""The continuous-batching decoder step (int4 weights, paged KV cache, mixed prefill + decode)
against per-sequence execution on the CPU oracle: every sequence of a packed step must come out as
if it had been run alone through the causal forward, lm_head and greedy argmax."""
import numpy as np
import pytest

import oracle_lib as O
from gpu_util import TOL, max_rel
from logismos_b200.decoder import BlockAllocator, DecoderModel
from logismos_b200.embed import ComputeError
from stella_weights import TINY, make_weights, quantize_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup():
    w = make_weights(TINY, 77)
    qw, deq = quantize_weights(TINY, w)
    oracle = O.OracleStella(TINY, deq)
    return qw, deq, oracle


def oracle_last(oracle, deq, ids):
    h = oracle.forward(np.asarray(ids, np.uint32), causal=True)[-1]
    logits = O.linear_t(h, deq["lm_head"], None, 1, TINY["vocab"], TINY["hidden"])
    return h, logits


def check_step(model, oracle, deq, histories, order):
    hs, lg, toks = model.last_hidden(), model.last_logits(), model._toks
    for row, sid in enumerate(order):
        h_ref, l_ref = oracle_last(oracle, deq, histories[sid])
        assert max_rel(hs[row], h_ref) <= TOL, (sid, len(histories[sid]))
        assert max_rel(lg[row], l_ref) <= TOL
        # greedy is exact on the GPU's own logits (first maximum wins) ...
        assert toks[row] == O.greedy(lg[row])
        # ... and agrees with the oracle's choice up to the logit tolerance
        assert l_ref[toks[row]] >= l_ref.max() - TOL * np.abs(l_ref).max()


def test_mixed_prefill_and_decode_steps_equal_per_sequence_execution(setup):
    qw, deq, oracle = setup
    rng = np.random.default_rng(1)
    alloc = BlockAllocator(64, 16, seed=3)
    model = DecoderModel(TINY, qw, n_pool_blocks=64, max_blocks_per_seq=16, max_step_tokens=512, max_step_seqs=8)
    hist = {}

    def run(entries):
        """entries: list of (seq id, new ids)."""
        ids, cached, new, tabs, order = [], [], [], [], []
        for sid, toks in entries:
            prev = hist.setdefault(sid, [])
            cached.append(len(prev)); new.append(len(toks)); ids.extend(toks)
            prev.extend(int(t) for t in toks)
            tabs.append(alloc.ensure(sid, len(prev))); order.append(sid)
        model._toks = model.step(ids, cached, new, np.stack(tabs))
        assert model.device_status() == 0
        check_step(model, oracle, deq, hist, order)
        return dict(zip(order, model._toks.tolist()))

    # step 1: three prefill chunks
    nxt = run([(0, rng.integers(0, 1000, 40)), (1, rng.integers(0, 1000, 7)), (2, rng.integers(0, 1000, 100))])
    # steps 2..: decode the three (crossing 16-token block boundaries), a new prefill joins in step 2,
    # caller order mixes decode and prefill entries
    nxt = run([(0, [nxt[0]]), (3, rng.integers(0, 1000, 33)), (1, [nxt[1]]), (2, [nxt[2]])])
    for _ in range(10):
        nxt = run([(sid, [nxt[sid]]) for sid in (2, 0, 3, 1)])
    assert len(hist[1]) == 18 and model.launches_last_step() > 0
    # a single-token sequence is a decode against an empty cache
    run([(9, [5])])
    # a prompt fed in chunks: every chunk after the first continues a cached prefix (positions, cache
    # slots, keys and values read through the block table), mixed with decode rows and with a chunk that
    # starts another sequence; every step is compared with the oracle run on the whole history, so
    # chunked == whole prompt == oracle
    prompt = rng.integers(0, 1000, 150)
    run([(11, prompt[:64]), (0, [nxt[0]])])
    run([(2, [nxt[2]]), (11, prompt[64:129]), (12, rng.integers(0, 1000, 20))])
    last = run([(11, prompt[129:])])
    h_chunked = model.last_hidden()[0].copy()
    whole = run([(13, prompt)])
    assert max_rel(model.last_hidden()[0], h_chunked) <= TOL and whole[13] == last[11]
    model.close()


def test_step_rejects_what_it_cannot_run(setup):
    qw, _, _ = setup
    model = DecoderModel(TINY, qw, n_pool_blocks=8, max_blocks_per_seq=8, max_step_tokens=64, max_step_seqs=2)
    tab = np.array([[0, 1, 2, 3, 4, 5, 6, 7]], np.int32)
    with pytest.raises(ComputeError):   # block table row with a missing entry
        model.step([1] * 20, [0], [20], np.array([[0, -1, -1, -1, -1, -1, -1, -1]], np.int32))
    with pytest.raises(ComputeError):   # more tokens than the step workspace
        model.step([1] * 65, [0], [65], tab)
    with pytest.raises(Exception):      # beyond the block table
        model.step([1], [128], [1], tab)
    model.close()
