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


def test_turbo3_cache_mode_runs_the_same_steps_at_the_codec_accuracy(setup):
    """kv_turbo3: the cache holds TurboQuant 3-bit rows (4.57 times smaller) and every sequence attends
    through the decoding gather. The K/V rows carry the codec's error (3 bits per value), so the stack is
    compared with the fp32 oracle at the codec's accuracy, not at the bf16 bar: the kernel-level tests
    (test_gpu_paged, test_gpu_attention) hold the cache bytes and the attention over them to the oracle."""
    from gpu_util import cosine
    qw, deq, oracle = setup
    rng = np.random.default_rng(4)
    alloc = BlockAllocator(64, 16, seed=3)
    model = DecoderModel(TINY, qw, n_pool_blocks=64, max_blocks_per_seq=16, max_step_tokens=256, max_step_seqs=4, kv_turbo3=True)
    hist = {0: rng.integers(0, 1000, 60).tolist(), 1: rng.integers(0, 1000, 130).tolist()}
    # sequence 1 enters in two chunks (the second continues a cached, quantised prefix), sequence 0 whole
    toks = model.step(hist[0] + hist[1][:64], [0, 0], [60, 64], np.stack([alloc.ensure(0, 60), alloc.ensure(1, 64)]))
    assert model.device_status() == 0
    hist[0].append(int(toks[0]))
    toks = model.step([hist[0][-1]] + hist[1][64:], [60, 64], [1, 66], np.stack([alloc.ensure(0, 61), alloc.ensure(1, 130)]))
    assert model.device_status() == 0
    hist[1].append(int(toks[1])); hist[0].append(int(toks[0]))
    for _ in range(3):
        toks = model.step([hist[0][-1], hist[1][-1]], [len(hist[0]) - 1, len(hist[1]) - 1], [1, 1],
                          np.stack([alloc.ensure(0, len(hist[0])), alloc.ensure(1, len(hist[1]))]))
        assert model.device_status() == 0
        hs = model.last_hidden()
        for row, sid in enumerate((0, 1)):
            h_ref, _ = oracle_last(oracle, deq, hist[sid])
            assert np.isfinite(hs[row]).all() and cosine(hs[row], h_ref) >= 0.9, (sid, cosine(hs[row], h_ref))
        hist[0].append(int(toks[0])); hist[1].append(int(toks[1]))
    model.close()
