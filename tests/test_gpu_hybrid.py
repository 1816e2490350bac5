"""The hybrid decoder step (linear-attention layers with recurrent state slots, gated full-attention
layers over the paged KV cache, int4 weights, mixed prefill + decode) against per-sequence
execution on the CPU oracle: every sequence of a packed step must come out as if its whole history
had been run alone through the stack, lm_head and greedy argmax."""
import numpy as np
import pytest

import oracle_lib as O
from gpu_util import TOL, max_rel
from hybrid_weights import TINY_HYBRID, TINY_HYBRID_128, make_hybrid
from logismos_b200.decoder import BlockAllocator
from logismos_b200.embed import ComputeError
from logismos_b200.hybrid import HybridModel, SlotAllocator

pytestmark = pytest.mark.gpu


def drive(cfg, seed, n_decode_steps):
    qw, deq = make_hybrid(cfg, seed)
    oracle = O.OracleHybrid(cfg, deq)
    rng = np.random.default_rng(seed)
    blocks, slots = BlockAllocator(64, 16, seed=3), SlotAllocator(8)
    model = HybridModel(cfg, qw, n_pool_blocks=64, max_blocks_per_seq=16, max_step_tokens=512, max_step_seqs=8, n_state_slots=8)
    hist = {}

    def run(entries):
        ids, cached, new, tabs, sl, order = [], [], [], [], [], []
        for sid, toks in entries:
            prev = hist.setdefault(sid, [])
            cached.append(len(prev)); new.append(len(toks)); ids.extend(toks)
            prev.extend(int(t) for t in toks)
            tabs.append(blocks.ensure(sid, len(prev))); sl.append(slots.get(sid)); order.append(sid)
        toks = model.step(ids, cached, new, np.stack(tabs), sl)
        assert model.device_status() == 0
        hs, lg = model.last_hidden(), model.last_logits()
        for row, sid in enumerate(order):
            h_ref, l_ref = oracle.forward(np.asarray(hist[sid], np.uint32))
            assert max_rel(hs[row], h_ref[-1]) <= TOL, (sid, len(hist[sid]))
            assert max_rel(lg[row], l_ref) <= TOL
            assert toks[row] == O.greedy(lg[row])
            assert l_ref[toks[row]] >= l_ref.max() - TOL * np.abs(l_ref).max()
        return dict(zip(order, toks.tolist()))

    V = cfg["vocab"]
    nxt = run([(0, rng.integers(0, V, 40)), (1, rng.integers(0, V, 7)), (2, rng.integers(0, V, 100))])
    nxt = run([(0, [nxt[0]]), (3, rng.integers(0, V, 33)), (1, [nxt[1]]), (2, [nxt[2]])])
    for _ in range(n_decode_steps):
        nxt = run([(sid, [nxt[sid]]) for sid in (2, 0, 3, 1)])
    # a finished sequence gives its slot and blocks to a new one, which must start from the zero state
    slots.release(1); blocks.release(1)
    nxt.update(run([(7, rng.integers(0, V, 21)), (0, [nxt[0]])]))
    run([(7, [nxt[7]]), (2, [nxt[2]])])
    # a single-token sequence is a decode against an empty cache and a zero state
    run([(9, [5])])
    assert model.launches_last_step() > 0
    # a prompt fed in chunks: every chunk after the first continues a cached prefix (positions, cache
    # slots, keys read through the block table, recurrent state carried in the slot), mixed with decode
    # rows and with a chunk that starts another sequence; each step is compared with the oracle run on
    # the whole history, so chunked == whole prompt == oracle
    slots.release(9); blocks.release(9); slots.release(7); blocks.release(7)
    prompt = rng.integers(0, V, 150)
    run([(11, prompt[:64]), (0, [nxt[0]])])
    nxt.update(run([(2, [nxt[2]]), (11, prompt[64:129]), (12, rng.integers(0, V, 20))]))
    last = run([(11, prompt[129:])])
    h_chunked = model.last_hidden()[0].copy()
    slots.release(12); blocks.release(12)
    whole = run([(13, prompt)])
    assert max_rel(model.last_hidden()[0], h_chunked) <= TOL and whole[13] == last[11]
    model.close()


def test_mixed_steps_equal_per_sequence_execution_head_dim_256():
    drive(TINY_HYBRID, 21, 8)


def test_mixed_steps_equal_per_sequence_execution_head_dim_128():
    drive(TINY_HYBRID_128, 22, 4)


@pytest.mark.parametrize("keep_bf16_copy", [True, False])
def test_every_linear_route_gives_the_same_model(keep_bf16_copy):
    """Steps of up to 128 rows run every projection through the fused-dequant kernel, larger steps
    through the dense GEMM over the persistent bf16 copy of the weights or, without one, over a
    per-layer expansion: all against the oracle."""
    cfg = TINY_HYBRID
    qw, deq = make_hybrid(cfg, 41)
    oracle = O.OracleHybrid(cfg, deq)
    rng = np.random.default_rng(9)
    model = HybridModel(cfg, qw, n_pool_blocks=64, max_blocks_per_seq=24, max_step_tokens=512, max_step_seqs=4, n_state_slots=4,
                        keep_bf16_copy=keep_bf16_copy)
    blocks = BlockAllocator(64, 24, seed=5)
    for sid, n in enumerate((200, 330, 60)):
        ids = rng.integers(0, cfg["vocab"], n)
        toks = model.step(ids, [0], [n], blocks.ensure(sid, n)[None, :], [sid])
        assert model.device_status() == 0
        h_ref, l_ref = oracle.forward(ids.astype(np.uint32))
        assert max_rel(model.last_hidden()[0], h_ref[-1]) <= TOL, n
        assert max_rel(model.last_logits()[0], l_ref) <= TOL
        assert toks[0] == O.greedy(model.last_logits()[0])
    model.close()


def test_the_same_sequence_in_steps_on_both_sides_of_every_routing_threshold():
    """The executor picks kernels by the number of rows in a step (GEMV lm_head up to 16 rows, fused-dequant
    linears up to 32, fused input projection and one-launch decode recurrence up to 64, dense GEMMs
    above). The same prompt and the same decode token, replicated into steps of 1, 16, 17, 33, 64, 65 and 129
    rows, must give every row the oracle's hidden state and logits, a token that maximises the oracle's
    logits, and logits that drift across the step sizes by no more than the parity tolerance."""
    cfg = TINY_HYBRID
    qw, deq = make_hybrid(cfg, 51)
    oracle = O.OracleHybrid(cfg, deq)
    rng = np.random.default_rng(4)
    prompt = rng.integers(0, cfg["vocab"], 12).astype(np.uint32)
    h_ref, l_ref = oracle.forward(prompt)
    t_ref = int(O.greedy(l_ref))
    h2_ref, l2_ref = oracle.forward(np.concatenate([prompt, [t_ref]]).astype(np.uint32))
    first = None
    for n in (1, 16, 17, 33, 64, 65, 129):
        model = HybridModel(cfg, qw, n_pool_blocks=n + 2, max_blocks_per_seq=2, max_step_tokens=n * len(prompt), max_step_seqs=n, n_state_slots=n)
        tabs = np.stack([np.array([i, n], np.int32) for i in range(n)])   # one block per sequence (13 tokens), the second entry unused
        toks = model.step(np.tile(prompt, n), [0] * n, [len(prompt)] * n, tabs, list(range(n)))
        assert model.device_status() == 0
        hs, lg = model.last_hidden(), model.last_logits()
        for r in range(n):
            assert max_rel(hs[r], h_ref[-1]) <= TOL and max_rel(lg[r], l_ref) <= TOL, (n, r)
        assert l_ref[toks].min() >= l_ref.max() - TOL * np.abs(l_ref).max(), n
        toks = model.step([t_ref] * n, [len(prompt)] * n, [1] * n, tabs, list(range(n)))   # the decode step, same token everywhere
        assert model.device_status() == 0
        hs, lg = model.last_hidden(), model.last_logits()
        for r in range(n):
            assert max_rel(hs[r], h2_ref[-1]) <= TOL and max_rel(lg[r], l2_ref) <= TOL, (n, r)
        assert l2_ref[toks].min() >= l2_ref.max() - TOL * np.abs(l2_ref).max(), n   # every row decodes a maximum of the oracle's logits
        if first is None:
            first = lg[0].copy()
        else:
            assert max_rel(lg[0], first) <= TOL, n                            # drift across routes
        model.close()


def test_step_rejects_what_it_cannot_run():
    qw, _ = make_hybrid(TINY_HYBRID_128, 3)
    model = HybridModel(TINY_HYBRID_128, qw, n_pool_blocks=8, max_blocks_per_seq=8, max_step_tokens=64, max_step_seqs=2, n_state_slots=2)
    tab = np.array([[0, 1, 2, 3, 4, 5, 6, 7]], np.int32)
    with pytest.raises(ComputeError):   # state slot outside the pool
        model.step([1], [0], [1], tab, [2])
    with pytest.raises(ComputeError):   # one slot for two sequences
        model.step([1, 2], [0, 0], [1, 1], np.concatenate([tab, tab]), [1, 1])
    with pytest.raises(ComputeError):   # more tokens than the step workspace
        model.step([1] * 65, [0], [65], tab, [0])
    with pytest.raises(Exception):      # beyond the block table
        model.step([1], [128], [1], tab, [0])
    model.close()
