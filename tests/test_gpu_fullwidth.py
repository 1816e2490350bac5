"""The two decoder executors at the WIDTH of their benchmark configurations (a few layers deep): one
mixed step with decode rows that have real cached history, a prefill chunk that starts a sequence and
one that continues a cached prefix, compared per sequence with the CPU oracle run on the whole
history: hidden states and logits element-wise per row, and the emitted token against the oracle's
own logits.

  ragged continuous-batching step: hidden 1536, 12 query / 2 KV heads of 128, SwiGLU 8960, vocab
      151936, int4 group-32 weights (2 of the 28 layers)
  hybrid serving stack: hidden 2048, 16 linear-attention heads of 128, 16 query / 2 KV heads of
      256, SwiGLU 6144, vocab 151936, int4 group-32 weights (4 of the 48 layers = one 3:1 group)
"""
import numpy as np
import pytest

import oracle_lib as O
from gpu_util import TOL, cosine, max_rel, row_rel
from hybrid_weights import make_hybrid
from logismos_b200.decoder import BlockAllocator, DecoderModel
from logismos_b200.hybrid import HYBRID_SERVING, HybridModel
from stella_weights import STELLA_1_5B, make_weights, quantize_weights

pytestmark = pytest.mark.gpu


def check_rows(hs, lg, toks, refs):
    """refs: per row (hidden_ref [hidden], logits_ref [vocab])."""
    for row, (h_ref, l_ref) in enumerate(refs):
        assert row_rel(hs[row], h_ref) <= TOL and cosine(hs[row], h_ref) >= 0.9995, row
        assert max_rel(lg[row], l_ref) <= TOL and cosine(lg[row], l_ref) >= 0.9995, row
        assert toks[row] == O.greedy(lg[row])
        # the emitted token is the oracle's choice, or within the logit tolerance of it
        assert l_ref[toks[row]] >= l_ref.max() - TOL * np.abs(l_ref).max(), row


def test_ragged_step_decoder_at_benchmark_width():
    cfg = dict(STELLA_1_5B, vocab=151936, n_layers=2)
    w = make_weights(cfg, 301)
    qw, deq = quantize_weights(cfg, w)
    oracle = O.OracleStella(cfg, deq)
    rng = np.random.default_rng(302)
    V = cfg["vocab"]
    alloc = BlockAllocator(256, 64, seed=1)
    model = DecoderModel(cfg, qw, n_pool_blocks=256, max_blocks_per_seq=64, max_step_tokens=1024, max_step_seqs=8)
    hist = {0: rng.integers(0, V, 70).tolist(), 1: rng.integers(0, V, 300).tolist(), 2: rng.integers(0, V, 33).tolist(),
            3: rng.integers(0, V, 150).tolist()}
    # step 1: the histories enter the cache (sequence 3 only its first 64 tokens)
    ids = hist[0] + hist[1] + hist[2] + hist[3][:64]
    toks = model.step(ids, [0, 0, 0, 0], [70, 300, 33, 64],
                      np.stack([alloc.ensure(i, n) for i, n in ((0, 70), (1, 300), (2, 33), (3, 64))]))
    assert model.device_status() == 0
    # step 2: three decode rows on that history, a 512-token prompt that starts, and the rest of sequence 3
    for i in range(3):
        hist[i].append(int(toks[i]))
    hist[4] = rng.integers(0, V, 512).tolist()
    entries = [(0, 70, 1), (4, 0, 512), (1, 300, 1), (3, 64, 86), (2, 33, 1)]
    ids = [t for sid, c, n in entries for t in hist[sid][c:c + n]]
    toks = model.step(ids, [c for _, c, _ in entries], [n for _, _, n in entries],
                      np.stack([alloc.ensure(sid, c + n) for sid, c, n in entries]))
    assert model.device_status() == 0
    refs = []
    for sid, c, n in entries:
        h = oracle.forward(np.asarray(hist[sid], np.uint32), causal=True)[-1]
        refs.append((h, O.linear_t(h, deq["lm_head"], None, 1, V, cfg["hidden"])))
    check_rows(model.last_hidden(), model.last_logits(), toks, refs)
    model.close()


def test_hybrid_decoder_at_serving_width():
    cfg = dict(HYBRID_SERVING, n_layers=4, max_pos=1024)
    qw, deq = make_hybrid(cfg, 311)
    oracle = O.OracleHybrid(cfg, deq)
    rng = np.random.default_rng(312)
    V = cfg["vocab"]
    alloc = BlockAllocator(128, 32, seed=2)
    model = HybridModel(cfg, qw, n_pool_blocks=128, max_blocks_per_seq=32, max_step_tokens=512, max_step_seqs=8, n_state_slots=8)
    hist = {0: rng.integers(0, V, 40).tolist(), 1: rng.integers(0, V, 130).tolist(), 2: rng.integers(0, V, 17).tolist(),
            3: rng.integers(0, V, 200).tolist()}
    ids = hist[0] + hist[1] + hist[2] + hist[3][:128]
    toks = model.step(ids, [0, 0, 0, 0], [40, 130, 17, 128],
                      np.stack([alloc.ensure(i, n) for i, n in ((0, 40), (1, 130), (2, 17), (3, 128))]), [0, 1, 2, 3])
    assert model.device_status() == 0
    for i in range(3):
        hist[i].append(int(toks[i]))
    hist[4] = rng.integers(0, V, 100).tolist()
    entries = [(3, 128, 72), (0, 40, 1), (1, 130, 1), (4, 0, 100), (2, 17, 1)]
    ids = [t for sid, c, n in entries for t in hist[sid][c:c + n]]
    toks = model.step(ids, [c for _, c, _ in entries], [n for _, _, n in entries],
                      np.stack([alloc.ensure(sid, c + n) for sid, c, n in entries]), [sid for sid, _, _ in entries])
    assert model.device_status() == 0
    refs = []
    for sid, c, n in entries:
        h_ref, l_ref = oracle.forward(np.asarray(hist[sid], np.uint32))
        refs.append((h_ref[-1], l_ref))
    check_rows(model.last_hidden(), model.last_logits(), toks, refs)
    # decode steps at this width (fused int4 linears, recurrence over the slots, paged decode at head_dim 256)
    for _ in range(2):
        for (sid, c, n), t in zip(entries, toks):
            hist[sid].append(int(t))
        entries = [(sid, len(hist[sid]) - 1, 1) for sid, _, _ in entries]
        toks = model.step([hist[sid][-1] for sid, _, _ in entries], [c for _, c, _ in entries], [1] * 5,
                          np.stack([alloc.ensure(sid, c + 1) for sid, c, _ in entries]), [sid for sid, _, _ in entries])
        assert model.device_status() == 0
    refs = []
    for sid, c, n in entries:
        h_ref, l_ref = oracle.forward(np.asarray(hist[sid], np.uint32))
        refs.append((h_ref[-1], l_ref))
    check_rows(model.last_hidden(), model.last_logits(), toks, refs)
    model.close()
