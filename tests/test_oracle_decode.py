"""The oracle's restatement of the reference's logit processors and samplers against the decode
crate's own unit-test vectors (crates/decode/src/processors.rs:213-360, sampler.rs:66-100,
chain.rs:88-130, lib.rs:90-92)."""
import numpy as np

import oracle_lib as O

NEG = -np.inf


def test_temperature_divides_and_one_is_identity():  # processors.rs:213-228
    assert O.temperature([1.0, 2.0, 3.0], 2.0).tolist() == [0.5, 1.0, 1.5]
    assert O.temperature([1.0, 2.0, 3.0], 1.0).tolist() == [1.0, 2.0, 3.0]
    # a temperature of zero is clamped to 1e-6 instead of producing infinities (:12-15, :20)
    assert np.isfinite(O.temperature([1.0, -2.0], 0.0)).all()


def test_top_k_masks_below_kth():  # processors.rs:231-242
    out = O.top_k([1.0, 3.0, 2.0, 5.0, 4.0], 2)
    assert out.tolist() == [NEG, NEG, NEG, 5.0, 4.0]
    assert O.top_k([1.0, 3.0, 2.0], 0).tolist() == [1.0, 3.0, 2.0]   # k == 0 and k >= n: identity (:52-54)
    assert O.top_k([1.0, 3.0, 2.0], 3).tolist() == [1.0, 3.0, 2.0]
    assert O.top_k([2.0, 5.0, 5.0, 1.0], 1).tolist() == [NEG, 5.0, 5.0, NEG]  # ties with the threshold survive (:77)


def test_top_k_masks_nan_logit():  # processors.rs:245-262
    out = O.top_k([1.0, np.nan, 5.0, 4.0, 3.0], 2)
    assert out.tolist() == [NEG, NEG, 5.0, 4.0, NEG]


def test_top_p_nucleus_keeps_dominant_prefix():  # processors.rs:303-312
    assert O.top_p([10.0, 0.0, 0.0, 0.0], 0.5).tolist() == [10.0, NEG, NEG, NEG]
    assert O.top_p([1.0, 2.0], 1.0).tolist() == [1.0, 2.0]
    # four near-equal probabilities: the cumulative sum reaches 0.5 after two entries (chain.rs:104-110)
    assert O.top_p([3.0, 2.9, 2.8, 2.7], 0.5).tolist()[:2] == [3.0, np.float32(2.9)]
    assert O.top_p([3.0, 2.9, 2.8, 2.7], 0.5).tolist()[2:] == [NEG, NEG]
    # equal probabilities are taken in index order (stable sort)
    assert O.top_p([1.0, 1.0, 1.0, 1.0], 0.4).tolist() == [1.0, 1.0, NEG, NEG]


def test_min_p_masks_tails():  # processors.rs:315-325
    assert O.min_p([5.0, 0.0, 0.0, 0.0], 0.5).tolist() == [5.0, NEG, NEG, NEG]
    assert O.min_p([5.0, 0.0], 0.0).tolist() == [5.0, 0.0]


def test_repetition_penalty():  # processors.rs:328-349
    assert O.repetition_penalty([2.0, 4.0, 1.0], [1], 2.0).tolist() == [2.0, 2.0, 1.0]
    assert O.repetition_penalty([-2.0, -4.0, 1.0], [1], 2.0).tolist() == [-2.0, -8.0, 1.0]
    assert O.repetition_penalty([2.0, 4.0, 1.0], [1, 1, 9], 2.0).tolist() == [2.0, 1.0, 1.0]  # listed twice: twice; out of range: skipped
    assert O.repetition_penalty([2.0, 4.0], [1], 1.0).tolist() == [2.0, 4.0]


def test_multinomial_walks_the_cdf():  # sampler.rs:31-58
    logits = np.array([1.0, 2.0, 3.0, 4.0], np.float32)
    p = np.exp(logits - 4.0); p /= p.sum()
    cdf = np.cumsum(p)
    for u in (0.0, 0.01, 0.05, 0.2, 0.35, 0.36, 0.9, 0.999999):
        assert O.multinomial(logits, u) == int(np.searchsorted(cdf, u, side="right"))
    # one dominant token takes (almost) every draw (sampler.rs:85-99)
    hits = sum(O.multinomial([10.0, 0.0, 0.0, 0.0], u) == 0 for u in np.random.default_rng(7).random(100))
    assert hits > 90
    assert O.multinomial([NEG, NEG, 2.0, NEG], 0.7) == 2          # masked logits carry no mass
    assert O.multinomial([NEG, NEG, NEG], 0.3) == O.greedy(np.array([NEG, NEG, NEG], np.float32))  # no mass: greedy (:43-45)
    assert O.multinomial([], 0.3) == 0


def test_chain_order_temperature_then_top_p():  # chain.rs:88-121: both orders pick index 0 here
    base = np.array([3.0, 2.9, 2.8, 2.7], np.float32)
    a = O.top_p(O.temperature(base, 0.1), 0.5)
    b = O.temperature(O.top_p(base, 0.5), 0.1)
    assert O.greedy(a) == O.greedy(b) == 0
    assert np.isinf(a[1:]).all() and np.isfinite(b[:2]).all()
