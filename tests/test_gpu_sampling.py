"""The device sampling chain against the oracle's restatement of the reference's decode crate
(crates/decode/src/processors.rs, sampler.rs, chain.rs), row by row, at the decoder vocabulary size.
Temperature, top-k and the repetition penalty are bit-exact; top-p, min-p and the multinomial walk sum
probabilities in a different order than the reference's sequential sums, so a token exactly at a cut
may differ: any difference must sit at the cut (checked on the probabilities in float64)."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import DEV
from logismos_b200 import sampling as S
from logismos_b200.ops import InvalidOp

pytestmark = pytest.mark.gpu
V = 151936


def rows(seed, n_rows=5, n=V, scale=3.0):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((n_rows, n)) * scale).astype(np.float32)
    x[1] = np.round(x[1] * 2) / 2          # a row full of ties
    x[2, : n // 2] = -np.inf               # a row half masked by an earlier processor
    return x


def probs64(row):
    r = row.astype(np.float64)
    e = np.where(np.isfinite(r), np.exp(r - r[np.isfinite(r)].max()), 0.0)
    return e / e.sum()


def run(proc, x):
    t = torch.from_numpy(x.copy()).to(DEV)
    proc.process(t)
    torch.cuda.synchronize()
    return t.cpu().numpy()


def test_temperature_top_k_and_repetition_penalty_are_bit_exact():
    x = rows(1)
    for t in (0.7, 1.0, 0.0, 2.5):
        got = run(S.TemperatureScale(t), x)
        for r in range(x.shape[0]):
            assert np.array_equal(got[r], O.temperature(x[r], t), equal_nan=True)
    xn = x.copy(); xn[0, 5] = np.nan; xn[3, 77] = np.nan
    for k in (1, 2, 50, 1000, V - 1, V, 0):
        got = run(S.TopK(k), xn)
        for r in range(x.shape[0]):
            assert np.array_equal(got[r], O.top_k(xn[r], k), equal_nan=True), (k, r)
    rng = np.random.default_rng(2)
    toks = rng.integers(0, V, (x.shape[0], 40)).astype(np.uint32)
    toks[0, 3] = toks[0, 2]; toks[1, 0] = V + 5   # listed twice; outside the vocabulary
    counts = np.array([40, 7, 0, 40, 13], np.int32)
    xr = x.copy(); xr[2] = np.abs(xr[4])  # finite rows
    got = run(S.RepetitionPenalty(torch.from_numpy(toks.view(np.int32)).to(DEV), torch.from_numpy(counts).to(DEV), 1.3), xr)
    for r in range(x.shape[0]):
        assert np.array_equal(got[r], O.repetition_penalty(xr[r], toks[r, : counts[r]], 1.3)), r


SUM_TOL = 1e-3  # the reference normalises by, and accumulates, SEQUENTIAL fp32 sums over up to 151936 terms: its own cut sits 1e-4..3e-4 (relative) off the exact one


@pytest.mark.parametrize("p", [0.05, 0.5, 0.9, 0.999, 1.0, 0.0])
def test_top_p_keeps_the_reference_nucleus(p):
    """Both nuclei are prefixes of the same order (descending probability, ties by index). They may differ
    in length only where the cumulative mass (float64) is within the reference's own summation error of p:
    its softmax divides by a sequential fp32 sum, the device sums pairwise."""
    x = rows(3)
    got = run(S.TopP(p), x)
    for r in range(x.shape[0]):
        ref = O.top_p(x[r], p)
        kg, kr = np.isfinite(got[r]), np.isfinite(ref)
        assert np.array_equal(got[r][kg], x[r][kg])  # kept logits are untouched
        if np.array_equal(kg, kr):
            continue
        pr = probs64(x[r])
        order = np.argsort(-pr, kind="stable")
        cum = np.cumsum(pr[order])
        ng, nr = int(kg.sum()), int(kr.sum())
        assert kg[order[:ng]].all() and kr[order[:nr]].all(), (p, r)   # both are prefixes of the order
        lo, hi = sorted((ng, nr))
        assert cum[lo - 1] >= p * (1 - SUM_TOL) and cum[hi - 2] <= p * (1 + SUM_TOL), (p, r, ng, nr, cum[lo - 1], cum[hi - 2])


@pytest.mark.parametrize("p", [0.001, 0.05, 0.5, 1.0, 0.0])
def test_min_p_masks_the_reference_tail(p):
    x = rows(4)
    got = run(S.MinP(p), x)
    for r in range(x.shape[0]):
        ref = O.min_p(x[r], p)
        diff = np.flatnonzero(np.isfinite(got[r]) != np.isfinite(ref))
        if diff.size:
            pr = probs64(x[r])
            thr = min(max(p, 0.0), 1.0) * pr.max()
            assert np.all(np.abs(pr[diff] - thr) <= 1e-5 * thr), (p, r, diff[:5])


def test_multinomial_returns_the_reference_token_for_the_same_draw():
    x = rows(5, n_rows=6)
    x[5] = -np.inf; x[5, 1234] = 0.5     # all the mass on one token
    x[4] = -np.inf                       # no mass at all: greedy, which returns index 0
    rng = np.random.default_rng(6)
    t = torch.from_numpy(x).to(DEV)
    sampler = S.MultinomialSampler(seed=1)
    for trial in range(6):
        u = rng.random(6).astype(np.float32)
        if trial == 0:
            u[:] = [0.0, 0.999999, 0.5, 1e-7, 0.3, 0.9]
        got = sampler.sample(t, uniforms=torch.from_numpy(u).to(DEV)).cpu().numpy().view(np.uint32)
        for r in range(6):
            ref = O.multinomial(x[r], float(u[r]))
            if got[r] != ref:
                cdf = np.cumsum(probs64(x[r]))
                lo, hi = sorted((int(got[r]), ref))
                assert cdf[hi - 1] - cdf[lo] <= SUM_TOL and abs(cdf[lo] - u[r]) <= SUM_TOL, (trial, r, got[r], ref)
    # seeded draws are reproducible (sampler.rs:72-82)
    a = S.MultinomialSampler(seed=42); b = S.MultinomialSampler(seed=42)
    for _ in range(4):
        assert torch.equal(a.sample(t), b.sample(t))


def test_chain_runs_processors_in_order_then_samples():  # chain.rs:33-76, :88-121
    x = rows(7)
    base = torch.from_numpy(x.copy()).to(DEV)
    chain = S.DecodeChain(S.GreedySampler()).push(S.TemperatureScale(0.8)).push(S.TopK(50)).push(S.TopP(0.95))
    assert len(chain) == 3 and not chain.is_empty()
    toks = chain.step(base).cpu().numpy().view(np.uint32)
    for r in range(x.shape[0]):
        ref = O.top_p(O.top_k(O.temperature(x[r], 0.8), 50), 0.95)
        assert toks[r] == O.greedy(ref)
        assert np.isfinite(base[r].cpu().numpy()).sum() <= 50 + (x[r] == np.sort(x[r])[-50]).sum()
    # a peaked small row, the reference's own example: cooling then top-p keeps only index 0
    small = torch.tensor([[3.0, 2.9, 2.8, 2.7]], dtype=torch.float32, device=DEV)
    c2 = S.DecodeChain(S.GreedySampler()).push(S.TemperatureScale(0.1)).push(S.TopP(0.5))
    assert int(c2.step(small)[0]) == 0 and torch.isinf(small[0, 1:]).all()
    with pytest.raises(InvalidOp):
        S.TopK(5).process(torch.zeros((2, 8)))  # CPU tensor: no CPU arm
