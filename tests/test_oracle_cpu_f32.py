"""Pins the oracle's cpu_f32 restatement against the known-answer vectors of the reference's
own unit tests (crates/kernels/src/cpu_f32/tests.rs; the test each case mirrors is named)."""
import math

import numpy as np
import pytest

import oracle_lib as O

A = lambda *v: np.array(v, dtype=np.float32)


def test_embed_lookup_in_range_copies_rows():  # tests.rs:6-14
    out = O.embed_lookup(A(1, 2, 10, 20, 100, 200), 2, 3, [1, 0, 2])
    assert out.tolist() == [10, 20, 1, 2, 100, 200]


def test_embed_lookup_out_of_range_id_yields_zeroed_row():  # tests.rs:17-31
    out = O.embed_lookup(A(1, 2, 10, 20), 2, 2, [0, 5])
    assert out.tolist() == [1, 2, 0, 0]


def test_rms_norm_matches_manual():  # tests.rs:34-43
    y = O.rms_norm(A(1, 2, 3, 4), np.ones(4, np.float32), 1, 4, 1e-6)
    inv = np.float32(1.0) / np.sqrt(np.float32(30.0 / 4.0) + np.float32(1e-6))
    assert np.abs(y - A(1, 2, 3, 4) * inv).max() < 1e-6


def test_linear_matches_hand_computed():  # tests.rs:46-63
    y = O.linear(A(1, 2, 3, 4, 5, 6), A(1, 0, 0, 1, 1, 1), A(100, 200), 2, 2, 3)
    assert np.abs(y - A(104, 205, 110, 211)).max() < 1e-5


def test_linear_matches_linear_t_with_transposed_weight():  # tests.rs:66-81
    a = A(1, 2, 3, 4, 5, 6)
    l = O.linear(a, A(1, 0, 0, 1, 1, 1), None, 2, 2, 3)
    lt = O.linear_t(a, A(1, 0, 1, 0, 1, 1), None, 2, 2, 3)
    assert np.abs(l - lt).max() < 1e-5


def test_linear_t_matches_naive():  # tests.rs:84-92
    y = O.linear_t(A(1, 2, 3), A(1, 0, 0, 0, 1, 1), A(10, 20), 1, 2, 3)
    assert abs(y[0] - 11) < 1e-6 and abs(y[1] - 25) < 1e-6


@pytest.mark.parametrize("fn,a,b,bias,m,n,k", [
    ("linear", 5, 6, None, 2, 2, 3),      # tests.rs:95-109 a.len() mismatch
    ("linear", 6, 5, None, 2, 2, 3),      # tests.rs:112-117 b.len() mismatch
    ("linear", 6, 6, 1, 2, 2, 3),         # tests.rs:120-126 bias.len() mismatch
    ("linear_t", 2, 6, None, 1, 2, 3),    # tests.rs:207-212
    ("linear_t", 3, 5, None, 1, 2, 3),    # tests.rs:215-220
])
def test_linear_shape_mismatch_panics(fn, a, b, bias, m, n, k):
    with pytest.raises(O.OraclePanic):
        getattr(O, fn)(np.ones(a, np.float32), np.ones(b, np.float32),
                       None if bias is None else np.ones(bias, np.float32), m, n, k)


def test_linear_overflowing_shape_is_rejected_not_wrapped():  # tests.rs:129-153
    k = 2
    m = (2**64 - 1) // k + 2
    assert (m * k) % 2**64 == 2
    with pytest.raises(O.OraclePanic) as e:
        O.linear(A(1, 2), A(1, 2), None, m, 1, k)
    assert e.value.args[0] == 1  # rejected on a.len(), not wrapped


@pytest.mark.parametrize("fn", ["linear", "linear_t"])
def test_output_shape_overflow_is_rejected(fn):  # tests.rs:156-204
    n = 2
    m = (2**64 - 1) // n + 2
    with pytest.raises(O.OraclePanic) as e:
        getattr(O, fn)(np.zeros(0, np.float32), np.zeros(0, np.float32), None, m, n, 0)
    assert e.value.args[0] == 4


def test_softmax_rows_sum_to_one():  # tests.rs:223-230
    y = O.softmax_last_dim(A(0, 1, 2, -1, 0, 1), 2, 3).reshape(2, 3)
    assert np.abs(y.sum(1) - 1).max() < 1e-6


def test_softmax_fully_masked_row_is_uniform_not_nan():  # tests.rs:233-247
    y = O.softmax_last_dim(np.full(4, -np.inf, np.float32), 1, 4)
    assert np.isfinite(y).all() and np.abs(y - 0.25).max() < 1e-6


def test_softmax_mixed_masked_and_unmasked_rows_both_finite():  # tests.rs:250-274
    ninf = -np.inf
    y = O.softmax_last_dim(A(ninf, ninf, ninf, 0, 1, 2), 2, 3).reshape(2, 3)
    assert np.isfinite(y).all() and np.abs(y.sum(1) - 1).max() < 1e-6


def test_rope_zero_pos_identity_halves():  # tests.rs:277-282
    x = A(1, 2, 3, 4)
    cos, sin = O.build_rope_table_f32(1, 4, 1_000_000.0)
    O.rope_halves_in_place(x, cos, sin, 1, 4)
    assert x.tolist() == [1, 2, 3, 4]


def test_rope_table_nonzero_position_matches_hand_computed_angles():  # tests.rs:285-326
    cos, sin = O.build_rope_table_f32(2, 4, 10_000.0)
    half = 2
    assert abs(cos[half] - math.cos(1.0)) < 1e-5 and abs(sin[half] - math.sin(1.0)) < 1e-5
    assert abs(cos[half + 1] - math.cos(0.01)) < 1e-5 and abs(sin[half + 1] - math.sin(0.01)) < 1e-5


def test_rope_table_is_f64_evaluated_then_cast():  # mod.rs:606-615
    cos, sin = O.build_rope_table_f32(64, 128, 1e6)
    pos, i = 37, 11
    ang = pos * (1e6 ** (-(2.0 * i) / 128.0))
    assert cos[pos * 64 + i] == np.float32(math.cos(ang)) and sin[pos * 64 + i] == np.float32(math.sin(ang))


def test_rope_rotation_is_inverse():  # tests.rs:329-343
    x = A(1, 2); orig = x.copy()
    c = A(math.sqrt(0.5)); s = A(math.sqrt(0.5))
    O.rope_halves_in_place(x, c, s, 1, 2)
    O.rope_halves_in_place(x, c, -s, 1, 2)
    assert np.abs(x - orig).max() < 1e-5


def test_mean_pool_respects_mask():  # tests.rs:346-351
    assert O.mean_pool_masked(A(1, 2, 3, 4, 5, 6), [1, 0, 1], 3, 2).tolist() == [3, 4]


def test_mean_pool_all_zero_mask_stays_finite():  # tests.rs:354-370
    assert O.mean_pool_masked(A(1, 2, 3, 4, 5, 6), [0, 0, 0], 3, 2).tolist() == [0, 0]


def test_l2_normalize_projects_to_unit():  # tests.rs:373-378
    v = A(3, 4); O.l2_normalize_in_place(v)
    assert abs(v[0] - 0.6) < 1e-6 and abs(v[1] - 0.8) < 1e-6


def test_l2_normalize_zero_vector_is_finite():  # mod.rs:587 clamp
    v = np.zeros(4, np.float32); O.l2_normalize_in_place(v)
    assert np.isfinite(v).all()


def test_mask_additive_broadcasts_across_heads():  # tests.rs:381-392
    s = np.ones(12, np.float32)
    O.mask_additive_in_place(s, [1, 0, 1, 1, 1, 1], 4, 3)
    assert np.isfinite(s[0]) and s[1] == -np.inf and np.isfinite(s[2]) and s[4] == -np.inf
    assert np.isfinite(s[6:]).all()


def test_mask_additive_zero_n_and_empty_mask_are_noops():  # tests.rs:395-404, :430-444
    s = np.zeros(0, np.float32)
    O.mask_additive_in_place(s, np.zeros(0, np.uint8), 4, 0)
    s = np.ones(12, np.float32)
    O.mask_additive_in_place(s, np.zeros(0, np.uint8), 4, 3)
    assert (s.view(np.uint32) == np.float32(1).view(np.uint32)).all()


def test_mask_additive_non_dividing_rows_panics():  # tests.rs:407-427
    with pytest.raises(O.OraclePanic):
        O.mask_additive_in_place(np.ones(15, np.float32), [1, 0, 1, 1, 1, 1], 5, 3)


def test_hadamard_mismatched_lengths_panics():  # tests.rs:447-462
    with pytest.raises(O.OraclePanic):
        O.hadamard(A(1, 2, 3), A(1, 2))


def test_silu_matches_manual():  # tests.rs:465-470
    y = O.silu(A(0, 1, -1))
    assert abs(y[0]) < 1e-6
    assert abs(y[1] - 1 / (1 + math.exp(-1))) < 1e-6 and abs(y[2] + 1 / (1 + math.exp(1))) < 1e-6


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (7, 19, 33), (97, 130, 300), (128, 1536, 1536), (5, 8960, 64)])
def test_sgemm_against_float64(m, n, k):
    """The blocked SGEMM standing in for matrixmultiply::sgemm agrees with a float64 product."""
    rng = np.random.default_rng(m * 1000 + n)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    want = a.astype(np.float64) @ w.astype(np.float64).T + bias
    got = O.linear_t(a, w, bias, m, n, k).reshape(m, n)
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max()) * math.sqrt(k)
    got2 = O.linear(a, np.ascontiguousarray(w.T), bias, m, n, k).reshape(m, n)
    assert np.abs(got2 - want).max() <= 1e-5 * max(1.0, np.abs(want).max()) * math.sqrt(k)
