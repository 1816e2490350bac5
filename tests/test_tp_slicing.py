"""Weight slicing for the tensor-parallel hybrid decoder: the rank slices partition every
projection (input projections by rows, output projections by whole 32-value groups of columns)."""
import numpy as np
import pytest

from hybrid_weights import TINY_HYBRID, make_hybrid
from logismos_b200.tp import slice_hybrid_weights

CFG = dict(TINY_HYBRID, gdn_heads=16)


def test_slicing_partitions_every_projection():
    qw, _ = make_hybrid(CFG, 4)
    parts = [slice_hybrid_weights(CFG, qw, 2, r) for r in range(2)]
    for l, lw in enumerate(qw["layers"]):
        for n in ("wq", "wk", "wv", "wgate", "w_gate", "w_up"):
            assert np.array_equal(np.concatenate([p[1]["layers"][l][n][0] for p in parts]), lw[n][0])
            assert np.array_equal(np.concatenate([p[1]["layers"][l][n][1] for p in parts]), lw[n][1])
        for n in ("wo", "w_down"):
            assert np.array_equal(np.concatenate([p[1]["layers"][l][n][0] for p in parts], axis=1), lw[n][0])
            assert np.array_equal(np.concatenate([p[1]["layers"][l][n][1] for p in parts], axis=1), lw[n][1])
    assert parts[0][0]["n_heads"] == 2 and parts[0][0]["gdn_heads"] == 8 and parts[0][0]["intermediate"] == 512
    with pytest.raises(ValueError):
        slice_hybrid_weights(dict(CFG, n_kv_heads=1), qw, 2, 0)
