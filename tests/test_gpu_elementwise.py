"""Parity of the memory-bound encoder kernels against the oracle's cpu_f32 restatement."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import DEV, TOL, bf16_cuda, max_rel, to_np
from logismos_b200 import ops

pytestmark = pytest.mark.gpu


def test_embed_lookup_is_a_bit_exact_gather_with_zero_rows_for_bad_ids():
    rng = np.random.default_rng(0)
    vocab, hidden = 1000, 1536
    table_t, table = bf16_cuda(rng.standard_normal((vocab, hidden)) * 0.02)
    ids = rng.integers(0, vocab, 77).astype(np.uint32)
    ids[[3, 50]] = [vocab, 2**32 - 1]  # out of range -> zero rows (cpu_f32/mod.rs:96-104)
    out = ops.embed_lookup(table_t, torch.from_numpy(ids.view(np.int32)).to(DEV))
    ref = O.embed_lookup(table, hidden, vocab, ids).reshape(77, hidden)
    assert (to_np(out).view(np.uint32) == ref.view(np.uint32)).all()


@pytest.mark.parametrize("rows,n", [(1, 4), (5, 1536), (33, 2048), (3, 8192), (7, 100),
                                    (1500, 1536), (1030, 2048), (1024, 512), (1100, 100), (1025, 1028)])  # tall: a warp per row
def test_rms_norm_f32(rows, n):
    rng = np.random.default_rng(rows + n)
    x = rng.standard_normal((rows, n)).astype(np.float32) * 3; w = rng.standard_normal(n).astype(np.float32)
    ref = O.rms_norm(x, w, rows, n, 1e-6).reshape(rows, n)
    yf = ops.rms_norm_f32(torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV), 1e-6, out_f32=True)
    assert max_rel(to_np(yf), ref) < 1e-5
    yb = ops.rms_norm_f32(torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV), 1e-6)
    assert max_rel(to_np(yb), ref) < 8e-3  # one bf16 rounding


@pytest.mark.parametrize("d", [128, 256, 40])  # 40: not a multiple of 16, the narrow-access kernel
def test_rope_halves_on_packed_qkv_rows(d):
    rng = np.random.default_rng(2)
    T, nh, nkv = 37, 6, 2
    stride = (nh + 2 * nkv) * d
    qkv_t, qkv = bf16_cuda(rng.standard_normal((T, stride)))
    pos = rng.integers(0, 300, T).astype(np.int32)
    cos, sin = O.build_rope_table_f32(512, d, 1e6)
    got = ops.rope_halves_(qkv_t.clone(), torch.from_numpy(cos.reshape(512, d // 2)).to(DEV),
                           torch.from_numpy(sin.reshape(512, d // 2)).to(DEV), torch.from_numpy(pos).to(DEV), nh + nkv, d)
    ref = qkv.copy()
    rot = np.ascontiguousarray(ref[:, : (nh + nkv) * d]).reshape(T * (nh + nkv), d)
    cr, sr = O.rope_gather(cos, sin, 512, d, np.repeat(pos, nh + nkv))
    O.rope_halves_in_place(rot.reshape(-1), cr, sr, T * (nh + nkv), d)
    ref[:, : (nh + nkv) * d] = rot.reshape(T, -1)
    g = to_np(got)
    assert max_rel(g[:, : (nh + nkv) * d], ref[:, : (nh + nkv) * d]) < 8e-3
    assert (g[:, (nh + nkv) * d:] == qkv[:, (nh + nkv) * d:]).all()  # v heads untouched


def test_rope_position_beyond_table_is_reported():  # RopeTable::gather (rope.rs:57-66)
    qkv_t, _ = bf16_cuda(np.ones((2, 256)))
    cos, sin = O.build_rope_table_f32(4, 128, 1e6)
    with pytest.raises(ops.InvalidOp):
        ops.rope_halves_(qkv_t, torch.from_numpy(cos.reshape(4, 64)).to(DEV), torch.from_numpy(sin.reshape(4, 64)).to(DEV),
                         torch.tensor([0, 4], dtype=torch.int32, device=DEV), 2, 128)


def test_swiglu():
    rng = np.random.default_rng(3)
    T, inter = 19, 8960
    gu_t, gu = bf16_cuda(rng.standard_normal((T, 2 * inter)) * 2)
    ref = O.hadamard(O.silu(gu[:, :inter].ravel()), gu[:, inter:].ravel()).reshape(T, inter)
    assert max_rel(to_np(ops.swiglu(gu_t)), ref) < 8e-3


def test_pool_head_matches_encode_raw_tail_including_empty_sequence():
    rng = np.random.default_rng(4)
    hidden, dim = 1536, 1024
    cu = np.array([0, 5, 5, 40, 41], np.int32)
    hs = rng.standard_normal((41, hidden)).astype(np.float32)
    hw_t, hw = bf16_cuda(rng.standard_normal((dim, hidden)) * 0.02)
    hb = (rng.standard_normal(dim) * 0.02).astype(np.float32)
    got = to_np(ops.pool_head(torch.from_numpy(hs).to(DEV), torch.from_numpy(cu).to(DEV), hw_t, torch.from_numpy(hb).to(DEV)))
    for i in range(4):
        seg = hs[cu[i]:cu[i + 1]]
        p = O.mean_pool_masked(seg, np.ones(len(seg), np.uint8), len(seg), hidden) if len(seg) else np.zeros(hidden, np.float32)
        O.l2_normalize_in_place(p)
        y = O.linear_t(p, hw, hb, 1, dim, hidden)
        O.l2_normalize_in_place(y)
        assert np.abs(got[i] - y).max() < 2e-5
    assert np.isfinite(got).all()


def test_greedy_argmax_first_max_wins_and_nan_is_never_selected():  # decode/src/lib.rs:73-92
    rng = np.random.default_rng(5)
    logits = rng.standard_normal((6, 151936)).astype(np.float32)
    logits[0, [100, 70000]] = 9.0          # tie: first index wins
    logits[1, 5] = np.nan; logits[1, 9] = 50.0
    logits[2, :] = -np.inf                 # nothing exceeds -inf -> 0
    logits[3, :] = np.nan
    logits[4, 151935] = 99.0
    got = ops.greedy(torch.from_numpy(logits).to(DEV)).cpu().numpy()
    assert got.tolist() == [O.greedy(r) for r in logits]
    assert got[0] == 100 and got[2] == 0 and got[3] == 0 and got[4] == 151935
    lb, lbf = bf16_cuda(logits[5:6])
    assert int(ops.greedy(lb).cpu()[0]) == O.greedy(lbf[0])
