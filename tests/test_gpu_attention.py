"""Ragged attention (encoder / prefill) against the oracle's restatement of
QwenAttention::forward's score / softmax / PV stage."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import DEV, TOL, bf16_cuda, max_rel, to_np
from logismos_b200 import ops

pytestmark = pytest.mark.gpu


def run_case(lens, nh, nkv, causal, seed, d=128):
    rng = np.random.default_rng(seed)
    T = int(sum(lens))
    stride = (nh + 2 * nkv) * d
    qkv_t, qkv = bf16_cuda(rng.standard_normal((T, stride)))
    cu = np.zeros(len(lens) + 1, np.int32); cu[1:] = np.cumsum(lens)
    out = to_np(ops.varlen_attention(qkv_t, torch.from_numpy(cu).to(DEV), nh, nkv, d, causal=causal))
    for i, L in enumerate(lens):
        if L == 0:
            continue
        seg = qkv[cu[i]:cu[i + 1]]
        q = np.ascontiguousarray(seg[:, : nh * d]); k = np.ascontiguousarray(seg[:, nh * d:(nh + nkv) * d])
        v = np.ascontiguousarray(seg[:, (nh + nkv) * d:])
        ref = O.sdpa(q, k, v, nh, nkv, d, causal=causal)
        assert max_rel(out[cu[i]:cu[i + 1]], ref) <= TOL, (i, L)


@pytest.mark.parametrize("causal", [False, True])
def test_stella_head_layout_ragged_lengths(causal):  # 12 q heads / 2 kv heads, lengths in [32, 512] + edges
    run_case([32, 512, 1, 63, 64, 65, 200, 0, 129], 12, 2, causal, 1)


@pytest.mark.parametrize("nh,nkv", [(16, 2), (4, 4), (8, 1)])
def test_other_gqa_layouts(nh, nkv):
    run_case([100, 17, 300], nh, nkv, False, nh)
    run_case([70, 260], nh, nkv, True, nh + 1)


@pytest.mark.parametrize("causal", [False, True])
def test_head_dim_256(causal):  # the hybrid decoder's full-attention layers: 16 q / 2 kv heads of 256
    run_case([70, 1, 33, 200, 64], 16, 2, causal, 21, d=256)
    run_case([129], 4, 4, causal, 22, d=256)


def test_rejects_unsupported_head_dim():
    qkv = torch.zeros((4, 3 * 64), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception):
        ops.varlen_attention(qkv, torch.tensor([0, 4], dtype=torch.int32, device=DEV), 1, 1, 64)
