"""GPU-vs-CPU parity of the four fp16 ops, with the reference's shapes, input distribution and
metric (crates/kernels/tests/matmul_parity.rs:83-136, op_parity.rs:80-160):
max |g - c| / max(|c|, 1e-3) <= 5e-3, inputs uniform(-1, 1) in fp16."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from logismos_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel_err(g, c):
    g = g.astype(np.float32); c = c.astype(np.float32)
    return float((np.abs(g - c) / np.maximum(np.abs(c), 1e-3)).max())


@pytest.mark.parametrize("m,n,k", [(32, 48, 64), (64, 64, 64), (256, 256, 256), (17, 23, 31), (128, 16, 512)])
def test_matmul_parity(m, n, k):  # matmul_parity.rs:103-150; (17,23,31) takes the naive kernel
    rng = np.random.default_rng(m * 7 + n)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16); b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    d = ops.matmul(torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)).cpu().numpy()
    assert rel_err(d, O.matmul_fp16_ref(a, b, m, n, k)) <= 5e-3


def test_matmul_long_reduction_per_tensor_metric():
    """K = 4096, beyond the reference's test sizes: near-zero outputs make the per-element metric
    meaningless there, so the bar is max |g - c| over max |c|."""
    rng = np.random.default_rng(9)
    m, n, k = 128, 16, 4096
    a = rng.uniform(-1, 1, (m, k)).astype(np.float16); b = rng.uniform(-1, 1, (k, n)).astype(np.float16)
    d = ops.matmul(torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV)).cpu().numpy().astype(np.float32)
    c = O.matmul_fp16_ref(a, b, m, n, k).astype(np.float32)
    assert np.abs(d - c).max() / np.abs(c).max() <= 5e-3


def test_matmul_rejects_bad_operands():  # praxis/src/matmul.rs:31-82, :154-166
    a = torch.zeros((16, 16), dtype=torch.float16, device=DEV)
    with pytest.raises(ops.InvalidOp):
        ops.matmul(a, torch.zeros((16, 16), dtype=torch.float16))  # mixed placement
    with pytest.raises(ops.InvalidOp):
        ops.matmul(a, torch.zeros((8, 16), dtype=torch.float16, device=DEV))  # inner dims
    with pytest.raises(ops.InvalidOp):
        ops.matmul(a.float(), a.float())  # dtype
    with pytest.raises(ops.InvalidOp):
        ops.matmul(a[:, ::2], a)  # non-contiguous


def test_rms_norm_parity():  # op_parity.rs:80-110 (8 x 1024)
    rng = np.random.default_rng(1)
    x = rng.uniform(-1, 1, (8, 1024)).astype(np.float16); w = rng.uniform(-1, 1, 1024).astype(np.float16)
    y = ops.rms_norm(torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV), 1e-5).cpu().numpy()
    assert rel_err(y, O.rms_norm_fp16_ref(x, w, 8, 1024, 1e-5)) <= 5e-3


def test_softmax_parity_and_fully_masked_row():  # op_parity.rs:121-150 (4 x 512) + the uniform-row contract
    rng = np.random.default_rng(2)
    x = rng.uniform(-1, 1, (4, 512)).astype(np.float16)
    x[2, :] = -np.inf
    y = ops.softmax(torch.from_numpy(x).to(DEV)).cpu().numpy()
    assert rel_err(y, O.softmax_fp16_ref(x, 4, 512)) <= 5e-3
    assert np.isfinite(y).all() and abs(float(y[2].astype(np.float32).sum()) - 1) < 2e-2


def test_rope_parity():  # op_parity.rs:156-190: (2, 64, 8, 128), theta 1e4, interleaved pairs
    rng = np.random.default_rng(3)
    b, s, h, d = 2, 64, 8, 128
    x = rng.uniform(-1, 1, (b, s, h, d)).astype(np.float16)
    table = O.build_cos_sin_table(s, d, 10000.0)
    y = ops.rope_apply(torch.from_numpy(x).to(DEV), torch.from_numpy(table.reshape(s, d)).to(DEV)).cpu().numpy()
    ref = x.copy(); O.rope_apply_fp16_ref(ref.reshape(-1), table, b, s, h, d)
    assert rel_err(y, ref) <= 5e-3
