"""int4 group-32 dequant GEMV / skinny GEMM against the oracle (the benchmark shapes and batch
sizes; value distributions of the benchmark configuration)."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import DEV, TOL, bf16_cuda, max_rel, to_np
from logismos_b200 import ops

pytestmark = pytest.mark.gpu


def make_case(n, k, b, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(-8, 8, (n, k), dtype=np.int8)
    scales = np.abs(rng.standard_normal((n, k // 32)) * 0.02).astype(np.float16)
    x_t, x = bf16_cuda(rng.standard_normal((b, k)))
    packed = O.int4_pack(codes)
    return codes, packed, scales, x_t, x


def run(packed, scales, x_t):
    return to_np(ops.gemv_int4(torch.from_numpy(packed).to(DEV), torch.from_numpy(scales).to(DEV), x_t))


@pytest.mark.parametrize("n,k", [(1536, 1536), (8960, 1536), (1536, 8960)])
@pytest.mark.parametrize("b", [1, 4, 16, 64])
def test_benchmark_shapes(n, k, b):
    codes, packed, scales, x_t, x = make_case(n, k, b, n + k + b)
    y = run(packed, scales, x_t)
    ref = O.int4_gemv(packed, scales.view(np.uint16), x)
    assert max_rel(y, ref) <= TOL
    # tighter: the only rounding left is the bf16 store of y
    assert np.abs(y - ref).max() <= 2 ** -8 * np.abs(ref).max() + 1e-6


@pytest.mark.parametrize("n,k", [(1536, 1536), (151936, 1536), (96, 8960)])
def test_activations_of_any_magnitude_keep_full_precision(n, k):
    """Rows of tiny and of huge activations in one batch (1e-6 ... 1e5, and one all-zero row): every
    row is checked against the oracle relative to ITS OWN magnitude (the staged operands are scaled per
    row by a power of two, so no row falls into the subnormals of fp16)."""
    rng = np.random.default_rng(n + k)
    codes = rng.integers(-8, 8, (n, k), dtype=np.int8)
    scales = np.abs(rng.standard_normal((n, k // 32)) * 0.02).astype(np.float16)
    mags = np.array([1e-6, 1e-4, 3e-3, 1.0, 50.0, 1e5, 0.0, 2e-5], np.float64)
    x_t, x = bf16_cuda(rng.standard_normal((8, k)) * mags[:, None])
    packed = O.int4_pack(codes)
    y = to_np(ops.gemv_int4(torch.from_numpy(packed).to(DEV), torch.from_numpy(scales).to(DEV), x_t, out_f32=True))
    rows = np.arange(n) if n <= 2048 else rng.choice(n, 2048, replace=False)
    ref = O.int4_gemv(np.ascontiguousarray(packed[rows]), np.ascontiguousarray(scales[rows]).view(np.uint16), x)
    for b in range(8):
        den = np.abs(ref[b]).max()
        if den == 0:
            assert (y[b, rows] == 0).all()
        else:
            assert np.abs(y[b, rows] - ref[b]).max() / den <= 1e-4, (b, mags[b])


@pytest.mark.parametrize("n,k,b", [(16, 128, 1), (17, 256, 3), (40, 384, 9), (100, 4224, 33), (31, 640, 64)])
def test_ragged_shapes(n, k, b):
    codes, packed, scales, x_t, x = make_case(n, k, b, 11 * n + b)
    assert max_rel(run(packed, scales, x_t), O.int4_gemv(packed, scales.view(np.uint16), x)) <= TOL


def test_unpacking_is_bit_exact():
    """With unit scales and a one-hot activation the output IS the signed code: every nibble
    position of every row must come back exactly."""
    n, k = 64, 256
    rng = np.random.default_rng(7)
    codes = rng.integers(-8, 8, (n, k), dtype=np.int8)
    packed = O.int4_pack(codes)
    scales = np.ones((n, k // 32), np.float16)
    got = np.empty((n, k), np.float32)
    for k0 in range(0, k, 64):
        x = np.zeros((64, k), np.float32); x[np.arange(64), k0 + np.arange(64)] = 1.0
        x_t, _ = bf16_cuda(x)
        got[:, k0:k0 + 64] = run(packed, scales, x_t).T
    assert (got == codes.astype(np.float32)).all()
    assert (O.int4_unpack(packed) == codes).all()


def test_extreme_codes_and_zero_scales():
    n, k = 32, 256
    codes = np.full((n, k), -8, np.int8); codes[::2] = 7
    packed = O.int4_pack(codes)
    scales = np.full((n, k // 32), 0.5, np.float16); scales[5] = 0
    x_t, x = bf16_cuda(np.ones((2, k)))
    y = run(packed, scales, x_t)
    ref = O.int4_gemv(packed, scales.view(np.uint16), x)
    assert (y == O.bf16_round(ref)).all() and (y[:, 5] == 0).all()


def test_shape_guards():
    c = torch.zeros((16, 50), dtype=torch.uint8, device=DEV)  # k = 100, not a multiple of 128
    with pytest.raises(Exception):
        ops.gemv_int4(c, torch.zeros((16, 3), dtype=torch.float16, device=DEV), torch.zeros((1, 100), dtype=torch.bfloat16, device=DEV))


def test_lm_head_shape_linearity_and_sampled_rows():
    """(151936, 1536), the HBM-bound benchmark shape: sampled rows against the oracle, and the
    size-independent property y(x1 + x2) = y(x1) + y(x2) over all rows."""
    n, k = 151936, 1536
    rng = np.random.default_rng(9)
    packed = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    scales = np.abs(rng.standard_normal((n, k // 32)) * 0.02).astype(np.float16)
    p_t = torch.from_numpy(packed).to(DEV); s_t = torch.from_numpy(scales).to(DEV)
    x1 = np.zeros((1, k), np.float32); x2 = np.zeros((1, k), np.float32)
    x1[0, ::2] = rng.integers(-4, 5, k // 2); x2[0, 1::2] = rng.integers(-4, 5, k // 2)  # exact in bf16
    y1 = to_np(ops.gemv_int4(p_t, s_t, bf16_cuda(x1)[0])).astype(np.float64)
    y2 = to_np(ops.gemv_int4(p_t, s_t, bf16_cuda(x2)[0])).astype(np.float64)
    y12 = to_np(ops.gemv_int4(p_t, s_t, bf16_cuda(x1 + x2)[0])).astype(np.float64)
    assert np.abs(y12 - (y1 + y2)).max() <= 3 * 2 ** -8 * np.abs(y12).max()
    rows = np.concatenate([[0, 1, 15, 16, n - 17, n - 1], rng.integers(0, n, 250)])
    ref = O.int4_gemv(np.ascontiguousarray(packed[rows]), np.ascontiguousarray(scales[rows]).view(np.uint16), x1 + x2)
    assert max_rel(y12[:, rows], ref) <= TOL


@pytest.mark.parametrize("n,k,b", [(75795, 256, 3), (75795, 384, 16), (75776, 128, 9), (80001, 256, 24), (75795, 512, 16), (75809, 768, 1),
                                   (75795, 2048, 2), (75809, 2048, 16)])  # rows 1 KB apart: the wide-slot kernel
def test_tall_ragged_matrix_every_row(n, k, b):
    """Matrices tall enough for the routes where a warp carries two 16-row tiles side by side (at
    least 32 row tiles per SM; one or two k steps per ring slot), with a row count that is not a
    multiple of 32 or 16, at batch sizes on both sides of the 16-row limit of those routes: every row
    against the oracle."""
    _, packed, scales, x_t, x = make_case(n, k, b, seed=n + b)
    y = run(packed, scales, x_t)
    ref = O.int4_gemv(packed, scales.view(np.uint16), x)
    assert max_rel(y, ref) <= TOL


@pytest.mark.parametrize("n,k,b", [(1536, 1536, 64), (8960, 1536, 17), (1536, 8960, 33), (151936, 1536, 64), (1000, 1536, 40), (256, 640, 64),
                                   (1536, 8960, 1), (1536, 8960, 4), (2048, 6144, 16), (1536, 1536, 8), (8960, 1536, 12), (17920, 1536, 16)])
def test_skinny_route_by_shape_and_rows(n, k, b):
    """The entry point that picks the kernel by shape and row count (k a multiple of 256): above 16 rows,
    for k >= 3 n at any batch and from 8 rows up to n = 16384 the fused-dequant tensor-core linear through
    a zeroed fp32 workspace, which it must leave zeroed; other shapes stay on the GEMV. Same oracle,
    same bar."""
    expect = int(k % 256 == 0 and n % 4 == 0 and (b > 16 or k >= 3 * n or (b >= 8 and n <= 16384)))
    assert ops.lib.logismos_skinny_int4_route(b, n, k) == expect
    codes, packed, scales, x_t, x = make_case(n, k, b, n + 3 * b)
    ws = torch.zeros(b * n, dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pk, sc = torch.from_numpy(packed).to(DEV), torch.from_numpy(scales).to(DEV)
    y = to_np(ops.skinny_int4(pk, sc, x_t, ws, status=status))
    assert int(status.item()) == 0 and float(ws.abs().max()) == 0.0
    rows = np.arange(n) if n <= 4096 else np.random.default_rng(0).choice(n, 4096, replace=False)
    ref = O.int4_gemv(np.ascontiguousarray(packed[rows]), np.ascontiguousarray(scales[rows]).view(np.uint16), x)
    assert max_rel(y[:, rows], ref) <= TOL
    y2 = to_np(ops.skinny_int4(pk, sc, x_t, ws, status=status))   # the workspace is reusable as left
    assert max_rel(y2[:, rows], ref) <= TOL
