"""The fused-dequant tensor-core linear for small token counts (acc += A dequant(W)^T, int4 group-32
weights) against the oracle: linear_t on the dequantised matrix."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import DEV, TOL, bf16_cuda, max_rel, to_np
from logismos_b200 import ops

pytestmark = pytest.mark.gpu


def make_case(m, n, k, seed, scale=0.02):
    rng = np.random.default_rng(seed)
    codes = rng.integers(-8, 8, (n, k), dtype=np.int8)
    scales = np.abs(rng.standard_normal((n, k // 32)) * scale).astype(np.float16)
    a_t, a = bf16_cuda(rng.standard_normal((m, k)))
    packed = O.int4_pack(codes)
    ref = O.linear_t(a, O.int4_dequant(packed, scales), None, m, n, k).reshape(m, n)
    return torch.from_numpy(packed).to(DEV), torch.from_numpy(scales).to(DEV), a_t, ref


# every token tile (64 / 128 / 256), ragged token counts and weight-row counts, one to many slices of k
@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (7, 2048, 2048), (32, 9216, 2048), (64, 32, 2048), (65, 2048, 6144), (100, 200, 512),
                                   (128, 12288, 2048), (200, 1536, 8960), (256, 2048, 2048), (16, 151936, 1536)])
def test_accumulates_linear_on_dequantised_weights(m, n, k):
    codes, scales, a_t, ref = make_case(m, n, k, m + n + k)
    acc = torch.zeros((m, n), dtype=torch.float32, device=DEV)
    status = ops.qlinear_int4_acc_(acc, a_t, codes, scales)
    assert int(status.item()) == 0
    got = to_np(acc)
    assert max_rel(got, ref) <= TOL
    # weights enter the MMA as bf16(code) * bf16(scale): two roundings of 2^-9 per product, random in sign
    assert np.abs(got - ref).max() <= 2 ** -7 * np.abs(ref).max()
    # a second call accumulates on top (the residual-stream use) and recycles barriers and TMEM cleanly
    ops.qlinear_int4_acc_(acc, a_t, codes, scales)
    assert np.abs(to_np(acc) - 2 * ref).max() <= 2 ** -6 * np.abs(ref).max()


@pytest.mark.parametrize("m,n,k", [(16, 8224, 2048), (64, 8224, 2048), (3, 256, 256)])
def test_static_weight_promise_changes_nothing_but_the_fetch_order(m, n, k):
    """The entry point that fills its weight ring ahead of the dependency wait, launched right behind
    another kernel of this library, gives the same sums as the plain entry point (whole-tile spans, so
    the summation order is fixed)."""
    from logismos_b200._lib import lib
    codes, scales, a_t, ref = make_case(m, n, k, 3 * m + n + k)
    lib.logismos_set_deterministic(1)
    try:
        outs = []
        for static in (False, True):
            acc = torch.zeros((m, n), dtype=torch.float32, device=DEV)
            warm = torch.zeros((m, n), dtype=torch.float32, device=DEV)
            ops.qlinear_int4_acc_(warm, a_t, codes, scales, sync=False)            # the kernel ahead of it
            status = ops.qlinear_int4_acc_(acc, a_t, codes, scales, static_w=static)
            assert int(status.item()) == 0
            outs.append(to_np(acc))
        assert np.array_equal(outs[0], outs[1]) and max_rel(outs[0], ref) <= TOL
    finally:
        lib.logismos_set_deterministic(0)


@pytest.mark.parametrize("m", [16, 64, 91, 128])
def test_back_to_back_launches_on_a_vocabulary_sized_matrix_never_expire_a_wait(m):
    """A thousand back-to-back launches of the static-weights entry point per tile configuration (32-, 64-
    and 128-token tiles) on a 151936 x 2048 matrix, the accumulator cleared between them as the lm_head of a
    decode step does: the status word stays 0 and the last accumulation is right. (Rare expired waits in
    the 128-token configuration were once the symptom of lanes leaving a polling loop in different
    iterations ahead of a warp-wide tensor-memory instruction, and of the weight ring filled early.)"""
    from logismos_b200._lib import lib
    n, k = 151936, 2048
    g = torch.Generator(device="cpu").manual_seed(m)
    codes = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, generator=g).to(DEV)
    scales = (torch.rand((n, k // 32), generator=g) * 0.02).to(torch.float16).to(DEV)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16).to(DEV)
    acc = torch.zeros((m, n), dtype=torch.float32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    s = torch.cuda.current_stream().cuda_stream
    for it in range(250):
        for _ in range(4):
            acc.zero_()
            assert lib.logismos_launch_qlinear_int4_g32_acc_f32_static(x.data_ptr(), codes.data_ptr(), scales.data_ptr(), acc.data_ptr(), m, n, k, k, n,
                                                                       status.data_ptr(), s) == 0
        assert int(status.item()) == 0, (it, hex(int(status.item())))
    rows = torch.arange(0, n, 997, device=DEV)
    w = (ops.dequant_int4(codes[rows].contiguous(), scales[rows].contiguous())).float()
    ref = x.float() @ w.t()
    assert float((acc[:, rows] - ref).abs().max()) <= 2e-2 * float(ref.abs().max())


def test_exact_for_exactly_representable_inputs():
    """Power-of-two scales and small integer activations: every product and partial sum is exact in
    bf16 / fp32, so the result must equal the integer dot product bit for bit (nibble order, sign
    handling, swizzled tile layout, slices of k)."""
    rng = np.random.default_rng(3)
    m, n, k = 33, 384, 1024
    codes = rng.integers(-8, 8, (n, k), dtype=np.int8)
    scales = (2.0 ** rng.integers(-3, 2, (n, k // 32))).astype(np.float16)
    a = rng.integers(-4, 5, (m, k)).astype(np.float32)
    a_t, a_r = bf16_cuda(a)
    assert np.array_equal(a, a_r)
    acc = torch.zeros((m, n), dtype=torch.float32, device=DEV)
    ops.qlinear_int4_acc_(acc, a_t, torch.from_numpy(O.int4_pack(codes)).to(DEV), torch.from_numpy(scales).to(DEV))
    w = codes.astype(np.float64) * np.repeat(scales.astype(np.float64), 32, axis=1)
    assert np.array_equal(to_np(acc).astype(np.float64), a.astype(np.float64) @ w.T)


def test_strided_rows_and_finish_kernels():
    m, n, k = 40, 256, 512
    codes, scales, a_t, ref = make_case(m, n, k, 9)
    wide = torch.zeros((m, k + 64), dtype=torch.bfloat16, device=DEV)
    wide[:, :k] = a_t
    acc_wide = torch.zeros((m, n + 32), dtype=torch.float32, device=DEV)
    ops.qlinear_int4_acc_(acc_wide[:, :n], wide[:, :k], codes, scales)
    assert max_rel(to_np(acc_wide[:, :n]), ref) <= TOL and float(acc_wide[:, n:].abs().max()) == 0.0
    acc = acc_wide[:, :n].contiguous()
    bias = torch.from_numpy(np.random.default_rng(1).standard_normal(n).astype(np.float32)).to(DEV)
    out = to_np(ops.qlinear_finish(acc.clone(), bias))
    assert np.abs(out - (to_np(acc) + to_np(bias))).max() <= 2 ** -8 * np.abs(out).max()
    work = acc.clone()
    sw = to_np(ops.qlinear_finish(work, None, swiglu=True))
    assert float(work.abs().max()) == 0.0           # the workspace is handed back zeroed
    v = to_np(acc).reshape(m, n // 64, 2, 32)
    want = (v[:, :, 0] / (1 + np.exp(-v[:, :, 0])) * v[:, :, 1]).reshape(m, n // 2)
    assert np.abs(sw - want).max() <= 2 ** -7 * np.abs(want).max() + 1e-6


def test_shape_guards():
    codes, scales, a_t, _ = make_case(4, 128, 256, 1)
    acc = torch.zeros((4, 128), dtype=torch.float32, device=DEV)
    with pytest.raises(ops.InvalidOp):
        ops.qlinear_int4_acc_(acc[:, :64], a_t, codes, scales)
    big = torch.zeros((257, 256), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ops.InvalidOp):
        ops.qlinear_int4_acc_(torch.zeros((257, 128), dtype=torch.float32, device=DEV), big, codes, scales)
