"""The tcgen05 GEMM (C = A W^T + b) against the oracle's linear_t and the on-device naive anchor."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import DEV, TOL, bf16_cuda, max_rel, to_np
from logismos_b200 import ops

pytestmark = pytest.mark.gpu


def case(m, n, k, seed, bias=True):
    rng = np.random.default_rng(seed)
    a_t, a = bf16_cuda(rng.standard_normal((m, k)))
    w_t, w = bf16_cuda(rng.standard_normal((n, k)) * 0.05)
    b = (rng.standard_normal(n) * 0.5).astype(np.float32) if bias else None
    return a_t, a, w_t, w, b


# M ragged against the 128-row tile, N exercising every tile width (128 / 192 / 256) and a ragged last
# tile, K from one stage to the longest reduction of the model
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (1, 16, 64), (100, 1536, 1536), (333, 2048, 1536), (129, 192, 128),
                                   (2176, 1536, 1536), (257, 1536, 8960), (64, 400, 256), (700, 17920, 512)])
def test_bf16_epilogue_matches_oracle_linear_t(m, n, k):
    a_t, a, w_t, w, b = case(m, n, k, m + n + k)
    got = to_np(ops.linear_t(a_t, w_t, torch.from_numpy(b).to(DEV)))
    ref = O.linear_t(a, w, b, m, n, k).reshape(m, n)
    assert max_rel(got, ref) <= TOL
    assert np.abs(got - ref).max() <= 2 ** -8 * np.abs(ref).max() + 1e-5  # only the bf16 store rounds


@pytest.mark.parametrize("m,n,k,kind", [(64, 2048, 2048, "bf16"), (300, 1536, 1536, "resid"), (64, 12288, 2048, "swiglu"), (2, 256, 64, "bf16")])
def test_static_weight_promise_changes_nothing_but_the_fetch_order(m, n, k, kind):
    """With the static-weights flag the kernel requests its first weight stages ahead of the dependency
    wait; launched behind a kernel of this library that rewrites the ACTIVATIONS (so the early start
    really overlaps a producer), the result equals the one without the flag bit for bit."""
    from logismos_b200._lib import lib
    a_t, a, w_t, w, b = case(m, n, k, 5 * m + n + k, bias=False)
    lib.logismos_set_deterministic(1)   # no split over k: a fixed summation order
    try:
        outs = []
        for static in (False, True):
            res = torch.zeros((m, n), dtype=torch.float32, device=DEV) if kind == "resid" else None
            x = torch.zeros((m, k), dtype=torch.float32, device=DEV)
            src = a_t.float().contiguous()
            # the producer ahead of the GEMM: this library's rms_norm (unit gains) of rows pre-scaled to unit RMS
            rms = src.pow(2).mean(dim=1, keepdim=True).sqrt()
            x.copy_(src / rms)
            ones = torch.ones(k, dtype=torch.float32, device=DEV)
            torch.cuda.synchronize()
            h = ops.rms_norm_f32(x, ones, 0.0, sync=False)
            outs.append(to_np(ops.linear_t(h, w_t, residual=res, swiglu=(kind == "swiglu"), static_w=static)))
        assert np.array_equal(outs[0], outs[1])
    finally:
        lib.logismos_set_deterministic(0)


def test_matches_the_naive_anchor_on_device():
    a_t, a, w_t, w, b = case(300, 768, 1024, 5)
    bt = torch.from_numpy(b).to(DEV)
    fast = to_np(ops.linear_t(a_t, w_t, bt)); slow = to_np(ops.linear_t(a_t, w_t, bt, naive=True))
    assert np.abs(fast - slow).max() <= 2 ** -7 * np.abs(slow).max()


@pytest.mark.parametrize("m,n,k", [(200, 1536, 1536), (77, 1536, 8960), (130, 512, 64)])
def test_residual_epilogue_accumulates_into_fp32(m, n, k):
    a_t, a, w_t, w, _ = case(m, n, k, 3 * m + n, bias=False)
    rng = np.random.default_rng(1)
    x0 = rng.standard_normal((m, n)).astype(np.float32)
    x_t = torch.from_numpy(x0.copy()).to(DEV)
    ops.linear_t(a_t, w_t, residual=x_t)
    ref = x0 + O.linear_t(a, w, None, m, n, k).reshape(m, n)
    assert np.abs(to_np(x_t) - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max())
    ops.linear_t(a_t, w_t, residual=x_t)  # twice: the accumulator buffers and barriers recycle cleanly
    assert np.abs(to_np(x_t) - (ref + ref - x0)).max() <= 2e-4 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("m,inter,k", [(150, 1024, 512), (2176, 8960, 1536), (33, 96, 64)])
def test_swiglu_epilogue(m, inter, k):
    rng = np.random.default_rng(m + inter)
    a_t, a = bf16_cuda(rng.standard_normal((m, k)))
    wg_t, wg = bf16_cuda(rng.standard_normal((inter, k)) * 0.05)
    wu_t, wu = bf16_cuda(rng.standard_normal((inter, k)) * 0.05)
    # gate/up rows interleaved in blocks of 32
    inter_w = torch.stack([wg_t.view(inter // 32, 32, k), wu_t.view(inter // 32, 32, k)], dim=1).reshape(2 * inter, k).contiguous()
    got = to_np(ops.linear_t(a_t, inter_w, swiglu=True))
    g = O.linear_t(a, wg, None, m, inter, k); u = O.linear_t(a, wu, None, m, inter, k)
    ref = O.hadamard(O.silu(g), u).reshape(m, inter)
    assert max_rel(got, ref) <= TOL


def test_shape_guards_reject_before_launch():
    a = torch.zeros((8, 100), dtype=torch.bfloat16, device=DEV)  # k not a multiple of 64
    w = torch.zeros((16, 100), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception):
        ops.linear_t(a, w)
    with pytest.raises(ops.InvalidOp):
        ops.linear_t(a.cpu(), w)
