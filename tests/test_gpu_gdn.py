"""Gated delta rule decode step against gated_delta_rule_recurrent_fwd restated in the oracle."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import DEV, bf16_cuda, max_rel, to_np
from logismos_b200 import ops

pytestmark = pytest.mark.gpu


def test_multi_step_decode_matches_recurrent_reference():
    rng = np.random.default_rng(0)
    n_seqs, heads, steps, D = 3, 4, 5, 128
    state0 = (rng.standard_normal((n_seqs, heads, D, D)) * 0.1).astype(np.float32)
    st = torch.from_numpy(state0.copy()).to(DEV)
    qs, ks, vs, gs, bs, outs = [], [], [], [], [], []
    for _ in range(steps):
        q = rng.standard_normal((n_seqs, heads, D)).astype(np.float32); k = rng.standard_normal((n_seqs, heads, D)).astype(np.float32)
        O.l2_norm_rows(q.reshape(-1), D); O.l2_norm_rows(k.reshape(-1), D)  # q/k L2-normalised per head
        q_t, q = bf16_cuda(q); k_t, k = bf16_cuda(k); v_t, v = bf16_cuda(rng.standard_normal((n_seqs, heads, D)))
        a = rng.standard_normal((n_seqs, heads)).astype(np.float32); b = rng.standard_normal((n_seqs, heads)).astype(np.float32)
        g, beta = O.gdn_gates(a, b, np.zeros(heads, np.float32), np.zeros(heads, np.float32))
        o = ops.gdn_decode_step_(st, q_t, k_t, v_t, torch.from_numpy(g).to(DEV), torch.from_numpy(beta).to(DEV), D ** -0.5)
        qs.append(q); ks.append(k); vs.append(v); gs.append(g); bs.append(beta); outs.append(to_np(o))
    final = to_np(st)
    for s in range(n_seqs):
        for h in range(heads):
            o_ref, s_ref = O.gdn_recurrent_fwd(np.stack([x[s, h] for x in qs]), np.stack([x[s, h] for x in ks]),
                                               np.stack([x[s, h] for x in vs]), np.array([x[s, h] for x in bs]),
                                               np.array([x[s, h] for x in gs]), D ** -0.5, state0[s, h], D, D)
            got = np.stack([x[s, h] for x in outs])
            assert max_rel(got, o_ref.reshape(steps, D)) <= 2e-2
            assert max_rel(final[s, h], s_ref.reshape(D, D)) <= 1e-4  # the state stays fp32


def test_zero_beta_only_decays_the_state():  # cpu.rs:296-313
    st0 = np.full((1, 1, 128, 128), 2.0, np.float32)
    st = torch.from_numpy(st0.copy()).to(DEV)
    one, _ = bf16_cuda(np.ones((1, 1, 128)))
    ops.gdn_decode_step_(st, one, one, one, torch.zeros((1, 1), device=DEV), torch.zeros((1, 1), device=DEV), 1.0)
    assert (to_np(st) == st0).all()


def test_ragged_prefill_matches_chunk_reference_and_continues_into_decode():
    rng = np.random.default_rng(3)
    heads, D = 3, 128
    lens = [37, 1, 130]
    T = sum(lens)
    cu = np.zeros(4, np.int32); cu[1:] = np.cumsum(lens)
    q_t, _ = bf16_cuda(rng.standard_normal((T, heads, D))); k_t, _ = bf16_cuda(rng.standard_normal((T, heads, D)))
    v_t, v = bf16_cuda(rng.standard_normal((T, heads, D)))
    a = rng.standard_normal((T, heads)).astype(np.float32); b = rng.standard_normal((T, heads)).astype(np.float32)
    A_log = rng.uniform(-1, 0.5, heads).astype(np.float32); dt_bias = rng.standard_normal(heads).astype(np.float32)
    # gates and q/k normalisation on the GPU against the oracle
    g_t, beta_t = ops.gdn_prepare_(q_t, k_t, torch.from_numpy(a).to(DEV), torch.from_numpy(b).to(DEV),
                                   torch.from_numpy(A_log).to(DEV), torch.from_numpy(dt_bias).to(DEV))
    g_ref, beta_ref = O.gdn_gates(a, b, A_log, dt_bias)
    assert np.abs(to_np(g_t) - g_ref).max() <= 1e-5 * max(1, np.abs(g_ref).max()) and np.abs(to_np(beta_t) - beta_ref).max() <= 1e-6
    q, k = to_np(q_t), to_np(k_t)
    assert np.abs(np.linalg.norm(q, axis=-1) - 1).max() < 1e-2
    state0 = (rng.standard_normal((3, heads, D, D)) * 0.05).astype(np.float32)
    st = torch.from_numpy(state0.copy()).to(DEV)
    o = to_np(ops.gdn_prefill_(st, q_t, k_t, v_t, g_t, beta_t, torch.from_numpy(cu).to(DEV), D ** -0.5))
    g_np, beta_np = to_np(g_t), to_np(beta_t)
    final = to_np(st)
    for s in range(3):
        sl = slice(cu[s], cu[s + 1])
        for h in range(heads):
            o_ref, states = O.gdn_chunk_fwd(q[sl, h], k[sl, h], v[sl, h], beta_np[sl, h], g_np[sl, h], D ** -0.5, state0[s, h], D, D, 64)
            assert max_rel(o[sl, h], o_ref.reshape(-1, D)) <= 2e-2
            assert max_rel(final[s, h], states[-1].reshape(D, D)) <= 1e-4


def test_output_gate_fused_into_the_recurrence_equals_the_separate_gate():
    rng = np.random.default_rng(8)
    heads, D, lens = 2, 128, [19, 3]
    T = sum(lens)
    cu = torch.tensor([0, 19, 22], dtype=torch.int32, device=DEV)
    mk = lambda: bf16_cuda(rng.standard_normal((T, heads, D)))[0]
    q_t, k_t, v_t, z_t = mk(), mk(), mk(), mk()
    g_t = torch.from_numpy(-np.abs(rng.standard_normal((T, heads))).astype(np.float32)).to(DEV)
    beta_t = torch.from_numpy(rng.uniform(0, 1, (T, heads)).astype(np.float32)).to(DEV)
    st_a = torch.zeros((2, heads, D, D), dtype=torch.float32, device=DEV); st_b = st_a.clone()
    plain = to_np(ops.gdn_prefill_(st_a, q_t, k_t, v_t, g_t, beta_t, cu, D ** -0.5)).astype(np.float64)
    gated = to_np(ops.gdn_prefill_(st_b, q_t, k_t, v_t, g_t, beta_t, cu, D ** -0.5, gate_z=z_t))
    z = to_np(z_t).astype(np.float64)
    want = plain * z / (1 + np.exp(-z))
    assert torch.equal(st_a, st_b)                       # the gate does not touch the state
    assert np.abs(gated - want).max() <= 2 ** -6 * np.abs(want).max()  # two bf16 roundings apart at most


def test_finish_of_the_input_projection_workspace():
    """gdn_finish on an fp32 workspace [T, q|k|v|z|a|b] equals: L2-normalise q, k in fp32, round once to
    bf16, gates from a, b (the oracle's formulas), workspace handed back zeroed."""
    from logismos_b200._lib import check, lib
    rng = np.random.default_rng(12)
    T, heads, D = 21, 8, 128
    W = heads * D
    ld = 4 * W + 2 * heads
    acc_np = rng.standard_normal((T, ld)).astype(np.float32)
    acc = torch.from_numpy(acc_np.copy()).to(DEV)
    A_log = rng.uniform(-1, 0.5, heads).astype(np.float32); dt_bias = rng.standard_normal(heads).astype(np.float32)
    proj = torch.empty((T, 4 * W), dtype=torch.bfloat16, device=DEV)
    g = torch.empty((T, heads), dtype=torch.float32, device=DEV); beta = torch.empty_like(g)
    A_t, dt_t = torch.from_numpy(A_log).to(DEV), torch.from_numpy(dt_bias).to(DEV)
    check(lib.logismos_launch_gdn_finish(acc.data_ptr(), ld, A_t.data_ptr(), dt_t.data_ptr(), proj.data_ptr(), 4 * W, g.data_ptr(),
                                         beta.data_ptr(), T, heads, torch.cuda.current_stream().cuda_stream), "gdn_finish")
    torch.cuda.synchronize()
    assert float(acc.abs().max()) == 0.0
    got = to_np(proj)
    qk = acc_np[:, :2 * W].reshape(T, 2 * heads, D).astype(np.float64)
    qk = qk / np.maximum(np.linalg.norm(qk, axis=-1, keepdims=True), 1e-12)
    want = np.concatenate([qk.reshape(T, 2 * W), acc_np[:, 2 * W:4 * W]], axis=1)
    assert np.abs(got - want).max() <= 2 ** -8 * np.abs(want).max()
    g_ref, beta_ref = O.gdn_gates(np.ascontiguousarray(acc_np[:, 4 * W:4 * W + heads]), np.ascontiguousarray(acc_np[:, 4 * W + heads:]), A_log, dt_bias)
    assert np.abs(to_np(g) - g_ref).max() <= 1e-5 * max(1, np.abs(g_ref).max()) and np.abs(to_np(beta) - beta_ref).max() <= 1e-6


def test_decode_from_the_workspace_equals_finish_then_recurrence():
    """The one-launch decode path (normalisation, gates and the one-token recurrence straight from the fp32
    workspace) against the two-launch route on the same workspace: same outputs and states bit for bit,
    workspace and pair counters handed back zeroed; state slots permuted, one sequence fresh."""
    from logismos_b200._lib import check, lib
    rng = np.random.default_rng(31)
    T, heads, D = 37, 8, 128
    W = heads * D
    ld = 4 * W + 2 * heads
    acc_np = rng.standard_normal((T, ld)).astype(np.float32)
    A_t = torch.from_numpy(rng.uniform(-1, 0.5, heads).astype(np.float32)).to(DEV)
    dt_t = torch.from_numpy(rng.standard_normal(heads).astype(np.float32)).to(DEV)
    state0 = torch.from_numpy((rng.standard_normal((T + 3, heads, D, D)) * 0.05).astype(np.float32)).to(DEV)
    slots = torch.from_numpy(rng.permutation(T + 3)[:T].astype(np.int32)).to(DEV)
    fresh_np = np.zeros(T, np.uint8); fresh_np[5] = 1
    fresh = torch.from_numpy(fresh_np).to(DEV)
    cu = torch.arange(0, T + 1, dtype=torch.int32, device=DEV)
    s = lambda: torch.cuda.current_stream().cuda_stream
    # route A: finish, then the token-serial kernel (throughput shape) with the fused output gate
    acc = torch.from_numpy(acc_np.copy()).to(DEV)
    proj = torch.empty((T, 4 * W), dtype=torch.bfloat16, device=DEV)
    g = torch.empty((T, heads), dtype=torch.float32, device=DEV); beta = torch.empty_like(g)
    st_a = state0.clone(); o_a = torch.empty((T, W), dtype=torch.bfloat16, device=DEV)
    check(lib.logismos_launch_gdn_finish(acc.data_ptr(), ld, A_t.data_ptr(), dt_t.data_ptr(), proj.data_ptr(), 4 * W, g.data_ptr(),
                                         beta.data_ptr(), T, heads, s()), "gdn_finish")
    p = proj.data_ptr()
    check(lib.logismos_launch_gdn_prefill(st_a.data_ptr(), p, p + 2 * W, p + 4 * W, g.data_ptr(), beta.data_ptr(), o_a.data_ptr(), p + 6 * W,
                                          cu.data_ptr(), slots.data_ptr(), fresh.data_ptr(), T, heads, 4 * W, D ** -0.5, 1, s()), "gdn_prefill")
    # route B: one launch
    acc_b = torch.from_numpy(acc_np.copy()).to(DEV)
    pairs = torch.zeros(T * heads, dtype=torch.int32, device=DEV)
    st_b = state0.clone(); o_b = torch.empty((T, W), dtype=torch.bfloat16, device=DEV)
    torch.cuda.synchronize()
    check(lib.logismos_launch_gdn_decode_from_acc(st_b.data_ptr(), acc_b.data_ptr(), ld, A_t.data_ptr(), dt_t.data_ptr(), o_b.data_ptr(),
                                                  slots.data_ptr(), fresh.data_ptr(), pairs.data_ptr(), T, heads, D ** -0.5, s()), "gdn_decode_from_acc")
    torch.cuda.synchronize()
    assert float(acc_b.abs().max()) == 0.0 and int(pairs.abs().max()) == 0
    assert np.array_equal(to_np(o_a), to_np(o_b))
    assert np.array_equal(to_np(st_a), to_np(st_b))
    assert np.isfinite(to_np(o_b)).all()


def test_both_kernel_shapes_agree_with_the_reference():
    """The throughput shape (64 columns per CTA, key rows in quarters) and the latency shape (32 columns, one per thread) against the oracle's recurrence, from a non-zero state, ragged lengths that
    end inside and on the eight-token staging chunks."""
    rng = np.random.default_rng(17)
    heads, D = 2, 128
    lens = [8, 13, 1, 24]
    T = sum(lens)
    cu = np.zeros(len(lens) + 1, np.int32); cu[1:] = np.cumsum(lens)
    nrm = lambda x: x / np.linalg.norm(x, axis=-1, keepdims=True)
    q_t, q = bf16_cuda(nrm(rng.standard_normal((T, heads, D)))); k_t, k = bf16_cuda(nrm(rng.standard_normal((T, heads, D))))
    v_t, v = bf16_cuda(rng.standard_normal((T, heads, D)))
    g = (-np.abs(rng.standard_normal((T, heads))) * 0.3).astype(np.float32); beta = rng.uniform(0, 1, (T, heads)).astype(np.float32)
    state0 = (rng.standard_normal((len(lens), heads, D, D)) * 0.05).astype(np.float32)
    outs = []
    for mode in (1, 2):
        st = torch.from_numpy(state0.copy()).to(DEV)
        o = to_np(ops.gdn_prefill_(st, q_t, k_t, v_t, torch.from_numpy(g).to(DEV), torch.from_numpy(beta).to(DEV),
                                   torch.from_numpy(cu).to(DEV), D ** -0.5, mode=mode))
        outs.append((o, to_np(st)))
        for s in range(len(lens)):
            sl = slice(cu[s], cu[s + 1])
            for h in range(heads):
                o_ref, states = O.gdn_chunk_fwd(q[sl, h], k[sl, h], v[sl, h], beta[sl, h], g[sl, h], D ** -0.5, state0[s, h], D, D, 64)
                assert max_rel(o[sl, h], o_ref.reshape(-1, D)) <= 2e-2, (mode, s, h)
                assert max_rel(outs[-1][1][s, h], states[-1].reshape(D, D)) <= 1e-4, (mode, s, h)
    assert np.abs(outs[0][1] - outs[1][1]).max() <= 1e-5 * np.abs(outs[0][1]).max()


def test_static_state_promise_changes_nothing_but_the_fetch_order():
    """With the static-state flag the recurrence reads its states ahead of the dependency wait. After a
    synchronisation (nothing in flight writes them) and right behind the kernel that prepares q, k and
    the gates, outputs and final states equal those without the flag bit for bit."""
    rng = np.random.default_rng(23)
    heads, D, n = 4, 128, 24
    nrm = lambda x: x / np.linalg.norm(x, axis=-1, keepdims=True)
    q_t, _ = bf16_cuda(rng.standard_normal((n, heads, D))); k_t, _ = bf16_cuda(rng.standard_normal((n, heads, D)))
    v_t, _ = bf16_cuda(rng.standard_normal((n, heads, D)))
    a = torch.from_numpy(rng.standard_normal((n, heads)).astype(np.float32)).to(DEV)
    b = torch.from_numpy(rng.standard_normal((n, heads)).astype(np.float32)).to(DEV)
    A_log = torch.from_numpy(rng.uniform(-1, 1, heads).astype(np.float32)).to(DEV)
    dt_bias = torch.from_numpy(rng.uniform(-1, 1, heads).astype(np.float32)).to(DEV)
    cu = torch.arange(0, n + 1, dtype=torch.int32, device=DEV)
    state0 = torch.from_numpy((rng.standard_normal((n, heads, D, D)) * 0.05).astype(np.float32)).to(DEV)
    outs = []
    for static in (False, True):
        st, qq, kk = state0.clone(), q_t.clone(), k_t.clone()
        torch.cuda.synchronize()
        g, beta = ops.gdn_prepare_(qq, kk, a, b, A_log, dt_bias, sync=False)          # normalises q, k in place; the producer
        o = ops.gdn_prefill_(st, qq, kk, v_t, g, beta, cu, D ** -0.5, mode=1, static_state=static)
        outs.append((to_np(o), to_np(st)))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    assert np.isfinite(outs[0][0]).all()


@pytest.mark.parametrize("split", [True, False])
def test_chunk_parallel_form_matches_the_recurrence(split):
    """The chunk-parallel kernels (triangular solve + tensor-core products per 64 tokens; as two launches
    through a scratch buffer, and as one launch) against the oracle's recurrence: lengths below, at and
    across chunk boundaries, an empty sequence, a non-zero incoming state, strong and weak decays, the
    fused output gate; and against the token-serial kernel."""
    rng = np.random.default_rng(23)
    heads, D = 2, 128
    lens = [64, 5, 150, 0, 1, 200]
    T = sum(lens)
    cu = np.zeros(len(lens) + 1, np.int32); cu[1:] = np.cumsum(lens)
    nrm = lambda x: x / np.linalg.norm(x, axis=-1, keepdims=True)
    q_t, q = bf16_cuda(nrm(rng.standard_normal((T, heads, D)))); k_t, k = bf16_cuda(nrm(rng.standard_normal((T, heads, D))))
    v_t, v = bf16_cuda(rng.standard_normal((T, heads, D)))
    z_t, z = bf16_cuda(rng.standard_normal((T, heads, D)))
    g = (-np.abs(rng.standard_normal((T, heads))) * np.where(rng.uniform(size=(T, heads)) < 0.1, 3.0, 0.05)).astype(np.float32)
    beta = rng.uniform(0, 1, (T, heads)).astype(np.float32)
    state0 = (rng.standard_normal((len(lens), heads, D, D)) * 0.05).astype(np.float32)
    g_t, beta_t, cu_t = torch.from_numpy(g).to(DEV), torch.from_numpy(beta).to(DEV), torch.from_numpy(cu).to(DEV)
    st = torch.from_numpy(state0.copy()).to(DEV)
    o = to_np(ops.gdn_chunked_(st, q_t, k_t, v_t, g_t, beta_t, cu_t, D ** -0.5, split=split))
    final = to_np(st)
    for s in range(len(lens)):
        sl = slice(cu[s], cu[s + 1])
        if lens[s] == 0:
            assert np.array_equal(final[s], state0[s])   # an empty sequence leaves its state alone
            continue
        for h in range(heads):
            o_ref, states = O.gdn_chunk_fwd(q[sl, h], k[sl, h], v[sl, h], beta[sl, h], g[sl, h], D ** -0.5, state0[s, h], D, D, 64)
            assert max_rel(o[sl, h], o_ref.reshape(-1, D)) <= 2e-2, (s, h)
            assert max_rel(final[s, h], states[-1].reshape(D, D)) <= 1e-2, (s, h)
    # the gate, and agreement with the token-serial kernel on the same inputs
    st_a = torch.from_numpy(state0.copy()).to(DEV); st_b = st_a.clone()
    o_chunk = to_np(ops.gdn_chunked_(st_a, q_t, k_t, v_t, g_t, beta_t, cu_t, D ** -0.5, gate_z=z_t, split=split))
    o_serial = to_np(ops.gdn_prefill_(st_b, q_t, k_t, v_t, g_t, beta_t, cu_t, D ** -0.5, gate_z=z_t))
    assert max_rel(o_chunk, o_serial) <= 2e-2
    assert max_rel(to_np(st_a), to_np(st_b)) <= 1e-2


def test_two_launch_chunk_form_equals_the_one_launch_form_on_many_chunks():
    """Both forms do the same arithmetic in the same order per chunk, so on a batch with many chunks per
    sequence (the scratch slots of several sequences interleaved in batch order) outputs and final states
    agree to rounding of the intermediates they both round (bf16 W, P; fp32 U)."""
    rng = np.random.default_rng(29)
    heads, D = 4, 128
    lens = [700, 64, 129, 1000, 63]
    T = sum(lens)
    cu = np.zeros(len(lens) + 1, np.int32); cu[1:] = np.cumsum(lens)
    nrm = lambda x: x / np.linalg.norm(x, axis=-1, keepdims=True)
    q_t, _ = bf16_cuda(nrm(rng.standard_normal((T, heads, D)))); k_t, _ = bf16_cuda(nrm(rng.standard_normal((T, heads, D))))
    v_t, _ = bf16_cuda(rng.standard_normal((T, heads, D))); z_t, _ = bf16_cuda(rng.standard_normal((T, heads, D)))
    g_t = torch.from_numpy((-np.abs(rng.standard_normal((T, heads))) * 0.1).astype(np.float32)).to(DEV)
    beta_t = torch.from_numpy(rng.uniform(0, 1, (T, heads)).astype(np.float32)).to(DEV)
    cu_t = torch.from_numpy(cu).to(DEV)
    state0 = torch.from_numpy((rng.standard_normal((len(lens), heads, D, D)) * 0.05).astype(np.float32)).to(DEV)
    res = []
    for split in (True, False):
        st = state0.clone()
        o = ops.gdn_chunked_(st, q_t, k_t, v_t, g_t, beta_t, cu_t, D ** -0.5, gate_z=z_t, split=split)
        res.append((to_np(o), to_np(st)))
    assert np.array_equal(res[0][0], res[1][0]) and np.array_equal(res[0][1], res[1][1])
