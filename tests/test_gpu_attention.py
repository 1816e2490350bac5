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


# ---- the tcgen05 kernel (head_dim 128): same oracle, same cases ----

def run_case_tc(lens, nh, nkv, causal, seed, d=128):
    rng = np.random.default_rng(seed)
    T = int(sum(lens))
    stride = (nh + 2 * nkv) * d
    qkv_t, qkv = bf16_cuda(rng.standard_normal((T, stride)))
    cu = np.zeros(len(lens) + 1, np.int32); cu[1:] = np.cumsum(lens)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = to_np(ops.varlen_attention_tc(qkv_t, torch.from_numpy(cu).to(DEV), nh, nkv, causal=causal, status=status, head_dim=d))
    assert int(status.item()) == 0
    for i, L in enumerate(lens):
        if L == 0:
            continue
        seg = qkv[cu[i]:cu[i + 1]]
        q = np.ascontiguousarray(seg[:, : nh * d]); k = np.ascontiguousarray(seg[:, nh * d:(nh + nkv) * d])
        v = np.ascontiguousarray(seg[:, (nh + nkv) * d:])
        ref = O.sdpa(q, k, v, nh, nkv, d, causal=causal)
        assert max_rel(out[cu[i]:cu[i + 1]], ref) <= TOL, (i, L)


@pytest.mark.parametrize("causal", [False, True])
def test_tc_stella_head_layout_ragged_lengths(causal):  # lengths around the 128-key block and 8-key padding edges
    run_case_tc([32, 512, 1, 63, 64, 65, 200, 0, 129, 127, 128, 7, 8, 9, 385], 12, 2, causal, 1)


@pytest.mark.parametrize("nh,nkv", [(16, 2), (4, 4), (8, 1)])
def test_tc_other_gqa_layouts(nh, nkv):
    run_case_tc([100, 17, 300], nh, nkv, False, nh)
    run_case_tc([70, 260], nh, nkv, True, nh + 1)


@pytest.mark.parametrize("causal", [False, True])
def test_tc_head_dim_256(causal):  # the hybrid decoder's full-attention layers: 16 q / 2 kv heads of 256
    run_case_tc([70, 1, 33, 200, 64, 0, 385, 128], 16, 2, causal, 21, d=256)
    run_case_tc([129], 4, 4, causal, 22, d=256)
    run_case_tc([900], 2, 1, causal, 23, d=256)


def test_tc_long_sequence_and_large_scores():
    """1100 keys (nine key blocks: both S buffers and both ring stages wrap several times) and inputs
    scaled so that the running maximum moves between blocks (the O rescale path)."""
    run_case_tc([1100, 5], 4, 2, False, 31)
    run_case_tc([700], 2, 1, True, 32)
    rng = np.random.default_rng(33)
    T, nh, nkv, d = 400, 2, 1, 128
    x = rng.standard_normal((T, (nh + 2 * nkv) * d)) * np.linspace(0.2, 3.0, T)[:, None]  # later keys score higher
    qkv_t, qkv = bf16_cuda(x)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    out = to_np(ops.varlen_attention_tc(qkv_t, cu, nh, nkv))
    ref = O.sdpa(np.ascontiguousarray(qkv[:, : nh * d]), np.ascontiguousarray(qkv[:, nh * d:(nh + nkv) * d]),
                 np.ascontiguousarray(qkv[:, (nh + nkv) * d:]), nh, nkv, d, causal=False)
    assert max_rel(out, ref) <= TOL


def test_tc_agrees_with_the_mma_sync_kernel_on_a_full_batch():
    rng = np.random.default_rng(5)
    lens = rng.integers(32, 513, 8)
    T = int(lens.sum())
    qkv_t, _ = bf16_cuda(rng.standard_normal((T, 16 * 128)))
    cu = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).to(DEV)
    a = to_np(ops.varlen_attention_tc(qkv_t, cu, 12, 2)).astype(np.float32)
    b = to_np(ops.varlen_attention(qkv_t, cu, 12, 2, 128)).astype(np.float32)
    assert max_rel(a, b) <= TOL


def test_tc_rejects_bad_arguments():
    qkv = torch.zeros((4, 3 * 128), dtype=torch.bfloat16, device=DEV)
    cu = torch.tensor([0, 4], dtype=torch.int32, device=DEV)
    with pytest.raises(Exception):
        ops.varlen_attention_tc(qkv, cu, 3, 2)  # heads % kv heads


@pytest.mark.parametrize("d,causal", [(128, False), (256, True)])
def test_tc_with_fused_rope_equals_rope_then_attention(d, causal):
    """The entry point that rotates q and k inside the V-transposing launch: bit-identical qkv and output
    to the RoPE launch followed by the plain entry point; a position beyond the table is reported."""
    rng = np.random.default_rng(41)
    lens = [70, 1, 200, 33]
    T, nh, nkv = sum(lens), 4, 2
    qkv_t, _ = bf16_cuda(rng.standard_normal((T, (nh + 2 * nkv) * d)))
    cu = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).to(DEV)
    pos = torch.from_numpy(np.concatenate([np.arange(L) for L in lens]).astype(np.int32)).to(DEV)
    cos, sin = O.build_rope_table_f32(256, d, 1e6)
    cos_t = torch.from_numpy(cos.reshape(256, d // 2)).to(DEV); sin_t = torch.from_numpy(sin.reshape(256, d // 2)).to(DEV)
    a_qkv = ops.rope_halves_(qkv_t.clone(), cos_t, sin_t, pos, nh + nkv, d)
    a_out = ops.varlen_attention_tc(a_qkv, cu, nh, nkv, causal=causal, head_dim=d)
    b_qkv = qkv_t.clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    b_out = ops.rope_varlen_attention_tc_(b_qkv, cos_t, sin_t, pos, cu, nh, nkv, causal=causal, head_dim=d, status=status)
    assert int(status.item()) == 0
    assert torch.equal(a_qkv, b_qkv) and torch.equal(a_out, b_out)
    bad = pos.clone(); bad[5] = 256
    ops.rope_varlen_attention_tc_(qkv_t.clone(), cos_t, sin_t, bad, cu, nh, nkv, causal=causal, head_dim=d, status=status)
    assert int(status.item()) == 1


# ---- prefill chunks that continue a cached sequence: keys and values read through the block tables ----

def run_case_prefix(cached, new, nh, nkv, d, seed, poison=False):
    """Sequence i holds cached[i] + new[i] tokens in a NaN-prefilled paged pool (seeded random block
    tables); the queries are its last new[i] positions. Reference: the oracle's causal attention over
    the whole sequence, rows of the chunk."""
    rng = np.random.default_rng(seed)
    n = len(cached)
    kv = [c + m for c, m in zip(cached, new)]
    nblk = [-(-L // 16) for L in kv]
    n_pool = sum(nblk) + 3
    perm = rng.permutation(n_pool).astype(np.int32)
    tables = np.full((n, max(max(nblk), 1) + 1), -1, np.int32)
    o = 0
    for i in range(n):
        tables[i, :nblk[i]] = perm[o:o + nblk[i]]; o += nblk[i]
    row = nkv * d
    kp = torch.full((n_pool, 16, row), float("nan"), dtype=torch.bfloat16, device=DEV); vp = torch.full_like(kp, float("nan"))
    qs, refs = [], []
    for i in range(n):
        L = kv[i]
        if L == 0:
            continue
        q_t, q = bf16_cuda(rng.standard_normal((L, nh * d)))
        k_t, k = bf16_cuda(rng.standard_normal((L, row))); v_t, v = bf16_cuda(rng.standard_normal((L, row)))
        p = np.arange(L)
        ops.paged_kv_store(k_t, v_t, kp, vp, torch.from_numpy(tables[i, p // 16].astype(np.int64) * 16 + p % 16).to(DEV))
        qs.append(q_t[cached[i]:])
        refs.append(O.sdpa(q, k, v, nh, nkv, d, causal=True)[cached[i]:] if new[i] else np.zeros((0, nh * d), np.float32))
    q_all = torch.cat(qs).contiguous() if qs else torch.zeros((0, nh * d), dtype=torch.bfloat16, device=DEV)
    cu = np.zeros(n + 1, np.int32); cu[1:] = np.cumsum(new)
    if poison:
        tables[0, 0] = n_pool + 5
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = to_np(ops.paged_prefix_attention(q_all, torch.from_numpy(cu).to(DEV), torch.tensor(kv, dtype=torch.int32, device=DEV), kp, vp,
                                           torch.from_numpy(tables).to(DEV), nh, nkv, d, status=status))
    if poison:
        assert int(status.item()) == 1
        return
    assert int(status.item()) == 0
    j = 0
    for i in range(n):
        if kv[i] == 0:
            continue
        if new[i]:
            assert max_rel(out[cu[i]:cu[i + 1]], refs[j]) <= TOL, (i, cached[i], new[i])
        j += 1


@pytest.mark.parametrize("d", [128, 256])
def test_paged_prefix_attention_chunks_against_cached_prefixes(d):
    # prefixes and chunks around the 128-key tile, the 16-token block and the 8-key padding edges; a chunk
    # that starts its sequence (cached 0) and a single-token chunk ride along
    run_case_prefix([100, 0, 128, 17, 500, 3, 255], [60, 70, 1, 129, 200, 8, 130], 16 if d == 256 else 12, 2, d, 51)
    run_case_prefix([1000], [300], 4, 4, d, 52)


def test_paged_prefix_attention_equals_the_unpaged_kernel_for_fresh_sequences():
    run_case_prefix([0, 0, 0], [200, 33, 128], 8, 2, 128, 53)


def test_paged_prefix_attention_reports_a_block_outside_the_pool():
    run_case_prefix([40, 10], [20, 30], 4, 2, 128, 54, poison=True)


@pytest.mark.parametrize("d", [128, 256])
def test_attention_over_a_turbo3_cache_equals_attention_over_the_decoded_rows(d):
    """Keys and values stored as TurboQuant 3-bit rows; prefill chunks and decode tokens (one query) read
    them through the block tables. Reference: the oracle's causal attention over the rows the oracle's
    own codec decodes (the quantisation error is the codec's, not the kernel's)."""
    rng = np.random.default_rng(61)
    nh, nkv = 8, 2
    cached, new = [90, 0, 200, 33], [40, 70, 1, 1]
    n = len(cached)
    kv = [c + m for c, m in zip(cached, new)]
    nblk = [-(-L // 16) for L in kv]
    n_pool = sum(nblk) + 2
    perm = rng.permutation(n_pool).astype(np.int32)
    tables = np.full((n, max(nblk) + 1), -1, np.int32)
    o = 0
    for i in range(n):
        tables[i, :nblk[i]] = perm[o:o + nblk[i]]; o += nblk[i]
    row = nkv * d
    rb = int(ops.lib.logismos_turbo3_row_bytes(row))
    kp = torch.zeros((n_pool, 16, rb), dtype=torch.uint8, device=DEV); vp = torch.zeros_like(kp)
    qs, refs = [], []
    for i in range(n):
        L = kv[i]
        q_t, q = bf16_cuda(rng.standard_normal((L, nh * d)))
        k_t, k = bf16_cuda(rng.standard_normal((L, row))); v_t, v = bf16_cuda(rng.standard_normal((L, row)))
        p = np.arange(L)
        ops.paged_kv_store_turbo3(k_t, v_t, kp, vp, torch.from_numpy(tables[i, p // 16].astype(np.int64) * 16 + p % 16).to(DEV))
        kd = O.bf16_round(O.turbo3_decode(O.turbo3_encode(k.reshape(L, row // 128, 128))).reshape(L, row))
        vd = O.bf16_round(O.turbo3_decode(O.turbo3_encode(v.reshape(L, row // 128, 128))).reshape(L, row))
        qs.append(q_t[cached[i]:])
        refs.append(O.sdpa(q, kd, vd, nh, nkv, d, causal=True)[cached[i]:])
    cu = np.zeros(n + 1, np.int32); cu[1:] = np.cumsum(new)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = to_np(ops.paged_prefix_attention(torch.cat(qs).contiguous(), torch.from_numpy(cu).to(DEV), torch.tensor(kv, dtype=torch.int32, device=DEV),
                                           kp, vp, torch.from_numpy(tables).to(DEV), nh, nkv, d, status=status, turbo3=True))
    assert int(status.item()) == 0
    for i in range(n):
        assert max_rel(out[cu[i]:cu[i + 1]], refs[i]) <= TOL, i
