"""Paged KV cache and paged-attention decode.

Bit-exact rows: store/gather/append against the oracle's paged cache, which is itself pinned to
the reference's FlatKvCache semantics. Decode output: against the oracle's single-query attention
on the gathered prefix, within the floating-point bar."""
import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import DEV, TOL, bf16_cuda, max_rel, to_np
from logismos_b200 import ops

pytestmark = pytest.mark.gpu
BS = 16


def bits(t):
    return t.detach().cpu().view(torch.int16).numpy().view(np.uint16)


def test_store_and_gather_equal_the_flat_cache_bit_for_bit():
    rng = np.random.default_rng(0)
    row, n_blocks = 256, 40
    kp = torch.zeros((n_blocks, BS, row), dtype=torch.bfloat16, device=DEV); vp = torch.zeros_like(kp)
    lens = [70, 1, 33]
    perm = rng.permutation(n_blocks).astype(np.int32)
    tables = -np.ones((3, 8), np.int32); o = 0
    for i, L in enumerate(lens):
        nb = -(-L // BS); tables[i, :nb] = perm[o:o + nb]; o += nb
    cu, pos, slots, sid = O.build_packing(np.zeros(3, np.int32), np.array(lens, np.int32), tables, BS, n_blocks)
    k_t, _ = bf16_cuda(rng.standard_normal((cu[-1], row))); v_t, _ = bf16_cuda(rng.standard_normal((cu[-1], row)))
    ops.paged_kv_store(k_t, v_t, kp, vp, torch.from_numpy(slots).to(DEV))
    kp_np = bits(kp).reshape(n_blocks, BS, row); vp_np = bits(vp).reshape(n_blocks, BS, row)
    for i, L in enumerate(lens):
        flat = O.FlatKvCache(1, row * 2, 128)
        flat.put(0, bits(k_t[cu[i]:cu[i + 1]]), bits(v_t[cu[i]:cu[i + 1]]))
        for n in sorted({0, 1, L // 2, L}):
            fk, fv = flat.get(0, n)
            gk, gv = ops.paged_kv_gather(kp, vp, torch.from_numpy(tables[i]).to(DEV), n)
            assert (bits(gk).view(np.uint8).reshape(n, row * 2) == fk).all() and (bits(gv).view(np.uint8).reshape(n, row * 2) == fv).all()
            ok, ov = O.paged_gather(kp_np.view(np.uint8).reshape(n_blocks, BS, row * 2), vp_np.view(np.uint8).reshape(n_blocks, BS, row * 2), BS, tables[i], n)
            assert (ok == fk).all() and (ov == fv).all()
    with pytest.raises(ops.InvalidOp):  # a slot outside the pool is reported, not written
        ops.paged_kv_store(k_t[:1], v_t[:1], kp, vp, torch.tensor([n_blocks * BS], dtype=torch.int64, device=DEV))
    with pytest.raises(ops.InvalidOp):
        ops.paged_kv_gather(kp, vp, torch.tensor([-1], dtype=torch.int32, device=DEV), 3)


def decode_case(ctx_lens, nh, nkv, chunk, seed, append=True, d=128):
    rng = np.random.default_rng(seed)
    n = len(ctx_lens)
    row = nkv * d
    blocks = [-(-L // BS) for L in ctx_lens]
    n_pool = sum(blocks) + 3
    perm = rng.permutation(n_pool).astype(np.int32)
    maxb = max(blocks) + 1
    tables = -np.ones((n, maxb), np.int32); o = 0
    for i, nb in enumerate(blocks):
        tables[i, :nb] = perm[o:o + nb]; o += nb
    # pool pre-filled with NaN: rows never written must not leak into any result
    kp = torch.full((n_pool, BS, row), float("nan"), dtype=torch.bfloat16, device=DEV); vp = torch.full_like(kp, float("nan"))
    hist_k, hist_v = [], []
    for i, L in enumerate(ctx_lens):
        kk_t, kk = bf16_cuda(rng.standard_normal((L, row))); vv_t, vv = bf16_cuda(rng.standard_normal((L, row)))
        hist_k.append(kk); hist_v.append(vv)
        n_old = L - 1 if append else L
        if n_old > 0:
            p = np.arange(n_old)
            slots = tables[i, p // BS].astype(np.int64) * BS + p % BS
            ops.paged_kv_store(kk_t[:n_old].contiguous(), vv_t[:n_old].contiguous(), kp, vp, torch.from_numpy(slots).to(DEV))
    q_t, q = bf16_cuda(rng.standard_normal((n, nh * d)))
    new_k = new_v = None
    if append:
        new_k, _ = bf16_cuda(np.stack([hist_k[i][-1] for i in range(n)])); new_v, _ = bf16_cuda(np.stack([hist_v[i][-1] for i in range(n)]))
    off, total = ops.build_decode_chunks(ctx_lens, chunk)
    out = to_np(ops.paged_attention_decode(q_t, kp, vp, new_k, new_v, torch.from_numpy(tables).to(DEV),
                                           torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), off.to(DEV), total, chunk, nh, nkv, d))
    assert np.isfinite(out).all()
    for i, L in enumerate(ctx_lens):
        ref = O.decode_attention(q[i], hist_k[i], hist_v[i], nh, nkv, d)
        assert max_rel(out[i], ref) <= TOL, (i, L)
        # the appended row is now in the cache, bit for bit, and gather returns the whole history
        gk, gv = ops.paged_kv_gather(kp, vp, torch.from_numpy(tables[i]).to(DEV), L)
        assert (to_np(gk) == hist_k[i]).all() and (to_np(gv) == hist_v[i]).all()


@pytest.mark.parametrize("chunk", [64, 512, 1024, 2048])  # 1024 and 2048: the executors' choice for large steps
def test_decode_with_fused_append_gqa8(chunk):  # the benchmark head layout: 16 q heads, 2 kv heads
    decode_case([1, 15, 16, 17, 128, 129, 700, 1000, 2049, 64, 513], 16, 2, chunk, 3)


def test_decode_without_append_and_other_layouts():
    decode_case([5, 300, 77], 16, 2, 256, 4, append=False)
    decode_case([40, 1025], 12, 2, 512, 5)   # Stella layout, 6 q heads per kv head
    decode_case([33, 200], 8, 8, 128, 6)     # no grouping
    decode_case([90], 16, 1, 64, 7)          # 16 q heads on one kv head


def test_decode_head_dim_256():  # 16 q / 2 kv heads of 256, the hybrid decoder's full-attention layout
    decode_case([1, 16, 17, 300, 1100, 64], 16, 2, 256, 31, d=256)
    decode_case([2049, 5000, 1024, 1025, 7], 16, 2, 2048, 33, d=256)
    decode_case([2049, 1500], 16, 2, 1024, 34, d=256)
    decode_case([45, 513], 8, 2, 512, 32, append=False, d=256)


def test_block_id_outside_the_pool_is_reported_not_dereferenced():
    d, nh, nkv = 128, 16, 2
    kp = torch.zeros((4, BS, nkv * d), dtype=torch.bfloat16, device=DEV); vp = torch.zeros_like(kp)
    q = torch.zeros((1, nh * d), dtype=torch.bfloat16, device=DEV)
    tables = torch.tensor([[0, 9, 1]], dtype=torch.int32, device=DEV)  # 9 >= 4 pool blocks
    off, total = ops.build_decode_chunks([40], 64)
    with pytest.raises(ops.InvalidOp):
        ops.paged_attention_decode(q, kp, vp, None, None, tables, torch.tensor([40], dtype=torch.int32, device=DEV), off.to(DEV), total, 64, nh, nkv, d)


def test_long_context_split_over_many_chunks():
    decode_case([32768, 128, 9000], 16, 2, 512, 8)
    decode_case([32768, 128, 9000], 16, 2, 2048, 9)


def test_turbo3_cache_rows_are_byte_identical_to_the_reference_codec():
    """KvCache::put / get with TurboQuant 3-bit rows: the pool bytes equal the oracle's
    encode_turbo3_0_head output for every head chunk, and the gathered rows equal its decode (rounded to
    bf16), through a shuffled block table; untouched slots stay untouched."""
    rng = np.random.default_rng(17)
    L, nkv, d = 75, 2, 256            # 4 chunks of 128 per row
    row = nkv * d
    scale = np.exp(rng.uniform(-3, 3, (L, 1)))           # rows of very different magnitude
    k_t, k = bf16_cuda(rng.standard_normal((L, row)) * scale); v_t, v = bf16_cuda(rng.standard_normal((L, row)) * 0.3)
    k[5] = 0; k_t[5] = 0                                 # an all-zero head row: norm 0
    rb = int(ops.lib.logismos_turbo3_row_bytes(row))
    assert rb == 4 * 56
    n_blocks = 9
    kp = torch.full((n_blocks, 16, rb), 0xAB, dtype=torch.uint8, device=DEV); vp = torch.full_like(kp, 0xCD)
    table = np.array([7, 2, 5, 0, 8], np.int32)
    p = np.arange(L)
    slots = table[p // 16].astype(np.int64) * 16 + p % 16
    ops.paged_kv_store_turbo3(k_t, v_t, kp, vp, torch.from_numpy(slots).to(DEV))
    kb, vb = kp.cpu().numpy().reshape(-1, rb), vp.cpu().numpy().reshape(-1, rb)
    ref_k = O.turbo3_encode(k.reshape(L, 4, 128)).reshape(L, rb); ref_v = O.turbo3_encode(v.reshape(L, 4, 128)).reshape(L, rb)
    assert np.array_equal(kb[slots], ref_k) and np.array_equal(vb[slots], ref_v)
    untouched = np.setdiff1d(np.arange(n_blocks * 16), slots)
    assert (kb[untouched] == 0xAB).all() and (vb[untouched] == 0xCD).all()
    ko, vo = ops.paged_kv_gather_turbo3(kp, vp, torch.from_numpy(table).to(DEV), L, row)
    dk = O.bf16_round(O.turbo3_decode(ref_k.reshape(L, 4, 56)).reshape(L, row)); dv = O.bf16_round(O.turbo3_decode(ref_v.reshape(L, 4, 56)).reshape(L, row))
    assert np.array_equal(to_np(ko), dk) and np.array_equal(to_np(vo), dv)
    # the codec is lossy by design (3 bits): the reference's own bar is a mean squared error below 0.05 on
    # small-amplitude data (crates/quant/src/lib.rs:682-697); relative to the row norm it stays bounded
    rel = np.linalg.norm(to_np(vo) - v, axis=1) / np.maximum(np.linalg.norm(v, axis=1), 1e-9)
    assert rel.max() < 0.5
    with pytest.raises(Exception):
        ops.paged_kv_store_turbo3(k_t, v_t, kp, vp, torch.full((L,), n_blocks * 16, dtype=torch.int64, device=DEV))
