"""The paged-decode entry point that allocates nothing, for hosts that cannot allocate device
memory where they decode (an engine whose allocator has already given every free byte of HBM to
the KV pool and the weights; a decode thread that must not hit the device-wide synchronisation an
allocation implies). Its per-chunk partials live in a buffer built into the library, so the test
checks what such a caller relies on: through the C ABI, the results equal those of the entry point
that takes caller scratch and, directly, the CPU oracle's decode attention over each sequence's
gathered history, on two calls in a row that share the built-in buffer (the second call meets the
first call's leftovers), and a request beyond the buffer's size is refused cleanly.
Collected last on purpose: a failure here cannot hide the other tests from a run that stops at the
first failure."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle_lib as O
from gpu_util import DEV, TOL, max_rel, to_np
from logismos_b200 import ops
from logismos_b200._lib import lib

pytestmark = pytest.mark.gpu
BS, D = 16, 128
LIMIT = 8 * 1024 * 1024


def P(t):
    return C.c_void_p(0) if t is None else C.c_void_p(t.data_ptr())


def make_case(ctx_lens, nh, nkv, chunk, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    n = len(ctx_lens)
    row = nkv * D
    blocks = [-(-L // BS) for L in ctx_lens]
    n_pool = sum(blocks) + 2
    perm = torch.randperm(n_pool, generator=g).to(torch.int32)
    tables = torch.full((n, max(blocks)), -1, dtype=torch.int32)
    o = 0
    for i, nb in enumerate(blocks):
        tables[i, :nb] = perm[o:o + nb]
        o += nb
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).to(DEV)
    off, total = ops.build_decode_chunks(ctx_lens, chunk)
    return dict(q=mk(n, nh * D), kp=mk(n_pool, BS, row), vp=mk(n_pool, BS, row), nk=mk(n, row), nv=mk(n, row),
                tables=tables.to(DEV), ctx=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), off=off.to(DEV),
                total=total, chunk=chunk, n=n, nh=nh, nkv=nkv, n_pool=n_pool, maxb=tables.shape[1])


def run_both(c):
    """(with caller scratch, without) outputs of the same case, each on its own copy of the pools."""
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = []
    for noalloc in (False, True):
        kp, vp = c["kp"].clone(), c["vp"].clone()
        out = torch.zeros_like(c["q"])
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        common = (P(c["q"]), P(kp), P(vp), P(c["nk"]), P(c["nv"]), P(c["tables"]), P(c["ctx"]), P(c["off"]), P(out))
        tail = (P(status), c["n"], c["total"], c["chunk"], c["maxb"], c["n_pool"], c["nh"], c["nkv"], D, st)
        if noalloc:
            rc = lib.logismos_launch_paged_attention_decode_noalloc_bf16(*common, *tail)
        else:
            need = lib.logismos_paged_decode_scratch_bytes(c["total"], c["nh"], D)
            scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV)
            rc = lib.logismos_launch_paged_attention_decode_bf16(*common, P(scratch), *tail)
        torch.cuda.synchronize()
        assert rc == 0 and int(status.item()) == 0
        outs.append((to_np(out), kp, vp))
    return outs


def test_two_calls_in_a_row_match_the_entry_point_with_caller_scratch():
    # call 1: long contexts, many chunks, fills a good part of the built-in buffer
    first = make_case([3000, 17, 1500, 640], 16, 2, 64, seed=1)
    # call 2: a different, smaller problem that reads and writes where call 1 left its partials
    second = make_case([700, 129], 12, 2, 128, seed=2)
    for case in (first, second):
        assert case["total"] > case["n"]  # at least one sequence is split, so the scratch path is exercised
        (ref, kp_r, vp_r), (got, kp_g, vp_g) = run_both(case)
        assert np.isfinite(got).all()
        assert max_rel(got, ref) <= TOL
        assert (got == ref).all()  # the same kernels on the same inputs: nothing may depend on the buffer's history
        assert torch.equal(kp_r, kp_g) and torch.equal(vp_r, vp_g)  # the fused append wrote the same rows
        # and against the oracle itself: every sequence's history (the appended token included) gathered
        # from the pools through its block table, last-row causal attention on the CPU
        kp, vp, tab, q = to_np(kp_g), to_np(vp_g), case["tables"].cpu().numpy(), to_np(case["q"])
        for i, L in enumerate(case["ctx"].cpu().tolist()):
            pos = np.arange(L)
            rows = tab[i, pos // BS].astype(np.int64) * BS + pos % BS
            k = np.ascontiguousarray(kp.reshape(-1, kp.shape[-1])[rows]); v = np.ascontiguousarray(vp.reshape(-1, vp.shape[-1])[rows])
            assert np.array_equal(k[-1], to_np(case["nk"])[i]) and np.array_equal(v[-1], to_np(case["nv"])[i])
            assert max_rel(got[i], O.decode_attention(q[i], k, v, case["nh"], case["nkv"], D)) <= TOL, (i, L)


def test_a_request_beyond_the_built_in_buffer_is_refused_without_launching():
    nh = 16
    too_many = LIMIT // (nh * (D + 2) * 4) + 1
    assert lib.logismos_paged_decode_scratch_bytes(too_many, nh, D) > LIMIT
    z = C.c_void_p(0)
    rc = lib.logismos_launch_paged_attention_decode_noalloc_bf16(z, z, z, z, z, z, z, z, z, z, 4, too_many, 512, 8, 8, nh, 2, D, z)
    assert rc == 2  # cudaErrorMemoryAllocation: classified as OutOfMemory by lg_error_kind_from_raw
    assert lib.lg_error_kind_name(lib.lg_error_kind_from_raw(rc)).decode() == "OutOfMemory"
    torch.cuda.synchronize()  # nothing was launched, the context is untouched
