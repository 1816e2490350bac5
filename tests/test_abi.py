"""CPU-side checks of the C-ABI library: it loads, exports every symbol the headers declare, the
host-only entry points compute the same indices as the oracle, and shape guards reject bad
shapes before any launch (no GPU needed: none of these calls touches a device)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle_lib as O
from logismos_b200._lib import lib, library_path

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in sorted(os.listdir(os.path.join(ROOT, "include"))):
        text = open(os.path.join(ROOT, "include", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b((?:lg|logismos)_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    assert os.path.exists(library_path()), "run python -m logismos_b200.build"
    dll = C.CDLL(library_path())
    syms = declared_symbols()
    assert len(syms) > 50
    missing = [s for s in sorted(syms) if not hasattr(dll, s)]
    assert not missing, missing


def test_the_four_reference_launcher_symbols_keep_their_names():
    dll = C.CDLL(library_path())
    for s in ("logismos_launch_matmul_naive_fp16", "logismos_launch_matmul_wmma_fp16", "logismos_launch_rms_norm_fp16",
              "logismos_launch_softmax_fp16", "logismos_launch_rope_fp16"):
        assert hasattr(dll, s)


def test_launcher_shape_guards_reject_without_launching():  # matmul/mod.rs:213-247, rope/mod.rs:215-269
    z = C.c_void_p(0)
    assert lib.logismos_launch_matmul_naive_fp16(z, z, z, 0, 4, 4, z) == 1
    assert lib.logismos_launch_matmul_naive_fp16(z, z, z, -1, 4, 4, z) == 1
    assert lib.logismos_launch_matmul_naive_fp16(z, z, z, 65536, 65536, 4, z) == 1   # M*N > i32::MAX
    assert lib.logismos_launch_matmul_wmma_fp16(z, z, z, 24, 16, 16, z) == 1         # not multiples of 16
    assert lib.logismos_launch_rope_fp16(z, z, 2**31 - 1, 2**31 - 1, 2, 2, z) == 1    # product overflows i64
    assert lib.logismos_launch_rope_fp16(z, z, 46341, 46341, 1, 2, z) == 1            # > i32::MAX
    assert lib.logismos_launch_rope_fp16(z, z, 1, 1, 1, 0, z) == 1
    assert lib.logismos_launch_rms_norm_fp16(z, z, z, 0, 8, 1e-5, z) == 1
    assert lib.logismos_launch_gemv_int4_g32_bf16(z, z, z, z, 1, 16, 100, z) == 1     # k % 128
    assert lib.logismos_launch_gemv_int4_g32_bf16(z, z, z, z, 65, 16, 128, z) == 1    # batch > 64
    assert lib.logismos_launch_linear_t_bf16(z, z, z, z, 8, 16, 100, 100, 16, 0, z, z) == 1  # k % 64
    assert lib.logismos_launch_varlen_attention_bf16(z, z, z, 1, 8, 4, 3, 128, 1024, 512, 768, 0, z) == 1  # heads % kv
    assert lib.logismos_launch_varlen_attention_bf16(z, z, z, 1, 8, 4, 2, 64, 512, 256, 384, 0, z) == 1    # head_dim
    assert lib.logismos_launch_varlen_attention_tc_bf16(z, z, z, z, 8, 1, 8, 4, 2, 64, 512, 256, 384, 0, z, z) == 1   # head_dim
    assert lib.logismos_launch_varlen_attention_tc_bf16(z, z, z, z, 8, 1, 8, 4, 3, 128, 1024, 512, 768, 0, z, z) == 1  # heads % kv, no scratch
    assert lib.logismos_varlen_attention_tc_scratch_bytes(100, 3, 2, 128) == 256 + 2 * 128 * 128 * 2  # 100 + 24 -> 128 padded keys
    assert lib.logismos_varlen_attention_tc_scratch_bytes(100, 3, 2, 64) == 0
    assert lib.logismos_launch_paged_attention_decode_bf16(z, z, z, z, z, z, z, z, z, z, z, 1, 1, 100, 4, 4, 16, 2, 128, z) == 1


def test_runtime_shim_returns_a_status_on_a_machine_without_a_gpu():
    """Every lg_* call must come back with a status (never spin or abort), device or not: on a box
    without a driver the calls fail with a classified code, on a GPU box they succeed."""
    n = C.c_int32(-1)
    rc = lib.lg_device_count(C.byref(n))
    assert (rc == 0 and n.value >= 1) or (rc != 0 and n.value == 0)
    d = C.c_void_p(123)
    rc = lib.lg_malloc(2**31 - 1, 64, C.byref(d))  # an ordinal no machine has: fails before allocating
    assert rc != 0 and d.value is None
    assert lib.lg_device_set_current(2**31 - 1) != 0
    s = C.c_void_p(77)
    assert lib.lg_stream_create(2**31 - 1, C.byref(s)) != 0 and s.value is None
    ms = C.c_float(0)
    assert lib.lg_event_elapsed_ms(None, None, None) == 1  # null out-pointer: InvalidValue


def test_error_kind_names_need_no_device():
    name = lambda c: lib.lg_error_kind_name(lib.lg_error_kind_from_raw(c)).decode()
    assert name(2) == "OutOfMemory" and name(700) == "IllegalAddress" and name(719) == "LaunchFailure"


def test_build_packing_matches_oracle_bit_for_bit():
    rng = np.random.default_rng(0)
    bs, n_pool, n = 16, 4096, 68
    cached = np.concatenate([rng.integers(256, 8193, 64), np.zeros(4)]).astype(np.int32)   # 64 decode + 4 prefill
    new = np.concatenate([np.ones(64), np.full(4, 512)]).astype(np.int32)
    need = -(-(cached + new) // bs)
    n_pool = int(need.sum()) + 5
    perm = rng.permutation(n_pool).astype(np.int32)
    tables = -np.ones((n, int(need.max()) + 1), np.int32); o = 0
    for i in range(n):
        tables[i, :need[i]] = perm[o:o + need[i]]; o += need[i]
    want = O.build_packing(cached, new, tables, bs, n_pool)
    total = int(new.sum())
    cu = np.empty(n + 1, np.int32); pos = np.empty(total, np.int32); slots = np.empty(total, np.int64); sid = np.empty(total, np.int32)
    P = lambda a: a.ctypes.data_as(C.c_void_p)
    r = lib.logismos_build_packing(P(cached), P(new), n, P(tables), tables.shape[1], bs, n_pool, P(cu), P(pos), P(slots), P(sid))
    assert r == total == 2112
    for got, ref in zip((cu, pos, slots, sid), want):
        assert (got == ref).all()
    tables[3, cached[3] // bs] = n_pool  # the block the new token of sequence 3 lands in: out of range -> rejected
    assert lib.logismos_build_packing(P(cached), P(new), n, P(tables), tables.shape[1], bs, n_pool, P(cu), P(pos), P(slots), P(sid)) == -1


def test_build_decode_chunks():
    cl = np.array([1, 512, 513, 17, 32768], np.int32); off = np.empty(6, np.int32)
    P = lambda a: a.ctypes.data_as(C.c_void_p)
    assert lib.logismos_build_decode_chunks(P(cl), 5, 512, P(off)) == 69
    assert off.tolist() == [0, 1, 2, 4, 5, 69]
    cl[3] = 0  # a context counts the token being decoded: an empty one is rejected
    assert lib.logismos_build_decode_chunks(P(cl), 5, 512, P(off)) == -1
    assert lib.logismos_paged_decode_scratch_bytes(68, 16, 128) == 68 * 16 * 130 * 4


def test_skinny_int4_route_table():
    """The kernel choice of logismos_launch_skinny_int4_g32_bf16 (host arithmetic): the tensor-core route above
    16 rows, for k >= 3 n at every batch, and from 8 rows up to n = 16384; the GEMV otherwise and whenever
    the shape rules of the tensor-core kernel do not hold."""
    want = {(1536, 1536, 1): 0, (1536, 1536, 8): 1, (1536, 1536, 16): 1, (1536, 1536, 64): 1, (8960, 1536, 4): 0, (8960, 1536, 16): 1,
            (1536, 8960, 1): 1, (1536, 8960, 64): 1, (151936, 1536, 1): 0, (151936, 1536, 16): 0, (151936, 1536, 17): 1,
            (17920, 1536, 16): 0, (2048, 6144, 2): 1, (256, 640, 64): 0, (1001, 1536, 40): 0, (1536, 1536, 65): 0, (1536, 1536, 0): 0}
    for (n, k, b), route in want.items():
        assert lib.logismos_skinny_int4_route(b, n, k) == route, (n, k, b)


def test_process_wide_switches_and_scratch_sizes_need_no_device():
    assert lib.logismos_get_dependent_launch() in (0, 1)
    before = lib.logismos_get_dependent_launch()
    lib.logismos_set_dependent_launch(0); assert lib.logismos_get_dependent_launch() == 0
    lib.logismos_set_dependent_launch(1); assert lib.logismos_get_dependent_launch() == 1
    lib.logismos_set_dependent_launch(before)
    det = lib.logismos_get_deterministic()
    lib.logismos_set_deterministic(1); assert lib.logismos_get_deterministic() == 1
    lib.logismos_set_deterministic(det)
    # one slot of 57856 bytes per (64-token chunk, head); every sequence may end in a partial chunk
    assert lib.logismos_gdn_chunked_scratch_bytes(4096, 4, 16) == (64 + 4) * 16 * 57856
    assert lib.logismos_gdn_chunked_scratch_bytes(63, 1, 2) == 1 * 2 * 57856
    assert lib.logismos_gdn_chunked_scratch_bytes(-1, 1, 2) == 0 and lib.logismos_gdn_chunked_scratch_bytes(64, 1, 0) == 0
    assert lib.logismos_turbo3_row_bytes(256) == 112 and lib.logismos_turbo3_row_bytes(100) == 0


def test_python_ops_reject_cpu_operands_without_touching_a_device():  # praxis/src/matmul.rs:154-166
    import torch
    from logismos_b200 import ops
    a = torch.zeros((16, 16), dtype=torch.float16)
    with pytest.raises(ops.InvalidOp):
        ops.matmul(a, a)
    with pytest.raises(ops.InvalidOp):
        ops.softmax(a)
