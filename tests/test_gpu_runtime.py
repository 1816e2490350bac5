"""The CUDA runtime shim against the behaviour the reference's hipcore tests pin
(crates/hipcore/tests/device_smoke.rs:15-62; src/memory.rs tests :499-679; src/error.rs)."""
import ctypes as C

import numpy as np
import pytest

from logismos_b200._lib import lib

pytestmark = pytest.mark.gpu


class Props(C.Structure):
    _fields_ = [("isa", C.c_char * 32), ("name", C.c_char * 256), ("total_vram_bytes", C.c_uint64),
                ("compute_units", C.c_int32), ("wavefront_size", C.c_int32), ("max_threads_per_block", C.c_int32),
                ("max_shared_mem_per_block", C.c_uint64), ("clock_rate_khz", C.c_int32), ("pci_bus_id", C.c_int32)]


def test_device_props_describe_a_b200():  # device_smoke.rs:15-40 (there: gfx1100, wave32, >= 48 CUs, >= 40 GiB)
    n = C.c_int32()
    assert lib.lg_device_count(C.byref(n)) == 0 and n.value >= 1
    p = Props()
    assert lib.lg_device_props_get(0, C.byref(p)) == 0
    assert p.isa == b"sm_100" and p.wavefront_size == 32
    assert p.compute_units >= 140 and p.total_vram_bytes >= 170 * 2**30
    assert p.max_threads_per_block == 1024 and p.max_shared_mem_per_block >= 227 * 1024


def test_h2d_d2h_round_trip_and_zero_fill():  # device_smoke.rs:42-62, memory.rs:163-182
    src = np.arange(4096, dtype=np.float32)
    d = C.c_void_p()
    assert lib.lg_malloc(0, src.nbytes, C.byref(d)) == 0
    assert lib.lg_memcpy_h2d(0, d, src.ctypes.data_as(C.c_void_p), src.nbytes) == 0
    back = np.empty_like(src)
    assert lib.lg_memcpy_d2h(0, back.ctypes.data_as(C.c_void_p), d, src.nbytes) == 0
    assert (back == src).all()
    assert lib.lg_memset(0, d, 0, src.nbytes) == 0
    assert lib.lg_memcpy_d2h(0, back.ctypes.data_as(C.c_void_p), d, src.nbytes) == 0
    assert (back == 0).all()
    assert lib.lg_free(0, d) == 0


def test_async_copy_stream_and_events():  # memory.rs:216-291, stream.rs:140-213
    s = C.c_void_p(); e0 = C.c_void_p(); e1 = C.c_void_p()
    assert lib.lg_stream_create(0, C.byref(s)) == 0
    assert lib.lg_event_create(0, C.byref(e0)) == 0 and lib.lg_event_create(0, C.byref(e1)) == 0
    src = np.random.default_rng(0).integers(0, 255, 1 << 20, dtype=np.uint8)
    d = C.c_void_p()
    assert lib.lg_malloc(0, src.nbytes, C.byref(d)) == 0
    assert lib.lg_event_record(0, e0, s) == 0
    assert lib.lg_memcpy_h2d_async(0, d, src.ctypes.data_as(C.c_void_p), src.nbytes, s) == 0
    assert lib.lg_event_record(0, e1, s) == 0
    assert lib.lg_stream_synchronize(0, s) == 0 and lib.lg_event_synchronize(0, e1) == 0
    ms = C.c_float(-1)
    assert lib.lg_event_elapsed_ms(e0, e1, C.byref(ms)) == 0 and ms.value >= 0
    back = np.empty_like(src)
    assert lib.lg_memcpy_d2h(0, back.ctypes.data_as(C.c_void_p), d, src.nbytes) == 0
    assert (back == src).all()
    for ev in (e0, e1):
        assert lib.lg_event_destroy(0, ev) == 0
    assert lib.lg_stream_destroy(0, s) == 0 and lib.lg_free(0, d) == 0


def test_invalid_device_ordinal_fails_deterministically():  # device.rs:125-153 (Device::invalid_for_test)
    bad = 2**31 - 1
    d = C.c_void_p(123)
    rc = lib.lg_malloc(bad, 64, C.byref(d))
    assert rc != 0 and d.value is None
    assert lib.lg_device_set_current(bad) != 0
    assert lib.lg_device_set_current(0) == 0  # the context stays usable


def test_error_kind_mapping_uses_cuda_numbering():  # error.rs:126-177 re-derived for cudaError_t
    name = lambda c: lib.lg_error_kind_name(lib.lg_error_kind_from_raw(c)).decode()
    assert name(0) == "None" and name(1) == "InvalidValue" and name(2) == "OutOfMemory"
    assert name(700) == "IllegalAddress" and name(701) == "LaunchOutOfResources"
    assert name(702) == "LaunchTimeout" and name(719) == "LaunchFailure" and name(600) == "NotReady"
    assert name(35) == "InsufficientDriver" and name(3) == "NotInitialized" and name(4) == "Deinitialized"
    assert name(500) == "NotFound" and name(99999) == "Unknown"
