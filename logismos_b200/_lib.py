"""ctypes binding of liblogismos_kernels.so (the C ABI declared in include/*.h)."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liblogismos_kernels.so")

vp, i32, i64, u32, u64, f32, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_float, C.c_size_t


class LogismosError(RuntimeError):
    """A launcher or runtime call returned a non-zero status (kernels::Error::Launch in the
    reference, crates/kernels/src/error.rs:30-41): carries the raw code and its classified kind."""

    def __init__(self, op: str, code: int, kind: str = "", message: str = ""):
        self.op, self.code, self.kind = op, code, kind
        super().__init__(f"{op}: {kind or 'error'} (code {code}) {message}".strip())


class NoGpuBuild(LogismosError):
    """The CUDA library is absent (Error::NoGpuBuild, crates/kernels/src/error.rs:58-64)."""


def library_path() -> str:
    return _SO


class _LStella(C.Structure):
    pass


def _declare(l):
    sig = {
        # runtime shim
        "lg_device_count": [C.POINTER(i32)],
        "lg_device_set_current": [i32],
        "lg_device_props_get": [i32, vp],
        "lg_device_mem_info": [i32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)],
        "lg_device_synchronize": [i32],
        "lg_malloc": [i32, sz, C.POINTER(vp)],
        "lg_free": [i32, vp],
        "lg_memset": [i32, vp, i32, sz],
        "lg_memcpy_h2d": [i32, vp, vp, sz],
        "lg_memcpy_d2h": [i32, vp, vp, sz],
        "lg_memcpy_h2d_async": [i32, vp, vp, sz, vp],
        "lg_stream_create": [i32, C.POINTER(vp)],
        "lg_stream_synchronize": [i32, vp],
        "lg_stream_destroy": [i32, vp],
        "lg_event_create": [i32, C.POINTER(vp)],
        "lg_event_record": [i32, vp, vp],
        "lg_event_synchronize": [i32, vp],
        "lg_event_elapsed_ms": [vp, vp, C.POINTER(f32)],
        "lg_event_destroy": [i32, vp],
        "lg_error_kind_from_raw": [u32],
        # reference launchers
        "logismos_launch_matmul_naive_fp16": [vp, vp, vp, i32, i32, i32, vp],
        "logismos_launch_matmul_wmma_fp16": [vp, vp, vp, i32, i32, i32, vp],
        "logismos_launch_rms_norm_fp16": [vp, vp, vp, i32, i32, f32, vp],
        "logismos_launch_softmax_fp16": [vp, vp, i32, i32, vp],
        "logismos_launch_rope_fp16": [vp, vp, i32, i32, i32, i32, vp],
        # encoder path
        "logismos_launch_embed_lookup_bf16": [vp, vp, vp, i32, i32, i32, vp],
        "logismos_launch_rms_norm_f32": [vp, vp, vp, i32, i32, f32, i32, vp],
        "logismos_launch_linear_t_bf16": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp],
        "logismos_launch_linear_t_naive_bf16": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp],
        "logismos_launch_rope_halves_bf16": [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp],
        "logismos_launch_swiglu_bf16": [vp, vp, i32, i32, vp],
        "logismos_launch_varlen_attention_bf16": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp],
        "logismos_launch_varlen_attention_tc_bf16": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp],
        "logismos_launch_rope_varlen_attention_tc_bf16": [vp, vp, vp, vp, i32, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp],
        "logismos_launch_paged_prefix_attention_tc_bf16": [vp, i32, vp, vp, vp, vp, vp, i32, i32, vp, vp, i32, i32, i32, i32, i32, i32,
                                                           i32, i32, vp, vp],
        "logismos_launch_paged_prefix_attention_turbo3_bf16": [vp, i32, vp, vp, vp, vp, vp, i32, i32, vp, vp, i32, i32, i32, i32, i32, i32,
                                                               i32, i32, vp, vp],
        "logismos_launch_pool_head_f32": [vp, vp, vp, vp, vp, vp, i32, i32, i32, vp],
        # decode path
        "logismos_launch_gemv_int4_g32_bf16": [vp, vp, vp, vp, i32, i32, i32, vp],
        "logismos_launch_gemv_int4_g32_f32": [vp, vp, vp, vp, i32, i32, i32, vp],
        "logismos_launch_skinny_int4_g32_bf16": [vp, vp, vp, vp, i32, i32, i32, vp, vp, vp],
        "logismos_skinny_int4_route": [i32, i32, i32],
        "logismos_launch_dequant_int4_g32_bf16": [vp, vp, vp, i32, i32, vp],
        "logismos_launch_qlinear_int4_g32_acc_f32": [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp],
        "logismos_launch_qlinear_int4_g32_acc_f32_static": [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp],
        "logismos_launch_qlinear_finish_bf16": [vp, vp, vp, i32, i32, i32, i32, i32, vp],
        "logismos_launch_paged_attention_decode_bf16": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32,
                                                        i32, i32, i32, i32, i32, vp],
        "logismos_launch_paged_attention_decode_noalloc_bf16": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32,
                                                                i32, i32, i32, i32, i32, vp],
        "logismos_launch_paged_kv_store_bf16": [vp, vp, i32, vp, vp, vp, i32, i32, i64, vp, vp],
        "logismos_launch_paged_kv_gather_bf16": [vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp],
        "logismos_launch_paged_kv_store_turbo3": [vp, vp, i32, vp, vp, vp, i32, i32, i64, vp, vp],
        "logismos_launch_paged_kv_gather_turbo3": [vp, vp, vp, i32, i32, i32, i32, vp, vp, vp, vp],
        "logismos_launch_gather_rows_f32": [vp, vp, vp, i32, i32, i32, vp, vp],
        "logismos_launch_gdn_decode_step": [vp, vp, vp, vp, vp, vp, vp, i32, i32, f32, vp],
        "logismos_launch_gdn_prefill": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, i32, vp],
        "logismos_launch_gdn_decode_from_acc": [vp, vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, f32, vp],
        "logismos_launch_gdn_chunked": [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, vp, i32, vp],
        "logismos_launch_gdn_prepare": [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, vp],
        "logismos_launch_gated_mul_bf16": [vp, i32, vp, i32, i32, i32, i32, vp],
        "logismos_launch_greedy_argmax": [vp, i32, vp, i32, i32, vp],
        "logismos_launch_temperature_f32": [vp, i32, i32, f32, vp],
        "logismos_launch_top_k_f32": [vp, i32, i32, i32, vp],
        "logismos_launch_top_p_f32": [vp, i32, i32, f32, vp],
        "logismos_launch_min_p_f32": [vp, i32, i32, f32, vp],
        "logismos_launch_repetition_penalty_f32": [vp, i32, i32, vp, vp, i32, f32, vp],
        "logismos_launch_multinomial_f32": [vp, i32, i32, vp, vp, vp],
        # model
        "logismos_launch_quantize_int4_g32": [vp, vp, vp, i32, i32, vp],
        "lg_safetensors_open": [C.c_char_p, C.POINTER(vp)],
        "lg_safetensors_get": [vp, C.c_char_p, vp],
        "lg_stella_load": [i32, C.c_char_p, vp, C.POINTER(vp)],
        "lg_decoder_load": [i32, C.c_char_p, vp, C.POINTER(vp)],
        "lg_stella_create": [i32, vp, vp, C.POINTER(vp)],
        "lg_stella_encode_ids_batch": [vp, vp, vp, i32, i32, i32, vp],
        "lg_stella_forward_device": [vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp],
        "lg_stella_last_hidden": [vp, i32, vp],
        "lg_decoder_create": [i32, vp, vp, C.POINTER(vp)],
        "lg_decoder_step": [vp, vp, vp, vp, i32, vp, vp],
        "lg_decoder_replay_device": [vp, vp],
        "lg_decoder_last_hidden": [vp, i32, vp],
        "lg_decoder_last_logits": [vp, i32, vp],
        "logismos_launch_add_f32": [vp, vp, i64, vp],
        "logismos_launch_gdn_finish": [vp, i32, vp, vp, vp, i32, vp, vp, i32, i32, vp],
        "lg_hybrid_set_allreduce": [vp, vp, vp],
        "lg_hybrid_set_reduce_add": [vp, vp, vp],
        "lg_tp_comm_alloc": [i32, i32, u64, C.POINTER(vp), vp],
        "lg_tp_comm_open": [i32, vp, i32, i32, u64, vp, C.POINTER(vp)],
        "lg_tp_reduce_add_f32": [vp, vp, vp, u64, vp, vp],
        "lg_hybrid_create": [i32, vp, vp, C.POINTER(vp)],
        "lg_hybrid_step": [vp, vp, vp, vp, i32, vp, vp, vp],
        "lg_hybrid_replay_device": [vp, vp],
        "lg_hybrid_last_hidden": [vp, i32, vp],
        "lg_hybrid_last_logits": [vp, i32, vp],
    }
    for name, args in sig.items():
        fn = getattr(l, name)
        fn.argtypes = args
        fn.restype = u32
    l.lg_error_kind_name.argtypes = [u32]
    l.lg_error_kind_name.restype = C.c_char_p
    l.lg_error_string.argtypes = [u32]
    l.lg_error_string.restype = C.c_char_p
    l.lg_last_error.argtypes = []
    l.lg_last_error.restype = C.c_char_p
    l.logismos_paged_decode_scratch_bytes.argtypes = [i32, i32, i32]
    l.logismos_paged_decode_scratch_bytes.restype = sz
    l.logismos_varlen_attention_tc_scratch_bytes.argtypes = [i32, i32, i32, i32]
    l.logismos_varlen_attention_tc_scratch_bytes.restype = sz
    l.logismos_paged_prefix_attention_scratch_bytes.argtypes = [i32, i32, i32, i32]
    l.logismos_paged_prefix_attention_scratch_bytes.restype = sz
    l.logismos_turbo3_row_bytes.argtypes = [i32]
    l.logismos_turbo3_row_bytes.restype = sz
    l.logismos_build_packing.argtypes = [vp, vp, i32, vp, i32, i32, i32, vp, vp, vp, vp]
    l.logismos_build_packing.restype = i64
    l.logismos_build_decode_chunks.argtypes = [vp, i32, i32, vp]
    l.logismos_build_decode_chunks.restype = i32
    l.logismos_pick_decode_chunk.argtypes = [vp, i32, i32, i32]
    l.logismos_pick_decode_chunk.restype = i32
    l.lg_tp_comm_region_bytes.argtypes = [i32, u64]
    l.lg_tp_comm_region_bytes.restype = sz
    l.lg_tp_comm_destroy.argtypes = [vp, i32]
    l.lg_tp_comm_destroy.restype = None
    l.logismos_set_deterministic.argtypes = [i32]
    l.logismos_set_deterministic.restype = None
    l.logismos_get_deterministic.argtypes = []
    l.logismos_get_deterministic.restype = i32
    l.logismos_skinny_int4_route.restype = i32
    l.logismos_gdn_chunked_scratch_bytes.argtypes = [i32, i32, i32]
    l.logismos_gdn_chunked_scratch_bytes.restype = sz
    l.logismos_set_dependent_launch.argtypes = [i32]
    l.logismos_set_dependent_launch.restype = None
    l.logismos_get_dependent_launch.argtypes = []
    l.logismos_get_dependent_launch.restype = i32
    l.lg_safetensors_close.argtypes = [vp]
    l.lg_safetensors_close.restype = None
    l.lg_safetensors_len.argtypes = [vp]
    l.lg_safetensors_len.restype = i32
    l.lg_safetensors_name.argtypes = [vp, i32]
    l.lg_safetensors_name.restype = C.c_char_p
    l.lg_safetensors_data_region_start.argtypes = [vp]
    l.lg_safetensors_data_region_start.restype = u64
    l.lg_stella_destroy.argtypes = [vp]
    l.lg_stella_destroy.restype = None
    l.lg_decoder_destroy.argtypes = [vp]
    l.lg_decoder_destroy.restype = None
    l.lg_hybrid_destroy.argtypes = [vp]
    l.lg_hybrid_destroy.restype = None
    for name in ("lg_decoder_launches_last_step", "lg_decoder_device_status", "lg_hybrid_launches_last_step",
                 "lg_hybrid_device_status"):
        getattr(l, name).argtypes = [vp]
        getattr(l, name).restype = i32
    for name in ("lg_stella_default_dim", "lg_stella_max_tokens", "lg_stella_launches_per_forward",
                 "lg_stella_device_status"):
        getattr(l, name).argtypes = [vp]
        getattr(l, name).restype = i32
    l.lg_stella_supported_dims.argtypes = [vp, C.POINTER(i32), i32]
    l.lg_stella_supported_dims.restype = i32
    return l


class _Lazy:
    """Loads the shared library on first use; a missing library is an error, never a fallback."""

    def __init__(self):
        self._l = None

    def _load(self):
        if self._l is None:
            if not os.path.exists(_SO):
                raise NoGpuBuild("load", 0, "NoGpuBuild",
                                 f"{_SO} is missing: build it with `python -m logismos_b200.build` "
                                 "(there is no CPU fallback)")
            self._l = _declare(C.CDLL(_SO))
        return self._l

    def __getattr__(self, name):
        return getattr(self._load(), name)


lib = _Lazy()


def check(code: int, op: str):
    """Raise LogismosError for a non-zero launcher / runtime status."""
    if code:
        kind = lib.lg_error_kind_name(lib.lg_error_kind_from_raw(code)).decode()
        raise LogismosError(op, int(code), kind, lib.lg_error_string(code).decode())
