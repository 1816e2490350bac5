"""Weight loading over the C ABI: the safetensors reader (``lg_safetensors_*``) and the checkpoint
loaders of the executors (``lg_stella_load``, ``lg_decoder_load``).

Mirrors ``loader::safetensors::Reader`` (crates/loader/src/safetensors.rs:44-197: open / get / names
/ len, archive ordering by on-disk offset, a re-stat of the file before every access) and
``StellaModel::load`` (crates/embed/src/stella.rs:138-201). The parsing, the tensor accounting and the
quantisation run in the native library; this module only marshals.
"""
from __future__ import annotations

import ctypes as C
from typing import List

import numpy as np

from ._lib import lib

DTYPES = {0: ("F32", np.float32), 1: ("F16", np.float16), 2: ("BF16", np.uint16), 3: ("F8E4M3", np.uint8), 4: ("F8E5M2", np.uint8),
          5: ("I32", np.int32), 6: ("I8", np.int8), 8: ("U8", np.uint8)}


class LoaderError(IOError):
    """loader::Error (crates/loader/src/error.rs): I/O, format, unknown tensor, stale mapping."""


class _View(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("rank", C.c_int32), ("shape", C.c_int64 * 8), ("data", C.c_void_p), ("nbytes", C.c_uint64)]


class TensorView:
    """loader::TensorView: name, dtype name, shape and the bytes (a numpy view into the mapping: valid
    while the reader is open; BF16 and fp8 come as raw 16- / 8-bit integers)."""

    def __init__(self, name, dtype, shape, array):
        self.name, self.dtype, self.shape, self.array = name, dtype, shape, array


class Reader:
    def __init__(self, path: str):
        h = C.c_void_p()
        if lib.lg_safetensors_open(str(path).encode(), C.byref(h)):
            raise LoaderError(lib.lg_last_error().decode())
        self._h, self.path = h, str(path)

    def close(self):
        if getattr(self, "_h", None):
            lib.lg_safetensors_close(self._h)
            self._h = None

    __del__ = close

    def __len__(self) -> int:
        return int(lib.lg_safetensors_len(self._h))

    def names(self) -> List[str]:
        return [lib.lg_safetensors_name(self._h, i).decode() for i in range(len(self))]

    def data_region_start(self) -> int:
        return int(lib.lg_safetensors_data_region_start(self._h))

    def get(self, name: str) -> TensorView:
        v = _View()
        if lib.lg_safetensors_get(self._h, name.encode(), C.byref(v)):
            raise LoaderError(lib.lg_last_error().decode())
        dname, npdt = DTYPES[v.dtype]
        shape = tuple(int(v.shape[i]) for i in range(v.rank))
        n = int(v.nbytes)
        if n == 0:
            arr = np.zeros(shape, npdt)
        else:
            buf = (C.c_uint8 * n).from_address(v.data)
            arr = np.frombuffer(buf, dtype=np.uint8)
            # the data region of a file is only guaranteed byte alignment: copy when a wider view would be misaligned
            arr = (arr.view(npdt) if v.data % np.dtype(npdt).itemsize == 0 else arr.copy().view(npdt)).reshape(shape)
        return TensorView(name, dname, shape, arr)


def quantize_int4(w):
    """fp32 CUDA tensor [n, k] -> (codes uint8 [n, k/2], scales float16 [n, k/32]) on the device
    (``logismos_launch_quantize_int4_g32``)."""
    import torch
    from .ops import InvalidOp, _p, _stream
    from ._lib import check
    if not (isinstance(w, torch.Tensor) and w.is_cuda and w.dtype == torch.float32 and w.dim() == 2 and w.is_contiguous()):
        raise InvalidOp("quantize_int4: contiguous fp32 CUDA tensor [n, k]")
    n, k = w.shape
    codes = torch.empty((n, k // 2), dtype=torch.uint8, device=w.device)
    scales = torch.empty((n, k // 32), dtype=torch.float16, device=w.device)
    with torch.cuda.device(w.device):
        check(lib.logismos_launch_quantize_int4_g32(_p(w), _p(codes), _p(scales), n, k, _stream()), "quantize_int4")
        torch.cuda.current_stream().synchronize()
    return codes, scales
