"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import oracle_lib as O

DEV = "cuda:0"
TOL = 2e-2  # max-rel per tensor, the floating-point bar of the build (bf16 storage, fp32 accumulate)


def max_rel(got, ref):
    got = np.asarray(got, dtype=np.float64); ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def row_rel(got, ref):
    """Largest per-row relative error: max over rows of max|got - ref| / max|ref| within the row (a
    stricter bar than one ratio over the whole tensor: a row of small values cannot hide behind a row
    of large ones)."""
    got = np.asarray(got, dtype=np.float64); ref = np.asarray(ref, dtype=np.float64)
    got = got.reshape(-1, got.shape[-1]); ref = ref.reshape(-1, ref.shape[-1])
    den = np.maximum(np.abs(ref).max(axis=1), 1e-30)
    return float((np.abs(got - ref).max(axis=1) / den).max())


def cosine(a, b):
    a = np.asarray(a, np.float64).ravel(); b = np.asarray(b, np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def bf16_cuda(x):
    """fp32 numpy -> bf16 CUDA tensor (round to nearest even) and the rounded values as fp32 numpy."""
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.bfloat16)
    return t.to(DEV), t.to(torch.float32).numpy()


def to_np(t):
    return t.detach().to(torch.float32).cpu().numpy()
