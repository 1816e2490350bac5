"""Builds liblogismos_kernels.so / .a from csrc/ with nvcc for sm_100a.

The counterpart of the reference's crates/kernels/build.rs (:35-49, :71-84, :117-122): nvcc
instead of hipcc, `-gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -Xcompiler -fPIC`, the
objects archived as liblogismos_kernels.a and also linked into a shared library for loaders that
bind at run time. Environment: NVCC overrides the compiler, LOGISMOS_SKIP_CUDA_BUILD=1 skips the
build (the library is then absent and every op fails loudly at load time).

Run as a module:  python -m logismos_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
SO = os.path.join(HERE, "liblogismos_kernels.so")
AR = os.path.join(HERE, "liblogismos_kernels.a")

CU_SOURCES = ["cudacore.cu", "legacy_fp16.cu", "elementwise.cu", "gemv_int4.cu", "dequant_int4.cu", "gemm_tcgen05.cu", "qgemm_tcgen05.cu",
              "attention.cu", "attention_tcgen05.cu", "gdn.cu", "gdn_chunk.cu", "sampling.cu", "kvquant.cu", "stella_model.cu", "decoder_model.cu", "hybrid_model.cu", "tp_comm.cu"]
CPP_SOURCES = ["sched.cpp", "loader.cpp"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def _nvcc() -> str:
    n = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(n) and not shutil.which(n):
        raise RuntimeError("nvcc not found (set NVCC)")
    return n


def _sources():
    out = []
    for s in CU_SOURCES + CPP_SOURCES:
        p = os.path.join(CSRC, s)
        if os.path.exists(p):
            out.append(p)
    return out


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if os.environ.get("LOGISMOS_SKIP_CUDA_BUILD"):
        raise RuntimeError("LOGISMOS_SKIP_CUDA_BUILD is set: no GPU kernels are built")
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(ROOT, "include", h) for h in os.listdir(os.path.join(ROOT, "include"))]
    headers += [os.path.join(CSRC, h) for h in os.listdir(CSRC) if h.endswith((".cuh", ".h"))]
    jobs = []
    objs = []
    for src in _sources():
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or r.returncode:
                    sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
                if r.returncode:
                    raise RuntimeError("nvcc failed for " + cmd[-3])
    if force or jobs or _stale(SO, objs):
        subprocess.check_call([nvcc, "-shared", "-o", SO] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"])
        if os.path.exists(AR):
            os.remove(AR)
        subprocess.check_call(["ar", "rcs", AR] + objs)
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
