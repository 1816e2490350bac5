"""Kernel timing used by the benchmarks: CUDA events on the launch stream around a CUDA-graph replay."""
from __future__ import annotations

import torch

USE_GRAPH = True


def timeit(fn, iters, warmup=3, reps=3):
    """Seconds per launch. The `iters` launches (fn(0) .. fn(iters - 1)) are captured into one CUDA
    graph and the graph is replayed, so that host-side launch cost (Python, descriptor encoding) is not
    what is timed; a kernel of a few microseconds is otherwise hidden behind ~15 us of host work per
    call. For a launch that should read its operands from HBM, rotate them through fn's argument over
    more distinct bytes than the L2 holds within one pass of `iters` launches."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    st = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if not USE_GRAPH:
        e0.record(st)
        for i in range(iters):
            fn(i)
        e1.record(st)
        e1.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / iters
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(iters):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    st = torch.cuda.current_stream()
    e0.record(st)
    for _ in range(reps):
        g.replay()
    e1.record(st)
    e1.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (iters * reps)
