"""Kernel timer that amortises launch overhead by capturing N calls in a CUDA graph
(python/minisgl/benchmark/perf.py:10-51 of the reference), plus the timing hygiene every number here follows:
warm-up, L2 flush between timed iterations, CUDA events on the launching stream."""
from __future__ import annotations

from typing import Callable, List

import torch

_FLUSH = {}


def flush_l2(device=None) -> None:
    """Writes a buffer larger than the 126 MB L2 so that the next kernel starts from HBM."""
    key = str(device)
    buf = _FLUSH.get(key)
    if buf is None:
        buf = torch.empty(256 << 20, dtype=torch.uint8, device=device or "cuda")
        _FLUSH[key] = buf
    buf.zero_()


def time_kernel(fn: Callable[[], None], warmup: int = 3, iters: int = 10, flush: bool = True) -> List[float]:
    """Per-iteration milliseconds (CUDA events, sync on both sides)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flush:
            flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return out


def time_in_graph(fn: Callable[[], None], calls: int = 64, warmup: int = 3, replays: int = 5) -> float:
    """Milliseconds per call with `calls` invocations captured in one CUDA graph (launch overhead amortised)."""
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for _ in range(warmup):
            fn()
    s.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for _ in range(calls):
            fn()
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(replays):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (replays * calls)
