"""Shared helpers of the benchmark CLIs: device timing with CUDA events and JSON output."""
from __future__ import annotations

import json
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def time_cuda(fn, warmup: int = 3, iters: int = 10, flush_l2: bool = True) -> float:
    """Median device time of ``fn()`` in milliseconds: CUDA events on the current stream,
    ``warmup`` untimed calls, an L2-sized write between timed calls when ``flush_l2``."""
    scrub = torch.empty(256 * 2**20, dtype=torch.uint8, device="cuda") if flush_l2 else None
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if scrub is not None:
            scrub.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def write_json(path: str | None, payload: dict) -> None:
    if not path:
        return
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        json.dump(payload, f, indent=1)


def time_cuda_graph(fn, reps: int = 20, flush_l2: bool = True) -> float:
    """Device time of one ``fn()`` in milliseconds with host launch latency taken out: ``reps``
    calls are captured into a CUDA graph (each preceded by an L2-sized write when ``flush_l2``)
    and the graph is replayed; the same graph without the calls is timed and subtracted.
    Use for kernels of a few microseconds, where Python's per-launch cost would dominate."""
    scrub = torch.empty(256 * 2**20, dtype=torch.uint8, device="cuda") if flush_l2 else None
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.synchronize()

    def capture(with_fn: bool):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                if scrub is not None:
                    scrub.zero_()
                if with_fn:
                    fn()
        return g

    def run(g):
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    full = run(capture(True))
    base = run(capture(False)) if scrub is not None else 0.0
    return (full - base) / reps
