"""Per-operator profiling: the reference's unused ``ProfilingMode`` enum
(rl_engine/platforms/constants.py:57-61) made real.

``RL_ENGINE_PROFILE`` (or :func:`set_mode`) selects

* ``off`` (default): :func:`profile_range` returns a shared no-op context; the cost at a call
  site is one attribute test.
* ``basic``: every range is timed on the device with a pair of CUDA events recorded on the
  current stream (no synchronisation at the call site; the events are resolved when a summary
  is asked for). CPU ranges are timed with ``perf_counter``.
* ``detailed``: ``basic`` plus an NVTX range of the same name, so a captured timeline or a
  kernel profile shows which operator a kernel belongs to.

:func:`summary` returns ``{name: {"calls", "total_ms", "mean_ms", "max_ms"}}``; with
``across_ranks`` the totals are the maximum over the ranks of the default process group (a
multi-GPU time is the slowest rank's). Ranges opened while a CUDA graph is being captured are
counted but not timed (an event recorded into a graph has no time of its own).
"""
from __future__ import annotations

import os
import time
from contextlib import contextmanager, nullcontext
from typing import Dict, Iterator, Optional

from ..platforms.constants import ProfilingMode

_NULL = nullcontext()


class Profiler:
    def __init__(self, mode: Optional[str] = None):
        self.mode = ProfilingMode.OFF
        self._pending: list = []          # (name, start_event, stop_event) not yet resolved
        self._stats: Dict[str, list] = {}  # name -> [calls, total_ms, max_ms, untimed_calls]
        self.set_mode(mode if mode is not None else os.environ.get("RL_ENGINE_PROFILE", "off"))

    # ------------------------------------------------------------------ configuration
    def set_mode(self, mode) -> None:
        self.mode = mode if isinstance(mode, ProfilingMode) else ProfilingMode(str(mode).lower())
        self.enabled = self.mode in (ProfilingMode.BASIC, ProfilingMode.DETAILED)

    def reset(self) -> None:
        self._pending.clear()
        self._stats.clear()

    # ------------------------------------------------------------------ recording
    def _add(self, name: str, ms: Optional[float]) -> None:
        st = self._stats.setdefault(name, [0, 0.0, 0.0, 0])
        st[0] += 1
        if ms is None:
            st[3] += 1
        else:
            st[1] += ms
            st[2] = max(st[2], ms)

    @contextmanager
    def _range(self, name: str, device) -> Iterator[None]:
        import torch

        on_cuda = device is not None and getattr(device, "type", str(device)) == "cuda" and torch.cuda.is_available()
        nvtx = self.mode == ProfilingMode.DETAILED and on_cuda
        if nvtx:
            torch.cuda.nvtx.range_push(name)
        try:
            if on_cuda and torch.cuda.is_current_stream_capturing():
                yield
                self._add(name, None)
            elif on_cuda:
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                yield
                stop.record()
                self._pending.append((name, start, stop))
                if len(self._pending) >= 4096:
                    self._resolve()
            else:
                t0 = time.perf_counter()
                yield
                self._add(name, (time.perf_counter() - t0) * 1e3)
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()

    def range(self, name: str, device=None):
        """Context manager timing one operator call (a no-op object when profiling is off)."""
        if not self.enabled:
            return _NULL
        return self._range(name, device)

    def _resolve(self) -> None:
        if not self._pending:
            return
        self._pending[-1][2].synchronize()
        for name, start, stop in self._pending:
            stop.synchronize()
            self._add(name, start.elapsed_time(stop))
        self._pending.clear()

    # ------------------------------------------------------------------ reporting
    def summary(self, across_ranks: bool = False) -> Dict[str, dict]:
        self._resolve()
        names = sorted(self._stats)
        totals = [self._stats[n][1] for n in names]
        if across_ranks:
            import torch
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                # every rank runs the same operators: reduce the totals in name order
                dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
                t = torch.tensor(totals, dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                totals = t.cpu().tolist()
        out = {}
        for n, tot in zip(names, totals):
            calls, _, mx, untimed = self._stats[n]
            timed = calls - untimed
            out[n] = {"calls": calls, "total_ms": tot, "mean_ms": tot / timed if timed else 0.0, "max_ms": mx}
        return out

    def report(self, across_ranks: bool = False) -> str:
        """The summary as a table, heaviest operator first."""
        from tabulate import tabulate

        rows = sorted(self.summary(across_ranks).items(), key=lambda kv: -kv[1]["total_ms"])
        return tabulate([[n, s["calls"], f"{s['total_ms']:.3f}", f"{s['mean_ms']:.4f}", f"{s['max_ms']:.4f}"]
                         for n, s in rows], headers=["operator", "calls", "total ms", "mean ms", "max ms"],
                        tablefmt="github")


profiler = Profiler()


def set_mode(mode) -> None:
    profiler.set_mode(mode)


def profile_range(name: str, device=None):
    """``with profile_range("gemm_bi", x.device): ...``: see the module docstring."""
    if not profiler.enabled:
        return _NULL
    return profiler._range(name, device)


def profiled(name: str):
    """Decorator form: times every call of the function under ``name``; the device is taken
    from the first tensor argument."""
    def deco(fn):
        def wrapper(*args, **kwargs):
            if not profiler.enabled:
                return fn(*args, **kwargs)
            dev = None
            for a in args:
                d = getattr(a, "device", None)
                if d is not None:
                    dev = d
                    break
            with profiler._range(name, dev):
                return fn(*args, **kwargs)

        wrapper.__name__ = getattr(fn, "__name__", name)
        wrapper.__doc__ = fn.__doc__
        wrapper.__wrapped__ = fn
        return wrapper

    return deco
