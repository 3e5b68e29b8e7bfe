"""Host-side failure detection for multi-rank jobs.

The device kernels of this library never wait without a bound (``bounded_wait.cuh``), but a
rank that is gone should be noticed *before* the next launch, not by a device timeout. Every
rank calls ``PeerMonitor.check(step)`` between steps: it publishes ``alive/<rank>/<step>`` in
the job's key-value store and waits, with a short limit, for the same key of every other rank.
A rank that leaves on purpose publishes ``left/<rank>`` first, so the others raise
:class:`PeerLost` immediately instead of after the limit. Nothing here touches a GPU.

The reference has no failure handling beyond an OOM ``try/except`` in its benchmark
(benchmarks/benchmark_grpo_op.py:42-45).
"""
from __future__ import annotations

import datetime
from typing import Optional

import torch.distributed as dist


class PeerLost(RuntimeError):
    def __init__(self, rank: int, step: int, reason: str):
        super().__init__(f"rank {rank} is gone at step {step}: {reason}")
        self.rank, self.step, self.reason = rank, step, reason


class PeerMonitor:
    def __init__(self, store: Optional[dist.Store] = None, rank: Optional[int] = None,
                 world: Optional[int] = None, timeout_s: float = 2.0, prefix: str = "ka_health"):
        if store is None:
            from torch.distributed.distributed_c10d import _get_default_store

            store = _get_default_store()
        self.store = dist.PrefixStore(prefix, store)
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.timeout = datetime.timedelta(seconds=timeout_s)

    def announce_leave(self) -> None:
        """Tell the others that this rank stops taking part (call between steps)."""
        self.store.set(f"left/{self.rank}", b"1")

    def _left(self, r: int) -> bool:
        try:
            return self.store.check([f"left/{r}"])
        except RuntimeError:
            return False

    def check(self, step: int) -> None:
        """Raise :class:`PeerLost` unless every rank has reached ``step``."""
        self.store.set(f"alive/{self.rank}/{step}", b"1")
        for r in range(self.world):
            if r == self.rank:
                continue
            if self._left(r):
                raise PeerLost(r, step, "announced that it left")
            try:
                self.store.wait([f"alive/{r}/{step}"], self.timeout)
            except Exception as e:  # noqa: BLE001  (c10d raises DistStoreError / RuntimeError on timeout)
                reason = "announced that it left" if self._left(r) else f"no heartbeat within {self.timeout.total_seconds():.1f} s"
                raise PeerLost(r, step, reason) from e
