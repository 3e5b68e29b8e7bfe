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


    # ------------------------------------------------------------------ elastic shrink
    def survivors(self, step: int) -> list[int]:
        """Ranks that have reached ``step`` (this one included); never raises. A rank counts as
        gone when it announced that it left or shows no heartbeat within the limit."""
        self.store.set(f"alive/{self.rank}/{step}", b"1")
        alive = []
        for r in range(self.world):
            if r == self.rank:
                alive.append(r)
                continue
            if self._left(r):
                continue
            try:
                self.store.wait([f"alive/{r}/{step}"], self.timeout)
                alive.append(r)
            except Exception:  # noqa: BLE001
                pass
        return alive

    def agree_on_survivors(self, step: int) -> list[int]:
        """One list for every surviving rank: the lowest-ranked survivor (in each rank's own
        view) publishes its view, the others adopt it. Raises :class:`PeerLost` if this rank is
        not in the agreed list (it was too slow and has been dropped)."""
        mine = self.survivors(step)
        leader = mine[0]
        key = f"decision/{step}"
        if leader == self.rank:
            self.store.set(key, ",".join(str(r) for r in mine).encode())
            return mine
        try:
            self.store.wait([key], self.timeout * 3)
        except Exception as e:  # noqa: BLE001
            raise PeerLost(leader, step, "the lowest surviving rank published no decision") from e
        agreed = [int(x) for x in self.store.get(key).decode().split(",")]
        if self.rank not in agreed:
            raise PeerLost(self.rank, step, "this rank was dropped from the job by the survivors")
        return agreed


def shrink_group(monitor: PeerMonitor, step: int, power_of_two: Optional[bool] = None):
    """After a :class:`PeerLost`: agree on the surviving ranks and build a process group of
    them without the ones that are gone (``new_group`` with local synchronisation, so the
    departed ranks need not take part). Returns ``(group, ranks)``; a surviving rank that is
    not in ``ranks`` gets ``(None, ranks)`` and has to stand by. Call it between steps, with no
    collective in flight. The deterministic all-reduce accepts any number of CPU ranks; its
    CUDA kernel takes 1, 2, 4 or 8, so with ``power_of_two`` (the default when CUDA is in use)
    the group is the largest such prefix of the survivors."""
    ranks = monitor.agree_on_survivors(step)
    if power_of_two is None:
        import torch

        power_of_two = torch.cuda.is_available()
    if power_of_two:
        keep = 1
        while keep * 2 <= len(ranks):
            keep *= 2
        ranks = ranks[:keep]
    if monitor.rank not in ranks:
        return None, ranks
    group = dist.new_group(ranks, use_local_synchronization=True)
    return group, ranks
