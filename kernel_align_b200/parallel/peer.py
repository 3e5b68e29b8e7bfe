"""Peer memory for the fused compute+collective kernels: one symmetric buffer per rank that
every other rank of the node can load from and store to over NVLink.

``PeerArena`` wraps ``torch.distributed._symmetric_memory``: every rank allocates the same
number of bytes, the rendezvous maps all of them into every process, and kernels receive the
list of base addresses (``ptrs[r]`` is rank ``r``'s buffer as seen from this process). Kernels
only use plain peer loads/stores on these addresses.
"""
from __future__ import annotations

import os
import weakref
from typing import Optional

import torch
import torch.distributed as dist

# The kernels only use plain peer loads and stores (every cross-GPU sum follows a fixed order,
# which in-switch reduction does not give), so the arenas are not bound to an NVLink multicast
# object: a binding nobody uses only widens what a dying rank can disturb on its peers.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


_live_arenas: "weakref.WeakSet" = weakref.WeakSet()


def reset_all_arenas() -> None:
    """Clear every peer arena of this process (flags, exchange and gather buffers) after a
    device-side wait gave up and left them half written. Collective over the default group:
    every rank of the job calls it, with no kernel in flight."""
    torch.cuda.synchronize()
    dist.barrier()
    for arena in list(_live_arenas):
        arena.buf.zero_()
    torch.cuda.synchronize()
    dist.barrier()


class PeerArena:
    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup] = None, device=None):
        import torch.distributed._symmetric_memory as symm

        if not dist.is_initialized():
            raise RuntimeError("PeerArena needs an initialised process group")
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.buf = symm.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm.rendezvous(self.buf, self.group)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        _live_arenas.add(self)

    def zero(self) -> None:
        """Collectively clear the arena (after an aborted launch left flags half-written)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)


_vp_groups: dict = {}


def vocab_parallel_group(vocab: int, panel_rows: int = 32768, group: Optional[dist.ProcessGroup] = None):
    """The :class:`~kernel_align_b200.ops.fused_logp.VocabParallel` description for the
    current process group, with its exchange arena allocated once and cached."""
    from ..ops import fused_logp
    from .. import _native

    g = group if group is not None else dist.group.WORLD
    key = (id(g), vocab, panel_rows)
    vp = _vp_groups.get(key)
    if vp is None:
        world = dist.get_world_size(g)
        nbytes = _native.cuda().ka_lmhead_logp_exchange_bytes(world, panel_rows)
        arena = PeerArena(nbytes, g)
        vp = fused_logp.VocabParallel(rank=arena.rank, world=world, exchange_ptrs=arena.ptrs, epoch=1,
                                      panel_rows=panel_rows)
        vp.arena = arena  # keep the mapping alive
        vp.process_group = g
        _vp_groups[key] = vp
    return vp


def attach_gather_arena(vp, k: int) -> list[int]:
    """Allocate (collectively) the arena the fused log-prob kernel gathers row-sharded hidden
    states of width ``k`` into: two generations of one panel of rows and ids, with their flags.
    Its size depends on the panel and on ``k`` only, not on the number of rows."""
    from .. import _native

    nbytes = _native.cuda().ka_lmhead_logp_gather_bytes(vp.world, vp.panel_rows, k)
    if nbytes == 0:
        raise ValueError(f"panel_rows {vp.panel_rows} must be a multiple of 256 * world ({vp.world})")
    arena = PeerArena(nbytes, getattr(vp, "process_group", None))
    if not hasattr(vp, "gather_arenas"):
        vp.gather_arenas = {}
    vp.gather_arenas[k] = arena   # keep the mapping alive
    vp.gather_ptrs[k] = arena.ptrs
    return arena.ptrs


def gather_arena_bytes(vp, k: int) -> int:
    """Bytes of symmetric memory :func:`attach_gather_arena` holds per rank."""
    from .. import _native

    return int(_native.cuda().ka_lmhead_logp_gather_bytes(vp.world, vp.panel_rows, k))
