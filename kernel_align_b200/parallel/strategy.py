"""Process layouts for the ``DistributedStrategy`` values.

``make_layout(strategy, tp_size=, pp_size=)`` splits the ranks of the default process group
into tensor-parallel, pipeline-parallel and data-parallel groups and returns a
:class:`ParallelLayout`; ``build_model`` creates the matching model object (a
:class:`LlamaModel` sharded over the tensor-parallel group, or a :class:`PipelineStage`).
Ranks are laid out tensor-parallel fastest, then pipeline, then data parallel, so that the
tensor-parallel group (the one that exchanges tiles inside kernels) consists of neighbouring
ranks, i.e. GPUs of one NVSwitch domain.

    data_parallel       every rank holds the whole model        dp = world
    model_parallel      one tensor-parallel group               tp = world
    pipeline_parallel   one pipeline                            pp = world
    hybrid              tp x pp x dp with tp_size, pp_size given

The reference declares these four names (rl_engine/platforms/constants.py:63-67) and
implements none of them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..platforms.constants import DistributedStrategy


@dataclass
class ParallelLayout:
    strategy: DistributedStrategy
    tp_size: int
    pp_size: int
    dp_size: int
    tp_rank: int
    pp_rank: int
    dp_rank: int
    tp_group: Optional[dist.ProcessGroup]
    pp_group: Optional[dist.ProcessGroup]
    dp_group: Optional[dist.ProcessGroup]


def _sizes(strategy: DistributedStrategy, world: int, tp_size: Optional[int], pp_size: Optional[int]):
    if strategy == DistributedStrategy.DATA_PARALLEL:
        tp, pp = 1, 1
    elif strategy == DistributedStrategy.MODEL_PARALLEL:
        tp, pp = world, 1
    elif strategy == DistributedStrategy.PIPELINE_PARALLEL:
        tp, pp = 1, world
    else:
        tp = tp_size if tp_size is not None else min(8, world)
        pp = pp_size if pp_size is not None else 1
    if tp < 1 or pp < 1 or world % (tp * pp):
        raise ValueError(f"{world} ranks do not split into tp={tp} x pp={pp} x dp")
    if tp not in (1, 2, 4, 8):
        raise ValueError("the tensor-parallel size must be 1, 2, 4 or 8 (eight canonical slices)")
    return tp, pp, world // (tp * pp)


def make_layout(strategy, tp_size: Optional[int] = None, pp_size: Optional[int] = None) -> ParallelLayout:
    """Create the process groups of ``strategy`` (collective: every rank of the default group
    must call it with the same arguments)."""
    strategy = strategy if isinstance(strategy, DistributedStrategy) else DistributedStrategy(str(strategy).lower())
    if not (dist.is_available() and dist.is_initialized()):
        return ParallelLayout(strategy, 1, 1, 1, 0, 0, 0, None, None, None)      # a single process
    world, rank = dist.get_world_size(), dist.get_rank()
    tp, pp, dp = _sizes(strategy, world, tp_size, pp_size)
    tp_rank, pp_rank, dp_rank = rank % tp, (rank // tp) % pp, rank // (tp * pp)

    def groups(members_of):
        """new_group must be called by every rank for every group, in one order."""
        mine = None
        seen = []
        for r in range(world):
            members = members_of(r)
            if members in seen:
                continue
            seen.append(members)
            g = dist.new_group(members) if len(members) > 1 else None
            if rank in members:
                mine = g
        return mine

    tp_group = groups(lambda r: [r - r % tp + i for i in range(tp)])
    pp_group = groups(lambda r: [(r // (tp * pp)) * tp * pp + r % tp + i * tp for i in range(pp)])
    dp_group = groups(lambda r: [r % (tp * pp) + i * tp * pp for i in range(dp)])
    return ParallelLayout(strategy, tp, pp, dp, tp_rank, pp_rank, dp_rank, tp_group, pp_group, dp_group)


def build_model(cfg, layout: ParallelLayout, seed: int = 0, device=None):
    """The model object of this rank: a :class:`LlamaModel` over the tensor-parallel group, or,
    with pipeline stages, the :class:`PipelineStage` of this rank (its layers sharded over the
    tensor-parallel group when there is one: tp x pp x dp)."""
    from ..models.llama import LlamaModel
    from .tp_gemm import TPContext

    if layout.pp_size > 1:
        from .pipeline import PipelineStage

        tp = TPContext(group=layout.tp_group, device=device) if layout.tp_size > 1 else None
        return PipelineStage(cfg, layout.pp_rank, layout.pp_size, seed=seed, device=device, group=layout.pp_group, tp=tp)
    if layout.tp_size > 1:
        tp = TPContext(group=layout.tp_group, device=device)
    else:
        tp = TPContext.__new__(TPContext)
        dev = torch.device(device) if device is not None else \
            (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        tp.group, tp.rank, tp.world, tp.device, tp._arenas = None, 0, 1, dev, {}
    return LlamaModel(cfg, tp=tp, seed=seed, device=device)
