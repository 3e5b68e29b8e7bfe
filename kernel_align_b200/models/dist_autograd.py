"""Small differentiable collectives used around the model (plumbing over torch.distributed)."""
from __future__ import annotations

import torch
import torch.distributed as dist


class _AllGatherRows(torch.autograd.Function):
    """Concatenate every rank's rows. The consumers downstream (vocabulary-parallel log-prob)
    hand back the *complete* gradient on every rank, so backward just takes this rank's rows."""

    @staticmethod
    def forward(ctx, x_local, tp):
        ctx.rank, ctx.rows = tp.rank, x_local.shape[0]
        if x_local.device.type != "cuda":
            pieces = [torch.empty_like(x_local) for _ in range(tp.world)]
            dist.all_gather(pieces, x_local.contiguous(), group=tp.group)
            return torch.cat(pieces)
        out = torch.empty(tp.world * x_local.shape[0], *x_local.shape[1:], dtype=x_local.dtype, device=x_local.device)
        dist.all_gather_into_tensor(out, x_local.contiguous(), group=tp.group)
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad[ctx.rank * ctx.rows:(ctx.rank + 1) * ctx.rows].contiguous(), None


def all_gather_rows(x_local: torch.Tensor, tp) -> torch.Tensor:
    return _AllGatherRows.apply(x_local, tp)
