"""Differentiable tensor-parallel linear layers on the fused compute+collective kernels.

Activations between blocks are sequence-sharded (each rank holds ``rows_per_rank`` token rows):

    column_parallel_linear:  y[M, N/world]   = all_gather(x_local) @ W_shard^T     (AG -> GEMM)
    row_parallel_linear:     y_local[M/world, N] = reduce_scatter(x @ W_shard^T)   (GEMM -> RS)

Their backward passes are the mirrored fused kernels (the gradient of an all-gather is a
reduce-scatter and vice versa), so forward and backward both overlap NVLink traffic with the
MMAs and both use the fixed 8-slice reduction order. With one rank the same kernels run on
local buffers.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import gemm
from .tp_gemm import TPContext, all_gather_gemm, gemm_reduce_scatter


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, w, tp: TPContext):
        if tp.world == 1:
            y, x_full = gemm.gemm_bi(x_local, w), x_local
        else:
            y, x_full = all_gather_gemm(x_local, w, tp, return_gathered=True)
        ctx.save_for_backward(x_full, w)
        ctx.tp = tp
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # [M, N_local] x [N_local, K] summed over the ranks' N shards, rows scattered back
            dx = gemm_reduce_scatter(dy, w, tp, trans_b=True, keep_padding=True)
        if ctx.needs_input_grad[1]:
            dw = gemm.gemm_bi(dy, x_full, trans_a=True, trans_b=True)
        return dx, dw, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual, tp: TPContext):
        y = gemm_reduce_scatter(x, w, tp, residual=residual, keep_padding=True)
        ctx.save_for_backward(x, w)
        ctx.tp = tp
        ctx.has_residual = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy_local):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        dy_local = dy_local.contiguous()
        dx = dw = None
        if tp.world == 1:
            dy_full = dy_local
            if ctx.needs_input_grad[0]:
                dx = gemm.gemm_bi(dy_full, w, trans_b=True)
        else:
            dx, dy_full = all_gather_gemm(dy_local, w, tp, trans_b=True, return_gathered=True)
        if ctx.needs_input_grad[1]:
            dw = gemm.gemm_bi(dy_full[: x.shape[0]], x, trans_a=True, trans_b=True)
        dres = dy_local if ctx.has_residual and ctx.needs_input_grad[2] else None
        return (dx[: x.shape[0]] if dx is not None else None), dw, dres, None


def column_parallel_linear(x_local: torch.Tensor, w_shard: torch.Tensor, tp: TPContext) -> torch.Tensor:
    """``all_gather(x_local) @ w_shard.T``: ``[rows_per_rank, K] -> [world * rows_per_rank, N_local]``."""
    return _ColumnParallelFn.apply(x_local, w_shard, tp)


def row_parallel_linear(x: torch.Tensor, w_shard: torch.Tensor, tp: TPContext,
                        residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """This rank's rows of ``sum_ranks x_r @ w_r.T`` (+ residual): ``[M, K_local] -> [rows_per_rank, N]``."""
    return _RowParallelFn.apply(x, w_shard, residual, tp)
