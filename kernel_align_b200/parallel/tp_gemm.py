"""Tensor-parallel linear layers whose collective runs inside the GEMM kernel.

``gemm_reduce_scatter(x, w_shard, ctx)``: row-parallel linear (``x [M, K/world]``,
``w_shard [N, K/world]``) -> this rank's rows ``[M/world, N]`` of ``x_full @ w_full.T`` (+ residual).
``all_gather_gemm(x_local, w_shard, ctx)``: column-parallel linear on row-sharded input
(``x_local [M/world, K]``, ``w_shard [N/world, K]``) -> ``[M, N/world]``.

Kernels: ``csrc/sm100/tp_gemm.cu`` / ``gemm.cu``; peer buffers: :class:`PeerArena`. With
``world == 1`` the same kernels run on local buffers, which is what makes TP=1 and TP=8 agree
bit for bit: K is always reduced as 8 canonical slices in one fixed tree order.

CPU tensors take a PyTorch path with the same arithmetic contract (8 canonical K slices, each
partial rounded to bf16, the fixed tree, residual added after rounding), exchanging over the
process group's CPU backend (gloo): it is what the multi-process CPU tests run, and it is
invariant in the number of ranks for the same reason the kernels are.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_size_t, c_uint, c_ulonglong, c_void_p
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native
from ..ops.fused_logp import default_timeout_ns
from ..ops.gemm import status_buffer
from ..utils.profiler import profiled


class _LocalArena:
    """Stand-in for :class:`PeerArena` when there is a single rank."""

    def __init__(self, nbytes: int, device):
        self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.ptrs = [self.buf.data_ptr()]
        self.rank, self.world = 0, 1


class TPContext:
    """Process-group handle plus the exchange buffers of the fused TP kernels (allocated on
    first use per shape, then reused; each buffer carries its own call counter)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, device=None):
        if dist.is_available() and dist.is_initialized():
            self.group = group if group is not None else dist.group.WORLD
            self.rank = dist.get_rank(self.group)
            self.world = dist.get_world_size(self.group)
        else:
            self.group, self.rank, self.world = None, 0, 1
        if device is not None:
            self.device = torch.device(device)
        elif torch.cuda.is_available():
            self.device = torch.device("cuda", torch.cuda.current_device())
        else:
            self.device = torch.device("cpu")
        self._arenas: dict = {}

    def arena(self, key, nbytes: int):
        ent = self._arenas.get(key)
        if ent is None:
            if self.world == 1:
                ar = _LocalArena(nbytes, self.device)
            else:
                from .peer import PeerArena

                ar = PeerArena(nbytes, self.group, self.device)
            ent = [ar, 0]
            self._arenas[key] = ent
        ent[1] += 1
        return ent[0], ent[1]


def _lib():
    lib = _native.cuda()
    lib.ka_gemm_rs_exchange_bytes.restype = c_size_t
    lib.ka_gemm_rs_exchange_bytes.argtypes = [c_int, c_int, c_int]
    lib.ka_gemm_rs_rows_per_rank.restype = c_int
    lib.ka_gemm_rs_rows_per_rank.argtypes = [c_int, c_int]
    lib.ka_ag_gemm_exchange_bytes.restype = c_size_t
    lib.ka_ag_gemm_exchange_bytes.argtypes = [c_int, c_int, c_int]
    lib.ka_gemm_reduce_scatter.restype = c_int
    lib.ka_gemm_reduce_scatter.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p,
                                           c_void_p, c_int, c_int, c_int, c_int, c_int, c_uint, c_void_p, c_int,
                                           c_ulonglong, c_void_p]
    lib.ka_all_gather_gemm.restype = c_int
    lib.ka_all_gather_gemm.argtypes = [c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_void_p, c_int,
                                       c_int, c_int, c_int, c_int, c_uint, c_void_p, c_int, c_ulonglong, c_void_p]
    return lib


def _tree8(p: torch.Tensor) -> torch.Tensor:
    """``p [8, ...]`` fp32 -> ((0+1)+(2+3))+((4+5)+(6+7))."""
    return ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]))


def _gemm_reduce_scatter_cpu(x, w_shard, ctx, residual, trans_b, keep_padding):
    m, k_local = x.shape
    wf = w_shard.float().t() if trans_b else w_shard.float()          # [N, K_local]
    n = wf.shape[0]
    s_local = 8 // ctx.world
    ks = k_local // s_local
    xf = x.float()
    from ..ops import cpu_ops

    parts = torch.stack([cpu_ops.gemm_cpu(xf[:, i * ks:(i + 1) * ks].contiguous(),
                                          wf[:, i * ks:(i + 1) * ks].contiguous()).to(torch.bfloat16).float()
                         for i in range(s_local)])                       # this rank's slices, rounded
    if ctx.world > 1:
        gathered = [torch.empty_like(parts) for _ in range(ctx.world)]
        dist.all_gather(gathered, parts.contiguous(), group=ctx.group)
        parts = torch.cat(gathered)
    v = _tree8(parts)
    rpr = rows_per_rank(m, ctx.world)
    lo = ctx.rank * rpr
    rows_valid = max(0, min(rpr, m - lo))
    out = torch.zeros(rpr, n, dtype=torch.float32)
    out[:rows_valid] = v[lo:lo + rows_valid]
    if residual is not None:
        res = residual.float()
        if res.shape[0] < rpr:
            res = torch.cat([res, res.new_zeros(rpr - res.shape[0], n)])
        out = out.to(torch.bfloat16).float() + res[:rpr]
    out = out.to(torch.bfloat16)
    return out if keep_padding else out[:rows_valid]


@profiled("gemm_reduce_scatter")
def gemm_reduce_scatter(x: torch.Tensor, w_shard: torch.Tensor, ctx: TPContext,
                        residual: Optional[torch.Tensor] = None, trans_b: bool = False,
                        keep_padding: bool = False) -> torch.Tensor:
    """Rows ``[rank * M/world, (rank + 1) * M/world)`` of ``concat_k(x) @ concat_k(w).T`` (+ residual).

    ``w_shard`` is ``[N, K_local]``, or ``[K_local, N]`` with ``trans_b``. ``keep_padding`` returns
    all ``rows_per_rank`` rows (a multiple of 128) instead of cutting at the end of the matrix."""
    m, k_local = x.shape
    n = w_shard.shape[1] if trans_b else w_shard.shape[0]
    if k_local % (8 // ctx.world * 64) != 0:
        raise ValueError("the K shard must split into whole 64-wide blocks per canonical slice")
    if x.device.type != "cuda":
        return _gemm_reduce_scatter_cpu(x, w_shard, ctx, residual, trans_b, keep_padding)
    lib = _lib()
    x = x.contiguous()
    w = w_shard.contiguous()
    rpr = rows_per_rank(m, ctx.world)
    nbytes = lib.ka_gemm_rs_exchange_bytes(m, n, ctx.world)
    arena, epoch = ctx.arena(("rs", m, n), nbytes)
    rows_valid = max(0, min(rpr, m - ctx.rank * rpr))
    out = torch.empty(rpr, n, dtype=torch.bfloat16, device=x.device)
    res = None
    if residual is not None:
        res = residual.contiguous()
        if res.shape[0] < rpr:
            res = torch.cat([res, res.new_zeros(rpr - res.shape[0], n)])
    ptrs = (c_void_p * ctx.world)(*arena.ptrs)
    props = torch.cuda.get_device_properties(x.device)
    rc = lib.ka_gemm_reduce_scatter(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), int(trans_b), out.data_ptr(),
                                    res.data_ptr() if res is not None else None, ptrs, m, n, k_local, ctx.world,
                                    ctx.rank, epoch & 0xFFFFFFFF, status_buffer(x.device).data_ptr(),
                                    props.multi_processor_count, default_timeout_ns(),
                                    torch.cuda.current_stream(x.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"ka_gemm_reduce_scatter rejected its arguments (code {rc})")
    return out if keep_padding else out[:rows_valid]


def rows_per_rank(m: int, world: int) -> int:
    """Rows of a reduce-scattered ``[m, n]`` result that each rank owns (multiple of 128; the
    same rule as ``ka_gemm_rs_rows_per_rank``)."""
    per = (m + world - 1) // world
    return (per + 127) // 128 * 128


@profiled("all_gather_gemm")
def all_gather_gemm(x_local: torch.Tensor, w_shard: torch.Tensor, ctx: TPContext, trans_b: bool = False,
                    return_gathered: bool = False):
    """``all_gather(x_local, dim=0) @ w_shard.T``; ``x_local`` rows must be a multiple of 128.

    ``w_shard`` is ``[N_local, K]``, or ``[K, N_local]`` with ``trans_b``. With ``return_gathered``
    also returns a copy of the gathered activations ``[world * rows, K]``."""
    rows, k = x_local.shape
    n_local = w_shard.shape[1] if trans_b else w_shard.shape[0]
    if rows % 128 != 0:
        raise ValueError("rows per rank must be a multiple of 128")
    if x_local.device.type != "cuda":
        from ..ops.gemm import gemm_bi

        if ctx.world > 1:
            pieces = [torch.empty_like(x_local) for _ in range(ctx.world)]
            dist.all_gather(pieces, x_local.contiguous(), group=ctx.group)
            x_full = torch.cat(pieces)
        else:
            x_full = x_local
        out = gemm_bi(x_full, w_shard, trans_b=trans_b)
        return (out, x_full.clone()) if return_gathered else out
    lib = _lib()
    x = x_local.contiguous()
    w = w_shard.contiguous()
    nbytes = lib.ka_ag_gemm_exchange_bytes(rows, k, ctx.world)
    arena, epoch = ctx.arena(("ag", rows, k), nbytes)
    out = torch.empty(ctx.world * rows, n_local, dtype=torch.bfloat16, device=x.device)
    ptrs = (c_void_p * ctx.world)(*arena.ptrs)
    props = torch.cuda.get_device_properties(x.device)
    rc = lib.ka_all_gather_gemm(x.data_ptr(), w.data_ptr(), w.stride(0), int(trans_b), out.data_ptr(), out.stride(0), ptrs, rows,
                                n_local, k, ctx.world, ctx.rank, epoch & 0xFFFFFFFF,
                                status_buffer(x.device).data_ptr(), props.multi_processor_count,
                                default_timeout_ns(), torch.cuda.current_stream(x.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"ka_all_gather_gemm rejected its arguments (code {rc})")
    if return_gathered:
        nb = (ctx.world * rows * k * 2 + 255) // 256 * 256
        gen = epoch & 1
        gathered = arena.buf[gen * nb: gen * nb + ctx.world * rows * k * 2].view(torch.bfloat16).view(ctx.world * rows, k)
        return out, gathered.clone()
    return out
