"""Batch-invariant bf16 GEMM on tcgen05 (``csrc/sm100/gemm.cu``).

``gemm_bi(a, b)`` computes ``a @ b.T`` for ``a [M, K]`` and ``b [N, K]`` (the layout of a
``torch.nn.Linear`` weight). ``trans_a`` / ``trans_b`` select the other storage orders so the
backward GEMMs need no transpose pass:

    y  = gemm_bi(x, w)                                  # [M, K] x [N, K]^T
    dx = gemm_bi(dy, w, trans_b=True)                   # dy [M, N] times w stored as [N(=K'), K(=N')]
    dw = gemm_bi(dy, x, trans_a=True, trans_b=True)     # dy^T x, both stored token-major

A row of the result depends only on that row of ``a`` (fixed tiles, fixed K order, no split-K),
so the output is bitwise identical for any batch size. ``Linear`` is the autograd wrapper.

Decode-sized products (``M <= 64``, plain layouts, bf16 output) go to the weight-streaming
kernel of ``csrc/sm100/gemm_skinny.cu`` (operands swapped, one accumulation chain over K in the
same order), which gives the same bits; ``KA_GEMM_SKINNY=0`` keeps everything on the tiled kernel.
"""
from __future__ import annotations

import os
from ctypes import c_int, c_longlong, c_ulonglong, c_void_p

from typing import Optional

import torch

from .. import _native
from .fused_logp import default_timeout_ns
from ..utils.profiler import profiled

_status: dict[int, torch.Tensor] = {}


def status_buffer(device: torch.device) -> torch.Tensor:
    """Per-device int32[8] block the GEMM kernels report bounded-wait failures into."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(8, dtype=torch.int32, device=device)
    return _status[idx]


def check_status(device: torch.device) -> None:
    st = status_buffer(device).cpu().tolist()
    if st[0] != 0:
        status_buffer(device).zero_()
        raise RuntimeError(f"gemm kernel gave up: code {st[0]} at site {st[1]}, block {st[2]}, aux {st[3:6]}")


def _fn():
    lib = _native.cuda()
    fn = lib.ka_gemm_bf16
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_int, c_int,
                   c_int, c_void_p, c_int, c_ulonglong, c_void_p]
    return fn


SKINNY_MAX_ROWS = 64


def _skinny_fn():
    fn = _native.cuda().ka_gemm_skinny_bf16
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p,
                   c_ulonglong, c_void_p]
    return fn


@profiled("gemm_skinny")
def _check_out(out: torch.Tensor, m: int, n: int, dtype: torch.dtype) -> None:
    if out.shape != (m, n) or out.dtype != dtype or out.stride(1) != 1 or out.stride(0) % 8 != 0 or \
            out.data_ptr() % 16 != 0:
        raise ValueError(f"out must be a [{m}, {n}] {dtype} view with unit column stride, a row stride that is a "
                         "multiple of 8 and a 16-byte aligned start")


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M <= 64, K] @ w[N, K].T`` on the weight-streaming kernel (bf16 in, bf16 out).
    ``out``: write into this ``[M, N]`` view (rows may be strided, e.g. a column block)."""
    m, k = a.shape
    n = w.shape[0]
    if m > SKINNY_MAX_ROWS or w.shape[1] != k:
        raise ValueError("gemm_skinny takes at most 64 rows and matching inner dimensions")
    a = a if a.stride(-1) == 1 else a.contiguous()
    w = w if w.stride(-1) == 1 else w.contiguous()
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    else:
        _check_out(out, m, n, torch.bfloat16)
    rc = _skinny_fn()(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), m, n, k,
                      status_buffer(a.device).data_ptr(), default_timeout_ns(),
                      torch.cuda.current_stream(a.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"ka_gemm_skinny_bf16 rejected its arguments (code {rc})")
    return out


@profiled("gemm_bi")
def gemm_bi(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
            out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``op(a) @ op(b).T`` with ``op(a) = a.T if trans_a`` (a stored ``[K, M]``) and
    ``op(b) = b.T if trans_b`` (b stored ``[K, N]``). 2-D bf16 inputs, row-major. ``out`` (CUDA):
    write the result into this view instead of a new tensor (rows may be strided)."""
    if a.device.type != "cuda":
        # the C++ library's GEMM: every dot product in one fixed order, so a row's result does not
        # depend on the batch here either (a BLAS call may block differently for different M)
        from . import cpu_ops

        af = a.float().t() if trans_a else a.float()
        bf = b.float().t() if trans_b else b.float()
        res = cpu_ops.gemm_cpu(af.contiguous(), bf.contiguous()).to(out_dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm_bi takes bf16 operands")
    a = a if a.stride(-1) == 1 else a.contiguous()
    b = b if b.stride(-1) == 1 else b.contiguous()
    k, m = (a.shape[0], a.shape[1]) if trans_a else (a.shape[1], a.shape[0])
    kb, n = (b.shape[0], b.shape[1]) if trans_b else (b.shape[1], b.shape[0])
    if k != kb:
        raise ValueError(f"inner dimensions differ: {k} vs {kb}")
    if (0 < m <= SKINNY_MAX_ROWS and not trans_a and not trans_b and out_dtype == torch.bfloat16
            and os.environ.get("KA_GEMM_SKINNY", "1") != "0"):
        return gemm_skinny(a, b, out=out)
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype, device=a.device)
    else:
        _check_out(out, m, n, out_dtype)
    props = torch.cuda.get_device_properties(a.device)
    rc = _fn()(a.data_ptr(), a.stride(0), int(trans_a), b.data_ptr(), b.stride(0), int(trans_b), out.data_ptr(),
               out.stride(0), int(out_dtype == torch.float32), m, n, k, status_buffer(a.device).data_ptr(),
               props.multi_processor_count, default_timeout_ns(), torch.cuda.current_stream(a.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"ka_gemm_bf16 rejected its arguments (code {rc})")
    return out


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return gemm_bi(x.reshape(-1, x.shape[-1]), w).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = gemm_bi(dy2, w, trans_b=True).reshape(x.shape) if ctx.needs_input_grad[0] else None
        dw = gemm_bi(dy2, x2, trans_a=True, trans_b=True) if ctx.needs_input_grad[1] else None
        return dx, dw


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` with autograd through the same kernel."""
    return _LinearFn.apply(x, w)
