"""Batch-invariant attention (causal or full, grouped KV heads, head_dim 128 on CUDA).

CUDA: ``csrc/sm100/attention.cu`` (TMA + tcgen05, fixed 128-wide KV tiles in increasing
order). CPU: ``csrc/cpu/attention_cpu.cpp``. The reference routes the op type "attention" to a
backend name only (rl_engine/kernels/registry.py:41-55).
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

from .. import _native
from .fused_logp import default_timeout_ns
from .gemm import status_buffer
from ..utils.profiler import profiled


@profiled("attention")
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True,
              scale: Optional[float] = None, return_lse: bool = False):
    """q ``[B, L, Hq, D]``, k / v ``[B, L, Hkv, D]`` -> ``[B, L, Hq, D]``.

    Inputs may be strided views of a fused projection as long as heads are contiguous
    (``stride(-1) == 1``, ``stride(-2) == D``) and the batch stride is ``L`` tokens.
    """
    b, l, hq, d = q.shape
    hkv = k.shape[2]
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(d)
    if q.device.type != "cuda":
        lib = _native.cpu()
        qf, kf, vf = (t.float().contiguous() for t in (q, k, v))
        out = torch.empty_like(qf)
        lse = torch.empty(b, hq, l, dtype=torch.float32) if return_lse else None
        fn = lib.ka_cpu_attention
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                       c_int]
        rc = fn(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), out.data_ptr(), lse.data_ptr() if return_lse else None,
                b, l, hq, hkv, d, sc, int(causal))
        if rc != 0:
            raise RuntimeError(f"ka_cpu_attention failed ({rc})")
        out = out.to(q.dtype)
        return (out, lse) if return_lse else out
    if d != 128 or q.dtype != torch.bfloat16:
        raise ValueError("the sm_100a attention kernel takes bf16 with head_dim 128")

    def tok_view(t, heads):
        ok = t.stride(3) == 1 and t.stride(2) == d and t.stride(0) == l * t.stride(1) and t.stride(1) % 8 == 0 \
            and t.data_ptr() % 16 == 0
        return t if ok else t.contiguous()

    q, k, v = tok_view(q, hq), tok_view(k, hkv), tok_view(v, hkv)
    out = torch.empty(b, l, hq, d, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(b, hq, l, dtype=torch.float32, device=q.device) if return_lse else None
    lib = _native.cuda()
    fn = lib.ka_attention_fwd
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_ulonglong, c_void_p]
    rc = fn(q.data_ptr(), q.stride(1), k.data_ptr(), k.stride(1), v.data_ptr(), v.stride(1), out.data_ptr(),
            out.stride(1), lse.data_ptr() if lse is not None else None, b, l, hq, hkv, d, sc, int(causal),
            status_buffer(q.device).data_ptr(), default_timeout_ns(), torch.cuda.current_stream(q.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"ka_attention_fwd rejected its arguments (code {rc})")
    return (out, lse) if return_lse else out


@profiled("attention_backward")
def attention_backward(q, k, v, out, d_out, lse, *, causal: bool = True, scale: Optional[float] = None):
    """``(dq, dk, dv)`` from the saved forward results. CUDA: the tcgen05 kernels of
    ``csrc/sm100/attention_bwd.cu`` (a dQ kernel and a dK/dV kernel, no atomics, fixed
    accumulation order); CPU: fp32 matmul math."""
    b, l, hq, d = q.shape
    hkv = k.shape[2]
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(d)
    if q.device.type != "cuda" or d != 128 or q.dtype != torch.bfloat16:
        return _attention_backward_math(q, k, v, out, d_out, lse, causal, sc)

    def tok(t):
        ok = t.stride(3) == 1 and t.stride(2) == d and t.stride(0) == l * t.stride(1) and t.stride(1) % 8 == 0 \
            and t.data_ptr() % 16 == 0
        return t if ok else t.contiguous()

    q, k, v, out, d_out = tok(q), tok(k), tok(v), tok(out), tok(d_out)
    dq = torch.empty(b, l, hq, d, dtype=torch.bfloat16, device=q.device)
    dk = torch.empty(b, l, hkv, d, dtype=torch.bfloat16, device=q.device)
    dv = torch.empty(b, l, hkv, d, dtype=torch.bfloat16, device=q.device)
    delta = torch.empty(b, hq, l, dtype=torch.float32, device=q.device)
    lse = lse.contiguous()
    fn = _native.cuda().ka_attention_bwd
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p,
                   c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong,
                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_ulonglong, c_void_p]
    rc = fn(q.data_ptr(), q.stride(1), k.data_ptr(), k.stride(1), v.data_ptr(), v.stride(1), out.data_ptr(),
            out.stride(1), d_out.data_ptr(), d_out.stride(1), lse.data_ptr(), delta.data_ptr(), dq.data_ptr(),
            dq.stride(1), dk.data_ptr(), dk.stride(1), dv.data_ptr(), dv.stride(1), b, l, hq, hkv, d, sc, int(causal),
            status_buffer(q.device).data_ptr(), default_timeout_ns(), torch.cuda.current_stream(q.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"ka_attention_bwd rejected its arguments (code {rc})")
    return dq, dk, dv


def _attention_backward_math(q, k, v, out, d_out, lse, causal, scale):
    """fp32 matmul formulation of the attention gradient, one sequence at a time (CPU path and
    test oracle). Deterministic: plain matmuls in a fixed order."""
    b, l, hq, d = q.shape
    hkv = k.shape[2]
    g = hq // hkv
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    mask = torch.ones(l, l, device=q.device, dtype=torch.bool).triu(1) if causal else None
    for bi in range(b):
        qf = q[bi].float().permute(1, 0, 2)                       # [hq, l, d]
        kf = k[bi].float().permute(1, 0, 2)                       # [hkv, l, d]
        vf = v[bi].float().permute(1, 0, 2)
        of = out[bi].float().permute(1, 0, 2)
        dof = d_out[bi].float().permute(1, 0, 2)
        kx = kf.repeat_interleave(g, 0)
        vx = vf.repeat_interleave(g, 0)
        s = torch.matmul(qf, kx.transpose(1, 2)) * scale           # [hq, l, l]
        p = torch.exp(s - lse[bi][:, :, None])
        if mask is not None:
            p = p.masked_fill(mask, 0.0)
        delta = (dof * of).sum(-1, keepdim=True)
        dp = torch.matmul(dof, vx.transpose(1, 2))
        ds = p * (dp - delta) * scale
        dq[bi] = torch.matmul(ds, kx).permute(1, 0, 2).to(q.dtype)
        dkx = torch.matmul(ds.transpose(1, 2), qf)                 # [hq, l, d]
        dvx = torch.matmul(p.transpose(1, 2), dof)
        dk[bi] = dkx.view(hkv, g, l, d).sum(1).permute(1, 0, 2).to(k.dtype)
        dv[bi] = dvx.view(hkv, g, l, d).sum(1).permute(1, 0, 2).to(v.dtype)
    return dq, dk, dv


class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        out, lse = attention(q, k, v, causal=causal, scale=scale, return_lse=True)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = attention_backward(q, k, v, out, d_out.contiguous(), lse, causal=ctx.causal, scale=ctx.scale)
        return dq, dk, dv, None, None


def attention_fn(q, k, v, *, causal: bool = True, scale: Optional[float] = None):
    """Differentiable attention: forward and backward on the tcgen05 kernels."""
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if not torch.is_grad_enabled() or not (q.requires_grad or k.requires_grad or v.requires_grad):
        return attention(q, k, v, causal=causal, scale=sc)
    return _AttentionFn.apply(q, k, v, causal, sc)
