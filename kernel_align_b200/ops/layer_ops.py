"""RMSNorm (with fused residual add), rotary embedding and SwiGLU.

CUDA: ``csrc/sm100/elementwise.cu`` (bf16 in/out, fp32 math, fixed-order reductions, one pass).
CPU: ``csrc/cpu/layer_ops_cpu.cpp`` with the same rounding points. The reference only names
these ops (README feature list, ``ActivationFunction.SILU`` in
rl_engine/platforms/constants.py:75-80).
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .. import _native
from ..utils.profiler import profiled


def _sms(t: torch.Tensor) -> int:
    return torch.cuda.get_device_properties(t.device).multi_processor_count


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _check(rc: int, name: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} failed ({rc})")


@profiled("rmsnorm")
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, residual: Optional[torch.Tensor] = None):
    """``y = rmsnorm(x + residual) * weight``. With ``residual`` returns ``(y, x + residual)``."""
    d = x.shape[-1]
    x2 = x.reshape(-1, d)
    rows = x2.shape[0]
    if x.device.type != "cuda":
        lib = _native.cpu()
        xf = x2.float().contiguous()
        rf = residual.reshape(-1, d).float().contiguous() if residual is not None else None
        wf = weight.float().contiguous()
        y = torch.empty_like(xf)
        ro = torch.empty_like(xf) if residual is not None else None
        fn = lib.ka_cpu_rmsnorm
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float]
        _check(fn(xf.data_ptr(), rf.data_ptr() if rf is not None else None, wf.data_ptr(), y.data_ptr(),
                  ro.data_ptr() if ro is not None else None, rows, d, float(eps)), "ka_cpu_rmsnorm")
        y = y.to(x.dtype).reshape(x.shape)
        return (y, ro.to(x.dtype).reshape(x.shape)) if residual is not None else y
    if x.dtype != torch.bfloat16:
        raise TypeError("the sm_100a rmsnorm takes bf16")
    x2 = x2.contiguous()
    r2 = residual.reshape(-1, d).contiguous() if residual is not None else None
    y = torch.empty_like(x2)
    ro = torch.empty_like(x2) if residual is not None else None
    lib = _native.cuda()
    fn = lib.ka_rmsnorm
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]
    _check(fn(x2.data_ptr(), r2.data_ptr() if r2 is not None else None, weight.contiguous().data_ptr(), y.data_ptr(),
              ro.data_ptr() if ro is not None else None, rows, d, float(eps), _sms(x), _stream(x)), "ka_rmsnorm")
    y = y.reshape(x.shape)
    return (y, ro.reshape(x.shape)) if residual is not None else y


def rope_tables(max_pos: int, head_dim: int, theta: float = 500000.0, device="cpu"):
    """``cos``/``sin`` tables ``[max_pos, head_dim/2]`` fp32, computed in float64 on the host so
    that every device sees the same values."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


@profiled("rope")
def rope_(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate ``x`` ``[tokens, heads, head_dim]`` in place ("rotate half" convention)."""
    tokens, heads, hd = x.shape
    pos = positions.reshape(-1).to(torch.int64).contiguous()
    if x.device.type != "cuda":
        lib = _native.cpu()
        xf = x.float().contiguous()
        fn = lib.ka_cpu_rope
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]
        _check(fn(xf.data_ptr(), pos.data_ptr(), cos.contiguous().data_ptr(), sin.contiguous().data_ptr(), tokens,
                  heads, hd), "ka_cpu_rope")
        x.copy_(xf.to(x.dtype))
        return x
    if x.dtype != torch.bfloat16 or x.stride(2) != 1 or x.stride(1) != hd:
        raise ValueError("rope_ takes bf16 [tokens, heads, head_dim] with contiguous heads")
    lib = _native.cuda()
    fn = lib.ka_rope
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    _check(fn(x.data_ptr(), x.stride(0), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), tokens, heads, hd, _sms(x),
              _stream(x)), "ka_rope")
    return x


@profiled("swiglu")
def swiglu(gate_up: torch.Tensor, up: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gate) * up``. Either one ``[..., 2F]`` tensor holding ``[gate | up]`` or two ``[..., F]``."""
    if up is None:
        f = gate_up.shape[-1] // 2
        g2 = gate_up.reshape(-1, 2 * f)
        gate_v, up_v, stride = g2[:, :f], g2[:, f:], 2 * f
        lead = gate_up.shape[:-1]
    else:
        f = gate_up.shape[-1]
        gate_v, up_v, stride = gate_up.reshape(-1, f).contiguous(), up.reshape(-1, f).contiguous(), f
        lead = gate_up.shape[:-1]
    rows = gate_v.shape[0]
    if gate_up.device.type != "cuda":
        lib = _native.cpu()
        gf, uf = gate_v.float().contiguous(), up_v.float().contiguous()
        out = torch.empty_like(gf)
        fn = lib.ka_cpu_swiglu
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong]
        _check(fn(gf.data_ptr(), uf.data_ptr(), out.data_ptr(), gf.numel()), "ka_cpu_swiglu")
        return out.to(gate_up.dtype).reshape(*lead, f)
    if gate_up.dtype != torch.bfloat16:
        raise TypeError("the sm_100a swiglu takes bf16")
    if up is None and not gate_up.is_contiguous():
        return swiglu(gate_up.contiguous())
    out = torch.empty(rows, f, dtype=torch.bfloat16, device=gate_up.device)
    lib = _native.cuda()
    fn = lib.ka_swiglu
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p]
    _check(fn(gate_v.data_ptr(), up_v.data_ptr(), stride, out.data_ptr(), rows, f, _sms(out), _stream(out)),
           "ka_swiglu")
    return out.reshape(*lead, f)


# --------------------------------------------------------------------------------------------
# Differentiable wrappers: on CUDA forward and backward both run the hand-written kernels; on
# CPU the forward is the C++ library and the backward the same formulas in PyTorch fp32.
# --------------------------------------------------------------------------------------------
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        ctx.save_for_backward(x, weight)
        ctx.eps = eps
        return rmsnorm(x, weight, eps)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        d = x.shape[-1]
        x2 = x.reshape(-1, d).contiguous()
        dy2 = dy.reshape(-1, d).contiguous()
        rows = x2.shape[0]
        if x.device.type != "cuda":
            xf, gf, wf = x2.float(), dy2.float(), weight.float()
            r = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + ctx.eps)
            gw = gf * wf
            dx = r * gw - xf * (r.pow(3) * (gw * xf).mean(-1, keepdim=True))
            dw = (gf * xf * r).sum(0)
            return dx.to(x.dtype).reshape(x.shape), dw.to(weight.dtype), None
        dx = torch.empty_like(x2)
        dw = torch.empty_like(weight)
        chunk = int(_native.cuda().ka_rmsnorm_bwd_chunk())
        part = torch.empty((rows + chunk - 1) // chunk, d, dtype=torch.float32, device=x.device)
        fn = _native.cuda().ka_rmsnorm_bwd
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]
        _check(fn(x2.data_ptr(), weight.contiguous().data_ptr(), dy2.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                  part.data_ptr(), rows, d, float(ctx.eps), _stream(x)), "ka_rmsnorm_bwd")
        return dx.reshape(x.shape), dw, None


def rmsnorm_fn(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """Differentiable RMSNorm (no fused residual; add the residual with ``+`` before it)."""
    if not (x.requires_grad or weight.requires_grad) or not torch.is_grad_enabled():
        return rmsnorm(x, weight, eps)
    return _RMSNormFn.apply(x, weight, eps)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, cos, sin):
        ctx.save_for_backward(positions, cos, sin)
        return rope_(x.clone(memory_format=torch.contiguous_format), positions, cos, sin)

    @staticmethod
    def backward(ctx, dy):
        positions, cos, sin = ctx.saved_tensors
        # the transpose of a rotation is the rotation by the opposite angle
        return rope_(dy.contiguous().clone(), positions, cos, -sin), None, None, None


def rope_fn(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Out-of-place, differentiable rotary embedding of ``x`` ``[tokens, heads, head_dim]``."""
    return _RopeFn.apply(x, positions, cos, sin)


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        ctx.save_for_backward(gate_up)
        return swiglu(gate_up)

    @staticmethod
    def backward(ctx, d_out):
        (gate_up,) = ctx.saved_tensors
        f = gate_up.shape[-1] // 2
        gu = gate_up.reshape(-1, 2 * f)
        d2 = d_out.reshape(-1, f).contiguous()
        rows = gu.shape[0]
        if gate_up.device.type != "cuda":
            g, u, d = gu[:, :f].float(), gu[:, f:].float(), d2.float()
            sg = torch.sigmoid(g)
            grad = torch.cat([d * u * sg * (1 + g * (1 - sg)), d * g * sg], 1)
            return grad.to(gate_up.dtype).reshape(gate_up.shape)
        grad = torch.empty_like(gu)
        fn = _native.cuda().ka_swiglu_bwd
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int,
                       c_void_p]
        _check(fn(gu.data_ptr(), gu.data_ptr() + 2 * f, 2 * f, d2.data_ptr(), grad.data_ptr(),
                  grad.data_ptr() + 2 * f, 2 * f, rows, f, _sms(gu), _stream(gu)), "ka_swiglu_bwd")
        return grad.reshape(gate_up.shape)


def swiglu_fn(gate_up: torch.Tensor) -> torch.Tensor:
    """Differentiable SwiGLU on a contiguous ``[..., 2F]`` tensor holding ``[gate | up]``."""
    if not gate_up.requires_grad or not torch.is_grad_enabled():
        return swiglu(gate_up)
    return _SwigluFn.apply(gate_up.contiguous())
