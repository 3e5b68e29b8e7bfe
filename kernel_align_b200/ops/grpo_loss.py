"""GRPO objective: group-normalised advantages and the clipped-ratio policy loss.

CUDA: ``csrc/sm100/grpo_loss.cu`` (fixed-order reductions, bitwise reproducible loss);
CPU: ``csrc/cpu/grpo_loss_cpu.cpp``. ``grpo_loss`` is differentiable with respect to
``logp_new``. The reference lists the GRPO loss in its README but ships no implementation.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from .. import _native
from ..utils.profiler import profiled


def group_advantages(rewards: torch.Tensor, group_size: int, eps: float = 1e-4) -> torch.Tensor:
    """``(r - mean_group) / (std_group + eps)`` over consecutive groups of ``group_size``
    rewards (unbiased standard deviation)."""
    r = rewards.reshape(-1).float().contiguous()
    if r.numel() % group_size:
        raise ValueError("the number of rewards must be a multiple of the group size")
    adv = torch.empty_like(r)
    n_groups = r.numel() // group_size
    if r.device.type == "cuda":
        fn = _native.cuda().ka_grpo_advantages
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_int, c_int, c_float, c_void_p]
        rc = fn(r.data_ptr(), adv.data_ptr(), n_groups, group_size, eps, torch.cuda.current_stream(r.device).cuda_stream)
    else:
        fn = _native.cpu().ka_cpu_grpo_advantages
        fn.restype = c_int
        fn.argtypes = [c_void_p, c_void_p, c_int, c_int, c_float]
        rc = fn(r.data_ptr(), adv.data_ptr(), n_groups, group_size, eps)
    if rc != 0:
        raise RuntimeError(f"grpo advantages failed ({rc})")
    return adv.reshape(rewards.shape)


class _GrpoLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logp_new, logp_old, logp_ref, adv, mask, eps_low, eps_high, beta, seq_mean):
        n_seq, seq_len = logp_new.shape
        ln = logp_new.detach().float().contiguous()
        lo = logp_old.detach().float().contiguous()
        lr = logp_ref.detach().float().contiguous() if logp_ref is not None else None
        a = adv.detach().float().contiguous()
        m = mask.to(torch.uint8).contiguous() if mask is not None else None
        out = torch.empty(3, dtype=torch.float32, device=ln.device)
        if ln.device.type == "cuda":
            raw = torch.empty_like(ln)
            ws = torch.empty(4 * n_seq, dtype=torch.float32, device=ln.device)
            fn = _native.cuda().ka_grpo_loss_fwd
            fn.restype = c_int
            fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float,
                           c_int, c_void_p, c_void_p, c_void_p, c_void_p]
            rc = fn(ln.data_ptr(), lo.data_ptr(), lr.data_ptr() if lr is not None else None, a.data_ptr(),
                    m.data_ptr() if m is not None else None, n_seq, seq_len, eps_low, eps_high, beta, int(seq_mean),
                    raw.data_ptr(), ws.data_ptr(), out.data_ptr(), torch.cuda.current_stream(ln.device).cuda_stream)
            if rc != 0:
                raise RuntimeError(f"ka_grpo_loss_fwd failed ({rc})")
            ctx.save_for_backward(raw, ws)
            ctx.cuda = True
        else:
            grad = torch.empty_like(ln)
            fn = _native.cpu().ka_cpu_grpo_loss
            fn.restype = c_int
            fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float,
                           c_int, c_void_p, c_void_p]
            rc = fn(ln.data_ptr(), lo.data_ptr(), lr.data_ptr() if lr is not None else None, a.data_ptr(),
                    m.data_ptr() if m is not None else None, n_seq, seq_len, eps_low, eps_high, beta, int(seq_mean),
                    grad.data_ptr(), out.data_ptr())
            if rc != 0:
                raise RuntimeError(f"ka_cpu_grpo_loss failed ({rc})")
            ctx.save_for_backward(grad)
            ctx.cuda = False
        ctx.shape = (n_seq, seq_len)
        ctx.mark_non_differentiable(out)
        return out[0].clone(), out

    @staticmethod
    def backward(ctx, g_loss, _g_stats):
        n_seq, seq_len = ctx.shape
        if ctx.cuda:
            raw, ws = ctx.saved_tensors
            grad = torch.empty_like(raw)
            up = g_loss.detach().float().reshape(1).contiguous()
            fn = _native.cuda().ka_grpo_loss_bwd
            fn.restype = c_int
            fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
            rc = fn(raw.data_ptr(), ws[3 * n_seq:].data_ptr(), up.data_ptr(), grad.data_ptr(), n_seq, seq_len,
                    torch.cuda.current_stream(raw.device).cuda_stream)
            if rc != 0:
                raise RuntimeError(f"ka_grpo_loss_bwd failed ({rc})")
        else:
            (g,) = ctx.saved_tensors
            grad = g * g_loss
        return grad, None, None, None, None, None, None, None, None


@profiled("grpo_loss")
def grpo_loss(logp_new: torch.Tensor, logp_old: torch.Tensor, advantages: torch.Tensor, *,
              mask: Optional[torch.Tensor] = None, logp_ref: Optional[torch.Tensor] = None, eps_low: float = 0.2,
              eps_high: Optional[float] = None, beta: float = 0.0, reduction: str = "token_mean",
              return_stats: bool = False):
    """Clipped-ratio GRPO loss. ``logp_*`` ``[G, L]`` fp32, ``advantages`` ``[G]``, ``mask`` ``[G, L]``.

    ``reduction``: ``"token_mean"`` (mean over all valid tokens) or ``"seq_mean"`` (mean over
    sequences of their token means). With ``return_stats`` also returns a tensor
    ``[loss, clip_fraction, valid_tokens]``.
    """
    if reduction not in ("token_mean", "seq_mean"):
        raise ValueError("reduction must be 'token_mean' or 'seq_mean'")
    hi = eps_low if eps_high is None else eps_high
    loss, stats = _GrpoLossFn.apply(logp_new, logp_old, logp_ref, advantages, mask, float(eps_low), float(hi),
                                    float(beta), reduction == "seq_mean")
    return (loss, stats) if return_stats else loss
