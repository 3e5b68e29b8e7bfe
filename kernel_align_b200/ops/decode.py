"""Single-token attention against a KV cache (rollout phase) and the fused AdamW update.

Kernels: ``csrc/sm100/decode_optim.cu``. CPU tensors fall back to the equivalent PyTorch math.
"""
from __future__ import annotations

import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .. import _native
from ..utils.profiler import profiled


@profiled("attention_decode")
def attention_decode(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, lens: torch.Tensor,
                     scale: float | None = None) -> torch.Tensor:
    """q ``[B, Hq, D]``; caches ``[B, max_len, Hkv, D]``; ``lens [B]`` int32 = keys to attend to."""
    b, hq, d = q.shape
    max_len, hkv = cache_k.shape[1], cache_k.shape[2]
    sc = float(scale) if scale is not None else 1.0 / math.sqrt(d)
    if q.device.type != "cuda":
        out = torch.empty_like(q)
        g = hq // hkv
        for i in range(b):
            n = int(lens[i])
            k = cache_k[i, :n].float().repeat_interleave(g, 1)  # [n, hq, d]
            v = cache_v[i, :n].float().repeat_interleave(g, 1)
            s = torch.einsum("hd,nhd->hn", q[i].float(), k) * sc
            out[i] = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), v).to(q.dtype)
        return out
    out = torch.empty_like(q)
    fn = _native.cuda().ka_attention_decode
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    rc = fn(q.contiguous().data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(), lens.to(torch.int32).contiguous().data_ptr(),
            out.data_ptr(), b, hq, hkv, d, max_len, sc, torch.cuda.current_stream(q.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"ka_attention_decode failed ({rc})")
    return out


@profiled("decode_qkv_rope_cache")
def decode_qkv_rope_cache(qkv: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, cos: torch.Tensor,
                          sin: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, hq: int,
                          hkv: int) -> torch.Tensor:
    """The step between the fused qkv projection and attention of a decode step, in one launch:
    ``qkv [B, (hq + 2 hkv) * D]`` is split, q and k are rotated at ``pos [B]`` (int64), k and v
    are written into cache row ``slot [1]`` (int64) of ``cache_k / cache_v [B, T, hkv, D]``.
    Returns the rotated ``q [B, hq, D]``. Position and slot are device tensors, so a CUDA graph
    can replay the launch. The same bits as ``rope_`` followed by ``index_copy_``."""
    b = qkv.shape[0]
    d = cache_k.shape[-1]
    if qkv.device.type != "cuda" or d != 128:
        from .layer_ops import rope_

        q = qkv[:, : hq * d].reshape(b, hq, d).contiguous()
        k = qkv[:, hq * d:(hq + hkv) * d].reshape(b, hkv, d).contiguous()
        v = qkv[:, (hq + hkv) * d:].reshape(b, 1, hkv, d)
        rope_(q, pos, cos, sin)
        rope_(k, pos, cos, sin)
        cache_k.index_copy_(1, slot, k.view(b, 1, hkv, d))
        cache_v.index_copy_(1, slot, v)
        return q
    if qkv.stride(1) != 1 or not cache_k.is_contiguous() or not cache_v.is_contiguous():
        raise ValueError("decode_qkv_rope_cache takes a row-major qkv and contiguous caches")
    q = torch.empty(b, hq, d, dtype=qkv.dtype, device=qkv.device)
    fn = _native.cuda().ka_decode_qkv_rope_cache
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                   c_int, c_int, c_int, c_void_p]
    rc = fn(qkv.data_ptr(), qkv.stride(0), pos.data_ptr(), slot.data_ptr(), cos.data_ptr(), sin.data_ptr(),
            q.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(), b, hq, hkv, cache_k.shape[1],
            torch.cuda.current_stream(qkv.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"ka_decode_qkv_rope_cache failed ({rc})")
    return q


class FusedAdamW:
    """AdamW over bf16 parameters with fp32 master weights and moments, one fused kernel per
    parameter tensor. Gradients may be fp32 (the deterministic all-reduce buckets) or bf16."""

    def __init__(self, params, lr: float = 1e-6, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0):
        self.params = [p for p in params if p.requires_grad]
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.step_count = 0
        self.state = [{"master": p.detach().float().clone(), "m": torch.zeros_like(p, dtype=torch.float32),
                       "v": torch.zeros_like(p, dtype=torch.float32)} for p in self.params]

    def zero_grad(self, set_to_none: bool = False) -> None:
        for p in self.params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        b1, b2 = self.betas
        for p, st in zip(self.params, self.state):
            if p.grad is None:
                continue
            g = p.grad.contiguous()
            if p.device.type != "cuda":
                gf = g.float() * grad_scale
                st["m"].mul_(b1).add_(gf, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(gf, gf, value=1 - b2)
                mh = st["m"] / (1 - b1 ** self.step_count)
                vh = st["v"] / (1 - b2 ** self.step_count)
                st["master"].mul_(1 - self.lr * self.weight_decay).addcdiv_(mh, vh.sqrt() + self.eps, value=-self.lr)
                p.copy_(st["master"].to(p.dtype))
                continue
            fn = _native.cuda().ka_adamw_step
            fn.restype = c_int
            fn.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_float, c_float, c_float,
                           c_float, c_float, c_int, c_float, c_int, c_void_p]
            sms = torch.cuda.get_device_properties(p.device).multi_processor_count
            rc = fn(p.data_ptr(), st["master"].data_ptr(), g.data_ptr(), int(g.dtype == torch.bfloat16),
                    st["m"].data_ptr(), st["v"].data_ptr(), p.numel(), self.lr, b1, b2, self.eps, self.weight_decay,
                    self.step_count, grad_scale, sms, torch.cuda.current_stream(p.device).cuda_stream)
            if rc != 0:
                raise RuntimeError(f"ka_adamw_step failed ({rc})")

    def state_dict(self) -> dict:
        return {"step": self.step_count, "lr": self.lr, "betas": self.betas, "eps": self.eps,
                "weight_decay": self.weight_decay,
                "state": [{k: v.clone() for k, v in st.items()} for st in self.state]}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = sd["step"]
        self.lr, self.betas, self.eps, self.weight_decay = sd["lr"], tuple(sd["betas"]), sd["eps"], sd["weight_decay"]
        for st, src in zip(self.state, sd["state"]):
            for k in st:
                st[k].copy_(src[k])
