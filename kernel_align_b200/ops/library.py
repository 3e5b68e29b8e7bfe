"""The operators as ``torch.library`` custom ops: ``torch.ops.kernel_align_b200.*``.

Importing this module registers forward-only ops with fake (meta) implementations, so the
kernels can appear in exported or compiled inference graphs without a graph break and with
correct shapes and dtypes under fake tensors:

    import kernel_align_b200.ops.library
    logp = torch.ops.kernel_align_b200.lmhead_logp(hidden, weight, ids, 1.0)
    tok = torch.ops.kernel_align_b200.sample(logits, 50, 0.9, 0.7, seed, step)

Each op calls the same Python entry point as the rest of the package (CUDA kernels for CUDA
tensors, the C++ library for CPU tensors). They are registered without an autograd formula:
training goes through the ``autograd.Function`` wrappers of the operator modules
(``lmhead_logp``, ``gemm.linear``, ``attention_fn``, ``rmsnorm_fn``, ...).

The reference names its backends by dotted path strings (rl_engine/kernels/registry.py:8-31)
and registers nothing with PyTorch.
"""
from __future__ import annotations

import torch
from torch import Tensor
from torch.library import custom_op

from . import attention as _attention
from . import fused_logp as _fused_logp
from . import gemm as _gemm
from . import layer_ops as _layer_ops
from . import logits_logp as _logits_logp
from . import sampling as _sampling

NS = "kernel_align_b200"


@custom_op(f"{NS}::lmhead_logp", mutates_args=())
def lmhead_logp(hidden: Tensor, weight: Tensor, ids: Tensor, scale: float) -> Tensor:
    with torch.no_grad():
        return _fused_logp.lmhead_logp(hidden, weight, ids, scale=scale)


@lmhead_logp.register_fake
def _(hidden, weight, ids, scale):
    return hidden.new_empty(hidden.shape[:-1], dtype=torch.float32)


@custom_op(f"{NS}::logits_logp", mutates_args=())
def logits_logp(logits: Tensor, ids: Tensor, scale: float) -> Tensor:
    return _logits_logp.logits_logp(logits, ids, scale=scale)


@logits_logp.register_fake
def _(logits, ids, scale):
    return logits.new_empty(logits.shape[:-1], dtype=torch.float32)


@custom_op(f"{NS}::sample", mutates_args=())
def sample(logits: Tensor, top_k: int, top_p: float, temperature: float, seed: int, step: int) -> Tensor:
    """``top_k <= 0`` and ``top_p >= 1`` switch the respective filter off."""
    return _sampling.sample(logits, top_k=top_k if top_k > 0 else None, top_p=top_p if top_p < 1.0 else None,
                            temperature=temperature, seed=seed, step=step)


@sample.register_fake
def _(logits, top_k, top_p, temperature, seed, step):
    return logits.new_empty(logits.shape[0], dtype=torch.int32)


@custom_op(f"{NS}::gemm_bi", mutates_args=())
def gemm_bi(a: Tensor, b: Tensor, trans_a: bool, trans_b: bool) -> Tensor:
    return _gemm.gemm_bi(a, b, trans_a=trans_a, trans_b=trans_b)


@gemm_bi.register_fake
def _(a, b, trans_a, trans_b):
    m = a.shape[1] if trans_a else a.shape[0]
    n = b.shape[1] if trans_b else b.shape[0]
    return a.new_empty(m, n, dtype=torch.bfloat16)


@custom_op(f"{NS}::attention", mutates_args=())
def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool, scale: float) -> Tensor:
    """``scale <= 0`` means ``1 / sqrt(head_dim)``."""
    return _attention.attention(q, k, v, causal=causal, scale=scale if scale > 0 else None)


@attention.register_fake
def _(q, k, v, causal, scale):
    return q.new_empty(q.shape)


@custom_op(f"{NS}::rmsnorm", mutates_args=())
def rmsnorm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    return _layer_ops.rmsnorm(x, weight, eps)


@rmsnorm.register_fake
def _(x, weight, eps):
    return torch.empty_like(x)


@custom_op(f"{NS}::swiglu", mutates_args=())
def swiglu(gate_up: Tensor) -> Tensor:
    return _layer_ops.swiglu(gate_up)


@swiglu.register_fake
def _(gate_up):
    return gate_up.new_empty(*gate_up.shape[:-1], gate_up.shape[-1] // 2)
