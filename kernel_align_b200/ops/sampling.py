"""Fused temperature / top-k / top-p sampling with a counter-based random stream.

``sample(logits, ...)`` draws one token per row in a single kernel launch
(``csrc/sm100/sampling.cu``; CPU: ``csrc/cpu/sampling_cpu.cpp``). The random number of a row
is Philox4x32-10 keyed by ``(seed, row id, step)``: sampling the same row under the same key
returns the same token whatever the batch it is part of, on GPU and on CPU alike.

Replaces the reference's FlashInfer route (rl_engine/kernels/sampling.py:47-75), with the
temperature applied once and ``top_p`` honoured on every path.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from ..utils.profiler import profiled


@profiled("sample")
def sample(
    logits: torch.Tensor,
    *,
    top_k: Optional[int] = None,
    top_p: Optional[float] = None,
    temperature: float = 1.0,
    seed: int = 0,
    step: int = 0,
    row_ids: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """logits ``[B, V]`` (fp32 / bf16 / fp16) -> int32 ``[B]`` token ids.

    ``temperature == 0`` or ``top_k == 1`` is greedy decoding. ``row_ids`` (int64 ``[B]``)
    names the rows for the random stream; it defaults to ``arange(B)``.
    """
    if logits.dim() != 2:
        raise ValueError("logits must be [batch, vocab]")
    b, v = logits.shape
    k = 0 if top_k is None else int(top_k)
    if top_k is not None and k < 1:
        raise ValueError("top_k must be >= 1")
    p = 1.0 if top_p is None else float(top_p)
    if not (0.0 < p <= 1.0):
        raise ValueError("top_p must be in (0, 1]")
    if temperature < 0:
        raise ValueError("temperature must be >= 0")
    if temperature == 0:
        k, p, inv_t = 1, 1.0, 1.0
    else:
        inv_t = 1.0 / float(temperature)
    if k >= v:
        k = 0
    if logits.device.type != "cuda":
        from . import cpu_ops

        return cpu_ops.sample_cpu(logits, inv_temperature=inv_t, top_k=k, top_p=p, seed=seed, step=step,
                                  row_ids=row_ids)
    x = logits if logits.stride(-1) == 1 else logits.contiguous()
    out = torch.empty(b, dtype=torch.int32, device=x.device)
    rid = None
    if row_ids is not None:
        rid = row_ids.to(device=x.device, dtype=torch.int64).contiguous()
    rc = _native.cuda().ka_sample(
        x.data_ptr(), _native.dtype_code(x.dtype), x.stride(0), b, v,
        rid.data_ptr() if rid is not None else None, inv_t, k, p,
        int(seed) & (2**64 - 1), int(step) & (2**64 - 1), out.data_ptr(),
        torch.cuda.current_stream(x.device).cuda_stream,
    )
    if rc != 0:
        raise RuntimeError(f"ka_sample failed ({rc})")
    return out
