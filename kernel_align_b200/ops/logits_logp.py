"""Per-token log-probability from materialised logits (``log_softmax(...).gather(...)``).

One streaming pass, no ``[rows, vocab]`` temporary: the CUDA kernel is
``csrc/sm100/logits_logp.cu``, the CPU path ``csrc/cpu/fused_logp_cpu.cpp``. This is the
operation behind the reference's ``SamplerBackend.compute_logp``
(rl_engine/kernels/sampling.py:91-112).
"""
from __future__ import annotations

import torch

from .. import _native
from ..utils.profiler import profiled


@profiled("logits_logp")
def logits_logp(logits: torch.Tensor, ids: torch.Tensor, *, scale: float = 1.0, return_lse: bool = False):
    """logits ``[..., V]`` (fp32 / bf16 / fp16), ids ``[...]`` -> fp32 ``[...]``.

    Ids outside ``[0, V)`` give 0. ``scale`` multiplies the logits (1 / temperature).
    """
    lead = logits.shape[:-1]
    v = logits.shape[-1]
    x = logits.reshape(-1, v)
    if ids.numel() != x.shape[0]:
        raise ValueError("ids must have one entry per row of logits")
    if x.device.type != "cuda":
        from . import cpu_ops

        res = cpu_ops.logits_logp_cpu(x, ids.reshape(-1), scale=scale, return_lse=return_lse)
        if return_lse:
            return res[0].reshape(lead), res[1].reshape(lead)
        return res.reshape(lead)
    if x.stride(-1) != 1:
        x = x.contiguous()
    rows = x.shape[0]
    ids64 = ids.reshape(-1).to(torch.int64).contiguous()
    logp = torch.empty(rows, dtype=torch.float32, device=x.device)
    lse = torch.empty(rows, dtype=torch.float32, device=x.device) if return_lse else None
    props = torch.cuda.get_device_properties(x.device)
    rc = _native.cuda().ka_logits_logp(
        x.data_ptr(), _native.dtype_code(x.dtype), x.stride(0), rows, v, ids64.data_ptr(), float(scale),
        logp.data_ptr(), lse.data_ptr() if lse is not None else None, props.multi_processor_count,
        torch.cuda.current_stream(x.device).cuda_stream,
    )
    if rc != 0:
        raise RuntimeError(f"ka_logits_logp failed ({rc})")
    if return_lse:
        return logp.reshape(lead), lse.reshape(lead)
    return logp.reshape(lead)
