"""``SamplerBackend``: the reference's sampling / log-prob module on the native operators.

API of ``rl_engine/kernels/sampling.py:9-112`` (``sample(logits, top_k, top_p, temperature,
deterministic)``, ``compute_logp(logits, token_ids)``) with its defects removed: the
temperature is applied once, ``top_p`` is honoured on every path, ``compute_logp`` accepts
2-D and 3-D logits and never builds a ``log_softmax`` temporary, CPU tensors run the C++ CPU
path instead of failing. On top of that, ``fused_logp(hidden, lm_head_weight, token_ids)``
computes the same log-probabilities straight from hidden states without materialising the
logits at all.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..ops import fused_logp as _fused
from ..ops import logits_logp as _ll
from ..ops import sampling as _sampling
from ..platforms.constants import constants
from ..utils.logger import logger


class SamplerBackend(nn.Module):
    def __init__(self, seed: int = 0):
        super().__init__()
        self.backend = constants.BackendLib.NATIVE.value
        self.seed = int(seed)
        self.step = 0
        logger.info_once("SamplerBackend: native sm_100a kernels (C++ CPU path for CPU tensors)")

    def manual_seed(self, seed: int, step: int = 0) -> "SamplerBackend":
        """Re-key the random stream; (seed, step) fully determine later draws."""
        self.seed, self.step = int(seed), int(step)
        return self

    def rng_state(self) -> dict:
        return {"seed": self.seed, "step": self.step}

    def set_rng_state(self, state: dict) -> None:
        self.seed, self.step = int(state["seed"]), int(state["step"])

    @torch.inference_mode()
    def sample(self, logits, top_k: Optional[int] = None, top_p: Optional[float] = None,
               temperature: float = 1.0, deterministic: bool = True, *, row_ids=None,
               step: Optional[int] = None) -> torch.Tensor:
        """One token id (int32) per row of ``logits`` ``[B, V]``.

        Every draw is reproducible, so ``deterministic`` is accepted and ignored. Each call
        consumes one step of the stream unless ``step`` is given explicitly.
        """
        if logits.dim() == 1:
            logits = logits.unsqueeze(0)
        use_step = self.step if step is None else int(step)
        out = _sampling.sample(logits, top_k=top_k, top_p=top_p, temperature=temperature,
                               seed=self.seed, step=use_step, row_ids=row_ids)
        if step is None:
            self.step += 1
        return out

    @torch.inference_mode()
    def sample_with(self, method, logits, *, top_k: int = 50, top_p: float = 0.9, temperature: float = 1.0,
                    **kw) -> torch.Tensor:
        """``sample`` selected by a ``SamplingMethod`` value (``constants.SamplingMethod``):
        ``greedy`` takes the arg-max, ``temperature`` draws from the full distribution,
        ``top_k`` / ``top_p`` (= ``nucleus``) / ``top_k_top_p`` apply the named filters."""
        from ..platforms.constants import SamplingMethod

        m = method if isinstance(method, SamplingMethod) else SamplingMethod(str(method).lower())
        if m == SamplingMethod.GREEDY:
            return self.sample(logits, top_k=1, temperature=temperature, **kw)
        if m == SamplingMethod.TEMPERATURE:
            return self.sample(logits, temperature=temperature, **kw)
        if m == SamplingMethod.TOP_K:
            return self.sample(logits, top_k=top_k, temperature=temperature, **kw)
        if m in (SamplingMethod.TOP_P, SamplingMethod.NUCLEUS):
            return self.sample(logits, top_p=top_p, temperature=temperature, **kw)
        return self.sample(logits, top_k=top_k, top_p=top_p, temperature=temperature, **kw)

    def compute_logp(self, logits, token_ids, temperature: float = 1.0) -> torch.Tensor:
        """Log-probability of ``token_ids`` under ``softmax(logits / temperature)``.

        logits ``[G, L, V]`` or ``[N, V]``; returns fp32 ``[G, L]`` (``[N]`` for 2-D input).
        """
        return _ll.logits_logp(logits, token_ids, scale=1.0 / float(temperature))

    @torch.inference_mode()
    def fused_logp(self, hidden, lm_head_weight, token_ids, temperature: float = 1.0, **kw) -> torch.Tensor:
        """Same quantity from hidden states ``[..., K]`` and the LM-head weight ``[V, K]``."""
        return _fused.lmhead_logp(hidden, lm_head_weight, token_ids, scale=1.0 / float(temperature), **kw)
