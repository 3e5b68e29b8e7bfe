"""``RolloutExecutor``: operator selection and the rollout (generation) phase.

Keeps the reference's entry point (rl_engine/executors/rollout.py:8-35):
``RolloutExecutor(model_config)``, ``execute_rollout()`` returning
``{"status": "success", "kernels": [logp_op, attention_op]}``. When a policy model is
attached, ``execute_rollout`` actually generates: it decodes ``max_new_tokens`` tokens per
prompt with the fused sampler and returns the sequences and their log-probabilities.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..kernels.registry import kernel_registry
from ..utils.logger import logger


class RolloutExecutor:
    def __init__(self, model_config: Optional[dict] = None, model=None, sampler=None):
        self.config = dict(model_config or {})
        self.model = model
        self.sampler = sampler
        logger.info("Initializing high-performance RolloutExecutor...")

    def _select_operators(self) -> Tuple[str, str]:
        logp_be = kernel_registry.dispatch("fused_logp")
        attn_be = kernel_registry.dispatch("attention")
        logger.info_once(f"Selected Logp backend: {logp_be}")
        logger.info_once(f"Selected Attention backend: {attn_be}")
        return logp_be, attn_be

    def execute_rollout(self, prompts: Optional[torch.Tensor] = None, **gen_kwargs) -> dict:
        """Without a model: report the operators a rollout would use (the reference's
        behaviour). With a model and ``prompts`` ``[B, P]``: run the generation loop."""
        logp_op, attn_op = self._select_operators()
        result = {"status": "success", "kernels": [logp_op, attn_op]}
        if self.model is None or prompts is None:
            logger.info_once(f"Starting rollout via {logp_op}...")
            return result
        from .generation import generate

        cfg = {**self.config, **gen_kwargs}
        out = generate(self.model, prompts, sampler=self.sampler,
                       max_new_tokens=int(cfg.get("max_new_tokens", 16)),
                       temperature=float(cfg.get("temperature", 1.0)),
                       top_k=cfg.get("top_k"), top_p=cfg.get("top_p"),
                       group_size=int(cfg.get("group_size", 1)))
        result.update(out)
        return result
