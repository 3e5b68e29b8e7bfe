"""Operator registry: op-type strings to the native operator that serves them.

Keeps the reference's surface (``rl_engine/kernels/registry.py:20-61``): an ``OpBackend``
enum whose failed lookups raise ``ValueError`` listing the valid names,
``KernelRegistry.dispatch(op_type) -> str`` and ``get_op_path(backend)``, and the
``kernel_registry`` singleton. The difference is that every entry here resolves to code that
exists: ``resolve()`` imports the dotted path and returns the callable. The five names of
the reference (``FLASH_ATTN``, ``FLASHINFER``, ...) are accepted as aliases of the native
operators, so ``dispatch("fused_logp")`` still answers ``"FLASHINFER"``-style callers through
``dispatch_legacy``.
"""
from __future__ import annotations

import importlib
from enum import Enum, EnumMeta
from typing import Callable, Dict

from ..platforms.device import device_ctx
from ..utils.logger import logger


class _LookupMeta(EnumMeta):
    def __getitem__(cls, name: str):
        try:
            return super().__getitem__(name)
        except KeyError:
            valid = ", ".join(cls.__members__)
            raise ValueError(f"Operator '{name}' not found. Supported backends: {valid}") from None


class OpBackend(Enum, metaclass=_LookupMeta):
    # sm_100a operators (dotted path of the Python entry point)
    SM100_FUSED_LOGP = "kernel_align_b200.ops.fused_logp.lmhead_logp"
    SM100_LOGITS_LOGP = "kernel_align_b200.ops.logits_logp.logits_logp"
    SM100_SAMPLING = "kernel_align_b200.ops.sampling.sample"
    SM100_ATTENTION = "kernel_align_b200.ops.attention.attention"
    SM100_GEMM = "kernel_align_b200.ops.gemm.gemm_bi"
    SM100_RMSNORM = "kernel_align_b200.ops.layer_ops.rmsnorm"
    SM100_ROPE = "kernel_align_b200.ops.layer_ops.rope_"
    SM100_SWIGLU = "kernel_align_b200.ops.layer_ops.swiglu"
    SM100_GRPO_LOSS = "kernel_align_b200.ops.grpo_loss.grpo_loss"
    SM100_ALLREDUCE = "kernel_align_b200.parallel.collectives.all_reduce_det"
    SM100_GEMM_RS = "kernel_align_b200.parallel.tp_gemm.gemm_reduce_scatter"
    SM100_AG_GEMM = "kernel_align_b200.parallel.tp_gemm.all_gather_gemm"
    SM100_ATTENTION_BWD = "kernel_align_b200.ops.attention.attention_backward"
    SM100_ATTENTION_DECODE = "kernel_align_b200.ops.decode.attention_decode"
    SM100_GEMM_SKINNY = "kernel_align_b200.ops.gemm.gemm_skinny"
    SM100_ADVANTAGES = "kernel_align_b200.ops.grpo_loss.group_advantages"
    # names the reference exposes: enum aliases of the native operators above (same value),
    # so OpBackend["FLASHINFER"] is OpBackend.SM100_FUSED_LOGP
    FLASH_ATTN = "kernel_align_b200.ops.attention.attention"
    FLASHINFER = "kernel_align_b200.ops.fused_logp.lmhead_logp"
    ROCM_AITER = "kernel_align_b200.ops.fused_logp.lmhead_logp"
    ROCM_CK = "kernel_align_b200.ops.attention.attention"
    TRITON_GENERIC = "kernel_align_b200.ops.gemm.gemm_bi"


# op_type keyword -> operator, first match wins (order matters: "logits_logp" before "logp")
_ROUTES: list[tuple[str, OpBackend]] = [
    ("logits_logp", OpBackend.SM100_LOGITS_LOGP),
    ("logp", OpBackend.SM100_FUSED_LOGP),
    ("sampl", OpBackend.SM100_SAMPLING),
    ("reduce_scatter", OpBackend.SM100_GEMM_RS),
    ("gemm_rs", OpBackend.SM100_GEMM_RS),
    ("all_gather", OpBackend.SM100_AG_GEMM),
    ("ag_gemm", OpBackend.SM100_AG_GEMM),
    ("all_reduce", OpBackend.SM100_ALLREDUCE),
    ("allreduce", OpBackend.SM100_ALLREDUCE),
    ("attention_backward", OpBackend.SM100_ATTENTION_BWD),
    ("attention_bwd", OpBackend.SM100_ATTENTION_BWD),
    ("decode_attention", OpBackend.SM100_ATTENTION_DECODE),
    ("attention_decode", OpBackend.SM100_ATTENTION_DECODE),
    ("skinny", OpBackend.SM100_GEMM_SKINNY),
    ("advantage", OpBackend.SM100_ADVANTAGES),
    ("rmsnorm", OpBackend.SM100_RMSNORM),
    ("norm", OpBackend.SM100_RMSNORM),
    ("rope", OpBackend.SM100_ROPE),
    ("swiglu", OpBackend.SM100_SWIGLU),
    ("ffn", OpBackend.SM100_SWIGLU),
    ("loss", OpBackend.SM100_GRPO_LOSS),
    ("gemm", OpBackend.SM100_GEMM),
    ("linear", OpBackend.SM100_GEMM),
    ("matmul", OpBackend.SM100_GEMM),
    ("attention", OpBackend.SM100_ATTENTION),
    ("attn", OpBackend.SM100_ATTENTION),
]


class KernelRegistry:
    """Routes an op-type string to the operator that implements it on this build."""

    def __init__(self) -> None:
        self._runtime_overrides: Dict[OpBackend, str] = {}
        logger.info(f"KernelRegistry initialized for {device_ctx.device_type}")

    def dispatch(self, op_type: str) -> str:
        """Name of the operator serving ``op_type``; unknown types go to attention, as in the
        reference where everything that is not a log-prob op is an attention op."""
        key = op_type.lower()
        for needle, backend in _ROUTES:
            if needle in key:
                return backend.name
        return OpBackend.SM100_ATTENTION.name

    def dispatch_legacy(self, op_type: str) -> str:
        """The reference's two-way answer (``FLASHINFER`` for log-prob ops, ``FLASH_ATTN``
        otherwise), for callers that compare against those strings."""
        return "FLASHINFER" if "logp" in op_type else "FLASH_ATTN"

    def override(self, backend: OpBackend, dotted_path: str) -> None:
        """Route ``backend`` to another callable for the rest of the process."""
        self._runtime_overrides[backend] = dotted_path

    def get_op_path(self, backend: OpBackend) -> str:
        return self._runtime_overrides.get(backend, backend.value)

    def resolve(self, backend: "OpBackend | str") -> Callable:
        """Import and return the callable behind a backend (or its name)."""
        if isinstance(backend, str):
            backend = OpBackend[backend]
        module, _, attr = self.get_op_path(backend).rpartition(".")
        return getattr(importlib.import_module(module), attr)


kernel_registry = KernelRegistry()
