"""Vocabulary of the engine: string enums grouped under one ``constants`` namespace.

The twelve enum classes and their member values are those of the reference's
``rl_engine/platforms/constants.py:6-97``, so that configuration written against it keeps
working. Here they are generated from one table (``_VOCABULARY``): a member is written either
as its value (the member name is the upper-cased value) or as ``NAME=value``. On this build
only ``DeviceType.CUDA`` / ``CPU`` and ``BackendLib.NATIVE`` are ever selected at run time
(one sm_100a code path and a C++ CPU path, no multi-vendor dispatch); several of the enums
drive real behaviour: ``ProfilingMode`` (``utils.profiler``), ``DistributedStrategy``
(``parallel.strategy``), ``SamplingMethod`` (``SamplerBackend.sample_with``), ``PrecisionType``
(``DeviceContext.dtype_of``), ``CheckpointFormat.PT`` (``utils.checkpoint``).
"""
from __future__ import annotations

from enum import Enum


class _StrEnum(str, Enum):
    def __str__(self) -> str:  # "cuda", not "DeviceType.CUDA"
        return str(self.value)


_VOCABULARY = {
    "DeviceType": "cuda rocm npu tpu xpu cpu",
    "BackendLib": "flashinfer aiter triton cann native",
    "PrecisionType": "FP32=float32 FP16=float16 BF16=bfloat16 int8 int4",
    "SamplingMethod": "top_k top_p top_k_top_p greedy temperature nucleus",
    "MemoryFormat": "contiguous channels_last preserve",
    "OperatorFusionLevel": "none partial full",
    "KernelOptimizationLevel": "default aggressive custom",
    "LoggingLevel": "debug info warning error critical",
    "ProfilingMode": "off basic detailed custom",
    "DistributedStrategy": "data_parallel model_parallel pipeline_parallel hybrid",
    "CheckpointFormat": "pt onnx torchscript custom",
    "ActivationFunction": "relu gelu silu tanh sigmoid",
}


def _build(name: str, spec: str) -> type:
    members = {}
    for item in spec.split():
        key, _, value = item.rpartition("=")
        members[(key or value).upper()] = value
    cls = _StrEnum(name, members, module=__name__)
    cls.__doc__ = f"{name}: " + ", ".join(members.values())
    return cls


DeviceType = _build("DeviceType", _VOCABULARY["DeviceType"])
BackendLib = _build("BackendLib", _VOCABULARY["BackendLib"])
PrecisionType = _build("PrecisionType", _VOCABULARY["PrecisionType"])
SamplingMethod = _build("SamplingMethod", _VOCABULARY["SamplingMethod"])
MemoryFormat = _build("MemoryFormat", _VOCABULARY["MemoryFormat"])
OperatorFusionLevel = _build("OperatorFusionLevel", _VOCABULARY["OperatorFusionLevel"])
KernelOptimizationLevel = _build("KernelOptimizationLevel", _VOCABULARY["KernelOptimizationLevel"])
LoggingLevel = _build("LoggingLevel", _VOCABULARY["LoggingLevel"])
ProfilingMode = _build("ProfilingMode", _VOCABULARY["ProfilingMode"])
DistributedStrategy = _build("DistributedStrategy", _VOCABULARY["DistributedStrategy"])
CheckpointFormat = _build("CheckpointFormat", _VOCABULARY["CheckpointFormat"])
ActivationFunction = _build("ActivationFunction", _VOCABULARY["ActivationFunction"])


class Constants:
    """Namespace object: ``constants.DeviceType.CUDA`` and so on."""


for _name in _VOCABULARY:
    setattr(Constants, _name, globals()[_name])

constants = Constants()
