"""Vocabulary of the engine: string enums grouped under one ``constants`` namespace.

The twelve enum classes and their values match the reference's
``rl_engine/platforms/constants.py:6-97`` so that configuration written against it keeps
working. On this build only ``DeviceType.CUDA`` / ``CPU`` and ``BackendLib.NATIVE`` are ever
selected at run time: there is one sm_100a code path and a C++ CPU path, no multi-vendor
dispatch. The names of the other members are kept as accepted spellings.
"""
from __future__ import annotations

from enum import Enum


class _StrEnum(str, Enum):
    def __str__(self) -> str:  # "cuda", not "DeviceType.CUDA"
        return str(self.value)


class DeviceType(_StrEnum):
    CUDA = "cuda"
    ROCM = "rocm"
    NPU = "npu"
    TPU = "tpu"
    XPU = "xpu"
    CPU = "cpu"


class BackendLib(_StrEnum):
    FLASHINFER = "flashinfer"
    AITER = "aiter"
    TRITON = "triton"
    CANN = "cann"
    NATIVE = "native"


class PrecisionType(_StrEnum):
    FP32 = "float32"
    FP16 = "float16"
    BF16 = "bfloat16"
    INT8 = "int8"
    INT4 = "int4"


class SamplingMethod(_StrEnum):
    TOP_K = "top_k"
    TOP_P = "top_p"
    TOP_K_TOP_P = "top_k_top_p"
    GREEDY = "greedy"
    TEMPERATURE = "temperature"
    NUCLEUS = "nucleus"


class MemoryFormat(_StrEnum):
    CONTIGUOUS = "contiguous"
    CHANNELS_LAST = "channels_last"
    PRESERVE = "preserve"


class OperatorFusionLevel(_StrEnum):
    NONE = "none"
    PARTIAL = "partial"
    FULL = "full"


class KernelOptimizationLevel(_StrEnum):
    DEFAULT = "default"
    AGGRESSIVE = "aggressive"
    CUSTOM = "custom"


class LoggingLevel(_StrEnum):
    DEBUG = "debug"
    INFO = "info"
    WARNING = "warning"
    ERROR = "error"
    CRITICAL = "critical"


class ProfilingMode(_StrEnum):
    OFF = "off"
    BASIC = "basic"
    DETAILED = "detailed"
    CUSTOM = "custom"


class DistributedStrategy(_StrEnum):
    DATA_PARALLEL = "data_parallel"
    MODEL_PARALLEL = "model_parallel"
    PIPELINE_PARALLEL = "pipeline_parallel"
    HYBRID = "hybrid"


class CheckpointFormat(_StrEnum):
    PT = "pt"
    ONNX = "onnx"
    TORCHSCRIPT = "torchscript"
    CUSTOM = "custom"


class ActivationFunction(_StrEnum):
    RELU = "relu"
    GELU = "gelu"
    SILU = "silu"
    TANH = "tanh"
    SIGMOID = "sigmoid"


class Constants:
    """Namespace object: ``constants.DeviceType.CUDA`` and so on."""

    DeviceType = DeviceType
    BackendLib = BackendLib
    PrecisionType = PrecisionType
    SamplingMethod = SamplingMethod
    MemoryFormat = MemoryFormat
    OperatorFusionLevel = OperatorFusionLevel
    KernelOptimizationLevel = KernelOptimizationLevel
    LoggingLevel = LoggingLevel
    ProfilingMode = ProfilingMode
    DistributedStrategy = DistributedStrategy
    CheckpointFormat = CheckpointFormat
    ActivationFunction = ActivationFunction


constants = Constants()
