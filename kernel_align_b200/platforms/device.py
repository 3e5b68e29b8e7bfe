"""Device context: what this process runs on and where it sits in the job.

Same role and attribute names as the reference's ``rl_engine/platforms/device.py:8-44``
(``device``, ``is_rocm``, ``backend_version``, ``device_type``, ``get_preferred_dtype``) with
the pieces a multi-GPU B200 job needs on top: compute capability, SM count, HBM size, and
the distributed ``rank`` / ``world_size`` / ``local_rank`` (read live, so they are right
both before and after ``torch.distributed`` is initialised). The preferred dtype on Blackwell
is bf16: tcgen05 runs bf16 and fp16 at the same rate and bf16 needs no loss scaling.
"""
from __future__ import annotations

import os

import torch

from ..utils.logger import current_rank, logger
from .constants import DeviceType


class DeviceContext:
    def __init__(self) -> None:
        self.is_rocm = False  # single sm_100a code path: kept for API compatibility
        self.backend_version = "N/A"
        self.capability: tuple[int, int] | None = None
        self.sm_count = 0
        self.total_memory = 0
        self.name = "cpu"
        if torch.cuda.is_available():
            self.local_rank = int(os.environ.get("LOCAL_RANK", "0")) % max(1, torch.cuda.device_count())
            self.device = torch.device(DeviceType.CUDA.value, self.local_rank)
            self.device_type = DeviceType.CUDA.value
            self.backend_version = torch.version.cuda or "N/A"
            props = torch.cuda.get_device_properties(self.device)
            self.capability = (props.major, props.minor)
            self.sm_count = props.multi_processor_count
            self.total_memory = props.total_memory
            self.name = props.name
            logger.info_once(
                f"RL-Engine on {self.name} (sm_{props.major}{props.minor}, {self.sm_count} SMs, "
                f"{self.total_memory / 2**30:.0f} GiB, CUDA {self.backend_version})"
            )
            if self.capability[0] != 10:
                logger.warn_once(
                    "the CUDA kernels of this build are compiled for sm_100a only; "
                    f"this device is sm_{props.major}{props.minor}"
                )
        else:
            self.local_rank = 0
            self.device = torch.device(DeviceType.CPU.value)
            self.device_type = DeviceType.CPU.value
            logger.warn_once("No GPU detected. RL-Engine is running its C++ CPU path.")

    # Distributed coordinates are properties so that they track torch.distributed's state.
    @property
    def rank(self) -> int:
        return current_rank()

    @property
    def world_size(self) -> int:
        try:
            import torch.distributed as dist

            if dist.is_available() and dist.is_initialized():
                return dist.get_world_size()
        except Exception:
            pass
        return int(os.environ.get("WORLD_SIZE", "1"))

    @property
    def is_blackwell(self) -> bool:
        return self.capability is not None and self.capability[0] == 10

    @staticmethod
    def dtype_of(precision) -> torch.dtype:
        """The torch dtype of a ``PrecisionType`` value (fp32 / fp16 / bf16 / int8); ``int4`` has
        no torch dtype and is rejected."""
        from .constants import PrecisionType

        p = precision if isinstance(precision, PrecisionType) else PrecisionType(str(precision).lower())
        table = {PrecisionType.FP32: torch.float32, PrecisionType.FP16: torch.float16,
                 PrecisionType.BF16: torch.bfloat16, PrecisionType.INT8: torch.int8}
        if p not in table:
            raise ValueError(f"no tensor dtype for precision {p.value}")
        return table[p]

    def get_preferred_dtype(self) -> torch.dtype:
        """bf16 on a GPU, fp32 on the CPU path."""
        return torch.bfloat16 if self.device.type == "cuda" else torch.float32


device_ctx = DeviceContext()
