"""RMSNorm entry point (see :mod:`kernel_align_b200.ops.layer_ops`)."""
from .layer_ops import rmsnorm  # noqa: F401
