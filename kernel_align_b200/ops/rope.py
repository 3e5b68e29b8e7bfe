"""Rotary embedding entry points (see :mod:`kernel_align_b200.ops.layer_ops`)."""
from .layer_ops import rope_, rope_tables  # noqa: F401

rope = rope_
