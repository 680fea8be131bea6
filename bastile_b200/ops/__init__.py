"""Kernel-backed ops; importing this package registers the Qwen3 patches
(src/bastile/ops/__init__.py:11-18)."""

from . import fused_linear_cross_entropy, rms_norm, rope, swiglu

__all__ = ["fused_linear_cross_entropy", "rms_norm", "rope", "swiglu"]
